// Cache manager: keys and values in pages, a block table per request and group, and
// slots for per-request state of fixed size.
//
// The reference keeps one token per slot with a GPU slot table [row, position] and CPU
// free lists (rust/engine/src/runner/kv_pool/naive_kvpool.rs:159-198, 334-505); its
// request handle separates reserving from committing, so that a failed step leaves the
// request releasable (rust/engine/src/runner/kv_pool/api.rs:287-325, 441-476).  Here
// the unit is a page of `page_size` tokens, and layers are gathered in groups with
// pages of their own: a group that needs every key keeps all its pages until the
// request ends; a group that needs only the last `window` keys gives a page back as
// soon as every later query is out of its reach.  Freed pages are handed out again
// last-in-first-out, so a page that has just been given back is the first to be used
// again (as naive_kvpool.rs:449-460 does with slots): what a new owner finds in a page
// is stale data, and only the lengths in the step's metadata say what may be read.
#pragma once
#include <algorithm>
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace lab {

struct CapacityError : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct StateError : std::logic_error {
  using std::logic_error::logic_error;
};

struct GroupConfig {
  int page_size = 16;
  int window = 0;  // 0: every key is kept; else only the last `window` keys are readable
  int num_pages = 0;
};

// A stack of free page (or slot) numbers that refuses double frees and unknown numbers.
class FreeStack {
 public:
  explicit FreeStack(int n = 0) { reset(n); }
  void reset(int n) {
    held_.assign(n, 0);
    free_.clear();
    for (int i = n - 1; i >= 0; --i) free_.push_back(i);  // low numbers go out first
  }
  int capacity() const { return (int)held_.size(); }
  int free_count() const { return (int)free_.size(); }
  int used_count() const { return capacity() - free_count(); }
  int take() {
    if (free_.empty()) throw CapacityError("no free entry");
    int v = free_.back();
    free_.pop_back();
    held_[v] = 1;
    return v;
  }
  void give(int v) {
    if (v < 0 || v >= capacity()) throw StateError("freeing entry " + std::to_string(v) + " outside the pool");
    if (!held_[v]) throw StateError("entry " + std::to_string(v) + " freed twice");
    held_[v] = 0;
    free_.push_back(v);
  }
  bool held(int v) const { return v >= 0 && v < capacity() && held_[v]; }

 private:
  std::vector<int> free_;
  std::vector<uint8_t> held_;
};

struct RequestCache {
  int64_t id = 0;
  int state_slot = -1;
  int committed = 0;  // tokens whose keys/values (and state) are final
  int reserved = 0;   // tokens that have pages (>= committed while a step is in flight)
  std::vector<std::vector<int>> tables;  // per group: page of logical block b, -1 once given back
  std::vector<int> first_live;           // per group: first block not yet given back
};

struct StepEntry {
  int64_t id;
  int n_tokens;
};

// Offsets (in int32 words) of the arrays of one packed step inside the staging buffer.
struct StepLayout {
  int tokens_cap = 0, requests_cap = 0;
  std::vector<int> table_width;  // per group
  int row_req = 0, row_pos = 0, q_start = 0, kv_len = 0, pos0 = 0, state_slot = 0;
  std::vector<int> row_slot, block_table;
  int total = 0;
};

class CacheManager {
 public:
  CacheManager(std::vector<GroupConfig> groups, int max_requests)
      : groups_(std::move(groups)), slots_(max_requests) {
    if (max_requests <= 0) throw std::invalid_argument("max_requests must be positive");
    for (auto& g : groups_) {
      if (g.page_size <= 0 || g.num_pages < 0 || g.window < 0) throw std::invalid_argument("bad group configuration");
      pools_.emplace_back(g.num_pages);
    }
  }

  int num_groups() const { return (int)groups_.size(); }
  const GroupConfig& group(int g) const { return groups_.at(g); }
  int max_requests() const { return slots_.capacity(); }
  bool has(int64_t id) const { return requests_.count(id) != 0; }
  int free_pages(int g) const { return pools_.at(g).free_count(); }
  int used_pages(int g) const { return pools_.at(g).used_count(); }
  int free_state_slots() const { return slots_.free_count(); }
  int used_state_slots() const { return slots_.used_count(); }
  int live_requests() const { return (int)requests_.size(); }

  // A new request: takes a state slot, holds no pages yet.
  int open(int64_t id) {
    if (has(id)) throw StateError("request " + std::to_string(id) + " is already open");
    if (slots_.free_count() == 0) throw CapacityError("no free state slot for request " + std::to_string(id));
    RequestCache rc;
    rc.id = id;
    rc.state_slot = slots_.take();
    rc.tables.resize(groups_.size());
    rc.first_live.assign(groups_.size(), 0);
    requests_.emplace(id, std::move(rc));
    return requests_.at(id).state_slot;
  }

  const RequestCache& get(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw StateError("request " + std::to_string(id) + " is not open");
    return it->second;
  }

  static int blocks_for(int tokens, int page_size) { return (tokens + page_size - 1) / page_size; }

  // Pages group g must still hand out so that the request can hold `n` more tokens.
  int pages_needed(int64_t id, int g, int n) const {
    const RequestCache& rc = get(id);
    const int ps = groups_[g].page_size;
    return blocks_for(rc.reserved + n, ps) - (int)rc.tables[g].size();
  }

  // Most pages of group g that a request holds at any time if it grows to `tokens` tokens
  // in steps of at most `max_step` tokens.
  int pages_at_peak(int g, int tokens, int max_step) const {
    const GroupConfig& cfg = groups_[g];
    const int all = blocks_for(tokens, cfg.page_size);
    if (cfg.window == 0) return all;
    // Live positions never span more than window - 1 + max_step; such a span touches
    // at most ceil(span / page) + 1 pages.
    const int span = cfg.window - 1 + std::max(1, max_step);
    return std::min(all, blocks_for(span, cfg.page_size) + 1);
  }

  // True if all of `entries` could be reserved together right now.
  bool can_reserve(const std::vector<StepEntry>& entries) const {
    for (int g = 0; g < num_groups(); ++g) {
      long need = 0;
      for (const auto& e : entries) need += pages_needed(e.id, g, e.n_tokens);
      if (need > pools_[g].free_count()) return false;
    }
    return true;
  }

  // Gives the request pages for its next `n` tokens in every group; all or nothing.
  void reserve(int64_t id, int n) {
    if (n <= 0) throw std::invalid_argument("reserve needs a positive token count");
    RequestCache& rc = mut(id);
    for (int g = 0; g < num_groups(); ++g) {
      const int need = pages_needed(id, g, n);
      if (need > pools_[g].free_count())
        throw CapacityError("group " + std::to_string(g) + " has " + std::to_string(pools_[g].free_count()) +
                            " free pages, request " + std::to_string(id) + " needs " + std::to_string(need));
    }
    for (int g = 0; g < num_groups(); ++g) {
      const int need = pages_needed(id, g, n);
      for (int i = 0; i < need; ++i) rc.tables[g].push_back(pools_[g].take());
    }
    rc.reserved += n;
  }

  // The step that computed the reserved tokens has finished: they are final.  Pages that
  // no later query can reach go back to their pool.
  void commit(int64_t id, int n) {
    RequestCache& rc = mut(id);
    if (n < 0 || rc.committed + n > rc.reserved) throw StateError("commit beyond what was reserved");
    rc.committed += n;
    for (int g = 0; g < num_groups(); ++g) {
      const GroupConfig& cfg = groups_[g];
      if (cfg.window == 0) continue;
      // A later query sits at position >= committed and reads keys > position - window.
      const int first_needed = rc.committed - cfg.window + 1;
      while (rc.first_live[g] < (int)rc.tables[g].size() &&
             (rc.first_live[g] + 1) * cfg.page_size <= first_needed) {
        int& page = rc.tables[g][rc.first_live[g]];
        pools_[g].give(page);
        page = -1;
        ++rc.first_live[g];
      }
    }
  }

  // A step failed: what was reserved beyond the committed tokens is given back.
  void rollback(int64_t id) {
    RequestCache& rc = mut(id);
    for (int g = 0; g < num_groups(); ++g) {
      const int keep = blocks_for(rc.committed, groups_[g].page_size);
      while ((int)rc.tables[g].size() > keep) {
        const int page = rc.tables[g].back();
        if (page >= 0) pools_[g].give(page);
        rc.tables[g].pop_back();
      }
    }
    rc.reserved = rc.committed;
  }

  // The request ends: every page and its state slot go back.
  void close(int64_t id) {
    RequestCache& rc = mut(id);
    for (int g = 0; g < num_groups(); ++g)
      for (int page : rc.tables[g])
        if (page >= 0) pools_[g].give(page);
    slots_.give(rc.state_slot);
    requests_.erase(id);
  }

  std::vector<int> block_table(int64_t id, int g) const { return get(id).tables.at(g); }
  int held_pages(int64_t id, int g) const {
    int n = 0;
    for (int p : get(id).tables.at(g)) n += p >= 0;
    return n;
  }

  // Self-check for tests: every page is held by exactly one request or free.
  void check_consistency() const {
    for (int g = 0; g < num_groups(); ++g) {
      std::vector<int> owners(groups_[g].num_pages, 0);
      for (const auto& kv : requests_)
        for (int page : kv.second.tables[g])
          if (page >= 0) {
            if (page >= groups_[g].num_pages) throw StateError("page outside the pool in a block table");
            if (++owners[page] > 1) throw StateError("page " + std::to_string(page) + " is held twice");
            if (!pools_[g].held(page)) throw StateError("page in a block table is marked free");
          }
      int held = 0;
      for (int o : owners) held += o;
      if (held != pools_[g].used_count()) throw StateError("a page is lost: held by no request and not free");
    }
    if ((int)requests_.size() != slots_.used_count()) throw StateError("state slots and requests disagree");
  }

  // ---- packing a step -------------------------------------------------------------
  StepLayout layout(int tokens_cap, int requests_cap, const std::vector<int>& table_width) const {
    if ((int)table_width.size() != num_groups()) throw std::invalid_argument("one table width per group");
    StepLayout L;
    L.tokens_cap = tokens_cap;
    L.requests_cap = requests_cap;
    L.table_width = table_width;
    int at = 0;
    auto take = [&](int n) {
      int here = at;
      at += (n + 3) & ~3;  // keep every array 16-byte aligned
      return here;
    };
    L.row_req = take(tokens_cap);
    L.row_pos = take(tokens_cap);
    L.q_start = take(requests_cap + 1);
    L.kv_len = take(requests_cap);
    L.pos0 = take(requests_cap);
    L.state_slot = take(requests_cap);
    for (int g = 0; g < num_groups(); ++g) L.row_slot.push_back(take(tokens_cap));
    for (int g = 0; g < num_groups(); ++g) L.block_table.push_back(take(requests_cap * table_width[g]));
    L.total = at;
    return L;
  }

  // Writes the arrays of one step.  Every entry's tokens must be reserved already: they
  // are the last `n_tokens` reserved positions of the request.  Rows beyond the real
  // ones (up to pad_tokens / pad_requests) are filled so that kernels skip them:
  // position -1, slot -1, length 0.
  void pack(const std::vector<StepEntry>& entries, const StepLayout& L, int32_t* buf, int pad_tokens,
            int pad_requests) const {
    int total = 0;
    for (const auto& e : entries) total += e.n_tokens;
    const int B = (int)entries.size();
    if (total > L.tokens_cap || pad_tokens > L.tokens_cap || B > L.requests_cap || pad_requests > L.requests_cap)
      throw std::invalid_argument("step does not fit the staging layout");
    int row = 0;
    for (int b = 0; b < B; ++b) {
      const RequestCache& rc = get(entries[b].id);
      const int n = entries[b].n_tokens;
      const int start = rc.reserved - n;
      if (n <= 0 || start < rc.committed) throw StateError("entry was not reserved for this step");
      buf[L.q_start + b] = row;
      buf[L.kv_len + b] = start + n;
      buf[L.pos0 + b] = start;
      buf[L.state_slot + b] = rc.state_slot;
      for (int g = 0; g < num_groups(); ++g) {
        const int ps = groups_[g].page_size, width = L.table_width[g];
        const auto& table = rc.tables[g];
        if ((int)table.size() > width) throw std::invalid_argument("block table wider than the staging layout");
        int32_t* bt = buf + L.block_table[g] + (size_t)b * width;
        for (int i = 0; i < width; ++i) bt[i] = i < (int)table.size() ? table[i] : -1;
        for (int i = 0; i < n; ++i) {
          const int pos = start + i;
          const int page = table[pos / ps];
          if (page < 0) throw StateError("a new token falls on a page that was given back");
          buf[L.row_slot[g] + row + i] = page * ps + pos % ps;
        }
      }
      for (int i = 0; i < n; ++i) {
        buf[L.row_req + row + i] = b;
        buf[L.row_pos + row + i] = start + i;
      }
      row += n;
    }
    buf[L.q_start + B] = row;
    const int Bp = std::max(B, pad_requests), Tp = std::max(row, pad_tokens);
    for (int b = B; b < Bp; ++b) {
      buf[L.q_start + b + 1] = row + (b - B + 1 <= Tp - row ? b - B + 1 : Tp - row);
      buf[L.kv_len + b] = 0;
      buf[L.pos0 + b] = 0;
      buf[L.state_slot + b] = -1;
      for (int g = 0; g < num_groups(); ++g)
        for (int i = 0; i < L.table_width[g]; ++i) buf[L.block_table[g] + (size_t)b * L.table_width[g] + i] = -1;
    }
    for (int r = row; r < Tp; ++r) {
      buf[L.row_req + r] = std::min(B + (r - row), std::max(Bp - 1, 0));
      buf[L.row_pos + r] = -1;
      for (int g = 0; g < num_groups(); ++g) buf[L.row_slot[g] + r] = -1;
    }
  }

 private:
  RequestCache& mut(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end()) throw StateError("request " + std::to_string(id) + " is not open");
    return it->second;
  }

  std::vector<GroupConfig> groups_;
  std::vector<FreeStack> pools_;
  FreeStack slots_;
  std::unordered_map<int64_t, RequestCache> requests_;
};

}  // namespace lab
