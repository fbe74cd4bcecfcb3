// Scheduler: admits requests, cuts prompts into portions under a token budget, lets
// running requests decode, finishes them and gives their cache back.
//
// The policy is the reference runner's (rust/engine/src/runner/model_runner.rs:577-757
// admission, 698-897 drive loop; rust/engine/src/runner/model_runner/batch_policy.rs:36-87
// planning):
//   * at every step boundary finished requests are cleaned up first, then waiting
//     requests are looked at in arrival order;
//   * a step holds at most `max_batch_tokens` new tokens: one for every decoding request
//     first, the rest goes to portions of prompts in the order the requests became active;
//   * a request decodes once it has produced its first token; only the portion that
//     reaches the end of the prompt produces a token;
//   * a request ends when its budget of new tokens is used up or it produced an
//     end-of-sequence token (which is counted and returned).
// Lookahead (this engine's addition): while a pure decode step runs on the device, the next
// one may be planned and launched before the first one's tokens have reached the host
// (`plan_ahead`): the device feeds the sampled ids forward itself.  A request that turns out
// to have ended with the earlier step still takes part in the later one; that token is
// dropped, and its cache is given back when the later step is completed.
// What happens when pages run out is decided by `reserve_future`:
//   * true (the reference's way): a request is admitted only if the pages for its whole
//     life (prompt + new tokens - 1) are free beyond what running requests will still
//     take; otherwise it waits (a later, smaller one may pass it), and it fails when
//     nothing is running that could free pages.  Pages then never run out mid-run.
//   * false: a request is admitted when its next portion fits.  If a running request
//     finds no page for its step, the youngest running request is preempted: its cache
//     is given back and it returns to the head of the waiting queue with prompt +
//     tokens so far as its new prompt (recomputed later; its tokens are kept).  A
//     request that cannot get its pages even alone fails.
#pragma once
#include <deque>
#include <memory>
#include <optional>

#include "cache_manager.hpp"

namespace lab {

struct SchedulerConfig {
  int max_batch_tokens = 512;  // model_runner.rs:50
  int max_seq_len = 0;         // prompt + new tokens may not exceed this (0: no limit besides pages)
  int max_active = 0;          // 0: as many as there are state slots
  bool reserve_future = true;
};

enum class FinishReason { kNone = 0, kLength = 1, kEos = 2, kCapacity = 3, kInvalid = 4, kCancelled = 5 };

struct SchedRequest {
  int64_t id = 0;
  std::vector<int> tokens;  // prompt followed by generated tokens
  int prompt_len = 0;       // length of the original prompt
  int max_new = 1;          // model_runner.rs:612-625 (default one token)
  std::vector<int> eos;
  bool ignore_eos = false;
  int generated = 0;
  int computed = 0;  // tokens whose cache entries are committed
  bool decoding = false;
  int preemptions = 0;
  long arrival = 0;
  // lookahead: tokens sampled on the device that the host has not seen yet (0 or 1), steps whose
  // cache entries were committed at launch, and the end that an earlier step brought while a
  // later one was already running
  int unseen = 0;
  int committed_early = 0;
  FinishReason ended = FinishReason::kNone;
};

struct PlanEntry {
  int64_t id;
  int start;    // position of the first token of this portion
  int n;        // number of tokens
  bool sample;  // the portion reaches the end of the known tokens: its last row yields a token
};

struct Finished {
  int64_t id;
  std::vector<int> generated;
  FinishReason reason;
  int prompt_len;
  int preemptions;
  std::string message;
};

class Scheduler {
 public:
  Scheduler(std::shared_ptr<CacheManager> cache, SchedulerConfig cfg) : cache_(std::move(cache)), cfg_(cfg) {
    if (cfg_.max_batch_tokens <= 0) throw std::invalid_argument("max_batch_tokens must be positive");
  }

  void add(int64_t id, std::vector<int> prompt, int max_new, std::vector<int> eos, bool ignore_eos) {
    SchedRequest r;
    r.id = id;
    r.prompt_len = (int)prompt.size();
    r.tokens = std::move(prompt);
    r.max_new = max_new;
    r.eos = std::move(eos);
    r.ignore_eos = ignore_eos;
    r.arrival = arrivals_++;
    waiting_.push_back(std::move(r));
  }

  bool cancel(int64_t id) {
    for (auto it = waiting_.begin(); it != waiting_.end(); ++it)
      if (it->id == id) {
        finish(*it, FinishReason::kCancelled, "cancelled while waiting");
        waiting_.erase(it);
        return true;
      }
    for (auto it = active_.begin(); it != active_.end(); ++it)
      if (it->id == id) {
        cache_->close(id);
        finish(*it, FinishReason::kCancelled, "cancelled while running");
        active_.erase(it);
        return true;
      }
    return false;
  }

  bool idle() const { return waiting_.empty() && active_.empty(); }
  int num_waiting() const { return (int)waiting_.size(); }
  int num_active() const { return (int)active_.size(); }
  long preemptions() const { return preemptions_; }

  // Decides the next step and reserves its pages.  An empty plan with requests left
  // means that nothing can run (the caller should look at `take_finished`).
  std::vector<PlanEntry> plan() {
    admit();
    for (;;) {
      std::vector<PlanEntry> entries = cut();
      if (entries.empty()) return entries;
      if (reserve_all(entries)) return entries;
      // Pages ran out under running requests.
      if (active_.size() == 1) {
        SchedRequest& only = active_.front();
        cache_->close(only.id);
        finish(only, FinishReason::kCapacity, "the cache cannot hold this request even alone");
        active_.clear();
        admit();
        continue;
      }
      preempt_youngest();
    }
  }

  // Plans the step after `in_flight`, a pure decode step that has been launched and not yet
  // completed, on the assumption that none of its requests ends with it; reserves its pages.
  // Its input tokens are the ones `in_flight` samples (they stay on the device).  Returns an
  // empty plan, and changes nothing, when looking ahead is not possible: requests are waiting,
  // `in_flight` is not a decode step of all running requests, one of them reaches its number of
  // new tokens with it, or the pages for one more token each are not there.
  std::vector<PlanEntry> plan_ahead(const std::vector<PlanEntry>& in_flight) {
    if (!waiting_.empty() || in_flight.empty() || in_flight.size() != active_.size()) return {};
    if ((int)in_flight.size() > cfg_.max_batch_tokens) return {};
    for (size_t i = 0; i < in_flight.size(); ++i) {
      const PlanEntry& e = in_flight[i];
      const SchedRequest& r = active_[i];
      if (r.id != e.id || e.n != 1 || !e.sample || !r.decoding || r.unseen != 0 || r.committed_early != 0) return {};
      if (r.ended != FinishReason::kNone || r.generated + 1 >= r.max_new) return {};
      if (cfg_.max_seq_len > 0 && e.start + 2 > cfg_.max_seq_len) return {};
    }
    // The step is on its way: its cache entries will be written, so they count from now on.
    for (size_t i = 0; i < in_flight.size(); ++i) cache_->commit(in_flight[i].id, 1);
    std::vector<StepEntry> want;
    for (const auto& e : in_flight) want.push_back({e.id, 1});
    if (!cache_->can_reserve(want)) {
      for (auto& r : active_) {  // remembered, so that complete() does not commit them again
        r.computed += 1;
        r.committed_early = 1;
      }
      return {};
    }
    std::vector<PlanEntry> next;
    for (size_t i = 0; i < in_flight.size(); ++i) {
      SchedRequest& r = active_[i];
      r.computed += 1;
      r.committed_early = 1;
      r.unseen = 1;
      cache_->reserve(r.id, 1);
      next.push_back({r.id, r.computed, 1, true});
    }
    return next;
  }

  // Tokens of one planned portion.
  std::vector<int> portion(int64_t id, int start, int n) const {
    const SchedRequest& r = find_active(id);
    if (start < 0 || start + n > (int)r.tokens.size()) throw StateError("portion outside the request's tokens");
    return std::vector<int>(r.tokens.begin() + start, r.tokens.begin() + start + n);
  }

  // The step ran: commit the cache of every entry and take the sampled tokens (one per
  // entry with `sample`, in plan order).
  void complete(const std::vector<PlanEntry>& entries, const std::vector<int>& sampled) {
    size_t next = 0;
    for (const auto& e : entries) {
      SchedRequest& r = find_active_mut(e.id);
      if (r.committed_early > 0) {
        r.committed_early -= 1;  // plan_ahead counted this step's cache entries at its launch
      } else {
        cache_->commit(e.id, e.n);
        r.computed += e.n;
      }
      if (!e.sample) continue;
      if (next >= sampled.size()) throw StateError("fewer sampled tokens than sampling entries");
      const int tok = sampled[next++];
      if (r.ended != FinishReason::kNone) continue;  // it ended a step ago: this token is dropped
      r.tokens.push_back(tok);
      r.generated += 1;
      r.decoding = true;
    }
    if (next != sampled.size()) throw StateError("more sampled tokens than sampling entries");
    // Finished requests leave before any peer's next step (model_runner.rs:711-722), unless a
    // later step that is already running holds them: then they leave when that step completes.
    for (auto it = active_.begin(); it != active_.end();) {
      FinishReason why = it->ended;
      if (why == FinishReason::kNone) {
        if (it->generated > 0 && !it->ignore_eos &&
            std::find(it->eos.begin(), it->eos.end(), it->tokens.back()) != it->eos.end())
          why = FinishReason::kEos;
        else if (it->generated >= it->max_new)
          why = FinishReason::kLength;
      }
      const bool held = it->unseen > 0 && it->ended == FinishReason::kNone;  // a later step runs with it
      if (it->unseen > 0) it->unseen -= 1;  // the token the later step took from the device has arrived
      if (why != FinishReason::kNone && held) {
        it->ended = why;  // leaves with the later step's completion
        ++it;
      } else if (why != FinishReason::kNone) {
        cache_->close(it->id);
        finish(*it, why, "");
        it = active_.erase(it);
      } else {
        ++it;
      }
    }
  }

  // The step failed on the device or host: nothing of it counts.
  void abandon(const std::vector<PlanEntry>& entries) {
    for (const auto& e : entries) cache_->rollback(e.id);
  }

  std::vector<Finished> take_finished() {
    std::vector<Finished> out;
    out.swap(finished_);
    return out;
  }

  const SchedRequest& find_active(int64_t id) const {
    for (const auto& r : active_)
      if (r.id == id) return r;
    throw StateError("request " + std::to_string(id) + " is not running");
  }

 private:
  SchedRequest& find_active_mut(int64_t id) { return const_cast<SchedRequest&>(find_active(id)); }

  void finish(const SchedRequest& r, FinishReason why, std::string message) {
    Finished f;
    f.id = r.id;
    f.generated.assign(r.tokens.begin() + r.prompt_len, r.tokens.end());
    f.reason = why;
    f.prompt_len = r.prompt_len;
    f.preemptions = r.preemptions;
    f.message = std::move(message);
    finished_.push_back(std::move(f));
  }

  int final_length(const SchedRequest& r) const {
    // The last sampled token never needs a cache entry (model_runner.rs:577-694).
    return r.prompt_len + r.max_new - 1;
  }

  // Pages of group g that running requests will still take before they end.
  long future_pages(int g) const {
    long need = 0;
    for (const auto& r : active_) {
      const int peak = cache_->pages_at_peak(g, final_length(r), cfg_.max_batch_tokens);
      need += std::max(0, peak - cache_->held_pages(r.id, g));
    }
    return need;
  }

  void admit() {
    const int max_active = cfg_.max_active > 0 ? cfg_.max_active : cache_->max_requests();
    for (auto it = waiting_.begin(); it != waiting_.end();) {
      SchedRequest& r = *it;
      std::string bad;
      const int known = (int)r.tokens.size();
      if (known == 0) bad = "empty prompt";
      else if (r.max_new < 0) bad = "negative max_new_tokens";
      else if (cfg_.max_seq_len > 0 && final_length(r) > cfg_.max_seq_len)
        bad = "prompt + new tokens exceed the maximum sequence length";
      if (!bad.empty()) {
        finish(r, FinishReason::kInvalid, bad);
        it = waiting_.erase(it);
        continue;
      }
      if (r.max_new - r.generated <= 0) {  // nothing to do (max_new == 0)
        finish(r, FinishReason::kLength, "");
        it = waiting_.erase(it);
        continue;
      }
      if ((int)active_.size() >= max_active || cache_->free_state_slots() == 0) break;
      bool fits = true, ever = true;
      for (int g = 0; g < cache_->num_groups() && fits; ++g) {
        const int total = cache_->group(g).num_pages;
        if (cfg_.reserve_future) {
          const int peak = cache_->pages_at_peak(g, final_length(r), cfg_.max_batch_tokens);
          if (peak > total) ever = false;
          if (peak + future_pages(g) > cache_->free_pages(g)) fits = false;
        } else {
          const int first = std::min(known, cfg_.max_batch_tokens);
          const int need = CacheManager::blocks_for(first, cache_->group(g).page_size);
          if (need > total) ever = false;
          if (need > cache_->free_pages(g)) fits = false;
        }
      }
      if (!ever || (!fits && active_.empty())) {
        // Nothing is running that could free pages: waiting would last forever
        // (model_runner.rs:745-757).
        finish(r, FinishReason::kCapacity, "the cache cannot hold this request");
        it = waiting_.erase(it);
        continue;
      }
      if (!fits) {
        ++it;  // stays queued; a later, smaller request may still pass
        continue;
      }
      cache_->open(r.id);
      r.computed = 0;
      r.decoding = false;
      active_.push_back(std::move(r));
      it = waiting_.erase(it);
    }
  }

  // batch_policy.rs:36-87: decode tokens first, the rest of the budget to prompt portions.
  std::vector<PlanEntry> cut() const {
    std::vector<PlanEntry> entries;
    int decoders = 0;
    for (const auto& r : active_) decoders += r.decoding && r.computed < (int)r.tokens.size();
    int decode_budget = std::min(decoders, cfg_.max_batch_tokens);
    int prefill_budget = cfg_.max_batch_tokens - decode_budget;
    for (const auto& r : active_) {
      const int left = (int)r.tokens.size() - r.computed;
      if (left <= 0) continue;
      if (r.decoding) {
        if (decode_budget > 0) {
          --decode_budget;
          entries.push_back({r.id, r.computed, 1, left == 1});
        }
      } else {
        const int n = std::min(left, prefill_budget);
        if (n > 0) {
          prefill_budget -= n;
          entries.push_back({r.id, r.computed, n, n == left});
        }
      }
    }
    return entries;
  }

  bool reserve_all(const std::vector<PlanEntry>& entries) {
    std::vector<StepEntry> want;
    for (const auto& e : entries) want.push_back({e.id, e.n});
    if (!cache_->can_reserve(want)) return false;
    for (const auto& e : entries) cache_->reserve(e.id, e.n);
    return true;
  }

  void preempt_youngest() {
    auto victim = active_.begin();
    for (auto it = active_.begin(); it != active_.end(); ++it)
      if (it->arrival > victim->arrival) victim = it;
    cache_->close(victim->id);
    victim->computed = 0;
    victim->decoding = false;  // its known tokens are a prompt again
    victim->preemptions += 1;
    ++preemptions_;
    waiting_.push_front(std::move(*victim));
    active_.erase(victim);
  }

  std::shared_ptr<CacheManager> cache_;
  SchedulerConfig cfg_;
  std::deque<SchedRequest> waiting_;
  std::vector<SchedRequest> active_;
  std::vector<Finished> finished_;
  long arrivals_ = 0;
  long preemptions_ = 0;
};

}  // namespace lab
