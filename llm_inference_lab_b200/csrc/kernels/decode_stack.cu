// The layers of a decode step as ONE persistent kernel (bfloat16, heads of 64 or 128).
//
// A decode step of a few tokens (one per request) is a chain of small dependent operators: per layer
// two norms, four matrix products, the rotation with the cache write, and the attention.  Launched one
// by one, each costs more in launch and ramp-up than in work.  Here one CTA per SM stays resident for
// the whole stack of pre-norm layers and walks their phases,
//
//   1  h = rmsnorm(x) * w1;  q, k, v = h Wqkv^T + b;  q and k rotated;  k, v into their cache pages
//   2  attention of every request's one query row over its pages (keys split over CTAs)
//   3  x += attn Wo^T
//   4  h = rmsnorm(x) * w2;  act = silu(h Wg^T) * (h Wu^T)
//   5  x += act Wd^T
//
// with a grid-wide barrier in global memory between phases.  What makes it pay:
//   * the weights of a phase do not depend on the phase before it, so the warp that loads them (TMA
//     into a ring of shared-memory stages) never waits at a barrier: it runs ahead into the next
//     phases as far as the ring has room, and HBM keeps streaming across the phase changes;
//   * the few activation rows are the stationary operand: every CTA builds them in shared memory
//     itself (the norm is recomputed per CTA from the residual rows, a few KB), in the swizzled
//     layout the tensor core reads, so no norm kernel and no activation round trip per product;
//   * a product is cut in items (tile of 128 output features, slice of K) so that every SM has
//     work; the items of a tile leave 32-bit partial sums in global memory, count themselves, and
//     the one that finishes last sums them in the fixed order of the slices and applies the
//     epilogue (bias + rotation + cache write, residual add, or SiLU gate): no order depends on timing.
// Products run on tcgen05.mma (features on the 128-row side, tokens on the N side: 16, 32 or 64),
// accumulators in tensor memory; attention uses the mma.sync tile code of the decode kernel.
// Every wait (mbarriers, the grid barrier) is bounded: when one runs out, the kernel sets the error
// word and an abort flag that every CTA sees, lets all roles drain, frees its tensor memory and returns.
// The grid must be co-resident (cooperative launch, one CTA per SM).
//
// Formulas: rust/engine/src/runner/model/qwen2/engine.rs:1133-1296 (a layer), kernels.rs:546-582
// (RMSNorm), 587-631 (rotation), 635-698 (cache store), 1134-1256 (grouped decode attention),
// 898-942 (merge of key splits), 1469-1486 (SiLU gate).
#include <cstring>

#include "tcgen05.cuh"
#include "attention_mma.cuh"

namespace {

static_assert(D == 64 || D == 128, "the decode stack is built for heads of 64 and of 128");

constexpr int THREADS = 256;            // warp 0 loads, warp 1 issues MMAs and owns tensor memory,
constexpr int WORKERS = THREADS - 32;   // warps 2-5 run epilogues, warps 6-7 help with operands and attention
constexpr int TM = 128, BK = 64, UMMA_K = 16;
constexpr int STAGE_BYTES = TM * BK * 2;  // one k-tile of 128 weight rows
constexpr int STAGES = 6;
constexpr int WORK_BYTES = 112 * 1024;    // the activation operand of a product, or the attention's key/value tiles
constexpr int CHUNK = 16;                 // tokens an epilogue step works on
constexpr int EXCH_STRIDE = CHUNK + 1;
constexpr int EXCH_BYTES = (TM * EXCH_STRIDE * 4 + 127) / 128 * 128;
constexpr int OFF_RING = 0, OFF_WORK = STAGES * STAGE_BYTES, OFF_EXCH = OFF_WORK + WORK_BYTES, OFF_BAR = OFF_EXCH + EXCH_BYTES;
constexpr int SMEM = OFF_BAR + 256 + 1024;
constexpr int TMEM_COLS = 128;            // two accumulators of up to 64 columns
constexpr int MAX_GROUPS = 4;
constexpr int MAX_ROW_CHUNKS = 16;        // 16-byte chunks of a residual row one of its 16 lanes holds: rows up to 2,048 wide
// attention inside the stack: warps 2.. stream tiles of keys through private rings laid over the work area
constexpr int AW = D > 64 ? 6 : 4;
constexpr int AT_BN = D > 64 ? 16 : 32;
constexpr int AT_STAGES = D > 64 ? 2 : 3;
constexpr int AT_TILE_BYTES = AT_BN * ROW_BYTES;
constexpr int AT_WARP_BYTES = AT_STAGES * 2 * AT_TILE_BYTES;
static_assert(AW * AT_WARP_BYTES <= WORK_BYTES && AW * 16 * (D + 2) * 4 <= WORK_BYTES, "attention fits the work area");
constexpr unsigned long long BARRIER_LIMIT_NS = 1000000000ull;
constexpr int MAX_ATT_SPLITS = 8;          // splits of a request's keys over CTAs
constexpr int BAR_WORDS = 32;              // words between the barrier's three counters (a cache line each)

enum Phase : int { PH_QKV = 0, PH_ATTN = 1, PH_O = 2, PH_GATE_UP = 3, PH_DOWN = 4, PHASES = 5 };

// One layer call: its weights (as tensor maps over [rows, K] bfloat16 matrices), norms, cache.
struct alignas(64) LayerParams {
  CUtensorMap map_qkv, map_o, map_gate_up, map_down;
  const __nv_bfloat16* norm1;
  const __nv_bfloat16* norm2;
  const __nv_bfloat16* bias_qkv;   // may be null
  __nv_bfloat16* cache_k;          // [num_pages, n_kv, page_size, D]
  __nv_bfloat16* cache_v;
  float eps1, eps2;
  int group;                       // which cache group's slots and block table the call uses
  int window;                      // 0: every key
  int write_kv;                    // 0: the call reads a cache another call fills
  int pad_;
};

struct StackParams {
  const LayerParams* layers;
  int n_layers;
  int phase_begin, phase_end;      // phases [begin, end) of the n_layers * 5 are run
  int T, BN;                       // tokens of the step, and the N of the MMAs (16, 32 or 64, >= T)
  int hidden, n_q, n_kv, inter;
  int s_qkv, s_o, s_gate_up, s_down;   // slices of K per product
  int att_splits;
  __nv_bfloat16* x;                // [T, hidden] residual stream, in and out
  __nv_bfloat16* qbuf;             // [T, n_q * D]
  __nv_bfloat16* attn;             // [T, n_q * D]
  __nv_bfloat16* act;              // [T, inter]
  float* partial;                  // partial sums of the products' K slices
  float* att_acc;                  // attention: (acc, max, sum) of the key splits
  float* att_ml;
  int* counters;                   // zero between uses
  unsigned* barrier;               // arrivals and abort flag, each in a 128-byte line of its own; cleared before the launch
  unsigned long long* stamps;      // null, or [phases][4] + 1 nanosecond stamps of CTA 0: a phase's start, its first operand
                                   // built, its first item done, all its items done; and the end of the kernel
  const float2* table;             // [T, D / 2] (cos, sin)
  const int* row_slot[MAX_GROUPS];
  const int* block_table[MAX_GROUPS];
  int max_blocks[MAX_GROUPS];
  const int* q_start;              // [T + 1]
  const int* kv_len;               // [T]
  int page_size, num_pages;
  float scale_log2;
};

struct Bars {
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_slot;
  int abort;
  int snap[2];
  int flag;
};

// A product of a phase: weights [n_rows (x2 gated), K], cut in tiles of 128 rows (64 + 64 when gated) and S slices of K.
struct Product {
  const CUtensorMap* map;
  int n_out;        // output features
  int K;
  int tiles, S, k_tiles, ktps;
  bool gated, norm;
  const __nv_bfloat16* src;   // activation rows [T, K]
  const __nv_bfloat16* norm_w;
  float eps;
  int counter_base;
};

__device__ __forceinline__ Product product_of(const StackParams& p, const LayerParams& L, int kind) {
  Product g;
  g.gated = kind == PH_GATE_UP;
  g.norm = kind == PH_QKV || kind == PH_GATE_UP;
  g.eps = kind == PH_QKV ? L.eps1 : L.eps2;
  g.norm_w = kind == PH_QKV ? L.norm1 : L.norm2;
  const int qd = p.n_q * D;
  switch (kind) {
    case PH_QKV: g.map = &L.map_qkv; g.n_out = (p.n_q + 2 * p.n_kv) * D; g.K = p.hidden; g.S = p.s_qkv; g.src = p.x; g.counter_base = 0; break;
    case PH_O: g.map = &L.map_o; g.n_out = p.hidden; g.K = qd; g.S = p.s_o; g.src = p.attn; g.counter_base = 1024; break;
    case PH_GATE_UP: g.map = &L.map_gate_up; g.n_out = p.inter; g.K = p.hidden; g.S = p.s_gate_up; g.src = p.x; g.counter_base = 2048; break;
    default: g.map = &L.map_down; g.n_out = p.hidden; g.K = p.inter; g.S = p.s_down; g.src = p.act; g.counter_base = 3072; break;
  }
  const int rows = g.gated ? TM / 2 : TM;
  g.tiles = (g.n_out + rows - 1) / rows;
  g.k_tiles = (g.K + BK - 1) / BK;
  g.ktps = (g.k_tiles + g.S - 1) / g.S;
  return g;
}

__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* ptr) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ float ldcg_bf16(const __nv_bfloat16* ptr) {
  const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(ptr));
  return __bfloat162float(__ushort_as_bfloat16(raw));
}

// All workers meet; returns false (to every worker alike) once any wait of this CTA, or of another
// CTA at the grid barrier, has run out.
__device__ __forceinline__ bool sync_alive(Bars* bars, int& parity) {
  if (threadIdx.x == 32) bars->snap[parity] = bars->abort;
  named_sync(1, WORKERS);
  const bool alive = bars->snap[parity] == 0;
  parity ^= 1;
  return alive;
}

// Grid-wide barrier (workers only; the loading warp never waits here).  The host clears the count
// before the launch; the n-th barrier is passed when n * (CTAs) have arrived.  One release-add per
// CTA, then bounded polling with acquire loads.
__device__ __forceinline__ void grid_barrier(const StackParams& p, Bars* bars, unsigned& passed) {
  named_sync(1, WORKERS);
  if (threadIdx.x == 32 && !bars->abort) {
    unsigned* arrivals = p.barrier;
    unsigned* abort_word = p.barrier + BAR_WORDS;
    passed += 1;
    const unsigned target = passed * gridDim.x;
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(arrivals), "r"(1u) : "memory");
    uint64_t t0 = 0;
    for (unsigned polls = 1; ld_acquire(arrivals) < target; ++polls) {
      if ((polls & 1023u) != 0u) continue;   // the abort flag and the clock are looked at now and then
      if (ld_acquire(abort_word) != 0u) {
        bars->abort = 1;
        break;
      }
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > BARRIER_LIMIT_NS) {
        atomicExch(abort_word, 1u);
        bars->abort = 1;
        lab_set_error(LAB_ERR_WAIT_TIMEOUT);
        break;
      }
    }
  }
  // the workers' next meeting (sync_alive) orders everything after the barrier
}

// ---- the loading warp: every weight tile of every item of this CTA, in order ----------------------
__device__ void producer(const StackParams& p, Bars* bars, uint8_t* ring) {
  volatile int* abort_flag = &bars->abort;
  int it = 0;
  bool alive = true;
  for (int ph = p.phase_begin; ph < p.phase_end && alive; ++ph) {
    const int kind = ph % PHASES;
    if (kind == PH_ATTN) continue;
    const LayerParams& L = p.layers[ph / PHASES];
    const Product g = product_of(p, L, kind);
    const int items = g.tiles * g.S;
    for (int item = blockIdx.x; item < items && alive; item += gridDim.x) {
      const int tile = item % g.tiles, split = item / g.tiles;
      const int kt0 = split * g.ktps, kt1 = min(g.k_tiles, kt0 + g.ktps);
      for (int kt = kt0; kt < kt1; ++kt, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(&bars->empty[s], ((it / STAGES) & 1) ^ 1, abort_flag)) {
          alive = false;
          break;
        }
        mbar_expect_tx(&bars->full[s], STAGE_BYTES);
        uint8_t* dst = ring + s * STAGE_BYTES;
        if (g.gated) {
          tma_load_2d(dst, g.map, &bars->full[s], kt * BK, tile * (TM / 2));
          tma_load_2d(dst + (TM / 2) * BK * 2, g.map, &bars->full[s], kt * BK, g.n_out + tile * (TM / 2));
        } else {
          tma_load_2d(dst, g.map, &bars->full[s], kt * BK, tile * TM);
        }
      }
    }
  }
  if (*abort_flag) {
    // Let copies in flight land before the CTA's shared memory goes away.
    const int first = it > STAGES ? it - STAGES : 0;
    for (int i = first; i < it; ++i) {
      const uint64_t t0 = global_timer_ns();
      while (!mbar_try_wait(&bars->full[i % STAGES], (i / STAGES) & 1) && global_timer_ns() - t0 < 100000000ull) {
      }
    }
  }
}

// ---- the activation operand: rows of tokens, K-major, 128-byte swizzle, one k-tile after the other ----
// Row t, 16-byte chunk j of k-tile kt lies at kt * BN * 128 + (t / 8) * 1024 + (t % 8) * 128 + ((j ^ (t % 8)) * 16).
// Half a warp serves a row: its 16 lanes hold the row's chunks (all loads in flight at once), sum the
// squares among themselves, and write the slice's chunks normalised.  `norm_w_s`: the norm's weights,
// staged in shared memory before the phase began.
__device__ void build_operand(const StackParams& p, const Product& g, int kt0, int kt1, uint8_t* work,
                              const __nv_bfloat16* norm_w_s, int wi, int lane) {
  const int chunks_row = g.K / 8;                // 16-byte chunks of a whole row
  const int c0 = kt0 * 8, c1 = kt1 * 8;          // chunks of the slice (beyond the row's end: zeros)
  const int sub = lane >> 4, l16 = lane & 15;    // which of the warp's two rows, and the lane within it
  constexpr int ROWS_AT_ONCE = 2 * (WORKERS / 32);
  for (int t = wi * 2 + sub; t < p.BN; t += ROWS_AT_ONCE) {
    uint8_t* row_base = work + (t >> 3) * 1024 + (t & 7) * 128;
    const int sw = t & 7;
    auto put = [&](int c, uint4 v) {
      const int cc = c - c0;
      *reinterpret_cast<uint4*>(row_base + (cc >> 3) * (p.BN * 128) + (((cc & 7) ^ sw) << 4)) = v;
    };
    const bool real = t < p.T;
    const uint4* src = reinterpret_cast<const uint4*>(g.src + (size_t)(real ? t : 0) * g.K);
    if (!g.norm || !real) {
      for (int c = c0 + l16; c < c1; c += 16) put(c, (real && c < chunks_row) ? __ldcg(src + c) : make_uint4(0, 0, 0, 0));
      if (!g.norm) continue;
    }
    // RMSNorm of the whole row in 32-bit, one rounding at the end; the slice's chunks go to shared memory.
    // (Rows beyond the step's tokens walk along with zeros: the half-warps of a warp shuffle together.)
    uint4 held[MAX_ROW_CHUNKS];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_ROW_CHUNKS; ++i) {
      const int c = l16 + 16 * i;
      held[i] = (real && c < chunks_row) ? __ldcg(src + c) : make_uint4(0, 0, 0, 0);
    }
    const int used = (chunks_row + 15) >> 4;   // chunks a lane really holds
#pragma unroll
    for (int i = 0; i < MAX_ROW_CHUNKS; ++i) {
      if (i >= used) break;
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&held[i]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // within the half-warp
    if (!real) continue;
    const float inv = rsqrtf(ss / (float)g.K + g.eps);
#pragma unroll
    for (int i = 0; i < MAX_ROW_CHUNKS; ++i) {
      const int c = l16 + 16 * i;
      if (16 * i >= c1) break;
      if (c >= c0 && c < c1) {
        uint4 out = make_uint4(0, 0, 0, 0);
        if (c < chunks_row) {
          const uint4 rw = *reinterpret_cast<const uint4*>(norm_w_s + c * 8);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&held[i]);
          const __nv_bfloat162* hw = reinterpret_cast<const __nv_bfloat162*>(&rw);
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]), fw = __bfloat1622float2(hw[e]);
            w[e] = pack_bf16(f.x * inv * fw.x, f.y * inv * fw.y);
          }
          out = make_uint4(w[0], w[1], w[2], w[3]);
        }
        put(c, out);
      }
    }
  }
}

// The weights of the norm that opens phase `ph`, copied into the exchange buffer (free between
// epilogues): asked for before the grid barrier, so that they have arrived when the operand is built.
__device__ __forceinline__ void stage_norm_weights(const StackParams& p, int ph, float* exch, int worker_tid) {
  const int kind = ph % PHASES;
  if (kind != PH_QKV && kind != PH_GATE_UP) return;
  const LayerParams& L = p.layers[ph / PHASES];
  const __nv_bfloat16* w = kind == PH_QKV ? L.norm1 : L.norm2;
  const uint32_t dst = smem_u32(exch);
  for (int c = worker_tid; c < p.hidden / 8; c += WORKERS) cp_async16(dst + c * 16, w + c * 8, true);
  cp_async_commit();
}

// ---- epilogues: 16 tokens of this thread's row of the tile at a time -------------------------------
// x[tok, m] += v (32-bit add, one rounding)
__device__ __forceinline__ void apply_residual(const StackParams& p, int m, int tok0, const float* v) {
  if (m >= p.hidden) return;
  float old[CHUNK];
#pragma unroll
  for (int j = 0; j < CHUNK; ++j)   // every load before the first store: they are independent
    old[j] = tok0 + j < p.T ? ldcg_bf16(p.x + (size_t)(tok0 + j) * p.hidden + m) : 0.f;
#pragma unroll
  for (int j = 0; j < CHUNK; ++j)
    if (tok0 + j < p.T) p.x[(size_t)(tok0 + j) * p.hidden + m] = __float2bfloat16_rn(old[j] + v[j]);
}

// rows 0..63 of the tile are gate values, rows 64..127 the up values of the same 64 features
__device__ __forceinline__ void apply_gate(const StackParams& p, int tile, int row, int tok0, const float* v, float* exch,
                                           bool go) {
#pragma unroll
  for (int j = 0; j < CHUNK; ++j) exch[row * EXCH_STRIDE + j] = v[j];
  named_sync(2, 128);
  const int f = row & 63, half = row >> 6, feature = tile * (TM / 2) + f;
  if (go && feature < p.inter) {
#pragma unroll
    for (int j = 0; j < CHUNK / 2; ++j) {
      const int col = half * (CHUNK / 2) + j, tok = tok0 + col;
      if (tok < p.T)
        p.act[(size_t)tok * p.inter + feature] =
            __float2bfloat16_rn(silu_gate(exch[f * EXCH_STRIDE + col], exch[(64 + f) * EXCH_STRIDE + col]));
    }
  }
  named_sync(2, 128);
}

// bias, rounding, rotation of q and k (the halves of a head meet through the exchange buffer),
// q to its buffer, k and v into their cache slots
__device__ __forceinline__ void apply_qkv(const StackParams& p, const LayerParams& L, int m, int row, int tok0,
                                          const float* v, float* exch, bool go) {
  const int width = (p.n_q + 2 * p.n_kv) * D;
  const float b = (L.bias_qkv != nullptr && m < width) ? __bfloat162float(L.bias_qkv[m]) : 0.f;
#pragma unroll
  for (int j = 0; j < CHUNK; ++j) exch[row * EXCH_STRIDE + j] = round_to<__nv_bfloat16>(v[j] + b);
  named_sync(2, 128);
  if (go && m < width) {
    constexpr int half = D / 2;
    const int head = m / D, jj = m - head * D;
    const bool rotate = head < p.n_q + p.n_kv, is_lo = jj < half, to_cache = head >= p.n_q;
    const bool is_k = head < p.n_q + p.n_kv;
    const float* mine = exch + row * EXCH_STRIDE;
    const float* other = exch + (is_lo ? row + half : row - half) * EXCH_STRIDE;
    if (!to_cache || L.write_kv) {
      const int kvh = is_k ? head - p.n_q : head - p.n_q - p.n_kv;
      const int* slots = p.row_slot[L.group];
      float2 f[CHUNK];
      int slot[CHUNK];
#pragma unroll
      for (int j = 0; j < CHUNK; ++j) {   // angles and slots of the chunk's tokens first, then the stores
        const int tok = min(tok0 + j, p.T - 1);
        f[j] = rotate ? p.table[(size_t)tok * half + (is_lo ? jj : jj - half)] : make_float2(1.f, 0.f);
        slot[j] = to_cache ? slots[tok] : 0;
      }
#pragma unroll
      for (int j = 0; j < CHUNK; ++j) {
        const int tok = tok0 + j;
        if (tok < p.T) {
          float val = mine[j];
          if (rotate) {
            float lo, hi;
            if (is_lo) {
              rope_rotate(val, other[j], f[j].x, f[j].y, lo, hi);
              val = lo;
            } else {
              rope_rotate(other[j], val, f[j].x, f[j].y, lo, hi);
              val = hi;
            }
          }
          if (!to_cache) {
            p.qbuf[(size_t)tok * (p.n_q * D) + m] = __float2bfloat16_rn(val);
          } else if (slot[j] >= 0) {
            const int page = slot[j] / p.page_size, off = slot[j] - page * p.page_size;
            if (page >= p.num_pages) {
              lab_set_error(LAB_ERR_PAGE_RANGE);
            } else {
              __nv_bfloat16* cache = is_k ? L.cache_k : L.cache_v;
              cache[(((size_t)page * p.n_kv + kvh) * p.page_size + off) * D + jj] = __float2bfloat16_rn(val);
            }
          }
        }
      }
    }
  }
  named_sync(2, 128);
}

// ---- one item of a product: MMAs (warp 1) and epilogue (warps 2-5) -------------------------------------
__device__ void product_item(const StackParams& p, const LayerParams& L, const Product& g, int kind, int tile, int split,
                             int n_kt, Bars* bars, uint8_t* ring, uint8_t* work, float* exch, uint32_t tmem_base,
                             int& it, int local, int warp, int lane) {
  volatile int* abort_flag = &bars->abort;
  const int buf = local & 1;
  const uint32_t use = (uint32_t)(local >> 1);
  if (warp == 1) {
    const uint32_t idesc = umma_instr_desc(TM, p.BN);
    bool ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_empty[buf], (use & 1) ^ 1, abort_flag));
    tc_fence_after();
    const uint32_t acc = tmem_base + buf * 64;
    for (int kt = 0; kt < n_kt && ok; ++kt, ++it) {
      const int s = it % STAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->full[s], (it / STAGES) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint64_t desc_a = smem_desc_sw128(smem_u32(ring + s * STAGE_BYTES));
      const uint64_t desc_b = smem_desc_sw128(smem_u32(work + kt * p.BN * 128));
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16(acc, desc_a + 2 * k, desc_b + 2 * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
      umma_commit(&bars->empty[s]);
    }
    if (ok) umma_commit(&bars->acc_full[buf]);
    return;
  }
  if (warp < 2 || warp > 5) return;
  const int quarter = warp & 3, row = quarter * 32 + lane;
  const bool ok = mbar_wait(&bars->acc_full[buf], use & 1, abort_flag);
  tc_fence_after();
  const bool go = __all_sync(0xffffffffu, ok && !*abort_flag);
  const uint32_t lane_addr = tmem_base + buf * 64 + ((uint32_t)(quarter * 32) << 16);
  const int n_chunks = (p.T + CHUNK - 1) / CHUNK;
  const int m = g.gated ? 0 : tile * TM + row;   // this thread's output feature (gated: by the exchange)
  auto apply = [&](int c, const float* v, bool live) {
    if (kind == PH_QKV) apply_qkv(p, L, m, row, c * CHUNK, v, exch, live);
    else if (kind == PH_GATE_UP) apply_gate(p, tile, row, c * CHUNK, v, exch, live);
    else if (live) apply_residual(p, m, c * CHUNK, v);
  };
  auto release = [&]() {   // the accumulator has been read: the MMA warp may overwrite it
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
  };
  if (g.S == 1) {
    for (int c = 0; c < n_chunks; ++c) {
      float v[CHUNK];
      if (go) tmem_ld16(lane_addr + c * CHUNK, v);
      else
#pragma unroll
        for (int j = 0; j < CHUNK; ++j) v[j] = 0.f;
      if (c == n_chunks - 1) release();
      apply(c, v, go);
    }
    return;
  }
  // several slices of K: leave this slice's partial sums, count, and let the last one finish the tile
  float* mine = p.partial + ((size_t)(tile * g.S + split) * TM + row) * p.BN;
  for (int c = 0; c < n_chunks && go; ++c) {
    float v[CHUNK];
    tmem_ld16(lane_addr + c * CHUNK, v);
#pragma unroll
    for (int q4 = 0; q4 < CHUNK / 4; ++q4)
      reinterpret_cast<float4*>(mine + c * CHUNK)[q4] = make_float4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
  }
  release();
  __threadfence();
  named_sync(2, 128);
  if (threadIdx.x == 64) {
    int last = 0;
    if (go) {
      int* counter = p.counters + g.counter_base + tile;
      last = atomicAdd(counter, 1) == g.S - 1;
      if (last) *counter = 0;   // zero again for the next use
    }
    bars->flag = last;
  }
  named_sync(2, 128);
  if (bars->flag == 0) return;   // the same for all four epilogue warps
  __threadfence();
  for (int c = 0; c < n_chunks; ++c) {
    float v[CHUNK];
#pragma unroll
    for (int j = 0; j < CHUNK; ++j) v[j] = 0.f;
    for (int s0 = 0; s0 < g.S; s0 += 4) {   // four slices' loads in flight, summed in ascending order
      float4 f[4][CHUNK / 4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float4* from = reinterpret_cast<const float4*>(
            p.partial + ((size_t)(tile * g.S + min(s0 + u, g.S - 1)) * TM + row) * p.BN + c * CHUNK);
#pragma unroll
        for (int q4 = 0; q4 < CHUNK / 4; ++q4) f[u][q4] = __ldcg(from + q4);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u < g.S) {
#pragma unroll
          for (int q4 = 0; q4 < CHUNK / 4; ++q4) {
            v[4 * q4] += f[u][q4].x;
            v[4 * q4 + 1] += f[u][q4].y;
            v[4 * q4 + 2] += f[u][q4].z;
            v[4 * q4 + 3] += f[u][q4].w;
          }
        }
      }
    }
    apply(c, v, true);
  }
}

// ---- attention of one (request, kv head x tile of 16 query heads, split of the keys) ---------------------
__device__ void attention_item(const StackParams& p, const LayerParams& L, int b, int y, int split, uint8_t* work,
                               Bars* bars, int aw, int lane) {
  const int threads = AW * 32, tid = aw * 32 + lane;
  const int qs = p.q_start[b];
  const int group = p.n_q / p.n_kv, m_tiles = (group + 15) / 16;
  const int kvh = y / m_tiles, mt = y - kvh * m_tiles;
  const int kvl = p.kv_len[b];
  const int first = L.window > 0 ? max(0, kvl - L.window) : 0;
  const int* bt = p.block_table[L.group] + (size_t)b * p.max_blocks[L.group];
  const int head0 = kvh * group + mt * 16, n_heads = min(16, group - mt * 16);
  const int splits = p.att_splits;
  const int start = (first / AT_BN) * AT_BN;
  const int total_tiles = kvl > start ? (kvl - start + AT_BN - 1) / AT_BN : 0;
  const int tiles_per_split = (total_tiles + splits - 1) / splits;
  const int tile_lo = split * tiles_per_split, tile_hi = min(total_tiles, tile_lo + tiles_per_split);
  const int n_qd = p.n_q * D;

  const uint32_t ring = smem_u32(work) + aw * AT_WARP_BYTES;
  auto issue = [&](int t, int stage) {
    const uint32_t kd = ring + stage * 2 * AT_TILE_BYTES;
    load_kv_rows_warp<AT_BN>(kd, kd + AT_TILE_BYTES, L.cache_k, L.cache_v, bt, start + t * AT_BN, first, kvl, kvh, p.n_kv,
                             p.page_size, p.num_pages, lane);
  };
  int t_issue = tile_lo + aw;
  for (int staged = 0; staged < AT_STAGES - 1; ++staged) {
    if (t_issue < tile_hi) issue(t_issue, staged);
    cp_async_commit();
    t_issue += AW;
  }
  // q fragments from the buffer the projection's epilogue filled (other SMs wrote it: not through L1)
  uint32_t qf[KSTEPS][4];
  {
    const __nv_bfloat16* qrow = p.qbuf + (size_t)qs * n_qd;
    const int ra = lane >> 2, rb = ra + 8;
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
      const int c = k * 16 + 2 * (lane & 3);
      const uint32_t* pa = reinterpret_cast<const uint32_t*>(qrow + (size_t)(head0 + ra) * D + c);
      const uint32_t* pb = reinterpret_cast<const uint32_t*>(qrow + (size_t)(head0 + rb) * D + c);
      qf[k][0] = ra < n_heads ? __ldcg(pa) : 0u;
      qf[k][1] = rb < n_heads ? __ldcg(pb) : 0u;
      qf[k][2] = ra < n_heads ? __ldcg(pa + 4) : 0u;
      qf[k][3] = rb < n_heads ? __ldcg(pb + 4) : 0u;
    }
  }
  float o[DTILES][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
  for (int t = 0; t < DTILES; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[t][e] = 0.f;
  const int lo[2] = {first, first}, hi[2] = {kvl - 1, kvl - 1};
  int stage = 0;
  for (int t = tile_lo + aw; t < tile_hi; t += AW) {
    const int pre_stage = (stage + AT_STAGES - 1) % AT_STAGES;
    if (t_issue < tile_hi) issue(t_issue, pre_stage);
    cp_async_commit();
    t_issue += AW;
    cp_async_wait<AT_STAGES - 1>();
    __syncwarp();
    const uint32_t kd = ring + stage * 2 * AT_TILE_BYTES;
    const int key0 = start + t * AT_BN;
    tile_step<AT_BN>(qf, kd, kd + AT_TILE_BYTES, o, m, l, key0, lo, hi, p.scale_log2, lane,
                     key0 >= first && key0 + AT_BN <= kvl);
    __syncwarp();
    stage = (stage + 1) % AT_STAGES;
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  named_sync(3, threads);   // every warp is done with its ring: the memory is reused for the merge
  float* all = reinterpret_cast<float*>(work);
  float* mg = all + aw * 16 * (D + 2);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = (lane >> 2) + 8 * r;
#pragma unroll
    for (int t = 0; t < DTILES; ++t) {
      mg[row * (D + 2) + t * 8 + 2 * (lane & 3)] = o[t][2 * r];
      mg[row * (D + 2) + t * 8 + 2 * (lane & 3) + 1] = o[t][2 * r + 1];
    }
    if ((lane & 3) == 0) {
      mg[row * (D + 2) + D] = m[r];
      mg[row * (D + 2) + D + 1] = l[r];
    }
  }
  named_sync(3, threads);
  for (int i = tid; i < n_heads * D; i += threads) {
    const int row = i / D, dim = i - row * D;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < AW; ++w) big = fmaxf(big, all[(w * 16 + row) * (D + 2) + D]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < AW; ++w) {
      const float mw = all[(w * 16 + row) * (D + 2) + D];
      const float wt = (mw == -INFINITY) ? 0.f : fast_exp2(mw - big);
      num += wt * all[(w * 16 + row) * (D + 2) + dim];
      den += wt * all[(w * 16 + row) * (D + 2) + D + 1];
    }
    const int head = head0 + row;
    if (splits == 1) {
      p.attn[(size_t)qs * n_qd + (size_t)head * D + dim] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    } else {
      const size_t slot = ((size_t)b * p.n_q + head) * splits + split;
      p.att_acc[slot * D + dim] = num;
      if (dim == 0) {
        p.att_ml[slot * 2] = big;
        p.att_ml[slot * 2 + 1] = den;
      }
    }
  }
  if (splits > 1) {
    // the split that finishes last for this (request, kv head, tile of heads) merges them all, in ascending order
    __threadfence();
    named_sync(3, threads);
    if (tid == 0) {
      int* counter = p.counters + 4096 + b * (p.n_kv * m_tiles) + y;
      const int last = atomicAdd(counter, 1) == splits - 1;
      if (last) *counter = 0;
      bars->flag = last;
    }
    named_sync(3, threads);
    if (bars->flag) {
      __threadfence();
      for (int i = tid; i < n_heads * D; i += threads) {
        const int row = i / D, dim = i - row * D;
        const size_t slot0 = ((size_t)b * p.n_q + head0 + row) * splits;
        float ms[MAX_ATT_SPLITS], acc[MAX_ATT_SPLITS], ls[MAX_ATT_SPLITS];
#pragma unroll
        for (int sp = 0; sp < MAX_ATT_SPLITS; ++sp) {   // every load first, then the sum in ascending order
          const bool in = sp < splits;
          ms[sp] = in ? __ldcg(p.att_ml + (slot0 + sp) * 2) : -INFINITY;
          ls[sp] = in ? __ldcg(p.att_ml + (slot0 + sp) * 2 + 1) : 0.f;
          acc[sp] = in ? __ldcg(p.att_acc + (slot0 + sp) * D + dim) : 0.f;
        }
        float big = -INFINITY;
#pragma unroll
        for (int sp = 0; sp < MAX_ATT_SPLITS; ++sp) big = fmaxf(big, ms[sp]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int sp = 0; sp < MAX_ATT_SPLITS; ++sp) {
          const float wt = (ms[sp] == -INFINITY) ? 0.f : fast_exp2(ms[sp] - big);
          num += wt * acc[sp];
          den += wt * ls[sp];
        }
        p.attn[(size_t)qs * n_qd + (size_t)(head0 + row) * D + dim] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
      }
    }
  }
  named_sync(3, threads);   // rings, merge area and flag are free for the next item
}

// ---- every warp but the loading one ------------------------------------------------------------------------
__device__ void worker(const StackParams& p, Bars* bars, uint8_t* ring, uint8_t* work, float* exch, uint32_t tmem_base,
                       int warp, int lane) {
  unsigned gen = 0;   // barriers passed so far
  int it = 0, local = 0, parity = 0;
  for (int ph = p.phase_begin; ph < p.phase_end; ++ph) {
    stage_norm_weights(p, ph, exch, threadIdx.x - 32);   // the exchange buffer is idle between phases
    if (ph > p.phase_begin) grid_barrier(p, bars, gen);
    cp_async_wait<0>();
    if (!sync_alive(bars, parity)) break;
    const bool stamping = p.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 32;
    unsigned long long* stamp = p.stamps + 4 * (ph - p.phase_begin);
    if (stamping) stamp[0] = global_timer_ns();
    const int kind = ph % PHASES;
    const LayerParams& L = p.layers[ph / PHASES];
    if (kind == PH_ATTN) {
      if (warp >= 2 && warp < 2 + AW) {
        const int m_tiles = (p.n_q / p.n_kv + 15) / 16, Y = p.n_kv * m_tiles;
        const int items = p.T * Y * p.att_splits;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
          const int split = item % p.att_splits, rest = item / p.att_splits;
          attention_item(p, L, rest / Y, rest % Y, split, work, bars, warp - 2, lane);
        }
      }
      if (stamping) stamp[3] = global_timer_ns();
      continue;
    }
    const Product g = product_of(p, L, kind);
    const int items = g.tiles * g.S;
    bool alive = true;
    for (int item = blockIdx.x; item < items && alive; item += gridDim.x, ++local) {
      const int tile = item % g.tiles, split = item / g.tiles;
      const int kt0 = split * g.ktps, kt1 = min(g.k_tiles, kt0 + g.ktps);
      if (item != (int)blockIdx.x && g.norm) {   // the epilogue before this item used the exchange buffer
        stage_norm_weights(p, ph, exch, threadIdx.x - 32);
        cp_async_wait<0>();
        named_sync(1, WORKERS);
      }
      build_operand(p, g, kt0, kt1, work, reinterpret_cast<const __nv_bfloat16*>(exch), warp - 1, lane);
      proxy_fence();
      alive = sync_alive(bars, parity);
      if (stamping && item == (int)blockIdx.x) stamp[1] = global_timer_ns();
      if (alive) product_item(p, L, g, kind, tile, split, kt1 - kt0, bars, ring, work, exch, tmem_base, it, local, warp, lane);
      // the operand may be rebuilt only when the MMAs that read it have retired: the epilogue
      // warps get here after they have seen the accumulator complete
      alive = sync_alive(bars, parity) && alive;
      if (stamping && item == (int)blockIdx.x) stamp[2] = global_timer_ns();
    }
    if (stamping) stamp[3] = global_timer_ns();
    if (p.stamps != nullptr && threadIdx.x == 32)   // every CTA: when its share of the phase was done
      p.stamps[4 * (p.phase_end - p.phase_begin) + 1 + (size_t)(ph - p.phase_begin) * gridDim.x + blockIdx.x] = global_timer_ns();
    if (!alive) break;
  }
  if (p.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 32) p.stamps[4 * (p.phase_end - p.phase_begin)] = global_timer_ns();
}

__global__ void __launch_bounds__(THREADS, 1) decode_stack_kernel(const __grid_constant__ StackParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Bars* bars = reinterpret_cast<Bars*>(smem + OFF_BAR);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->acc_full[a], 1);
      mbar_init(&bars->acc_empty[a], 4);  // one arrival per epilogue warp
    }
    bars->abort = 0;
    bars->snap[0] = bars->snap[1] = 0;
    bars->flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(&bars->tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_slot;
  if (warp == 0) {
    if (lane == 0) producer(p, bars, smem + OFF_RING);
  } else {
    worker(p, bars, smem + OFF_RING, smem + OFF_WORK, reinterpret_cast<float*>(smem + OFF_EXCH), tmem_base, warp, lane);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

LAB_EXPORT int lab_decode_stack_head_dim() { return D; }
LAB_EXPORT int lab_decode_stack_layer_bytes() { return (int)sizeof(LayerParams); }
LAB_EXPORT int lab_decode_stack_work_bytes() { return WORK_BYTES; }
LAB_EXPORT int lab_decode_stack_max_hidden() { return MAX_ROW_CHUNKS * 16 * 8; }

// Fills one LayerParams (in host memory; the caller copies the array to the device).  Weights are
// contiguous bfloat16 matrices [rows, K]: w_qkv [(n_q + 2 n_kv) * D, hidden], w_o [hidden, n_q * D],
// w_gate_up [2 * inter, hidden] (gate rows, then up rows), w_down [hidden, inter].
LAB_EXPORT int lab_decode_stack_layer(void* dst, const void* w_qkv, const void* w_o, const void* w_gate_up,
                                      const void* w_down, const void* norm1, const void* norm2, const void* bias_qkv,
                                      void* cache_k, void* cache_v, int hidden, int n_q, int n_kv, int inter, float eps1,
                                      float eps2, int group, int window, int write_kv) {
  if (hidden % 8 || inter % 8 || group < 0 || group >= MAX_GROUPS) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)w_qkv) | ((uintptr_t)w_o) | ((uintptr_t)w_gate_up) | ((uintptr_t)w_down) | ((uintptr_t)norm1) |
       ((uintptr_t)norm2)) & 15)
    return (int)cudaErrorInvalidValue;
  LayerParams L = {};
  int rc;
  if ((rc = lab_make_map_bf16(&L.map_qkv, w_qkv, (long long)(n_q + 2 * n_kv) * D, hidden, hidden, TM))) return rc;
  if ((rc = lab_make_map_bf16(&L.map_o, w_o, hidden, (long long)n_q * D, (long long)n_q * D, TM))) return rc;
  if ((rc = lab_make_map_bf16(&L.map_gate_up, w_gate_up, 2ll * inter, hidden, hidden, TM / 2))) return rc;
  if ((rc = lab_make_map_bf16(&L.map_down, w_down, hidden, inter, inter, TM))) return rc;
  L.norm1 = (const __nv_bfloat16*)norm1;
  L.norm2 = (const __nv_bfloat16*)norm2;
  L.bias_qkv = (const __nv_bfloat16*)bias_qkv;
  L.cache_k = (__nv_bfloat16*)cache_k;
  L.cache_v = (__nv_bfloat16*)cache_v;
  L.eps1 = eps1;
  L.eps2 = eps2;
  L.group = group;
  L.window = window;
  L.write_kv = write_kv;
  memcpy(dst, &L, sizeof(L));
  return 0;
}

// How many CTAs of the stack kernel the device holds at once (one per SM): the size of its grid.
LAB_EXPORT int lab_decode_stack_grid() {
  static int grid = 0;
  if (grid == 0) {
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return 0;
    if (cudaFuncSetAttribute(decode_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_kernel, THREADS, SMEM) != cudaSuccess ||
        per_sm < 1)
      return 0;
    grid = sms;
  }
  return grid;
}

// Runs phases [phase_begin, phase_end) of the stack (5 per layer).  ints: T, BN, hidden, n_q, n_kv, inter,
// s_qkv, s_o, s_gate_up, s_down, att_splits, page_size, num_pages, n_groups, then per group max_blocks.
// ptrs: layers, x, qbuf, attn, act, partial, att_acc, att_ml, counters, barrier, table, q_start, kv_len,
// stamps (may be null), then per group row_slot, then per group block_table.
LAB_EXPORT int lab_decode_stack(const void* const* ptrs, const int* ints, int n_layers, int phase_begin, int phase_end,
                                float scale, cudaStream_t stream) {
  const int grid = lab_decode_stack_grid();
  if (grid <= 0) return (int)cudaErrorLaunchOutOfResources;
  StackParams p = {};
  p.n_layers = n_layers;
  p.phase_begin = phase_begin;
  p.phase_end = phase_end;
  p.T = ints[0];
  p.BN = ints[1];
  p.hidden = ints[2];
  p.n_q = ints[3];
  p.n_kv = ints[4];
  p.inter = ints[5];
  p.s_qkv = ints[6];
  p.s_o = ints[7];
  p.s_gate_up = ints[8];
  p.s_down = ints[9];
  p.att_splits = ints[10];
  p.page_size = ints[11];
  p.num_pages = ints[12];
  const int n_groups = ints[13];
  if (n_groups < 1 || n_groups > MAX_GROUPS) return (int)cudaErrorInvalidValue;
  if (p.T < 1 || p.T > 64 || (p.BN != 16 && p.BN != 32 && p.BN != 64) || p.BN < p.T) return (int)cudaErrorInvalidValue;
  if (phase_begin < 0 || phase_end > n_layers * PHASES || phase_begin >= phase_end) return (int)cudaErrorInvalidValue;
  if (p.hidden % 8 || p.hidden / 8 > MAX_ROW_CHUNKS * 16 || p.hidden * 2 > EXCH_BYTES || p.n_q % p.n_kv) return (int)cudaErrorInvalidValue;
  for (int s : {p.s_qkv, p.s_o, p.s_gate_up, p.s_down, p.att_splits})
    if (s < 1) return (int)cudaErrorInvalidValue;
  // the operand of an item (its slice of K for BN rows) must fit the work area, and no slice may be empty
  const int ks[4] = {p.hidden, p.n_q * D, p.hidden, p.inter};
  const int ss[4] = {p.s_qkv, p.s_o, p.s_gate_up, p.s_down};
  for (int i = 0; i < 4; ++i) {
    const int k_tiles = (ks[i] + BK - 1) / BK, ktps = (k_tiles + ss[i] - 1) / ss[i];
    if (ktps * p.BN * 128 > WORK_BYTES || (ss[i] - 1) * ktps >= k_tiles) return (int)cudaErrorInvalidValue;
  }
  p.layers = (const LayerParams*)ptrs[0];
  p.x = (__nv_bfloat16*)ptrs[1];
  p.qbuf = (__nv_bfloat16*)ptrs[2];
  p.attn = (__nv_bfloat16*)ptrs[3];
  p.act = (__nv_bfloat16*)ptrs[4];
  p.partial = (float*)ptrs[5];
  p.att_acc = (float*)ptrs[6];
  p.att_ml = (float*)ptrs[7];
  p.counters = (int*)ptrs[8];
  p.barrier = (unsigned*)ptrs[9];
  p.table = (const float2*)ptrs[10];
  p.q_start = (const int*)ptrs[11];
  p.kv_len = (const int*)ptrs[12];
  p.stamps = (unsigned long long*)ptrs[13];
  for (int g = 0; g < n_groups; ++g) {
    p.row_slot[g] = (const int*)ptrs[14 + g];
    p.block_table[g] = (const int*)ptrs[14 + n_groups + g];
    p.max_blocks[g] = ints[14 + g];
  }
  p.scale_log2 = scale * LOG2E;
  if (p.att_splits > MAX_ATT_SPLITS) return (int)cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(p.barrier, 0, 2 * BAR_WORDS * sizeof(unsigned), stream);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // every CTA resident at once: the grid barrier relies on it
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, decode_stack_kernel, p);
}
