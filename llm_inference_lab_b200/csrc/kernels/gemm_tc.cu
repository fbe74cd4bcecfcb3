// Matrix product on the 5th-generation tensor cores of sm_100a: TMA loads into
// 128-byte-swizzled shared memory, tcgen05.mma with the accumulator in tensor memory,
// tcgen05.ld for the epilogue.
//
//   out[t, n] = OutT( sum_k x[t, k] * w[n, k]  (+ bias[n]) )                 w is [out, in]
//   gated:      out[t, n] = T( silu(g) * u ),  g = x . w[n], u = x . w[inter + n]   (32-bit, one rounding)
//   split-K:    partial[z, t, n] = sum over the z-th slice of k   (32-bit, summed by the
//               kernel that consumes it, in a fixed order)
//   pick:       the output head of a step that wants tokens, not logits: every tile keeps, per
//               token, its best candidate (the logit, or logit / temperature + Gumbel noise) and
//               a second, tiny kernel picks each token's best over all tiles; the logits are
//               never written (kernels.rs:1489-1552 is the reference's two-stage arg-max over
//               logits it has stored)
//   q/k/v:      the fused projection of an attention layer with its epilogue: bias, rounding,
//               split-half rotary encoding of the q and k heads with cosines and sines from the
//               step's table, q to the activation, k and v straight into their cache pages
//               (rust/engine/src/runner/model/qwen2/kernels.rs:240-284 packed projection, 587-631
//               rotation, 635-698 cache store: three launches there, one here)
//
// Both operands are K-major bfloat16 ([rows, K] row-major), which is how activations and
// checkpoint weights ([out, in]) already lie, so nothing is transposed.  The operand on the
// M side of the MMA is cut in tiles of 128 rows, the one on the N side in tiles of BN rows.
// "Normal" orientation puts tokens on M and output features on N (prefill: many tokens);
// "swapped" puts output features on M and the few tokens of a decode step on N, so that a
// step with 1..256 tokens still fills the 128-row MMA and streams every weight once.
//
// Gated product: the weight matrix holds the gate rows, then the up rows.  In normal
// orientation a tile's N side is half gate rows, half up rows (two TMA loads), so a thread's
// accumulator row holds both; in swapped orientation a tile's M side is 64 gate rows over 64 up
// rows of the same features, and the epilogue warps exchange them through shared memory.
// The q/k/v epilogue needs a head whole inside a tile (heads of 64 or 128) and runs in normal
// orientation: a thread holds a token's row and rotates pairs of its own columns.  (Steps of few
// tokens keep the plain product with K in slices and the rotation kernel that sums them: in swapped
// orientation the epilogue measured slower both with nine CTAs that walk the whole of K, 0.875
// against 0.80 ms a decode step at batch 8, and with K in slices and the last CTA of a tile rotating
// and storing for all its tokens, 0.90 ms.  Nor did it pay to sum the slices of K inside a thread-block
// cluster, the other ranks' accumulators added on rank 0 through distributed shared memory so that the
// product leaves the kernel finished: at batch 8 a decode step took 0.807 ms with gate/up cut in two,
// 0.802 with q/k/v in four, 0.833 with the output projection in four and 0.870 with down in eight,
// against 0.785 ms with 32-bit partial products in global memory that the consuming kernel sums.)
//
// CTAs are persistent (one per SM at most) and walk the output tiles: warp 0 issues TMA loads
// into a ring of stages that runs on across tiles, warp 1 issues the MMAs (one elected lane)
// into one of two accumulators in tensor memory and owns the allocation, warps 2-5 read an
// accumulator back (each its quarter of the 128 lanes) and apply the epilogue while the MMAs
// of the next tile fill the other accumulator.  Every
// wait on an mbarrier is bounded: when it runs out the kernel records an error code, lets
// the other roles drain and frees its tensor memory before it returns.
//
// Formulas and rounding order: rust/engine/src/runner/model/qwen2/kernels.rs:156-178,
// 393-418 (32-bit accumulation, bias added in 32-bit, one rounding), 422-448 and 1469-1486
// (gate/up with the SiLU product), 300-387 (split-K partials merged in 32-bit).
#include <limits.h>

#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;  // rows of the M-side tile (UMMA M)
constexpr int BK = 64;   // bf16 elements per k-tile: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;

enum Mode : int { PLAIN = 0, GATED_SILU = 1, QKV_ROPE = 2, PICK = 3 };

// Where the q/k/v epilogue finds its angles and puts its results.
struct QkvStore {
  __nv_bfloat16* cache_k;   // [num_pages, n_kv, page_size, d]; null: this call does not write the cache
  __nv_bfloat16* cache_v;
  const int* row_slot;      // [tokens] page * page_size + offset of each row's key and value, -1: none
  const float2* table;      // [tokens, d / 2] (cos, sin) of position * inv_freq
  int n_q, n_kv, d, page_size, num_pages;
};

// What the picking head needs: one token per row, greedy where the temperature is 0 (ties to the
// smallest index, a NaN never wins, a row of NaNs gives INT32_MAX), else Gumbel-max with the hash of
// (seed, position, index) the sampling kernel uses.
struct PickArgs {
  int* tokens;                 // [rows] out
  const float* temperature;    // [rows] or null (greedy)
  const uint32_t* seeds;       // [rows]
  const int* positions;        // [rows]
  float* part_val;             // [rows, m_tiles] best candidate of each tile
  int* part_idx;
};

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

struct Params {
  void* out;            // [tokens, ld_out] of OutT, or partial [splits, tokens, ld_out] floats;
                        // q/k/v: the rotated q [tokens, ld_out]
  const __nv_bfloat16* bias;
  int m_rows;           // valid rows on the M side (tokens, or features when swapped)
  int n_rows;           // valid rows on the N side
  int ld_out;
  long long split_stride;  // elements between split-K partial planes (0: no split)
  int k_tiles;          // k-tiles in total
  int k_tiles_per_split;
  int up_offset;        // gated: row offset of the "up" half inside the weight matrix
  int m_tiles, n_tiles, splits;  // tiles on the M side, on the N side, and split-K planes
  QkvStore qkv;         // q/k/v epilogue only
  PickArgs pick;        // picking head only
};

// Element offset of (slot, kv head) in a cache of [pages, n_kv, page_size, d], or -1 (no slot; a
// slot outside the pool also sets the error word).
__device__ __forceinline__ long long cache_row_offset(const QkvStore& e, int slot, int kvh) {
  if (slot < 0) return -1;
  const int page = slot / e.page_size, off = slot - page * e.page_size;
  if (page >= e.num_pages) {
    lab_set_error(LAB_ERR_PAGE_RANGE);
    return -1;
  }
  return (((long long)page * e.n_kv + kvh) * e.page_size + off) * e.d;
}

// Normal orientation: this thread holds 32 consecutive "lo" columns and the 32 "hi" columns that pair
// with them (d / 2 further on) of token row m, of head `head` (q heads, then k heads, then v heads),
// from column `j0` of the head on.  Adds the bias, rounds (the value the projection alone would have
// stored), rotates q and k, rounds again and stores 2 x 64 bytes.
__device__ __forceinline__ void qkv_store_row(const Params& p, int m, int head, int j0, const uint32_t* rlo,
                                              const uint32_t* rhi) {
  const QkvStore& e = p.qkv;
  const int half = e.d / 2, col_lo = head * e.d + j0, col_hi = col_lo + half;
  __nv_bfloat16* dst;
  if (head < e.n_q) {
    dst = (__nv_bfloat16*)p.out + (size_t)m * p.ld_out + col_lo;
  } else {
    if (e.cache_k == nullptr) return;
    const bool is_k = head < e.n_q + e.n_kv;
    const long long at = cache_row_offset(e, e.row_slot[m], is_k ? head - e.n_q : head - e.n_q - e.n_kv);
    if (at < 0) return;
    dst = (is_k ? e.cache_k : e.cache_v) + at + j0;
  }
  const bool rotate = head < e.n_q + e.n_kv;
  const float2* cs = e.table + (size_t)m * half + j0;
#pragma unroll
  for (int q4 = 0; q4 < 4; ++q4) {
    uint32_t wl[4], wh[4];
    uint4 bl = make_uint4(0, 0, 0, 0), bh = bl;
    if (p.bias) {
      bl = reinterpret_cast<const uint4*>(p.bias + col_lo)[q4];
      bh = reinterpret_cast<const uint4*>(p.bias + col_hi)[q4];
    }
    const __nv_bfloat162* hbl = reinterpret_cast<const __nv_bfloat162*>(&bl);
    const __nv_bfloat162* hbh = reinterpret_cast<const __nv_bfloat162*>(&bh);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 fbl = __bfloat1622float2(hbl[k]), fbh = __bfloat1622float2(hbh[k]);
      float lo[2], hi[2];
      lo[0] = round_to<__nv_bfloat16>(__uint_as_float(rlo[q4 * 8 + 2 * k]) + fbl.x);
      lo[1] = round_to<__nv_bfloat16>(__uint_as_float(rlo[q4 * 8 + 2 * k + 1]) + fbl.y);
      hi[0] = round_to<__nv_bfloat16>(__uint_as_float(rhi[q4 * 8 + 2 * k]) + fbh.x);
      hi[1] = round_to<__nv_bfloat16>(__uint_as_float(rhi[q4 * 8 + 2 * k + 1]) + fbh.y);
      if (rotate) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const float2 f = cs[q4 * 8 + 2 * k + u];
          rope_rotate(lo[u], hi[u], f.x, f.y, lo[u], hi[u]);
        }
      }
      wl[k] = pack_bf16(lo[0], lo[1]);
      wh[k] = pack_bf16(hi[0], hi[1]);
    }
    reinterpret_cast<uint4*>(dst)[q4] = make_uint4(wl[0], wl[1], wl[2], wl[3]);
    reinterpret_cast<uint4*>(dst + half)[q4] = make_uint4(wh[0], wh[1], wh[2], wh[3]);
  }
}

template <int MODE, int BN, bool SWAP>
struct Shape {
  static constexpr int TM = BM;
  static constexpr int A_BYTES = TM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // swapped, gated or picking: the epilogue warps exchange rows of the tile through a buffer of their own
  static constexpr int EXCHANGE_BYTES = ((MODE == GATED_SILU || MODE == PICK) && SWAP) ? ((TM * (BN + 1) * 4 + 1023) / 1024) * 1024 : 0;
  static_assert(MODE != PICK || SWAP, "the picking head runs with the vocabulary on the 128-row side");
  static_assert(MODE != QKV_ROPE || !SWAP, "the q/k/v epilogue runs with tokens on the 128-row side");
  static constexpr int STAGES_RAW = (SMEM_BUDGET - EXCHANGE_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 10 ? 10 : STAGES_RAW;
  static constexpr int ACC_COLS = BN < 32 ? 32 : BN;
  static constexpr int ACC_BUFS = 2 * ACC_COLS <= 512 ? 2 : 1;  // accumulators in tensor memory
  static constexpr int TMEM_COLS = ACC_BUFS * ACC_COLS;         // a power of two >= 32
  static constexpr int SMEM = STAGES * STAGE_BYTES + EXCHANGE_BYTES + 1024 /*align*/ + 512 /*barriers*/;
  static_assert(STAGES >= 2, "the tile does not leave room for a pipeline");
  static_assert((2 * STAGES + 4) * 8 + 8 <= 512, "the barriers outgrow their 512 bytes");
};

// A persistent CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  Tiles are numbered with
// the M side fastest, so CTAs that run at the same time share the N-side operand in L2.
// Two accumulators in tensor memory let the epilogue of one tile run beside the MMAs of the next.
template <int MODE, int BN, bool SWAP, typename OutT>
__global__ void __launch_bounds__(THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                          const __grid_constant__ CUtensorMap map_b, Params p) {
  using S = Shape<MODE, BN, SWAP>;
  constexpr int TM = BM;
  constexpr bool GATED = MODE == GATED_SILU;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* exchange = reinterpret_cast<float*>(tiles + S::STAGES * S::STAGE_BYTES);
  uint64_t* full = (uint64_t*)(tiles + S::STAGES * S::STAGE_BYTES + S::EXCHANGE_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_full = empty + S::STAGES;       // [ACC_BUFS]
  uint64_t* acc_empty = acc_full + 2;           // [ACC_BUFS]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int M_ROWS = (GATED && SWAP) ? TM / 2 : TM;    // output rows per tile on the M side
  constexpr int N_ROWS = (GATED && !SWAP) ? BN / 2 : BN;   // rows of the N-side operand per tile
  const int total_tiles = p.m_tiles * p.n_tiles * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile index -> (row on the M side, row on the N side, first k-tile, number of k-tiles)
  auto locate = [&](int tile, int& m0, int& n0, int& kt0, int& n_kt, int& split) {
    const int mt = tile % p.m_tiles;
    const int rest = tile / p.m_tiles;
    const int nt = rest % p.n_tiles;
    split = rest / p.n_tiles;
    m0 = mt * M_ROWS;
    n0 = nt * N_ROWS;
    kt0 = split * p.k_tiles_per_split;
    int kt1 = kt0 + p.k_tiles_per_split;
    if (kt1 > p.k_tiles) kt1 = p.k_tiles;
    n_kt = kt1 > kt0 ? kt1 - kt0 : 0;
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: TMA loads ----
      // Weights do not depend on earlier kernels of the step: the first stages' weight tiles are
      // requested before the wait on the predecessor, the activation tiles after it.
      auto load_weights = [&](int s, int kx, int m0, int n0) {
        uint8_t* a_dst = tiles + s * S::STAGE_BYTES;
        uint8_t* b_dst = a_dst + S::A_BYTES;
        if (SWAP) {
          tma_load_2d(a_dst, &map_a, &full[s], kx, m0);
          if (GATED) tma_load_2d(a_dst + (TM / 2) * BK * 2, &map_a, &full[s], kx, p.up_offset + m0);
        } else {
          tma_load_2d(b_dst, &map_b, &full[s], kx, n0);
          if (GATED) tma_load_2d(b_dst + (BN / 2) * BK * 2, &map_b, &full[s], kx, p.up_offset + n0);
        }
      };
      auto load_activations = [&](int s, int kx, int m0, int n0) {
        uint8_t* a_dst = tiles + s * S::STAGE_BYTES;
        if (SWAP) tma_load_2d(a_dst + S::A_BYTES, &map_b, &full[s], kx, n0);
        else tma_load_2d(a_dst, &map_a, &full[s], kx, m0);
      };
      int it = 0;  // stages filled so far, over all tiles
      bool first_tile = true, alive = true;
      for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
        int m0, n0, kt0, n_kt, split;
        locate(tile, m0, n0, kt0, n_kt, split);
        int i = 0;
        if (first_tile) {
          const int ahead = n_kt < S::STAGES ? n_kt : S::STAGES;
          for (; i < ahead; ++i) {  // the ring is empty: no wait
            mbar_expect_tx(&full[i], S::STAGE_BYTES);
            load_weights(i, (kt0 + i) * BK, m0, n0);
          }
          pdl_wait();
          for (int j = 0; j < ahead; ++j) load_activations(j, (kt0 + j) * BK, m0, n0);
          it = ahead;
          first_tile = false;
        }
        for (; i < n_kt; ++i, ++it) {
          const int s = it % S::STAGES;
          const uint32_t ph = (it / S::STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) { alive = false; break; }
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          const int kx = (kt0 + i) * BK;
          load_weights(s, kx, m0, n0);
          load_activations(s, kx, m0, n0);
        }
      }
      if (first_tile) pdl_wait();
      if (*abort_flag) {
        // Let copies in flight land before the CTA's shared memory goes away.
        const int first = it > S::STAGES ? it - S::STAGES : 0;
        for (int i = first; i < it; ++i) {
          const uint64_t t0 = global_timer_ns();
          while (!mbar_try_wait(&full[i % S::STAGES], (i / S::STAGES) & 1) && global_timer_ns() - t0 < 100000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    {
      // ---- MMA issuer: the whole warp walks the loop, one elected lane issues ----
      constexpr uint32_t idesc = umma_instr_desc(TM, BN);
      auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
      };
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        int m0, n0, kt0, n_kt, split;
        locate(tile, m0, n0, kt0, n_kt, split);
        const int buf = local % S::ACC_BUFS;
        const uint32_t use = (uint32_t)(local / S::ACC_BUFS);
        // the epilogue must have drained this accumulator (passes at once on its first use)
        ok = wait_all(&acc_empty[buf], (use & 1) ^ 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc_addr = tmem_base + buf * S::ACC_COLS;
        for (int i = 0; i < n_kt; ++i, ++it) {
          const int s = it % S::STAGES;
          const uint32_t ph = (it / S::STAGES) & 1;
          ok = wait_all(&full[s], ph);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + s * S::STAGE_BYTES);
          // descriptors of the stage's first 16 elements of K; each further 16 lie 32 bytes on
          // (two 16-byte units of the address field)
          const uint64_t desc_a = smem_desc_sw128(a_addr), desc_b = smem_desc_sw128(a_addr + S::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(acc_addr, desc_a + 2 * k, desc_b + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
        }
        umma_commit(&acc_full[buf]);  // the accumulator is complete once every MMA has retired
      }
    }
  } else {
    // ---- epilogue: warps 2..5, each reads its quarter of the 128 accumulator lanes ----
    const int quarter = warp & 3;
    constexpr int QROWS = TM / 4;            // tile rows in a quarter: one per lane
    pdl_wait();  // the output may still be read by an earlier kernel until it has completed
    int local = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      int m0, n0, kt0, n_kt, split;
      locate(tile, m0, n0, kt0, n_kt, split);
      const int buf = local % S::ACC_BUFS;
      const uint32_t use = (uint32_t)(local / S::ACC_BUFS);
      const bool ok = mbar_wait(&acc_full[buf], use & 1, abort_flag);
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + buf * S::ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      const int m = m0 + quarter * QROWS + lane;  // this thread's row on the M side
      const bool partial = p.split_stride != 0;
      // Decided once per thread; the swapped gated and picking epilogues meet at named barriers, which every
      // epilogue thread reaches whatever it decided.
      const bool go = __all_sync(0xffffffffu, ok && !*abort_flag);
      bool released = false;
      auto release = [&]() {  // the accumulator has been read: the MMA warp may overwrite it (once per tile)
        if (released) return;
        released = true;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      };
      if constexpr (MODE == QKV_ROPE && !SWAP) {
        // thread = token row m; the tile's columns are whole heads (d divides BN): per head, 32 pairs
        // of columns (i, i + d / 2) at a time
        const int d = p.qkv.d, n_heads = p.qkv.n_q + 2 * p.qkv.n_kv;
        const int groups = d / 64;  // groups of 32 pairs per head
        bool more = go;
#pragma unroll 1
        for (int hh = 0; hh < BN / 64 && more; ++hh) {  // at most BN / 64 heads in a tile
          if (hh * d >= BN) break;
          const int head = n0 / d + hh;
          if (head >= n_heads) break;  // same for the whole warp
#pragma unroll 1
          for (int g = 0; g < groups; ++g) {
            uint32_t rlo[32], rhi[32];
            tmem_ld32_issue(lane_addr + hh * d + g * 32, rlo);
            tmem_ld32_issue(lane_addr + hh * d + d / 2 + g * 32, rhi);
            tmem_wait();
            if (g == groups - 1 && ((hh + 1) * d >= BN || head + 1 >= n_heads)) release();
            if (m < p.m_rows) qkv_store_row(p, m, head, g * 32, rlo, rhi);
          }
        }
        release();
      } else if constexpr (MODE == PICK) {
        // thread = vocabulary entry m; columns = tokens.  Every candidate of the tile goes through the
        // exchange buffer (an entry that may not win, beyond the vocabulary or the step's rows, as NaN:
        // a NaN never wins); then each token's best over the tile's 128 entries is found by a few
        // threads that scan a share of the rows in ascending order, so that ties go to the smaller index.
        const PickArgs& a = p.pick;
        const int tile_row = quarter * QROWS + lane;
#pragma unroll 1
        for (int c = 0; c < BN / 16 && go; ++c) {
          if (n0 + c * 16 >= p.n_rows) break;  // same for the whole warp
          float v[16];
          tmem_ld16(lane_addr + c * 16, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = n0 + c * 16 + j;
            float val = __int_as_float(0x7fc00000);
            if (m < p.m_rows && tok < p.n_rows) {
              val = v[j];
              const float temp = a.temperature ? a.temperature[tok] : 0.f;
              if (temp > 0.f) {
                const uint32_t key = mix32(mix32(a.seeds[tok] ^ 0x9E3779B9u) ^ (uint32_t)a.positions[tok]);
                const uint32_t h = mix32(key + (uint32_t)m * 0x85EBCA6Bu);
                const float u = ((float)(h >> 9) + 0.5f) * (1.f / 8388608.f);
                val = val * (1.f / temp) - logf(-logf(u));
              }
            }
            exchange[tile_row * (BN + 1) + c * 16 + j] = val;
          }
        }
        release();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // PARTS threads per token, each a share of the rows; then the shares of a token are combined
        constexpr int PARTS = 128 / BN > 0 ? 128 / BN : 1, SHARE = TM / PARTS;
        const int t = threadIdx.x - 64, col = t % BN, part = t / BN;
        float bv = -INFINITY;
        int bi = INT_MAX;
        if (go && part < PARTS && n0 + col < p.n_rows) {
#pragma unroll 8
          for (int r = part * SHARE; r < (part + 1) * SHARE; ++r) {
            const float val = exchange[r * (BN + 1) + col];
            if (better(val, m0 + r, bv, bi)) {
              bv = val;
              bi = m0 + r;
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // every share is read: the buffer's first rows take the results
        int* exch_idx = reinterpret_cast<int*>(exchange) + 128;
        exchange[t] = bv;
        exch_idx[t] = bi;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (go && t < BN && n0 + t < p.n_rows) {
          bv = -INFINITY;
          bi = INT_MAX;
#pragma unroll
          for (int q = 0; q < PARTS; ++q)
            if (better(exchange[q * BN + t], exch_idx[q * BN + t], bv, bi)) {
              bv = exchange[q * BN + t];
              bi = exch_idx[q * BN + t];
            }
          a.part_val[(size_t)(n0 + t) * p.m_tiles + m0 / TM] = bv;
          a.part_idx[(size_t)(n0 + t) * p.m_tiles + m0 / TM] = bi;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the buffer is free for the next tile
      } else if constexpr (!SWAP) {
        // thread = token row m; columns = output features, 32 at a time
        constexpr int OUT_COLS = GATED ? BN / 2 : BN;
        static_assert(OUT_COLS % 32 == 0, "normal orientation works on 32 output columns at a time");
        const int nbase = (n0 / N_ROWS) * OUT_COLS;
#pragma unroll 1
        for (int c = 0; c < OUT_COLS / 32 && go; ++c) {
          uint32_t r[32];
          float v[32];
          if (n_kt > 0) {
            tmem_ld32_issue(lane_addr + c * 32, r);
            if (GATED) {
              uint32_t ru[32];
              tmem_ld32_issue(lane_addr + BN / 2 + c * 32, ru);
              tmem_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = silu_gate(__uint_as_float(r[j]), __uint_as_float(ru[j]));
            } else {
              tmem_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
          if (c == OUT_COLS / 32 - 1) release();
          const int n = nbase + c * 32;
          if (m >= p.m_rows || n >= p.n_rows) continue;
          if (partial) {
            float* dst = (float*)p.out + split * p.split_stride + (size_t)m * p.ld_out + n;
            if (n + 32 <= p.n_rows && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n + j < p.n_rows) dst[j] = v[j];
            }
          } else {
            if (p.bias) {
              if (n + 32 <= p.n_rows && (((uintptr_t)(p.bias + n)) & 15) == 0) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                  const uint4 raw = reinterpret_cast<const uint4*>(p.bias + n)[q4];
                  const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(hb[e]);
                    v[q4 * 8 + 2 * e] += f.x;
                    v[q4 * 8 + 2 * e + 1] += f.y;
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n + j < p.n_rows) v[j] += __bfloat162float(p.bias[n + j]);
              }
            }
            OutT* dst = (OutT*)p.out + (size_t)m * p.ld_out + n;
            if (n + 32 <= p.n_rows && (((uintptr_t)dst) & 15) == 0) {
              if (sizeof(OutT) == 2) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                  uint32_t w[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(v[q4 * 8 + 2 * e], v[q4 * 8 + 2 * e + 1]);
                    w[e] = *reinterpret_cast<uint32_t*>(&h);
                  }
                  reinterpret_cast<uint4*>(dst)[q4] = make_uint4(w[0], w[1], w[2], w[3]);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n + j < p.n_rows) dst[j] = from_f32<OutT>(v[j]);
            }
          }
        }
        release();
      } else if constexpr (GATED) {
        // thread = output feature; columns = tokens.  Lanes 0..63 hold gate values, lanes 64..127
        // the up values of the same 64 features: all go through the exchange buffer, then each of
        // the 128 threads finishes one feature for half of the tokens.
        const int tile_row = quarter * QROWS + lane;
#pragma unroll 1
        for (int c = 0; c < BN / 16 && go; ++c) {
          if (n0 + c * 16 >= p.n_rows) break;  // same for the whole warp
          float v[16];
          tmem_ld16(lane_addr + c * 16, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) exchange[tile_row * (BN + 1) + c * 16 + j] = v[j];
        }
        release();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // the 128 threads share the tile's TM / 2 features: PARTS threads per feature, each a part of the tokens
        constexpr int HALF = TM / 2, PARTS = 128 / HALF;
        const int t = threadIdx.x - 64, f = t % HALF, h = t / HALF;
        if (go && m0 + f < p.m_rows) {
          __nv_bfloat16* dst = (__nv_bfloat16*)p.out + m0 + f;
          for (int col = h * (BN / PARTS); col < (h + 1) * (BN / PARTS); ++col) {
            const int tok = n0 + col;
            if (tok >= p.n_rows) break;
            dst[(size_t)tok * p.ld_out] =
                __float2bfloat16_rn(silu_gate(exchange[f * (BN + 1) + col], exchange[(HALF + f) * (BN + 1) + col]));
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the buffer is free for the next tile
      } else {
        // thread = output feature m; columns = tokens
        const float b = (p.bias && !partial && m < p.m_rows) ? __bfloat162float(p.bias[m]) : 0.f;
        int c = 0;
#pragma unroll 1
        for (; c < BN / 16 && go; ++c) {
          const int t = n0 + c * 16;
          if (t >= p.n_rows) break;  // same for the whole warp
          float v[16];
          if (n_kt > 0) tmem_ld16(lane_addr + c * 16, v);
          else
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
          if (c == BN / 16 - 1 || t + 16 >= p.n_rows) release();
          if (m >= p.m_rows) continue;
          if (partial) {
            float* dst = (float*)p.out + split * p.split_stride + m;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (t + j < p.n_rows) dst[(size_t)(t + j) * p.ld_out] = v[j];
          } else {
            OutT* dst = (OutT*)p.out + m;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (t + j < p.n_rows) dst[(size_t)(t + j) * p.ld_out] = from_f32<OutT>(v[j] + b);
          }
        }
        release();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, S::TMEM_COLS);
  }
}

// ---- host side -------------------------------------------------------------------------
template <int MODE, int BN, bool SWAP, typename OutT>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, dim3 grid, cudaStream_t stream) {
  using S = Shape<MODE, BN, SWAP>;
  static bool configured = false;
  auto kern = gemm_tc_kernel<MODE, BN, SWAP, OutT>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)lab_launch(kern, grid, dim3(THREADS), (size_t)S::SMEM, stream, ma, mb, p);
}

template <int MODE, bool SWAP, typename OutT>
int dispatch_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, dim3 grid, cudaStream_t s) {
  constexpr bool WIDE = !(MODE == GATED_SILU && SWAP);  // the gated exchange buffer is sized for up to 64 tokens
  switch (bn) {
    case 16: if constexpr (SWAP && MODE != QKV_ROPE) return launch<MODE, 16, SWAP, OutT>(ma, mb, p, grid, s); break;
    case 32: if constexpr (SWAP && MODE != QKV_ROPE) return launch<MODE, 32, SWAP, OutT>(ma, mb, p, grid, s); break;
    case 64: if constexpr (MODE != QKV_ROPE) return launch<MODE, 64, SWAP, OutT>(ma, mb, p, grid, s); break;
    case 128: if constexpr (WIDE) return launch<MODE, 128, SWAP, OutT>(ma, mb, p, grid, s); break;
    case 256: if constexpr (WIDE && MODE != PICK) return launch<MODE, 256, SWAP, OutT>(ma, mb, p, grid, s); break;
  }
  return (int)cudaErrorInvalidValue;
}

int sm_count() {
  static int count = 0;
  if (count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0)
      count = 148;
  }
  return count;
}

// Fills the tensor maps, the tile counts and the grid for an orientation; returns a CUDA error code.
int set_up(Params& p, CUtensorMap& ma, CUtensorMap& mb, dim3& grid, const void* x, const void* w, int tokens,
           int n_out, int w_rows, int K, int ldx, int gated, int swap, int bn, int splits) {
  p.k_tiles = (K + BK - 1) / BK;
  p.k_tiles_per_split = (p.k_tiles + splits - 1) / splits;
  p.up_offset = n_out;
  p.splits = splits;
  int rc;
  if (!swap) {
    const int box_b = gated ? bn / 2 : bn;
    if ((rc = lab_make_map_bf16(&ma, x, tokens, K, ldx, BM))) return rc;
    if ((rc = lab_make_map_bf16(&mb, w, w_rows, K, K, box_b))) return rc;
    p.m_rows = tokens;
    p.n_rows = n_out;
    p.m_tiles = (tokens + BM - 1) / BM;
    p.n_tiles = (n_out + box_b - 1) / box_b;
  } else {
    const int m_rows_tile = gated ? BM / 2 : BM;
    if ((rc = lab_make_map_bf16(&ma, w, w_rows, K, K, m_rows_tile))) return rc;
    if ((rc = lab_make_map_bf16(&mb, x, tokens, K, ldx, bn))) return rc;
    if (gated && bn > 64) return (int)cudaErrorInvalidValue;  // the exchange buffer is sized for up to 64 tokens
    p.m_rows = n_out;
    p.n_rows = tokens;
    p.m_tiles = (n_out + m_rows_tile - 1) / m_rows_tile;
    p.n_tiles = (tokens + bn - 1) / bn;
  }
  const long long tiles = (long long)p.m_tiles * p.n_tiles * splits;
  grid = dim3((unsigned)(tiles < sm_count() ? tiles : sm_count()));
  return 0;
}

// The second stage of the picking head: one block per token reduces the tiles' candidates.
__global__ void __launch_bounds__(128) pick_finish_kernel(int* __restrict__ tokens, const float* __restrict__ part_val,
                                                          const int* __restrict__ part_idx, int tiles) {
  __shared__ float sv[4];
  __shared__ int si[4];
  pdl_trigger();
  pdl_wait();
  const int tok = blockIdx.x;
  float bv = -INFINITY;
  int bi = INT_MAX;
  for (int c0 = threadIdx.x; c0 < tiles; c0 += 128 * 4) {   // four loads in flight
    float v[4];
    int i[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + 128 * u;
      v[u] = c < tiles ? part_val[(size_t)tok * tiles + c] : -INFINITY;
      i[u] = c < tiles ? part_idx[(size_t)tok * tiles + c] : INT_MAX;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (better(v[u], i[u], bv, bi)) {
        bv = v[u];
        bi = i[u];
      }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int q = 1; q < 4; ++q)
      if (better(sv[q], si[q], bv, bi)) {
        bv = sv[q];
        bi = si[q];
      }
    tokens[tok] = bi;
  }
}

// For tests of the bounded waits: one warp waits on a barrier that nobody ever arrives at, with a
// limit of `limit_ns`.  The wait gives up, the library's error word says that a wait ran out, and the
// kernel returns; the context stays usable.
__global__ void wait_probe_kernel(unsigned long long limit_ns, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_init_fence();
  }
  __syncthreads();
  const bool ok = mbar_wait(&bar, 0, &abort_flag, limit_ns);
  if (threadIdx.x == 0) *gave_up = ok ? 0 : 1;
}

}  // namespace

// x: [tokens, K] bf16 (row stride ldx), w: [n_out (x2 when gated), K] bf16 contiguous.
// out: bf16 or f32 [tokens, ld_out]; with splits > 1, `out` is the partial buffer
// [splits, tokens, ld_out] of floats (no bias, not gated).
// swap != 0: features on the M side (few tokens); bn: tile of the N side (16..256).
LAB_EXPORT int lab_gemm_tc(void* out, const void* x, const void* w, const void* bias, int tokens, int n_out, int K,
                           int ldx, int ld_out, int gated, int out_f32, int swap, int bn, int splits,
                           cudaStream_t stream) {
  if (tokens <= 0 || n_out <= 0) return 0;
  if (K % 8 || ldx % 8 || K <= 0) return (int)cudaErrorInvalidValue;            // 16-byte rows for TMA
  if ((((uintptr_t)x) | ((uintptr_t)w)) & 15) return (int)cudaErrorInvalidValue;  // 16-byte bases for TMA
  if (splits < 1 || (splits > 1 && (gated || !out_f32))) return (int)cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  Params p = {};
  p.out = out;
  p.bias = (const __nv_bfloat16*)bias;
  p.ld_out = ld_out;
  p.split_stride = splits > 1 ? (long long)tokens * ld_out : 0;
  dim3 grid;
  // A gated tile whose "gate" rows run past n_out would read "up" rows as gate: tiles are cut so
  // that valid outputs never mix the halves (rows >= n_out are masked in the epilogue), but the
  // up half must start at a row the map can address with the same box.
  const int rc = set_up(p, ma, mb, grid, x, w, tokens, n_out, gated ? 2 * n_out : n_out, K, ldx, gated, swap, bn, splits);
  if (rc) return rc;
  if (gated) {
    if (out_f32) return (int)cudaErrorInvalidValue;
    if (swap) return dispatch_bn<GATED_SILU, true, __nv_bfloat16>(bn, ma, mb, p, grid, stream);
    return dispatch_bn<GATED_SILU, false, __nv_bfloat16>(bn, ma, mb, p, grid, stream);
  }
  if (swap) {
    if (out_f32) return dispatch_bn<PLAIN, true, float>(bn, ma, mb, p, grid, stream);
    return dispatch_bn<PLAIN, true, __nv_bfloat16>(bn, ma, mb, p, grid, stream);
  }
  if (out_f32) return dispatch_bn<PLAIN, false, float>(bn, ma, mb, p, grid, stream);
  return dispatch_bn<PLAIN, false, __nv_bfloat16>(bn, ma, mb, p, grid, stream);
}

// The output head of a step that wants tokens: tokens[t] = the pick over n_out logits x[t] . w[n] (greedy where
// temperature is null or 0, else Gumbel-max with seeds and positions).  tokens <= bn <= 128.
// part_val / part_idx: [tokens * ceil(n_out / 128)] scratch.  Two launches: the product, and the pick over its tiles.
LAB_EXPORT int lab_gemm_tc_pick(int* out_tokens, const void* x, const void* w, int tokens, int n_out, int K, int ldx,
                                const float* temperature, const void* seeds, const int* positions, float* part_val,
                                int* part_idx, int bn, cudaStream_t stream) {
  if (tokens <= 0 || n_out <= 0) return 0;
  if (K % 8 || ldx % 8 || K <= 0 || tokens > bn || bn > 128) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)x) | ((uintptr_t)w)) & 15) return (int)cudaErrorInvalidValue;
  if (!part_val || !part_idx || (temperature && (!seeds || !positions))) return (int)cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  Params p = {};
  p.pick.tokens = out_tokens;
  p.pick.temperature = temperature;
  p.pick.seeds = (const uint32_t*)seeds;
  p.pick.positions = positions;
  p.pick.part_val = part_val;
  p.pick.part_idx = part_idx;
  dim3 grid;
  int rc = set_up(p, ma, mb, grid, x, w, tokens, n_out, n_out, K, ldx, 0, 1, bn, 1);
  if (rc) return rc;
  if ((rc = dispatch_bn<PICK, true, float>(bn, ma, mb, p, grid, stream))) return rc;
  return (int)lab_launch(pick_finish_kernel, dim3(tokens), dim3(128), 0, stream, out_tokens, (const float*)part_val,
                         (const int*)part_idx, p.m_tiles);
}

// The fused q/k/v projection of an attention layer with its epilogue.
//   x: [tokens, K] bf16 (row stride ldx); w: [(n_q + 2 n_kv) * d, K] bf16 contiguous (q rows, k rows, v rows);
//   bias: the same width, or null; q_out: [tokens, ld_q] bf16 receives the rotated q;
//   table: [tokens, d / 2] (cos, sin) pairs; row_slot: [tokens] cache slots (page * page_size + offset,
//   -1: none); cache_k / cache_v: [num_pages, n_kv, page_size, d], or null when the call does not write.
// Heads of 64 or 128 (a head must lie whole inside a tile), rotation over the whole head.
LAB_EXPORT int lab_gemm_tc_qkv(void* q_out, const void* x, const void* w, const void* bias, int tokens, int n_q,
                               int n_kv, int d, int K, int ldx, int ld_q, const void* table, const int* row_slot,
                               void* cache_k, void* cache_v, int page_size, int num_pages, int bn,
                               cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if ((d != 64 && d != 128) || n_q <= 0 || n_kv <= 0) return (int)cudaErrorInvalidValue;
  if (K % 8 || ldx % 8 || K <= 0 || ld_q % 8) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)bias) | ((uintptr_t)q_out) | ((uintptr_t)cache_k) |
       ((uintptr_t)cache_v) | ((uintptr_t)table)) & 15)
    return (int)cudaErrorInvalidValue;
  if (table == nullptr || ((cache_k != nullptr) && (cache_v == nullptr || row_slot == nullptr || page_size <= 0)))
    return (int)cudaErrorInvalidValue;
  if (bn % d) return (int)cudaErrorInvalidValue;   // whole heads in a tile
  const int n_out = (n_q + 2 * n_kv) * d;
  CUtensorMap ma, mb;
  Params p = {};
  p.out = q_out;
  p.bias = (const __nv_bfloat16*)bias;
  p.ld_out = ld_q;
  p.split_stride = 0;
  p.qkv.cache_k = (__nv_bfloat16*)cache_k;
  p.qkv.cache_v = (__nv_bfloat16*)cache_v;
  p.qkv.row_slot = row_slot;
  p.qkv.table = (const float2*)table;
  p.qkv.n_q = n_q;
  p.qkv.n_kv = n_kv;
  p.qkv.d = d;
  p.qkv.page_size = page_size;
  p.qkv.num_pages = num_pages;
  dim3 grid;
  const int rc = set_up(p, ma, mb, grid, x, w, tokens, n_out, n_out, K, ldx, 0, 0, bn, 1);
  if (rc) return rc;
  return dispatch_bn<QKV_ROPE, false, __nv_bfloat16>(bn, ma, mb, p, grid, stream);
}

// Launches the wait that nothing ends (see wait_probe_kernel); the limit is capped at 50 ms.
LAB_EXPORT int lab_gemm_tc_wait_probe(unsigned long long limit_ns, int* gave_up, cudaStream_t stream) {
  if (limit_ns > 50000000ull) limit_ns = 50000000ull;
  wait_probe_kernel<<<1, 32, 0, stream>>>(limit_ns, gave_up);
  return (int)cudaGetLastError();
}
