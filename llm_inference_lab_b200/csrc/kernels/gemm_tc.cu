// Matrix product on the 5th-generation tensor cores of sm_100a: TMA loads into
// 128-byte-swizzled shared memory, tcgen05.mma with the accumulator in tensor memory,
// tcgen05.ld for the epilogue.
//
//   out[t, n] = OutT( sum_k x[t, k] * w[n, k]  (+ bias[n]) )                 w is [out, in]
//   gated:      out[t, n] = T( silu(g) * u ),  g = x . w[n], u = x . w[inter + n]   (32-bit, one rounding)
//   split-K:    partial[z, t, n] = sum over the z-th slice of k   (32-bit, summed by the
//               kernel that consumes it, in a fixed order)
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
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;  // rows of the M-side tile (UMMA M)
constexpr int BK = 64;   // bf16 elements per k-tile: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;

struct Params {
  void* out;            // [tokens, ld_out] of OutT, or partial [splits, tokens, ld_out] floats
  const __nv_bfloat16* bias;
  int m_rows;           // valid rows on the M side (tokens, or features when swapped)
  int n_rows;           // valid rows on the N side
  int ld_out;
  long long split_stride;  // elements between split-K partial planes (0: no split)
  int k_tiles;          // k-tiles in total
  int k_tiles_per_split;
  int up_offset;        // gated: row offset of the "up" half inside the weight matrix
  int m_tiles, n_tiles, splits;  // tiles on the M side, on the N side, and split-K planes
};

// TM: rows of the M-side tile, 128 or (swapped orientation only) 64.  With 64 rows an output has twice
// the tiles, so a decode step's products spread over more SMs and a CTA's share of the weights fits
// its shared memory whole: all of it is requested before the wait on the preceding kernel.  The
// accumulator of an M = 64 MMA lies in lanes 0..15 of each quarter of tensor memory (row r in lane
// 32 * (r / 16) + r % 16), so each epilogue warp still reads its own quarter.
template <int TM, int BN, bool GATED, bool SWAP>
struct Shape {
  static_assert(TM == 128 || (TM == 64 && SWAP), "64-row tiles exist in swapped orientation only");
  static constexpr int A_BYTES = TM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // gated + swapped: the epilogue warps exchange gate and up values through a buffer of their own
  static constexpr int EXCHANGE_BYTES = (GATED && SWAP) ? ((TM * (BN + 1) * 4 + 1023) / 1024) * 1024 : 0;
  static constexpr int STAGES_RAW = (SMEM_BUDGET - EXCHANGE_BYTES) / STAGE_BYTES;
  static constexpr int STAGES_CAP = TM == 64 ? 16 : 10;
  static constexpr int STAGES = STAGES_RAW > STAGES_CAP ? STAGES_CAP : STAGES_RAW;
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
template <int TM, int BN, bool GATED, bool SWAP, typename OutT>
__global__ void __launch_bounds__(THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                          const __grid_constant__ CUtensorMap map_b, Params p) {
  using S = Shape<TM, BN, GATED, SWAP>;
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
    constexpr int QROWS = TM / 4;            // tile rows in a quarter: its first QROWS lanes
    const bool has_row = lane < QROWS;
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
      const int m = m0 + quarter * QROWS + lane;  // this thread's row on the M side (if has_row)
      const bool partial = p.split_stride != 0;
      // Decided once per thread; the gated swapped epilogue meets at named barriers, which every
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
      if constexpr (!SWAP) {
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
          if (has_row) {
#pragma unroll
            for (int j = 0; j < 16; ++j) exchange[tile_row * (BN + 1) + c * 16 + j] = v[j];
          }
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
        const float b = (p.bias && !partial && has_row && m < p.m_rows) ? __bfloat162float(p.bias[m]) : 0.f;
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
          if (!has_row || m >= p.m_rows) continue;
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
template <int TM, int BN, bool GATED, bool SWAP, typename OutT>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, dim3 grid, cudaStream_t stream) {
  using S = Shape<TM, BN, GATED, SWAP>;
  static bool configured = false;
  auto kern = gemm_tc_kernel<TM, BN, GATED, SWAP, OutT>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)lab_launch(kern, grid, dim3(THREADS), (size_t)S::SMEM, stream, ma, mb, p);
}

template <bool GATED, bool SWAP, typename OutT>
int dispatch_bn(int bm, int bn, const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, dim3 grid,
                cudaStream_t s) {
  if constexpr (SWAP) {
    if (bm == 64) {
      switch (bn) {
        case 16: return launch<64, 16, GATED, SWAP, OutT>(ma, mb, p, grid, s);
        case 32: return launch<64, 32, GATED, SWAP, OutT>(ma, mb, p, grid, s);
        case 64: return launch<64, 64, GATED, SWAP, OutT>(ma, mb, p, grid, s);
      }
      return (int)cudaErrorInvalidValue;
    }
  }
  switch (bn) {
    case 16: if constexpr (SWAP) return launch<128, 16, GATED, SWAP, OutT>(ma, mb, p, grid, s); break;
    case 32: if constexpr (SWAP) return launch<128, 32, GATED, SWAP, OutT>(ma, mb, p, grid, s); break;
    case 64: return launch<128, 64, GATED, SWAP, OutT>(ma, mb, p, grid, s);
    case 128: if constexpr (!(GATED && SWAP)) return launch<128, 128, GATED, SWAP, OutT>(ma, mb, p, grid, s); break;
    case 256: if constexpr (!(GATED && SWAP)) return launch<128, 256, GATED, SWAP, OutT>(ma, mb, p, grid, s); break;
  }
  return (int)cudaErrorInvalidValue;
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
// swap != 0: features on the M side (few tokens); bn: tile of the N side (16..256); bm: rows of the
// M-side tile, 128, or 64 (swapped orientation with bn <= 64 only).
LAB_EXPORT int lab_gemm_tc(void* out, const void* x, const void* w, const void* bias, int tokens, int n_out, int K,
                           int ldx, int ld_out, int gated, int out_f32, int swap, int bm, int bn, int splits,
                           cudaStream_t stream) {
  if (tokens <= 0 || n_out <= 0) return 0;
  if (bm != 128 && !(bm == 64 && swap && bn <= 64)) return (int)cudaErrorInvalidValue;
  if (K % 8 || ldx % 8 || K <= 0) return (int)cudaErrorInvalidValue;            // 16-byte rows for TMA
  if ((((uintptr_t)x) | ((uintptr_t)w)) & 15) return (int)cudaErrorInvalidValue;  // 16-byte bases for TMA
  if (splits < 1 || (splits > 1 && (gated || !out_f32))) return (int)cudaErrorInvalidValue;
  const int w_rows = gated ? 2 * n_out : n_out;
  CUtensorMap ma, mb;
  Params p;
  p.out = out;
  p.bias = (const __nv_bfloat16*)bias;
  p.ld_out = ld_out;
  p.k_tiles = (K + BK - 1) / BK;
  p.k_tiles_per_split = (p.k_tiles + splits - 1) / splits;
  p.split_stride = splits > 1 ? (long long)tokens * ld_out : 0;
  p.up_offset = n_out;
  dim3 grid;
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
    const int m_rows_tile = gated ? bm / 2 : bm;
    if ((rc = lab_make_map_bf16(&ma, w, w_rows, K, K, m_rows_tile))) return rc;
    if ((rc = lab_make_map_bf16(&mb, x, tokens, K, ldx, bn))) return rc;
    if (gated && bn > 64) return (int)cudaErrorInvalidValue;  // the exchange buffer is sized for up to 64 tokens
    p.m_rows = n_out;
    p.n_rows = tokens;
    p.m_tiles = (n_out + m_rows_tile - 1) / m_rows_tile;
    p.n_tiles = (tokens + bn - 1) / bn;
  }
  p.splits = splits;
  {
    static int sm_count = 0;
    if (sm_count == 0) {
      int dev = 0;
      if (cudaGetDevice(&dev) != cudaSuccess ||
          cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0)
        sm_count = 148;
    }
    const long long tiles = (long long)p.m_tiles * p.n_tiles * splits;
    grid = dim3((unsigned)(tiles < sm_count ? tiles : sm_count));
  }
  // A gated tile whose "gate" rows run past n_out would read "up" rows as gate: tiles are cut so
  // that valid outputs never mix the halves (rows >= n_out are masked in the epilogue), but the
  // up half must start at a row the map can address with the same box.
  if (gated) {
    if (out_f32) return (int)cudaErrorInvalidValue;
    if (swap) return dispatch_bn<true, true, __nv_bfloat16>(bm, bn, ma, mb, p, grid, stream);
    return dispatch_bn<true, false, __nv_bfloat16>(bm, bn, ma, mb, p, grid, stream);
  }
  if (swap) {
    if (out_f32) return dispatch_bn<false, true, float>(bm, bn, ma, mb, p, grid, stream);
    return dispatch_bn<false, true, __nv_bfloat16>(bm, bn, ma, mb, p, grid, stream);
  }
  if (out_f32) return dispatch_bn<false, false, float>(bm, bn, ma, mb, p, grid, stream);
  return dispatch_bn<false, false, __nv_bfloat16>(bm, bn, ma, mb, p, grid, stream);
}

// Launches the wait that nothing ends (see wait_probe_kernel); the limit is capped at 50 ms.
LAB_EXPORT int lab_gemm_tc_wait_probe(unsigned long long limit_ns, int* gave_up, cudaStream_t stream) {
  if (limit_ns > 50000000ull) limit_ns = 50000000ull;
  wait_probe_kernel<<<1, 32, 0, stream>>>(limit_ns, gave_up);
  return (int)cudaGetLastError();
}
