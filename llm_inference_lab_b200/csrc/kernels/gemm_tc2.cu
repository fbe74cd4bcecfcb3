// Matrix product for steps with many tokens on pairs of SMs: tcgen05.mma.cta_group::2.
//
//   out[t, n] = OutT( sum_k x[t, k] * w[n, k]  (+ bias[n]) )                 w is [out, in]
//   gated:      out[t, n] = T( silu(g) * u ),  g = x . w[n], u = x . w[inter + n]   (32-bit, one rounding)
//   split-K:    partial[z, t, n] = sum over the z-th slice of k   (32-bit, summed by the consumer)
//
// A cluster of two CTAs works on one tile of 256 tokens x BN accumulator columns (256, or 224 or
// 192 where that fills the rounds of the pairs better).  Each CTA
// loads its own 128 token rows (A) and only HALF of the weight tile (BN / 2 of the BN rows of B);
// one MMA of M = 256, issued by the leader CTA, reads A from both CTAs' shared memory and each
// half of B from the CTA that holds it, and leaves each CTA the accumulator rows of its own
// tokens in its own tensor memory.  A CTA therefore fills 32 KB of shared memory per k-tile
// instead of the 48 KB of the single-CTA kernel with the same 128 x 256 accumulator, and filling
// shared memory from L2 is what bounds these products.  In a gated product the leader's half of B
// are the gate rows and its peer's half the up rows of the same 128 features.
//
// Per CTA: warp 0 loads (TMA; both CTAs' copies complete on the leader's barrier), warp 1 of the
// leader issues the MMAs (the whole warp walks the loop, an elected lane issues) and commits to
// the barriers of both CTAs (tcgen05.commit with multicast), warps 2-5 of each CTA read their
// accumulator back and store.  CTAs are persistent: a pair walks the tiles, with two accumulators
// in tensor memory, so the epilogue of one tile runs beside the MMAs of the next.  No load uses
// cluster multicast.  Every wait is bounded: when one runs out the kernel records an error code
// and lets the roles drain; both CTAs free their tensor memory after a cluster barrier.
//
// Formulas and rounding order: rust/engine/src/runner/model/qwen2/kernels.rs:156-178,
// 393-418 (32-bit accumulation, bias added in 32-bit, one rounding), 422-448 and 1469-1486
// (gate/up with the SiLU product), 300-387 (split-K partials merged in 32-bit).
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;   // token rows per CTA (the pair's MMA has M = 256)
constexpr int BK = 64;    // bf16 elements per k-tile: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;
constexpr int ACC_BUFS = 2;
constexpr int ACC_STRIDE = 256;                   // columns of tensor memory between the two accumulators
constexpr int TMEM_COLS = ACC_BUFS * ACC_STRIDE;  // two accumulators fill tensor memory
// BN: accumulator columns of a tile (256, 224 or 192); each CTA loads BN / 2 weight rows.  The host
// takes the width whose tiles fill the rounds of the pairs best: 608 half-tiles of gate/up at 2,048
// tokens are 4.1 rounds of 74 pairs at 256 columns and 4.8 rounds of shorter tiles at 224.
template <int BN>
struct Tile {
  static_assert(BN % 32 == 0 && BN <= ACC_STRIDE && BN >= 64, "N of an M = 256 MMA, halves in whole swizzle groups");
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 192 * 1024 / STAGE_BYTES > 8 ? 8 : 192 * 1024 / STAGE_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 512 /*barriers*/;
  // Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 256 over the pair, N = BN.
  static constexpr uint32_t IDESC =
      (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
  static_assert((2 * STAGES + 2 * ACC_BUFS) * 8 + 8 <= 512, "the barriers outgrow their 512 bytes");
};

// Arrival on a barrier of any CTA of the cluster (address in the cluster's shared window).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A tile into this CTA's shared memory; the bytes are counted on `bar_cluster_addr`, a barrier of
// the pair's leader.  No multicast: each CTA fetches what it holds.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// Called by every lane of a converged warp with the same arguments; one elected lane issues.
// The arrival reaches the barrier at this address in every CTA of `cta_mask`.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "{\n\t.reg .pred e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t}" ::
          "r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}
// D[tmem of both CTAs] (+)= A[both CTAs' smem] * B[both CTAs' smem]^T, bf16 inputs, 32-bit accumulate.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\t"
      "elect.sync _|e, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
struct Params {
  void* out;            // [tokens, ld_out] of OutT, or partial [splits, tokens, ld_out] floats
  const __nv_bfloat16* bias;
  int tokens, n_out;    // valid rows and output features
  int ld_out;
  long long split_stride;  // elements between split-K partial planes (0: no split)
  int k_tiles;          // k-tiles in total
  int k_tiles_per_split;
  int up_offset;        // gated: row offset of the "up" half inside the weight matrix
  int m_tiles, n_tiles, splits;  // tiles of 256 tokens, tiles of output features, split-K planes
};

template <bool GATED, typename OutT, int BN>
__global__ void __launch_bounds__(THREADS) gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a,
                                                           const __grid_constant__ CUtensorMap map_b, Params p) {
  constexpr int STAGES = Tile<BN>::STAGES, STAGE_BYTES = Tile<BN>::STAGE_BYTES;
  constexpr uint32_t IDESC = Tile<BN>::IDESC;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + STAGES * STAGE_BYTES);  // used in the leader only
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;          // [ACC_BUFS]
  uint64_t* acc_empty = acc_full + ACC_BUFS;    // [ACC_BUFS], used in the leader only
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + ACC_BUFS);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  constexpr int OUT_COLS = GATED ? BN / 2 : BN;   // output features per tile
  const int total_tiles = p.m_tiles * p.n_tiles * p.splits;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);    // the leader's producer announces the bytes of both CTAs
      mbar_init(&empty[s], 1);   // one commit of the leader's MMA warp, sent to both CTAs
    }
    for (int a = 0; a < ACC_BUFS; ++a) {
      mbar_init(&acc_full[a], 1);   // one commit, sent to both CTAs
      mbar_init(&acc_empty[a], 8);  // the four epilogue warps of each CTA
    }
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    // one warp of each CTA of the pair, with the same destination: the same columns in both
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync();  // both CTAs' barriers exist before either signals the other
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile index -> (first token row of the pair, first output feature, first k-tile, number of k-tiles)
  auto locate = [&](int tile, int& m0, int& n0, int& kt0, int& n_kt, int& split) {
    const int mt = tile % p.m_tiles;
    const int rest = tile / p.m_tiles;
    const int nt = rest % p.n_tiles;
    split = rest / p.n_tiles;
    m0 = mt * 2 * BM;
    n0 = nt * OUT_COLS;
    kt0 = split * p.k_tiles_per_split;
    int kt1 = kt0 + p.k_tiles_per_split;
    if (kt1 > p.k_tiles) kt1 = p.k_tiles;
    n_kt = kt1 > kt0 ? kt1 - kt0 : 0;
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: this CTA's token rows and its half of the weight rows ----
      pdl_wait();
      int it = 0;
      bool alive = true;
      for (int tile = pair; tile < total_tiles && alive; tile += n_pairs) {
        int m0, n0, kt0, n_kt, split;
        locate(tile, m0, n0, kt0, n_kt, split);
        const int a_row = m0 + (int)rank * BM;
        // gated: the leader holds the gate rows, its peer the up rows of the same features
        const int b_row = GATED ? (leader ? n0 : p.up_offset + n0) : n0 + (int)rank * (BN / 2);
        for (int i = 0; i < n_kt; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait<true>(&empty[s], ph ^ 1, abort_flag)) { alive = false; break; }
          if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          const uint32_t bar = map_to_rank(smem_u32(&full[s]), 0);
          uint8_t* a_dst = tiles + s * STAGE_BYTES;
          const int kx = (kt0 + i) * BK;
          tma_load_2d_pair(a_dst, &map_a, bar, kx, a_row);
          tma_load_2d_pair(a_dst + A_BYTES, &map_b, bar, kx, b_row);
        }
      }
    }
  } else if (warp == 1) {
    if (leader) {
      // ---- MMA issuer of the pair: the whole warp walks the loop, one elected lane issues ----
      auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, mbar_wait<true>(bar, parity, abort_flag));
      };
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++local) {
        int m0, n0, kt0, n_kt, split;
        locate(tile, m0, n0, kt0, n_kt, split);
        const int buf = local % ACC_BUFS;
        const uint32_t use = (uint32_t)(local / ACC_BUFS);
        // both CTAs' epilogues must have drained this accumulator (passes at once on its first use)
        ok = wait_all(&acc_empty[buf], (use & 1) ^ 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc_addr = tmem_base + buf * ACC_STRIDE;
        for (int i = 0; i < n_kt; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = wait_all(&full[s], ph);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
          // descriptors of the stage's first 16 elements of K; each further 16 lie 32 bytes on
          const uint64_t desc_a = smem_desc_sw128(a_addr), desc_b = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_pair(acc_addr, desc_a + 2 * k, desc_b + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s], 3);  // both CTAs may refill the stage once these MMAs have read it
        }
        umma_commit_pair(&acc_full[buf], 3);  // the accumulators of both CTAs are complete
      }
    }
  } else {
    // ---- epilogue: warps 2..5, each reads its quarter of this CTA's 128 accumulator lanes ----
    const int quarter = warp & 3;
    pdl_wait();  // the output may still be read by an earlier kernel until it has completed
    int local = 0;
    for (int tile = pair; tile < total_tiles; tile += n_pairs, ++local) {
      int m0, n0, kt0, n_kt, split;
      locate(tile, m0, n0, kt0, n_kt, split);
      const int buf = local % ACC_BUFS;
      const uint32_t use = (uint32_t)(local / ACC_BUFS);
      const bool ok = mbar_wait<true>(&acc_full[buf], use & 1, abort_flag);
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + buf * ACC_STRIDE + ((uint32_t)(quarter * 32) << 16);
      const int m = m0 + (int)rank * BM + quarter * 32 + lane;  // this thread's token row
      const bool partial = p.split_stride != 0;
      const bool go = __all_sync(0xffffffffu, ok && !*abort_flag);
      bool released = false;
      auto release = [&]() {  // the accumulator has been read: the leader's MMA warp may overwrite it
        if (released) return;
        released = true;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty[buf]), 0));
      };
      // 32 columns at a time; the last chunk of a tile whose width is no multiple of 32 reads on into
      // columns that belong to nothing (they lie inside the accumulator's 256) and stores only its own.
      constexpr int CHUNKS = (OUT_COLS + 31) / 32;
      const int n_end = min(p.n_out, n0 + OUT_COLS);
#pragma unroll 1
      for (int c = 0; c < CHUNKS && go; ++c) {
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
        if (c == CHUNKS - 1) release();
        const int n = n0 + c * 32;
        if (m >= p.tokens || n >= n_end) continue;
        if (partial) {
          float* dst = (float*)p.out + split * p.split_stride + (size_t)m * p.ld_out + n;
          const bool aligned = (((uintptr_t)dst) & 15) == 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (aligned && n + 4 * j + 4 <= n_end) {
              reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (n + 4 * j + e < n_end) dst[4 * j + e] = v[4 * j + e];
            }
          }
        } else {
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n + j < n_end) v[j] += __bfloat162float(p.bias[n + j]);
          }
          OutT* dst = (OutT*)p.out + (size_t)m * p.ld_out + n;
          const bool aligned = (((uintptr_t)dst) & 15) == 0;
          constexpr int PER = 16 / (int)sizeof(OutT);   // elements of a 16-byte store
#pragma unroll
          for (int g = 0; g < 32 / PER; ++g) {
            if (aligned && n + g * PER + PER <= n_end) {
              if constexpr (sizeof(OutT) == 2) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(v[g * 8 + 2 * e], v[g * 8 + 2 * e + 1]);
                  w[e] = *reinterpret_cast<uint32_t*>(&h);
                }
                reinterpret_cast<uint4*>(dst)[g] = make_uint4(w[0], w[1], w[2], w[3]);
              } else {
                reinterpret_cast<float4*>(dst)[g] = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
              }
            } else {
#pragma unroll
              for (int e = 0; e < PER; ++e)
                if (n + g * PER + e < n_end) dst[g * PER + e] = from_f32<OutT>(v[g * PER + e]);
            }
          }
        }
      }
      release();
    }
  }
  // Neither CTA leaves, nor frees its tensor memory, while its peer may still signal its barriers,
  // read its shared memory (the pair's MMA) or write its tensor memory.
  tc_fence_before();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------

template <bool GATED, typename OutT, int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, long long tiles, cudaStream_t stream) {
  constexpr int SMEM = Tile<BN>::SMEM;
  static int max_pairs = 0;  // clusters of two CTAs that the device holds at once
  auto kern = gemm_tc2_kernel<GATED, OutT, BN>;
  if (max_pairs == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2);
    probe.blockDim = dim3(THREADS);
    probe.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute pa[1];
    pa[0].id = cudaLaunchAttributeClusterDimension;
    pa[0].val.clusterDim.x = 2;
    pa[0].val.clusterDim.y = 1;
    pa[0].val.clusterDim.z = 1;
    probe.attrs = pa;
    probe.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &probe);
    if (e != cudaSuccess) return (int)e;
    if (n <= 0) return (int)cudaErrorLaunchOutOfResources;
    max_pairs = n;
  }
  const int pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_lab_pdl ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, ma, mb, p);
}

template <bool GATED, typename OutT>
int launch_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, long long tiles, cudaStream_t s) {
  switch (bn) {
    case 256: return launch<GATED, OutT, 256>(ma, mb, p, tiles, s);
    case 224: return launch<GATED, OutT, 224>(ma, mb, p, tiles, s);
    case 192: return launch<GATED, OutT, 192>(ma, mb, p, tiles, s);
  }
  return (int)cudaErrorInvalidValue;
}

// The tile width whose rounds over the pairs of SMs cost least, the wider on a tie.  A round of
// narrower tiles is shorter, but less than in proportion (measured per round against 256 columns:
// 224 columns 0.89 with a long K and no gain in the gated product, whose tiles have few k-tiles and
// an epilogue as long as their MMAs; 192 columns 0.84), so a narrower tile pays where it saves a
// round, fits the output's width or gives more pairs a tile.
int pick_bn(int tokens, int n_out, bool gated, int splits) {
  static int pairs = 0;
  if (pairs == 0) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2)
      sms = 148;
    pairs = sms / 2;
  }
  const long long m_tiles = (tokens + 2 * BM - 1) / (2 * BM);
  int best = 256;
  long long best_cost = -1;
  for (int bn : {256, 224, 192}) {
    const int out_cols = gated ? bn / 2 : bn;
    const long long tiles = m_tiles * ((n_out + out_cols - 1) / out_cols) * splits;
    const int round_cost = bn == 256 ? 256 : (bn == 224 ? (gated ? 256 : 240) : (gated ? 215 : 210));
    const long long cost = ((tiles + pairs - 1) / pairs) * round_cost;
    if (best_cost < 0 || cost < best_cost) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

}  // namespace

// x: [tokens, K] bf16 (row stride ldx), w: [n_out (x2 when gated), K] bf16 contiguous.
// out: bf16 or f32 [tokens, ld_out]; with splits > 1, `out` is the partial buffer
// [splits, tokens, ld_out] of floats (no bias, not gated).
// bn: accumulator columns of a tile, 256, 224 or 192; 0: the width that fills the rounds of the pairs best.
LAB_EXPORT int lab_gemm_tc2(void* out, const void* x, const void* w, const void* bias, int tokens, int n_out, int K,
                            int ldx, int ld_out, int gated, int out_f32, int splits, int bn, cudaStream_t stream) {
  if (tokens <= 0 || n_out <= 0) return 0;
  if (K % 8 || ldx % 8 || K <= 0) return (int)cudaErrorInvalidValue;            // 16-byte rows for TMA
  if ((((uintptr_t)x) | ((uintptr_t)w)) & 15) return (int)cudaErrorInvalidValue;  // 16-byte bases for TMA
  if (splits < 1 || (splits > 1 && (gated || !out_f32 || bias))) return (int)cudaErrorInvalidValue;
  if (gated && (out_f32 || bias)) return (int)cudaErrorInvalidValue;
  if (bn == 0) bn = pick_bn(tokens, n_out, gated != 0, splits);
  if (bn != 256 && bn != 224 && bn != 192) return (int)cudaErrorInvalidValue;
  const int w_rows = gated ? 2 * n_out : n_out;
  CUtensorMap ma, mb;
  int rc;
  if ((rc = lab_make_map_bf16(&ma, x, tokens, K, ldx, BM))) return rc;
  if ((rc = lab_make_map_bf16(&mb, w, w_rows, K, K, bn / 2))) return rc;
  Params p;
  p.out = out;
  p.bias = (const __nv_bfloat16*)bias;
  p.tokens = tokens;
  p.n_out = n_out;
  p.ld_out = ld_out;
  p.k_tiles = (K + BK - 1) / BK;
  p.k_tiles_per_split = (p.k_tiles + splits - 1) / splits;
  p.split_stride = splits > 1 ? (long long)tokens * ld_out : 0;
  p.up_offset = n_out;
  const int out_cols = gated ? bn / 2 : bn;
  p.m_tiles = (tokens + 2 * BM - 1) / (2 * BM);
  p.n_tiles = (n_out + out_cols - 1) / out_cols;
  p.splits = splits;
  const long long tiles = (long long)p.m_tiles * p.n_tiles * splits;
  if (gated) return launch_bn<true, __nv_bfloat16>(bn, ma, mb, p, tiles, stream);
  if (out_f32) return launch_bn<false, float>(bn, ma, mb, p, tiles, stream);
  return launch_bn<false, __nv_bfloat16>(bn, ma, mb, p, tiles, stream);
}
