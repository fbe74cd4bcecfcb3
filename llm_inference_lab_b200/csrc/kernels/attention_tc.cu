// Attention over the paged cache in bfloat16 on tensor cores, built for one head size
// (-DLAB_HEAD_DIM=d, a multiple of 16 up to 128): a causal prefill kernel for requests
// that bring several tokens, and a split-KV decode kernel (plus merge) for requests that
// bring one.  Both walk a request's block table, so keys and values may lie on any pages.
//
//   scores  s_j = (q . k_j) / sqrt(d) for keys j <= query position (and within the window)
//   softmax online in 32-bit (running max, sum and accumulator), p rounded to bfloat16
//           before the product with V, o = acc / sum rounded once
//   split-KV: each split leaves (acc, max, sum); merged as sum_s w_s acc_s / sum_s w_s sum_s
//           with w_s = exp(max_s - max)
// as the reference's tensor-core attention does (rust/engine/src/runner/model/qwen2/
// kernels.rs:946-1124 tile loop, 1134-1256 grouped decode, 1295-1452 prefill, 898-942 merge).
//
// The products run on mma.sync.m16n8k16 (bf16 in, f32 out): the score and PV products of a
// head of 64 are small next to the matrix products of the layer, and the kernels are bound
// by the softmax arithmetic (prefill) and by reading the cache (decode).
// Shared-memory rows are padded by 16 bytes, which keeps ldmatrix free of bank conflicts
// for every head size that is a multiple of 16.
#include "attention_mma.cuh"

namespace {

// ----------------------------------------------------------------------------------------
// Prefill: one CTA per (tile of 64 query rows, query head, request); 4 warps x 16 rows.
// ----------------------------------------------------------------------------------------
constexpr int PF_BM = 64, PF_BN = 64, PF_THREADS = 128;
constexpr int PF_TILE_BYTES = PF_BN * ROW_BYTES;
constexpr int PF_SMEM = PF_BM * ROW_BYTES + 4 * PF_TILE_BYTES;  // Q + 2 stages of (K, V)

__global__ void __launch_bounds__(PF_THREADS) attention_prefill_kernel(
    __nv_bfloat16* __restrict__ out, int out_stride, const __nv_bfloat16* __restrict__ q, int q_stride,
    const __nv_bfloat16* __restrict__ cache_k, const __nv_bfloat16* __restrict__ cache_v,
    const int* __restrict__ q_start, const int* __restrict__ kv_len_arr, const int* __restrict__ pos0_arr,
    const int* __restrict__ block_table, int max_blocks, int n_q, int n_kv, int page_size, int num_pages, int window,
    float scale_log2, int min_q_len) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.z, h = blockIdx.y;
  const int qs = q_start[b], ql = q_start[b + 1] - qs;
  // Later rows see more keys: their tiles are scheduled first, so that the longest CTAs do not
  // start last.
  const int r0 = (gridDim.x - 1 - blockIdx.x) * PF_BM;
  if (ql < min_q_len || r0 >= ql) return;
  const int kvh = h / (n_q / n_kv);
  const int p0 = pos0_arr[b], kvl = kv_len_arr[b];
  const int* bt = block_table + (size_t)b * max_blocks;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t q_s = smem_u32(smem);
  const uint32_t kv_s = q_s + PF_BM * ROW_BYTES;

  // Q tile -> shared memory (rows past the request's tokens are zeros)
  for (int c = tid; c < PF_BM * CPR; c += PF_THREADS) {
    const int row = c / CPR, col = c - row * CPR;
    const bool ok = r0 + row < ql;
    const __nv_bfloat16* src = q + (size_t)(qs + (ok ? r0 + row : 0)) * q_stride + (size_t)h * D + col * 8;
    cp_async16(q_s + row * ROW_BYTES + col * 16, src, ok);
  }
  cp_async_commit();

  const int last_row = min(r0 + PF_BM, ql) - 1;
  const int hi_all = p0 + last_row;
  const int lo_all = window > 0 ? max(0, p0 + r0 - window + 1) : 0;
  const int t_first = lo_all / PF_BN, t_last = hi_all / PF_BN;

  auto issue = [&](int t, int stage) {
    const uint32_t kd = kv_s + stage * 2 * PF_TILE_BYTES;
    constexpr int RW = PF_BN / (PF_THREADS / 32);  // rows of the tile each warp copies
    load_kv_rows_warp<RW>(kd + warp * RW * ROW_BYTES, kd + PF_TILE_BYTES + warp * RW * ROW_BYTES, cache_k, cache_v, bt,
                          t * PF_BN + warp * RW, lo_all, kvl, kvh, n_kv, page_size, num_pages, lane);
    cp_async_commit();
  };
  issue(t_first, 0);

  int lo[2], hi[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r0 + warp * 16 + (lane >> 2) + 8 * r;
    const int pos = p0 + row;
    hi[r] = row < ql ? pos : -1;
    lo[r] = window > 0 ? max(0, pos - window + 1) : 0;
  }
  float o[DTILES][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
  for (int t = 0; t < DTILES; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[t][e] = 0.f;

  uint32_t qf[KSTEPS][4];
  bool have_q = false;
  for (int t = t_first; t <= t_last; ++t) {
    const int stage = (t - t_first) & 1;
    if (t + 1 <= t_last) {
      issue(t + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (!have_q) {
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {
        const int row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int dcol = k * 16 + 8 * (lane >> 4);
        ldmatrix_x4(qf[k], q_s + row * ROW_BYTES + dcol * 2);
      }
      have_q = true;
    }
    // A warp whose rows all lie before this tile's first key has nothing to do in it.
    const int warp_hi = p0 + min(r0 + warp * 16 + 15, ql - 1);
    if (t * PF_BN <= warp_hi) {
      const uint32_t kd = kv_s + stage * 2 * PF_TILE_BYTES;
      // A tile that lies wholly before the warp's first row (and inside every row's window) needs no mask.
      const int first_row = r0 + warp * 16;
      const bool all_visible = first_row + 15 < ql && t * PF_BN + PF_BN - 1 <= p0 + first_row &&
                               (window == 0 || t * PF_BN >= p0 + first_row + 15 - window + 1);
      tile_step<PF_BN>(qf, kd, kd + PF_TILE_BYTES, o, m, l, t * PF_BN, lo, hi, scale_log2, lane, all_visible);
    }
    __syncthreads();  // the stage is refilled by the next iteration's prefetch
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    const int row = r0 + warp * 16 + (lane >> 2) + 8 * r;
    if (row >= ql) continue;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
    __nv_bfloat16* dst = out + (size_t)(qs + row) * out_stride + (size_t)h * D + 2 * (lane & 3);
#pragma unroll
    for (int t = 0; t < DTILES; ++t)
      *reinterpret_cast<uint32_t*>(dst + t * 8) = pack_bf16(o[t][2 * r] * inv, o[t][2 * r + 1] * inv);
  }
}

// ----------------------------------------------------------------------------------------
// Decode: one CTA per (split of the keys, kv head x tile of 16 query heads of its group,
// request with exactly one new token).  Each warp streams its own tiles of keys
// through a private ring of shared-memory stages; the warps' softmax states are merged at
// the end.  With several splits the CTA leaves (acc, max, sum) in scratch for the merge kernel.
// ----------------------------------------------------------------------------------------
// A warp's instructions depend on one another (ldmatrix, mma, shuffles, exp2, mma), so a tile takes
// a warp microseconds, and what keeps the memory system busy is the number of warps per SM.  Heads
// of up to 64: 4 warps with tiles of 32 keys, two CTAs per SM.  Larger heads: 12 warps with tiles of
// 16 keys in one CTA per SM, as many as registers and shared memory hold (measured at heads of 128,
// 32 requests of 4,096 keys, 4 kv heads: 47 us, 5.7 TB/s, against 67 us with 4 warps and tiles of 32).
#ifndef LAB_DC_BN
#define LAB_DC_BN (LAB_HEAD_DIM > 64 ? 16 : 32)
#endif
#ifndef LAB_DC_WARPS
#define LAB_DC_WARPS (LAB_HEAD_DIM > 64 ? 12 : 4)
#endif
constexpr int DC_BN = LAB_DC_BN, DC_WARPS = LAB_DC_WARPS, DC_THREADS = 32 * DC_WARPS;
constexpr int DC_TILE_BYTES = DC_BN * ROW_BYTES;
constexpr int DC_MERGE_BYTES = DC_WARPS * 16 * (D + 2) * 4;
constexpr int DC_MAX_CLUSTER = 8;  // the portable cluster size
// What the splits of a cluster send one another: from each split the elements this CTA merges (all
// shares together are at most 16 * D floats, rounded up per split) and 16 (max, sum) pairs.  The
// area lies outside the rings, because a peer may write here while this CTA still reads its tiles.
constexpr int DC_RECV_BYTES = ((16 * D + DC_MAX_CLUSTER * 33 + 8) * 4 + 15) / 16 * 16;
// Shared memory of a decode CTA.  In a cluster a warp meets two tiles at most (one or two rounds of
// the warps per CTA and split), so two stages do; the footprint matters: beyond about 100 KB the CTAs of consecutive
// launches no longer share SMs, and a launch of 128 CTAs measured 8.6 us instead of 5.5.
template <bool CLUSTER>
struct DcLayout {
  static constexpr int STAGES = CLUSTER ? 2 : (D <= 64 ? 3 : 2);
  static constexpr int WARP_BYTES = STAGES * 2 * DC_TILE_BYTES;
  static constexpr int RING_BYTES = DC_WARPS * WARP_BYTES > DC_MERGE_BYTES ? DC_WARPS * WARP_BYTES : DC_MERGE_BYTES;
  static constexpr int SMEM = RING_BYTES + (CLUSTER ? DC_RECV_BYTES : 0);  // rings (then the warps' states), receive area
};

// CLUSTER: the splits of one (request, kv head, tile of heads) are the CTAs of one thread-block
// cluster (grid x = cluster x = splits, at most 8).  Every CTA merges a share of the output
// elements: each split stores the (acc, max, sum) of those elements straight into the shared
// memory of the CTA that merges them (remote stores do not stall, remote loads would), and after
// one cluster barrier everyone finds all it needs at home: no scratch and no merge kernel.
template <bool CLUSTER = false>
__global__ void __launch_bounds__(DC_THREADS) attention_decode_kernel(
    __nv_bfloat16* __restrict__ out, int out_stride, const __nv_bfloat16* __restrict__ q, int q_stride,
    __nv_bfloat16* __restrict__ cache_k, __nv_bfloat16* __restrict__ cache_v,
    const int* __restrict__ q_start, const int* __restrict__ kv_len_arr, const int* __restrict__ block_table,
    int max_blocks, int n_q, int n_kv, int page_size, int num_pages, int window, float scale_log2, int splits,
    float* __restrict__ part_acc, float* __restrict__ part_ml) {
  extern __shared__ __align__(16) uint8_t smem[];
  using L = DcLayout<CLUSTER>;
  pdl_trigger();
  // Until pdl_wait() below only what no kernel of this step writes is read: the step's metadata
  // (row offsets, lengths, block tables) and keys and values of earlier steps.  The rows of this
  // step (q, and the tile that holds the newest key) come after the wait.
  const int b = blockIdx.z;
  const int qs = q_start[b];
  if (q_start[b + 1] - qs != 1) {
    pdl_wait();  // this kernel ends only after the one before it: what follows may count on both
    return;
  }
  const int group = n_q / n_kv, m_tiles = (group + 15) / 16;
  const int kvh = blockIdx.y / m_tiles, mt = blockIdx.y - kvh * m_tiles;
  const int split = blockIdx.x;
  const int kvl = kv_len_arr[b];
  const int first = window > 0 ? max(0, kvl - window) : 0;
  const int* bt = block_table + (size_t)b * max_blocks;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head0 = kvh * group + mt * 16;           // first query head of this CTA
  const int n_heads = min(16, group - mt * 16);      // valid rows

  // keys of this split: whole 32-key tiles counted from the 32-aligned start
  const int start = (first / DC_BN) * DC_BN;
  const int total_tiles = kvl > start ? (kvl - start + DC_BN - 1) / DC_BN : 0;
  const int tiles_per_split = (total_tiles + splits - 1) / splits;
  const int tile_lo = split * tiles_per_split;
  const int tile_hi = min(total_tiles, tile_lo + tiles_per_split);

  const uint32_t ring = smem_u32(smem) + warp * L::WARP_BYTES;
  auto issue = [&](int t, int stage) {
    const uint32_t kd = ring + stage * 2 * DC_TILE_BYTES;
    const int key0 = start + t * DC_BN;
    load_kv_rows_warp<DC_BN>(kd, kd + DC_TILE_BYTES, cache_k, cache_v, bt, key0, first, kvl, kvh, n_kv,
                             page_size, num_pages, lane);
  };
  // this warp's tiles: tile_lo + warp, + DC_WARPS, ...; the first copies start before anything else
  int t_issue = tile_lo + warp;
  int staged = 0;
  for (; staged < L::STAGES - 1; ++staged) {
    // a tile that reaches the newest key waits for the kernel that writes it
    if (t_issue < tile_hi && start + (t_issue + 1) * DC_BN >= kvl) break;
    if (t_issue < tile_hi) issue(t_issue, staged);
    cp_async_commit();
    t_issue += DC_WARPS;
  }
  pdl_wait();
  for (; staged < L::STAGES - 1; ++staged) {
    if (t_issue < tile_hi) issue(t_issue, staged);
    cp_async_commit();
    t_issue += DC_WARPS;
  }

  uint32_t qf[KSTEPS][4];
  {
    // q fragments straight from global memory: row r of the A operand is query head head0 + r
    const __nv_bfloat16* qrow = q + (size_t)qs * q_stride;
    const int ra = lane >> 2, rb = ra + 8;
#pragma unroll
    for (int k = 0; k < KSTEPS; ++k) {
      const int c = k * 16 + 2 * (lane & 3);
      const uint32_t* pa = reinterpret_cast<const uint32_t*>(qrow + (size_t)(head0 + ra) * D + c);
      const uint32_t* pb = reinterpret_cast<const uint32_t*>(qrow + (size_t)(head0 + rb) * D + c);
      qf[k][0] = ra < n_heads ? pa[0] : 0u;
      qf[k][1] = rb < n_heads ? pb[0] : 0u;
      qf[k][2] = ra < n_heads ? pa[4] : 0u;
      qf[k][3] = rb < n_heads ? pb[4] : 0u;
    }
  }
  float o[DTILES][4], m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
#pragma unroll
  for (int t = 0; t < DTILES; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[t][e] = 0.f;
  const int lo[2] = {first, first}, hi[2] = {kvl - 1, kvl - 1};

  int stage = 0;
  for (int t = tile_lo + warp; t < tile_hi; t += DC_WARPS) {
    // prefetch the tile L::STAGES - 1 ahead into the stage consumed last iteration
    const int pre_stage = (stage + L::STAGES - 1) % L::STAGES;
    if (t_issue < tile_hi) issue(t_issue, pre_stage);
    cp_async_commit();
    t_issue += DC_WARPS;
    cp_async_wait<L::STAGES - 1>();
    __syncwarp();
    const uint32_t kd = ring + stage * 2 * DC_TILE_BYTES;
    const int key0 = start + t * DC_BN;
    // every key of an inner tile is visible to the one query row: no mask to evaluate
    tile_step<DC_BN>(qf, kd, kd + DC_TILE_BYTES, o, m, l, key0, lo, hi, scale_log2, lane,
                     key0 >= first && key0 + DC_BN <= kvl);
    __syncwarp();
    stage = (stage + 1) % L::STAGES;
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  __syncthreads();  // every warp is done with its ring: the memory is reused for the merge
  float* mg = reinterpret_cast<float*>(smem) + warp * 16 * (D + 2);
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
  __syncthreads();
  const float* all = reinterpret_cast<const float*>(smem);
  [[maybe_unused]] const uint32_t recv_base = smem_u32(smem) + L::RING_BYTES;  // same offset in every CTA
  for (int i = tid; i < n_heads * D; i += DC_THREADS) {
    const int row = i / D, dim = i - row * D;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) big = fmaxf(big, all[(w * 16 + row) * (D + 2) + D]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) {
      const float mw = all[(w * 16 + row) * (D + 2) + D];
      const float wt = (mw == -INFINITY) ? 0.f : fast_exp2(mw - big);
      num += wt * all[(w * 16 + row) * (D + 2) + dim];
      den += wt * all[(w * 16 + row) * (D + 2) + D + 1];
    }
    const int head = head0 + row;
    if (splits == 1) {
      out[(size_t)qs * out_stride + (size_t)head * D + dim] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    } else if constexpr (CLUSTER) {
      // to the CTA that merges element i: slot `split` of its receive area
      const int share = (n_heads * D + splits - 1) / splits;
      const int dest = i / share;
      const uint32_t slot = recv_base + (uint32_t)(split * (share + 32)) * 4;
      st_cluster_f32(map_to_rank(slot + (uint32_t)(i - dest * share) * 4, dest), num);
      if (dim < splits) {  // the row's (max, sum) to every CTA of the cluster: thread `dim` serves CTA `dim`
        const uint32_t ml = map_to_rank(slot + (uint32_t)(share + 2 * row) * 4, dim);
        st_cluster_f32(ml, big);
        st_cluster_f32(ml + 4, den);
      }
    } else {
      const size_t slot = ((size_t)b * n_q + head) * splits + split;
      part_acc[slot * D + dim] = num;
      if (dim == 0) {
        part_ml[slot * 2] = big;
        part_ml[slot * 2 + 1] = den;
      }
    }
  }
  if constexpr (CLUSTER) {
    if (splits > 1) {
      cluster_sync();  // every split's stores have landed
      // This CTA's share of the output elements, one element per thread, from its own shared memory;
      // the sum runs in ascending split order, as in the merge kernel.
      const int items = n_heads * D, share = (items + splits - 1) / splits;
      const int lo_item = split * share, hi_item = min(items, lo_item + share);
      const float* recv = reinterpret_cast<const float*>(smem + L::RING_BYTES);
      for (int i = lo_item + tid; i < hi_item; i += DC_THREADS) {
        const int row = i / D, dim = i - row * D;
        float big = -INFINITY;
        for (int sp = 0; sp < splits; ++sp) big = fmaxf(big, recv[sp * (share + 32) + share + 2 * row]);
        float num = 0.f, den = 0.f;
        for (int sp = 0; sp < splits; ++sp) {
          const float* from = recv + sp * (share + 32);
          const float ms = from[share + 2 * row];
          const float wt = (ms == -INFINITY) ? 0.f : fast_exp2(ms - big);
          num += wt * from[i - lo_item];
          den += wt * from[share + 2 * row + 1];
        }
        out[(size_t)qs * out_stride + (size_t)(head0 + row) * D + dim] =
            __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
      }
    }
  }
}

// Merge of the splits: one block per (request, query head), D threads.
__global__ void attention_merge_kernel(__nv_bfloat16* __restrict__ out, int out_stride,
                                       const int* __restrict__ q_start, int n_q, int splits,
                                       const float* __restrict__ part_acc, const float* __restrict__ part_ml) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x, head = blockIdx.y, dim = threadIdx.x;
  const int qs = q_start[b];
  if (q_start[b + 1] - qs != 1) return;
  const size_t slot0 = ((size_t)b * n_q + head) * splits;
  float big = -INFINITY;
  for (int s0 = 0; s0 < splits; s0 += 8) {  // eight loads in flight
    float ms[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) ms[j] = s0 + j < splits ? part_ml[(slot0 + s0 + j) * 2] : -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) big = fmaxf(big, ms[j]);
  }
  float num = 0.f, den = 0.f;
  for (int s0 = 0; s0 < splits; s0 += 8) {  // the loads of eight splits first, then their sum in ascending order
    float ms[8], acc[8], ls[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = s0 + j < splits;
      ms[j] = in ? part_ml[(slot0 + s0 + j) * 2] : -INFINITY;
      acc[j] = in ? part_acc[(slot0 + s0 + j) * D + dim] : 0.f;
      ls[j] = in ? part_ml[(slot0 + s0 + j) * 2 + 1] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (s0 + j < splits) {
        const float wt = (ms[j] == -INFINITY) ? 0.f : fast_exp2(ms[j] - big);
        num += wt * acc[j];
        den += wt * ls[j];
      }
    }
  }
  out[(size_t)qs * out_stride + (size_t)head * D + dim] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
}

}  // namespace

LAB_EXPORT int lab_attention_head_dim() { return D; }
// What the caller needs to choose the splits: the keys a decode CTA takes in one round of its warps,
// and how many decode CTAs an SM holds (by shared memory).
LAB_EXPORT int lab_attention_decode_keys_per_round() { return DC_BN * DC_WARPS; }
LAB_EXPORT int lab_attention_decode_ctas_per_sm() { return DcLayout<false>::SMEM + 1024 <= 114 * 1024 ? 2 : 1; }

// Scratch the decode kernel needs with `splits` > 1: floats for part_acc and part_ml.
LAB_EXPORT long long lab_attention_decode_scratch_floats(int requests, int n_q, int splits) {
  return splits > 1 ? (long long)requests * n_q * splits * (D + 2) : 0;
}

LAB_EXPORT int lab_attention_prefill(void* out, int out_stride, const void* q, int q_stride, const void* cache_k,
                                     const void* cache_v, const int* q_start, const int* kv_len, const int* pos0,
                                     const int* block_table, int max_blocks, int requests, int max_q_len, int n_q,
                                     int n_kv, int page_size, int num_pages, int window, float scale, int min_q_len,
                                     cudaStream_t stream) {
  if (requests <= 0 || max_q_len <= 0) return 0;
  if (n_q % n_kv || q_stride % 8 || (((uintptr_t)q) & 15)) return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((max_q_len + PF_BM - 1) / PF_BM, n_q, requests);
  return (int)lab_launch(attention_prefill_kernel, grid, dim3(PF_THREADS), (size_t)PF_SMEM, stream,
                         (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,
                         (const __nv_bfloat16*)cache_k, (const __nv_bfloat16*)cache_v, q_start, kv_len, pos0,
                         block_table, max_blocks, n_q, n_kv, page_size, num_pages, window, scale * LOG2E, min_q_len);
}

static int decode_launch(void* out, int out_stride, const void* q, int q_stride, const void* cache_k,
                         const void* cache_v, const int* q_start, const int* kv_len, const int* block_table,
                         int max_blocks, int requests, int n_q, int n_kv, int page_size, int num_pages, int window,
                         float scale, int splits, float* scratch, bool may_cluster, cudaStream_t stream) {
  if (requests <= 0) return 0;
  const bool cluster = may_cluster && splits >= 2 && splits <= DC_MAX_CLUSTER;
  if (n_kv <= 0 || n_q % n_kv || splits < 1 || (splits > 1 && !cluster && scratch == nullptr)) return (int)cudaErrorInvalidValue;
  // The shared-memory limit is an attribute of the kernel on one device: set once per device.
  static bool configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
  if (!configured[device]) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         DcLayout<false>::SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               DcLayout<true>::SMEM);
    if (e != cudaSuccess) return (int)e;
    configured[device] = true;
  }
  const int group = n_q / n_kv, m_tiles = (group + 15) / 16;
  dim3 grid(splits, n_kv * m_tiles, requests);
  if (cluster) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DC_THREADS);
    cfg.dynamicSmemBytes = DcLayout<true>::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_lab_pdl ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, attention_decode_kernel<true>, (__nv_bfloat16*)out, out_stride,
                                   (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)cache_k, (__nv_bfloat16*)cache_v,
                                   q_start, kv_len, block_table, max_blocks, n_q, n_kv, page_size, num_pages, window,
                                   scale * LOG2E, splits, (float*)nullptr, (float*)nullptr);
  }
  float* part_acc = scratch;
  float* part_ml = scratch ? scratch + (size_t)requests * n_q * splits * D : nullptr;
  cudaError_t e = lab_launch(attention_decode_kernel<false>, grid, dim3(DC_THREADS), (size_t)DcLayout<false>::SMEM, stream,
                             (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,
                             (__nv_bfloat16*)cache_k, (__nv_bfloat16*)cache_v, q_start, kv_len, block_table,
                             max_blocks, n_q, n_kv, page_size, num_pages, window, scale * LOG2E, splits, part_acc,
                             part_ml);
  if (e != cudaSuccess) return (int)e;
  if (splits > 1)
    e = lab_launch(attention_merge_kernel, dim3(requests, n_q), dim3(D), 0, stream, (__nv_bfloat16*)out, out_stride,
                   q_start, n_q, splits, (const float*)part_acc, (const float*)part_ml);
  return (int)e;
}

// cluster_merge != 0 and 2 <= splits <= 8: the splits merge inside the kernel, through their cluster's
// shared memory (worth it while all CTAs of the launch are resident at once); else the merge kernel
// does it, from scratch: lab_attention_decode_scratch_floats(...) floats (may be null when unused).
LAB_EXPORT int lab_attention_decode(void* out, int out_stride, const void* q, int q_stride, const void* cache_k,
                                    const void* cache_v, const int* q_start, const int* kv_len,
                                    const int* block_table, int max_blocks, int requests, int n_q, int n_kv,
                                    int page_size, int num_pages, int window, float scale, int splits, float* scratch,
                                    int cluster_merge, cudaStream_t stream) {
  return decode_launch(out, out_stride, q, q_stride, cache_k, cache_v, q_start, kv_len, block_table, max_blocks,
                       requests, n_q, n_kv, page_size, num_pages, window, scale, splits, scratch, cluster_merge != 0,
                       stream);
}

// ----------------------------------------------------------------------------------------
// Split-KV decode attention for callers that must not allocate (declared in
// attention_noalloc.h; this entry point has no counterpart in the reference).
//
// The partial results of the splits normally live in a buffer the caller allocates.  Here
// they live in a fixed array that is part of this library's image on the device, so the
// call needs no allocation at all: no cudaMalloc, no cudaFree, no allocating library call.
// Every GPU that loads this library holds the array (LAB_NOALLOC_MAX_FLOATS floats, 4 MiB)
// until the process exits.
// ----------------------------------------------------------------------------------------
#define LAB_NOALLOC_MAX_FLOATS (1ll << 20)
#define LAB_NOALLOC_MAX_DEVICES 64
#define LAB_NOALLOC_TOO_LARGE (-2)
#define LAB_NOALLOC_BAD_DEVICE (-3)

static __device__ __align__(256) float g_noalloc_scratch[LAB_NOALLOC_MAX_FLOATS];
// In host code the array's name only stands for the symbol; its device address is looked up
// once per device and kept here.
static float* g_noalloc_address[LAB_NOALLOC_MAX_DEVICES];

LAB_EXPORT long long lab_attention_decode_noalloc_max_floats() { return LAB_NOALLOC_MAX_FLOATS; }

LAB_EXPORT const char* lab_attention_decode_noalloc_strerror(int code) {
  if (code == LAB_NOALLOC_TOO_LARGE)
    return "requests * query heads * splits * (head size + 2) exceeds the fixed scratch of 1048576 floats: "
           "use fewer splits or requests, or the entry point that takes a caller's buffer";
  if (code == LAB_NOALLOC_BAD_DEVICE) return "the current device's ordinal is beyond the 64 this entry point keeps addresses for";
  if (code == 0) return "ok";
  return cudaGetErrorString((cudaError_t)code);
}

LAB_EXPORT int lab_attention_decode_noalloc(void* out, int out_stride, const void* q, int q_stride,
                                            const void* cache_k, const void* cache_v, const int* q_start,
                                            const int* kv_len, const int* block_table, int max_blocks, int requests,
                                            int n_q, int n_kv, int page_size, int num_pages, int window, float scale,
                                            int splits, cudaStream_t stream) {
  if (splits < 1 || requests < 0 || n_q <= 0 || n_kv <= 0) return (int)cudaErrorInvalidValue;
  if (lab_attention_decode_scratch_floats(requests, n_q, splits) > LAB_NOALLOC_MAX_FLOATS) return LAB_NOALLOC_TOO_LARGE;
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= LAB_NOALLOC_MAX_DEVICES) return LAB_NOALLOC_BAD_DEVICE;
  if (g_noalloc_address[device] == nullptr) {
    // Set-up, once per device, with that device current: the first call on a device does it,
    // so that call should come before any stream capture.
    float* address = nullptr;
    e = cudaGetSymbolAddress((void**)&address, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_address[device] = address;
  }
  // Every split writes its (acc, max, sum) before the merge reads it, splits without keys
  // included, so nothing in the array has to start at zero and nothing is cleared.
  return decode_launch(out, out_stride, q, q_stride, cache_k, cache_v, q_start, kv_len, block_table, max_blocks,
                       requests, n_q, n_kv, page_size, num_pages, window, scale, splits, g_noalloc_address[device],
                       false, stream);
}
