// Plain attention over the paged cache: one kernel for any number of new tokens per
// request (whole prompts, portions, single decoded tokens), any head size that is a
// multiple of 8 up to 256, any number of heads and groups, with or without a window.
// It is the attention of the 32-bit path and the yardstick of the tensor-core kernels.
//
// One block per (query row, query head).  Keys are cut into chunks of 32 by absolute
// position; chunk c goes to warp c mod 4, one key per lane.  Each warp keeps a running
// (max, sum, accumulator) in 32-bit; the four are merged at the end in a fixed order.
// The partition depends only on the query's position, so the result for a position is
// the same whatever else is in the batch and however the prompt was cut.
//
// Formulas: rust/engine/src/runner/model/qwen2/kernels.rs:702-853 (scores scaled by
// 1/sqrt(d), mask key <= query, online softmax with max/sum/accumulator in 32-bit,
// o = acc / sum), 898-942 (merge of partial softmax states).  The window (keys with
// query - key < window) is this engine's addition.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_DPL = 8;  // dims per lane: head sizes up to 256

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) attention_plain_kernel(
    T* __restrict__ out, int out_stride, const T* __restrict__ q, int q_stride, const T* __restrict__ cache_k,
    const T* __restrict__ cache_v, const int* __restrict__ row_req, const int* __restrict__ row_pos,
    const int* __restrict__ block_table, int max_blocks, int n_q, int n_kv, int d, int page_size, int num_pages,
    int window, float scale) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  float* qs = smem;                      // [d]
  float* part = smem + d;                // [WARPS][d + 2]
  const int t = blockIdx.x, h = blockIdx.y, kvh = h / (n_q / n_kv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int req = row_req[t], p = row_pos[t];
  const int* bt = block_table + (size_t)req * max_blocks;

  for (int i = threadIdx.x; i < d; i += blockDim.x) qs[i] = to_f32<T>(q[(size_t)t * q_stride + (size_t)h * d + i]);
  __syncthreads();

  const int first = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  float m = -INFINITY, l = 0.f, acc[MAX_DPL];
#pragma unroll
  for (int i = 0; i < MAX_DPL; ++i) acc[i] = 0.f;

  for (int c = first / 32 + warp; c * 32 <= p; c += WARPS) {
    const int j = c * 32 + lane;
    const bool valid = j >= first && j <= p;
    long long base = -1;
    float s = -INFINITY;
    if (valid) {
      const int page = bt[j / page_size];
      if (page < 0 || page >= num_pages) {
        lab_set_error(LAB_ERR_PAGE_RANGE);
      } else {
        base = (((long long)page * n_kv + kvh) * page_size + (j % page_size)) * d;
        const T* kr = cache_k + base;
        float dot = 0.f;
        for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32<T>(kr[i]), dot);
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;  // no readable key in this chunk (same for the whole warp)
    const float pj = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) acc[i] *= corr;
    for (int jj = 0; jj < 32; ++jj) {
      const float pw = __shfl_sync(0xffffffffu, pj, jj);
      const long long bw = __shfl_sync(0xffffffffu, base, jj);
      if (pw == 0.f || bw < 0) continue;
      const T* vr = cache_v + bw;
#pragma unroll
      for (int i = 0; i < MAX_DPL; ++i) {
        const int dim = lane + 32 * i;
        if (dim < d) acc[i] = fmaf(pw, to_f32<T>(vr[dim]), acc[i]);
      }
    }
    m = m_new;
  }

  float* mine = part + warp * (d + 2);
#pragma unroll
  for (int i = 0; i < MAX_DPL; ++i) {
    const int dim = lane + 32 * i;
    if (dim < d) mine[dim] = acc[i];
  }
  if (lane == 0) {
    mine[d] = m;
    mine[d + 1] = l;
  }
  __syncthreads();
  float big = -INFINITY;
  for (int w = 0; w < WARPS; ++w) big = fmaxf(big, part[w * (d + 2) + d]);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float num = 0.f, den = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      const float mw = part[w * (d + 2) + d];
      const float wt = (mw == -INFINITY) ? 0.f : expf(mw - big);
      num += wt * part[w * (d + 2) + i];
      den += wt * part[w * (d + 2) + d + 1];
    }
    out[(size_t)t * out_stride + (size_t)h * d + i] = from_f32<T>(den > 0.f ? num / den : 0.f);
  }
}
}  // namespace

LAB_EXPORT int lab_attention_plain(void* out, int out_stride, const void* q, int q_stride, const void* cache_k,
                                   const void* cache_v, const int* row_req, const int* row_pos, const int* block_table,
                                   int max_blocks, int tokens, int n_q, int n_kv, int d, int page_size, int num_pages,
                                   int window, float scale, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d > 32 * MAX_DPL || d <= 0 || n_q % n_kv) return (int)cudaErrorInvalidValue;
  dim3 grid(tokens, n_q);
  const size_t smem = (size_t)(d + WARPS * (d + 2)) * sizeof(float);
  if (dtype == LAB_F32)
    return (int)lab_launch(attention_plain_kernel<float>, grid, dim3(WARPS * 32), smem, stream, (float*)out, out_stride,
                           (const float*)q, q_stride, (const float*)cache_k, (const float*)cache_v, row_req, row_pos,
                           block_table, max_blocks, n_q, n_kv, d, page_size, num_pages, window, scale);
  return (int)lab_launch(attention_plain_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), smem, stream,
                         (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)q, q_stride,
                         (const __nv_bfloat16*)cache_k, (const __nv_bfloat16*)cache_v, row_req, row_pos, block_table,
                         max_blocks, n_q, n_kv, d, page_size, num_pages, window, scale);
}
