// Row-wise kernels of the step: embedding gather, RMSNorm fused with the residual
// add (and with the sum of split-K partial products), rotary position encoding
// fused with the write of keys and values into cache pages.
//
// Formulas follow the reference's kernels, restated for paged storage:
//   embedding   rust/engine/src/runner/model/qwen2/kernels.rs:46-57, 113-150
//   rms_norm    kernels.rs:546-582   (32-bit sum, mean over the true width, two roundings)
//   add         kernels.rs:1454-1467 (32-bit add, one rounding)
//   rope        kernels.rs:587-631   (split-half pairing, 32-bit angle, cos/sin rounded to T)
//   store       rust/engine/src/runner/kv_pool/naive_kvpool.rs:880-954 (K cached after rotation)
#include "common.cuh"

// ----------------------------------------------------------------------------------------
// Embedding: out[t, :] = table[clamp(ids[t]), :]
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                             int hidden, int vocab) {
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* src = table + (size_t)id * hidden;
  T* dst = out + (size_t)t * hidden;
  const int bytes = hidden * (int)sizeof(T);
  if ((bytes & 15) == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = threadIdx.x; i < bytes / 16; i += blockDim.x) d4[i] = s4[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
  }
}

LAB_EXPORT int lab_embed(void* out, const void* table, const int* ids, int tokens, int hidden, int vocab, int dtype,
                         cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == LAB_F32)
    embed_kernel<float><<<tokens, 128, 0, stream>>>((float*)out, (const float*)table, ids, hidden, vocab);
  else
    embed_kernel<__nv_bfloat16><<<tokens, 128, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)table, ids,
                                                            hidden, vocab);
  LAB_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Residual add + RMSNorm.
//   r = x (+ delta) (+ sum_s partial[s])        32-bit add, rounded to T, written back to x
//   y = T( T(r * rsqrt(mean(r^2) + eps)) * w )
// `rows` (optional) gathers: output row i is computed from input row rows[i]; x is then
// left untouched (used for the final norm at the positions whose logits are wanted).
// `partial` (optional) holds `splits` 32-bit partial products [splits, tokens, hidden]
// of the preceding matrix product, summed here in a fixed order.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(T* __restrict__ y, T* __restrict__ x, const T* __restrict__ delta,
                                   const float* __restrict__ partial, int splits, size_t split_stride,
                                   const T* __restrict__ w, const int* __restrict__ rows, int n_in_rows, int hidden,
                                   float eps) {
  __shared__ float scratch[32];
  extern __shared__ float rowbuf[];  // hidden floats
  int in_row = blockIdx.x;
  if (rows) {
    in_row = rows[blockIdx.x];
    if (in_row < 0 || in_row >= n_in_rows) {
      if (threadIdx.x == 0) lab_set_error(LAB_ERR_ROW_RANGE);
      in_row = 0;
    }
  }
  T* xr = x + (size_t)in_row * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f32<T>(xr[i]);
    if (delta) v += to_f32<T>(delta[(size_t)in_row * hidden + i]);
    if (partial) {
      float p = 0.f;
      for (int s = 0; s < splits; ++s) p += partial[s * split_stride + (size_t)in_row * hidden + i];
      v += p;
    }
    if (delta || partial) {
      v = round_to<T>(v);
      if (!rows) xr[i] = from_f32<T>(v);
    }
    rowbuf[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  T* yr = y + (size_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float n = round_to<T>(rowbuf[i] * inv);
    yr[i] = from_f32<T>(n * to_f32<T>(w[i]));
  }
}

LAB_EXPORT int lab_add_rmsnorm(void* y, void* x, const void* delta, const float* partial, int splits,
                               long long split_stride, const void* w, const int* rows, int n_out_rows, int n_in_rows,
                               int hidden, float eps, int dtype, cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    add_rmsnorm_kernel<float><<<n_out_rows, threads, smem, stream>>>(
        (float*)y, (float*)x, (const float*)delta, partial, splits, (size_t)split_stride, (const float*)w, rows,
        n_in_rows, hidden, eps);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    add_rmsnorm_kernel<__nv_bfloat16><<<n_out_rows, threads, smem, stream>>>(
        (__nv_bfloat16*)y, (__nv_bfloat16*)x, (const __nv_bfloat16*)delta, partial, splits, (size_t)split_stride,
        (const __nv_bfloat16*)w, rows, n_in_rows, hidden, eps);
  }
  LAB_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Rotary encoding of q and k (split-half pairing over the first `rotary_dim` of each head)
// + write of rotated k and of v into the cache pages.
//   qkv: [tokens, (n_q + 2 n_kv) * d] rows of the fused projection (bias already added);
//        q is rotated in place.
//   cache_k / cache_v: [num_pages, n_kv, page_size, d]; slot = page * page_size + offset.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq, int rotary_dim,
                                     const int* __restrict__ slots, T* __restrict__ cache_k, T* __restrict__ cache_v,
                                     int n_q, int n_kv, int d, int page_size, int num_pages) {
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // [0, n_q) q heads, then n_kv k heads, then n_kv v heads
  T* src = qkv + (size_t)t * row_stride + (size_t)head * d;
  const float pos = (float)positions[t];
  const int half = rotary_dim / 2;
  if (head < n_q + n_kv) {
    T* dst = src;
    if (head >= n_q) {
      if (cache_k == nullptr) return;
      const int slot = slots[t];
      if (slot < 0) return;
      const int page = slot / page_size, off = slot - page * page_size;
      if (page >= num_pages) {
        if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
        return;
      }
      dst = cache_k + (((size_t)page * n_kv + (head - n_q)) * page_size + off) * d;
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      if (i < half) {
        const float ang = pos * inv_freq[i];
        float sn, cs;
        sincosf(ang, &sn, &cs);
        const float c = round_to<T>(cs), s = round_to<T>(sn);
        const float lo = to_f32<T>(src[i]), hi = to_f32<T>(src[i + half]);
        const float a = round_to<T>(round_to<T>(lo * c) - round_to<T>(hi * s));
        const float b = round_to<T>(round_to<T>(hi * c) + round_to<T>(lo * s));
        // Both halves are read before either is written: a thread owns the pair (i, i + half).
        dst[i] = from_f32<T>(a);
        dst[i + half] = from_f32<T>(b);
      } else if (i >= rotary_dim) {
        dst[i] = src[i];
      }
    }
  } else {
    if (cache_v == nullptr) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot - page * page_size;
    if (page >= num_pages) {
      if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
      return;
    }
    T* dst = cache_v + (((size_t)page * n_kv + (head - n_q - n_kv)) * page_size + off) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = src[i];
  }
}

LAB_EXPORT int lab_rope_kv_write(void* qkv, int row_stride, const int* positions, const float* inv_freq,
                                 int rotary_dim, const int* slots, void* cache_k, void* cache_v, int tokens, int n_q,
                                 int n_kv, int d, int page_size, int num_pages, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rotary_dim % 2 || rotary_dim > d) return (int)cudaErrorInvalidValue;
  dim3 grid(tokens, n_q + 2 * n_kv);
  const int threads = d >= 128 ? 128 : (d >= 64 ? 64 : 32);
  if (dtype == LAB_F32)
    rope_kv_write_kernel<float><<<grid, threads, 0, stream>>>((float*)qkv, row_stride, positions, inv_freq, rotary_dim,
                                                              slots, (float*)cache_k, (float*)cache_v, n_q, n_kv, d,
                                                              page_size, num_pages);
  else
    rope_kv_write_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (__nv_bfloat16*)qkv, row_stride, positions, inv_freq, rotary_dim, slots, (__nv_bfloat16*)cache_k,
        (__nv_bfloat16*)cache_v, n_q, n_kv, d, page_size, num_pages);
  LAB_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// out = T( T(silu(gate)) * up ) for separately stored gate and up (kernels.rs:1469-1486).
// gate_up: [tokens, 2 * inter] with gate in the first half of each row.
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / inter, c = i - t * inter;
  const float g = to_f32<T>(gate_up[t * 2 * inter + c]);
  const float u = to_f32<T>(gate_up[t * 2 * inter + inter + c]);
  const float a = round_to<T>(g / (1.f + expf(-g)));
  out[i] = from_f32<T>(a * u);
}

LAB_EXPORT int lab_silu_mul(void* out, const void* gate_up, int tokens, int inter, int dtype, cudaStream_t stream) {
  const size_t total = (size_t)tokens * inter;
  if (total == 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  if (dtype == LAB_F32)
    silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, (const float*)gate_up, inter, total);
  else
    silu_mul_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up,
                                                                  inter, total);
  LAB_LAUNCH_CHECK();
}
