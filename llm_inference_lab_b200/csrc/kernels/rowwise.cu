// Row-wise kernels of the step: embedding gather, RMSNorm fused with the residual
// add (and with the sum of split-K partial products), rotary position encoding
// fused with the write of keys and values into cache pages.
//
// Formulas follow the reference's kernels, restated for paged storage:
//   embedding   rust/engine/src/runner/model/qwen2/kernels.rs:46-57, 113-150
//   rms_norm    kernels.rs:546-582   (32-bit sum, mean over the true width)
//   add         kernels.rs:1454-1467 (32-bit add, one rounding)
//   rope        kernels.rs:587-631   (split-half pairing, 32-bit angle)
//   store       rust/engine/src/runner/kv_pool/naive_kvpool.rs:880-954 (K cached after rotation)
// Inside an operator everything stays in 32-bit and the result is rounded to the storage type once,
// at the operator's edge.  (The reference also rounds the normalised value before the weight, and
// cos, sin and the four products of a rotation: fewer roundings only come closer to the exact value.)
#include "common.cuh"

// ----------------------------------------------------------------------------------------
// Embedding: out[t, :] = table[clamp(ids[t]), :]
// ----------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(T* __restrict__ out, const T* __restrict__ table, const int* __restrict__ ids,
                             int hidden, int vocab) {
  pdl_trigger();
  pdl_wait();  // the ids may come from the previous step's sampling kernel
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
    return (int)lab_launch(embed_kernel<float>, dim3(tokens), dim3(128), 0, stream, (float*)out, (const float*)table,
                           ids, hidden, vocab);
  return (int)lab_launch(embed_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, (__nv_bfloat16*)out,
                         (const __nv_bfloat16*)table, ids, hidden, vocab);
}

// ----------------------------------------------------------------------------------------
// Residual add + RMSNorm.
//   r = x (+ delta) (+ sum_s partial[s])        32-bit add, rounded to T, written back to x
//   y = T( r * rsqrt(mean(r^2) + eps) * w )
// `rows` (optional) gathers: output row i is computed from input row rows[i]; x is then
// left untouched (used for the final norm at the positions whose logits are wanted).
// `partial` (optional) holds `splits` 32-bit partial products [splits, tokens, hidden]
// of the preceding matrix product, summed here in a fixed order.
// ----------------------------------------------------------------------------------------
// Sum of the split-K partial products of one element, in ascending split order; the loads of
// eight (then four) splits are issued together so that their latencies overlap.
__device__ __forceinline__ float sum_partials(const float* __restrict__ p, int splits, size_t stride) {
  float acc = 0.f;
  int s = 0;
  for (; s + 8 <= splits; s += 8) {
    float a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = p[(size_t)(s + j) * stride];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += a[j];
  }
  for (; s + 4 <= splits; s += 4) {
    const float a0 = p[(size_t)s * stride], a1 = p[(size_t)(s + 1) * stride], a2 = p[(size_t)(s + 2) * stride],
                a3 = p[(size_t)(s + 3) * stride];
    acc += a0;
    acc += a1;
    acc += a2;
    acc += a3;
  }
  for (; s < splits; ++s) acc += p[(size_t)s * stride];
  return acc;
}

template <typename T>
__global__ void add_rmsnorm_kernel(T* __restrict__ y, T* __restrict__ x, const T* __restrict__ delta,
                                   const float* __restrict__ partial, int splits, size_t split_stride,
                                   const T* __restrict__ w, const int* __restrict__ rows, int n_in_rows, int hidden,
                                   float eps) {
  __shared__ float scratch[32];
  extern __shared__ float rowbuf[];  // hidden floats
  pdl_trigger();
  // The norm weight depends on nothing that runs before this kernel: its first element per thread
  // is fetched while the kernel before this one is still finishing.
  const float w_first = threadIdx.x < hidden ? to_f32<T>(w[threadIdx.x]) : 0.f;
  pdl_wait();
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
    if (partial) v += sum_partials(partial + (size_t)in_row * hidden + i, splits, split_stride);
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
    yr[i] = from_f32<T>(rowbuf[i] * inv * (i == (int)threadIdx.x ? w_first : to_f32<T>(w[i])));
  }
}

// The same for bfloat16 rows whose width is a multiple of 8, for steps with many rows: a thread
// owns chunks of 8 elements (16-byte loads and stores) and keeps them in registers.
constexpr int NORM_VEC_THREADS = 128;
constexpr int NORM_VEC_MAX_CHUNKS = 8;  // per thread: widths up to 128 * 8 * 8 = 8192

__global__ void __launch_bounds__(NORM_VEC_THREADS) add_rmsnorm_vec_kernel(
    __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
    const float* __restrict__ partial, int splits, size_t split_stride, const __nv_bfloat16* __restrict__ w,
    const int* __restrict__ rows, int n_in_rows, int hidden, float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  int in_row = blockIdx.x;
  if (rows) {
    in_row = rows[blockIdx.x];
    if (in_row < 0 || in_row >= n_in_rows) {
      if (threadIdx.x == 0) lab_set_error(LAB_ERR_ROW_RANGE);
      in_row = 0;
    }
  }
  const int chunks = hidden / 8;
  const size_t base = (size_t)in_row * hidden;
  float v[NORM_VEC_MAX_CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NORM_VEC_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * NORM_VEC_THREADS;
    if (c >= chunks) break;
    const uint4 raw = *reinterpret_cast<const uint4*>(x + base + c * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      v[k][2 * e] = f.x;
      v[k][2 * e + 1] = f.y;
    }
    if (delta) {
      const uint4 rd = *reinterpret_cast<const uint4*>(delta + base + c * 8);
      const __nv_bfloat162* hd = reinterpret_cast<const __nv_bfloat162*>(&rd);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(hd[e]);
        v[k][2 * e] += f.x;
        v[k][2 * e + 1] += f.y;
      }
    }
    if (partial) {
      float p[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < splits; ++s) {  // ascending split order, as the scalar kernel
        const float4 a = *reinterpret_cast<const float4*>(partial + s * split_stride + base + c * 8);
        const float4 b = *reinterpret_cast<const float4*>(partial + s * split_stride + base + c * 8 + 4);
        p[0] += a.x; p[1] += a.y; p[2] += a.z; p[3] += a.w;
        p[4] += b.x; p[5] += b.y; p[6] += b.z; p[7] += b.w;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[k][e] += p[e];
    }
    if (delta || partial) {
      uint4 packed;
      __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        hp[e] = __floats2bfloat162_rn(v[k][2 * e], v[k][2 * e + 1]);
        const float2 f = __bfloat1622float2(hp[e]);
        v[k][2 * e] = f.x;
        v[k][2 * e + 1] = f.y;
      }
      if (!rows) *reinterpret_cast<uint4*>(x + base + c * 8) = packed;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[k][e] * v[k][e];
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  __nv_bfloat16* yr = y + (size_t)blockIdx.x * hidden;
#pragma unroll
  for (int k = 0; k < NORM_VEC_MAX_CHUNKS; ++k) {
    const int c = threadIdx.x + k * NORM_VEC_THREADS;
    if (c >= chunks) break;
    const uint4 rw = *reinterpret_cast<const uint4*>(w + c * 8);
    const __nv_bfloat162* hw = reinterpret_cast<const __nv_bfloat162*>(&rw);
    uint4 packed;
    __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 fw = __bfloat1622float2(hw[e]);
      hp[e] = __floats2bfloat162_rn(v[k][2 * e] * inv * fw.x, v[k][2 * e + 1] * inv * fw.y);
    }
    *reinterpret_cast<uint4*>(yr + c * 8) = packed;
  }
}

LAB_EXPORT int lab_add_rmsnorm(void* y, void* x, const void* delta, const float* partial, int splits,
                               long long split_stride, const void* w, const int* rows, int n_out_rows, int n_in_rows,
                               int hidden, float eps, int dtype, cudaStream_t stream) {
  if (n_out_rows <= 0) return 0;
  const bool aligned = ((((uintptr_t)y) | ((uintptr_t)x) | ((uintptr_t)delta) | ((uintptr_t)partial) | ((uintptr_t)w)) & 15) == 0;
  if (dtype == LAB_BF16 && n_out_rows > 64 && hidden % 8 == 0 && aligned &&
      hidden <= NORM_VEC_THREADS * NORM_VEC_MAX_CHUNKS * 8 && (split_stride % 4) == 0)
    return (int)lab_launch(add_rmsnorm_vec_kernel, dim3(n_out_rows), dim3(NORM_VEC_THREADS), 0, stream,
                           (__nv_bfloat16*)y, (__nv_bfloat16*)x, (const __nv_bfloat16*)delta, partial, splits,
                           (size_t)split_stride, (const __nv_bfloat16*)w, rows, n_in_rows, hidden, eps);
  int threads = (hidden + 31) / 32 * 32;   // one element per thread where the row allows it
  threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return (int)lab_launch(add_rmsnorm_kernel<float>, dim3(n_out_rows), dim3(threads), smem, stream, (float*)y,
                           (float*)x, (const float*)delta, partial, splits, (size_t)split_stride, (const float*)w,
                           rows, n_in_rows, hidden, eps);
  }
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return (int)lab_launch(add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_out_rows), dim3(threads), smem, stream,
                         (__nv_bfloat16*)y, (__nv_bfloat16*)x, (const __nv_bfloat16*)delta, partial, splits,
                         (size_t)split_stride, (const __nv_bfloat16*)w, rows, n_in_rows, hidden, eps);
}

// ----------------------------------------------------------------------------------------
// Rotary encoding of q and k (split-half pairing over the first `rotary_dim` of each head)
// + write of rotated k and of v into the cache pages.
//   qkv: [tokens, (n_q + 2 n_kv) * d] rows of the fused projection (bias already added);
//        q is rotated in place; without a cache to write, k is rotated in place as well.
//   cache_k / cache_v: [num_pages, n_kv, page_size, d]; slot = page * page_size + offset.
// ----------------------------------------------------------------------------------------
// The fused projection arrives either rounded to T in `qkv` (q is then rotated in place), or
// as `splits` 32-bit split-K partial products in `partial` ([splits, tokens, row_stride]) with
// the bias still to be added: the kernel sums them in ascending order, adds the bias in 32-bit,
// rounds once (the value the projection would have stored) and writes rotated q to `q_out`
// ([tokens, n_q * d]).
// Block (t, g) serves token t and heads [g * heads_per_block, ...): one head per block when a
// step has few tokens (more blocks in flight), all heads per block when it has many.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const float* __restrict__ partial,
                                     int splits, size_t split_stride, const T* __restrict__ bias,
                                     T* __restrict__ q_out, const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq, int rotary_dim,
                                     const int* __restrict__ slots, T* __restrict__ cache_k, T* __restrict__ cache_v,
                                     int n_q, int n_kv, int d, int page_size, int num_pages, int heads_per_block) {
  pdl_trigger();
  // Before pdl_wait() only what no kernel of this step writes is read (positions, slots, the
  // frequencies): the angle of this thread's first pair is ready when the projection arrives.
  const int t = blockIdx.x;
  const int n_heads = n_q + 2 * n_kv;  // [0, n_q) q heads, then n_kv k heads, then n_kv v heads
  const int head_lo = blockIdx.y * heads_per_block;
  const int head_hi = min(n_heads, head_lo + heads_per_block);
  auto value = [&](size_t col) -> float {
    if (partial) {
      float v = sum_partials(partial + (size_t)t * row_stride + col, splits, split_stride);
      if (bias) v += to_f32<T>(bias[col]);
      return round_to<T>(v);
    }
    return to_f32<T>(qkv[(size_t)t * row_stride + col]);
  };
  const float pos = rotary_dim > 0 ? (float)positions[t] : 0.f;   // no positions are read where nothing rotates
  long long cache_row = -1;  // element offset of (page, kv head 0, offset) in the cache, or -1: no write
  if (cache_k != nullptr && head_hi > n_q) {
    const int slot = slots[t];
    if (slot >= 0) {
      const int page = slot / page_size, off = slot - page * page_size;
      if (page >= num_pages) {
        if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
      } else {
        cache_row = ((long long)page * n_kv * page_size + off) * d;
      }
    }
  }
  const int items = (head_hi - head_lo) * d;
  float sn0 = 0.f, cs0 = 1.f;
  {
    const int i = threadIdx.x % d;
    if ((int)threadIdx.x < items && i < rotary_dim / 2) sincosf(pos * inv_freq[i], &sn0, &cs0);
  }
  pdl_wait();
  for (int e = threadIdx.x; e < items; e += blockDim.x) {
    const int head = head_lo + e / d, i = e % d;
    const size_t col0 = (size_t)head * d;
    T* dst;
    if (head < n_q) {
      dst = partial ? q_out + (size_t)t * n_q * d + col0 : qkv + (size_t)t * row_stride + col0;
    } else if (cache_k == nullptr) {
      // no cache to write: k is rotated where it lies (a caller that only encodes), v stays as it is
      if (partial || head >= n_q + n_kv) continue;
      dst = qkv + (size_t)t * row_stride + col0;
    } else {
      if (cache_row < 0) continue;
      const bool is_k = head < n_q + n_kv;
      const int kvh = is_k ? head - n_q : head - n_q - n_kv;
      dst = (is_k ? cache_k : cache_v) + cache_row + (long long)kvh * page_size * d;
    }
    const int half = (head < n_q + n_kv) ? rotary_dim / 2 : 0;  // v is not rotated
    if (i < half) {
      float sn = sn0, cs = cs0;
      if (e != (int)threadIdx.x) sincosf(pos * inv_freq[i], &sn, &cs);
      // Both halves are read before either is written: a thread owns the pair (i, i + half).
      const float lo = value(col0 + i), hi = value(col0 + i + half);
      float rlo, rhi;
      rope_rotate(lo, hi, cs, sn, rlo, rhi);
      dst[i] = from_f32<T>(rlo);
      dst[i + half] = from_f32<T>(rhi);
    } else if (i >= 2 * half) {
      dst[i] = from_f32<T>(value(col0 + i));
    }
  }
}

// cos and sin of pos * inv_freq[i] for every row of a step, formed once per step in 32-bit and
// read by the rotary kernels of all layers: table[t][i] = (cos, sin).
__global__ void rope_table_kernel(float2* __restrict__ table, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int half, int total) {
  pdl_trigger();
  pdl_wait();
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int t = e / half, i = e - t * half;
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
  table[e] = make_float2(cs, sn);
}

LAB_EXPORT int lab_rope_table(void* table, const int* positions, const float* inv_freq, int tokens, int half,
                              cudaStream_t stream) {
  const int total = tokens * half;
  if (total <= 0) return 0;
  return (int)lab_launch(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, (float2*)table, positions,
                         inv_freq, half, total);
}

// bfloat16, many rows: a thread rotates 8 pairs (or copies 8 values) with 16-byte loads and stores;
// cos and sin come from the step's table.  Needs rotary_dim / 2 and the head size to be multiples
// of 8 and 16-byte aligned rows.
__global__ void __launch_bounds__(256) rope_kv_write_vec_kernel(
    __nv_bfloat16* __restrict__ qkv, int row_stride, const float2* __restrict__ table, int rotary_dim,
    const int* __restrict__ slots, __nv_bfloat16* __restrict__ cache_k, __nv_bfloat16* __restrict__ cache_v, int n_q,
    int n_kv, int d, int page_size, int num_pages, int tokens) {
  pdl_trigger();
  pdl_wait();
  const int half = rotary_dim / 2;
  const int rot_items = half / 8, copy_items = (d - rotary_dim) / 8;
  const int per_head = rot_items + copy_items;          // q and k heads: pairs of chunks, then plain chunks
  const int per_v = d / 8;
  const int per_token = (n_q + n_kv) * per_head + n_kv * per_v;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (long long)tokens * per_token) return;
  const int t = (int)(e / per_token);
  int w = (int)(e - (long long)t * per_token);
  int head, item;
  bool is_v = false;
  if (w < (n_q + n_kv) * per_head) {
    head = w / per_head;
    item = w - head * per_head;
  } else {
    w -= (n_q + n_kv) * per_head;
    head = n_q + n_kv + w / per_v;
    item = w % per_v;
    is_v = true;
  }
  __nv_bfloat16* src = qkv + (size_t)t * row_stride + (size_t)head * d;
  __nv_bfloat16* dst = src;
  if (head >= n_q && cache_k == nullptr) {
    if (is_v) return;      // no cache to write: k is rotated where it lies, v stays as it is
  } else if (head >= n_q) {
    const int slot = slots[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot - page * page_size;
    if (page >= num_pages) {
      lab_set_error(LAB_ERR_PAGE_RANGE);
      return;
    }
    const int kvh = is_v ? head - n_q - n_kv : head - n_q;
    dst = (is_v ? cache_v : cache_k) + (((size_t)page * n_kv + kvh) * page_size + off) * d;
  }
  if (is_v || item >= rot_items) {
    const int i0 = is_v ? item * 8 : rotary_dim + (item - rot_items) * 8;
    if (dst != src) *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(src + i0);
    return;
  }
  const int i0 = item * 8;
  const uint4 rlo = *reinterpret_cast<const uint4*>(src + i0), rhi = *reinterpret_cast<const uint4*>(src + i0 + half);
  const __nv_bfloat16* lo = reinterpret_cast<const __nv_bfloat16*>(&rlo);
  const __nv_bfloat16* hi = reinterpret_cast<const __nv_bfloat16*>(&rhi);
  const float2* cs = table + (size_t)t * half + i0;
  uint4 olo, ohi;
  __nv_bfloat16* pl = reinterpret_cast<__nv_bfloat16*>(&olo);
  __nv_bfloat16* ph = reinterpret_cast<__nv_bfloat16*>(&ohi);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 f = cs[j];
    float rl, rh;
    rope_rotate(__bfloat162float(lo[j]), __bfloat162float(hi[j]), f.x, f.y, rl, rh);
    pl[j] = __float2bfloat16_rn(rl);
    ph[j] = __float2bfloat16_rn(rh);
  }
  *reinterpret_cast<uint4*>(dst + i0) = olo;
  *reinterpret_cast<uint4*>(dst + i0 + half) = ohi;
}

// table: optional [tokens, rotary_dim / 2] (cos, sin) pairs from lab_rope_table.
LAB_EXPORT int lab_rope_kv_write_table(void* qkv, int row_stride, const void* table, int rotary_dim, const int* slots,
                                       void* cache_k, void* cache_v, int tokens, int n_q, int n_kv, int d,
                                       int page_size, int num_pages, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rotary_dim % 16 || rotary_dim > d || d % 8 || row_stride % 8 || table == nullptr ||
      ((((uintptr_t)qkv) | ((uintptr_t)cache_k) | ((uintptr_t)cache_v)) & 15))
    return (int)cudaErrorInvalidValue;
  const int per_head = rotary_dim / 16 + (d - rotary_dim) / 8;
  const long long total = (long long)tokens * ((n_q + n_kv) * per_head + n_kv * (d / 8));
  return (int)lab_launch(rope_kv_write_vec_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                         (__nv_bfloat16*)qkv, row_stride, (const float2*)table, rotary_dim, slots,
                         (__nv_bfloat16*)cache_k, (__nv_bfloat16*)cache_v, n_q, n_kv, d, page_size, num_pages, tokens);
}

LAB_EXPORT int lab_rope_kv_write(void* qkv, int row_stride, const float* partial, int splits, long long split_stride,
                                 const void* bias, void* q_out, const int* positions, const float* inv_freq,
                                 int rotary_dim, const int* slots, void* cache_k, void* cache_v, int tokens, int n_q,
                                 int n_kv, int d, int page_size, int num_pages, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rotary_dim % 2 || rotary_dim > d) return (int)cudaErrorInvalidValue;
  if (partial && (q_out == nullptr || dtype == LAB_F32)) return (int)cudaErrorInvalidValue;
  const int n_heads = n_q + 2 * n_kv;
  const int heads_per_block = tokens >= 128 ? n_heads : 1;
  dim3 grid(tokens, (n_heads + heads_per_block - 1) / heads_per_block);
  const int threads = heads_per_block > 1 ? 256 : (d >= 128 ? 128 : (d >= 64 ? 64 : 32));
  if (dtype == LAB_F32)
    return (int)lab_launch(rope_kv_write_kernel<float>, grid, dim3(threads), 0, stream, (float*)qkv, row_stride,
                           partial, splits, (size_t)split_stride, (const float*)bias, (float*)q_out, positions,
                           inv_freq, rotary_dim, slots, (float*)cache_k, (float*)cache_v, n_q, n_kv, d, page_size,
                           num_pages, heads_per_block);
  return (int)lab_launch(rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)qkv,
                         row_stride, partial, splits, (size_t)split_stride, (const __nv_bfloat16*)bias,
                         (__nv_bfloat16*)q_out, positions, inv_freq, rotary_dim, slots, (__nv_bfloat16*)cache_k,
                         (__nv_bfloat16*)cache_v, n_q, n_kv, d, page_size, num_pages, heads_per_block);
}

// ----------------------------------------------------------------------------------------
// A copy from pinned host memory to the device on a stream: what a step's metadata takes.  Called
// directly, it costs the host a fraction of what the same copy costs through a tensor library.
// ----------------------------------------------------------------------------------------
LAB_EXPORT int lab_copy_to_device(void* dst, const void* pinned_src, long long bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  return (int)cudaMemcpyAsync(dst, pinned_src, (size_t)bytes, cudaMemcpyHostToDevice, stream);
}

