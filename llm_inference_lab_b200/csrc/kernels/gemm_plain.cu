// Plain matrix product on the ordinary arithmetic units (no tensor cores, no reduced
// precision): the matrix product of the 32-bit path, and the yardstick the tensor-core
// kernels are tested against.
//
//   out[m, n] = OutT( sum_k x[m, k] * w[n, k]  (+ bias[n]) )          w is [out, in]
//   gated:      out[m, n] = T( silu(g) * u ),  g = x . w[n], u = x . w[inter + n]   (32-bit, one rounding)
//
// The sum over k runs in ascending order with one fused multiply-add per term, so an
// output element does not depend on how the rows were batched.  Formulas:
// rust/engine/src/runner/model/qwen2/kernels.rs:156-178, 393-418 (linear, bias in 32-bit,
// one rounding), 422-448 (gate/up with the SiLU product), 1469-1486 (SiLU).
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename T, typename OutT, bool GATED>
__global__ void __launch_bounds__(256) gemm_plain_kernel(OutT* __restrict__ out, const T* __restrict__ x,
                                                         const T* __restrict__ w, const T* __restrict__ bias, int M,
                                                         int N, int K, int ldx, int ldo) {
  pdl_trigger();
  pdl_wait();
  __shared__ float xs[BK][BM + PAD];
  __shared__ float ws[GATED ? 2 : 1][BK][BN + PAD];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[GATED ? 2 : 1][4][4];
#pragma unroll
  for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.f;

  const int lr = tid >> 2, lk = (tid & 3) * 4;  // this thread loads row lr, k in [lk, lk + 4)
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int m = m0 + lr;
      xs[lk + e][lr] = (m < M && k < K) ? to_f32<T>(x[(size_t)m * ldx + k]) : 0.f;
      const int n = n0 + lr;
      ws[0][lk + e][lr] = (n < N && k < K) ? to_f32<T>(w[(size_t)n * K + k]) : 0.f;
      if (GATED) ws[GATED ? 1 : 0][lk + e][lr] = (n < N && k < K) ? to_f32<T>(w[(size_t)(N + n) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[GATED ? 2 : 1][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) b[g][j] = ws[g][k][tx * 4 + j];
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[g][i][j] = fmaf(a[i], b[g][j], acc[g][i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v;
      if (GATED) {
        const float g = acc[0][i][j], u = acc[GATED ? 1 : 0][i][j];
        v = g / (1.f + expf(-g)) * u;
      } else {
        v = acc[0][i][j] + (bias ? to_f32<T>(bias[n]) : 0.f);
      }
      out[(size_t)m * ldo + n] = from_f32<OutT>(v);
    }
  }
}

template <typename T, typename OutT>
int launch(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int ldx, int ldo, int gated,
           cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (gated)
    return (int)lab_launch(gemm_plain_kernel<T, OutT, true>, grid, dim3(256), 0, stream, (OutT*)out, (const T*)x,
                           (const T*)w, (const T*)nullptr, M, N, K, ldx, ldo);
  return (int)lab_launch(gemm_plain_kernel<T, OutT, false>, grid, dim3(256), 0, stream, (OutT*)out, (const T*)x,
                         (const T*)w, (const T*)bias, M, N, K, ldx, ldo);
}
}  // namespace

// N is the number of output columns; with gated != 0, w holds 2 N rows (gate rows, then up rows).
LAB_EXPORT int lab_gemm_plain(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int ldx,
                              int ldo, int gated, int dtype, int out_f32, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (dtype == LAB_F32) return launch<float, float>(out, x, w, bias, M, N, K, ldx, ldo, gated, stream);
  if (out_f32) return launch<__nv_bfloat16, float>(out, x, w, bias, M, N, K, ldx, ldo, gated, stream);
  return launch<__nv_bfloat16, __nv_bfloat16>(out, x, w, bias, M, N, K, ldx, ldo, gated, stream);
}
