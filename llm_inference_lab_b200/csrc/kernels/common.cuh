// Shared helpers of the sm_100a kernels: storage types, conversions, reductions,
// and the device-side error word.
//
// Storage type T is float or __nv_bfloat16.  Arithmetic that the model's
// numerics depend on (sums, softmax, norms, angles, residual adds) is done in
// float; `store<T>` rounds to nearest even at the operator's edge, as the
// reference rounds to its storage type at every operator boundary
// (rust/engine/README.md:430-447).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LAB_EXPORT extern "C" __attribute__((visibility("default")))

enum LabDtype : int { LAB_F32 = 0, LAB_BF16 = 1 };

// Error codes a kernel may leave in the error word (first one wins).
enum LabDeviceError : int {
  LAB_OK = 0,
  LAB_ERR_PAGE_RANGE = 1,      // a page or slot index outside the pool
  LAB_ERR_WAIT_TIMEOUT = 2,    // a bounded wait on an mbarrier ran out
  LAB_ERR_ROW_RANGE = 3,       // a gathered row index outside the batch
};

// One copy per shared library (each library is built from one .cu file).
static __device__ int g_lab_error_word;

__device__ __forceinline__ void lab_set_error(int code) { atomicCAS(&g_lab_error_word, 0, code); }

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Round a float to the storage type and back: the value an operator boundary leaves.
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

// Split-half rotary pair: (lo, hi) are elements i and i + rotary_dim / 2 of a head, (cs, sn) the cosine
// and sine of the pair's angle (rust/engine/src/runner/model/qwen2/kernels.rs:587-631).  One spelling
// for every kernel that rotates, so that all of them round alike.
__device__ __forceinline__ void rope_rotate(float lo, float hi, float cs, float sn, float& out_lo, float& out_hi) {
  out_lo = __fmaf_rn(lo, cs, -__fmul_rn(hi, sn));
  out_hi = __fmaf_rn(hi, cs, __fmul_rn(lo, sn));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 2^x by the hardware approximation (relative error about 2^-22; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// ---- thread-block clusters ---------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of `addr` (shared, this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, int rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads, same order for every call; `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

#define LAB_LAUNCH_CHECK() return (int)cudaGetLastError()

// ---- programmatic dependent launch --------------------------------------------------------
// Kernels of a step run back to back on one stream, each tiny next to its launch latency.
// Launched with the programmatic-serialization attribute, a kernel may start while its
// predecessor still runs: it signals `pdl_trigger()` at its top (its own successor may be
// scheduled), does whatever does not depend on earlier kernels of the step (barrier set-up,
// prefetch of weights), and calls `pdl_wait()` before it touches anything an earlier kernel
// wrote or may still read.  `pdl_wait()` returns once the predecessor grid has completed and
// its memory is visible; without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

static int g_lab_pdl = 1;
LAB_EXPORT void lab_set_pdl(int on) { g_lab_pdl = on; }

template <typename... KArgs, typename... Args>
static inline cudaError_t lab_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_lab_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Reads the error word of this library and clears it.  Synchronises the device.
LAB_EXPORT int lab_take_error_word(int* out) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(out, g_lab_error_word, sizeof(int));
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemcpyToSymbol(g_lab_error_word, &zero, sizeof(int));
}
