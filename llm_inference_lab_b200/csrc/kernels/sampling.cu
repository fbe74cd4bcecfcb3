// Picking the next token on the GPU: greedy and temperature sampling.
//
// Greedy is an argmax over 32-bit logits; ties go to the smallest index and a NaN never
// wins; a row without any finite candidate yields INT32_MAX, which the host reports
// (rust/engine/src/runner/model/qwen2/kernels.rs:1488-1552; engine.rs:844-851).
// The reference samples greedily only (rust/engine/src/runner/model_runner.rs:615-623).
// Temperature sampling is this engine's addition, by the Gumbel-max rule
//   token = argmax_i( logit_i / temperature - log(-log u_i) ),
// with u_i in (0, 1) from an integer hash of (seed, position, i): the draw for a
// position does not depend on the batch, on the step, or on the order of evaluation.
#include "common.cuh"
#include <limits.h>

namespace {
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__global__ void __launch_bounds__(1024) sample_kernel(int* __restrict__ tokens, const float* __restrict__ logits,
                                                      long long ld, int vocab, const float* __restrict__ temperature,
                                                      const uint32_t* __restrict__ seeds,
                                                      const int* __restrict__ positions) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row = blockIdx.x;
  const float* lr = logits + (size_t)row * ld;
  const float temp = temperature ? temperature[row] : 0.f;
  uint32_t key = 0;
  float inv_temp = 1.f;
  if (temp > 0.f) {
    key = mix32(mix32(seeds[row] ^ 0x9E3779B9u) ^ (uint32_t)positions[row]);
    inv_temp = 1.f / temp;
  }
  float bv = -INFINITY;
  int bi = INT_MAX;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    float v = lr[i];
    if (temp > 0.f) {
      const uint32_t h = mix32(key + (uint32_t)i * 0x85EBCA6Bu);
      const float u = ((float)(h >> 9) + 0.5f) * (1.f / 8388608.f);
      v = v * inv_temp - logf(-logf(u));
    }
    if (better(v, i, bv, bi)) { bv = v; bi = i; }  // a NaN compares false and never wins
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    bv = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : INT_MAX;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) tokens[row] = bi;
  }
}
}  // namespace

// temperature, seeds, positions: per row; temperature == nullptr or 0 means greedy.
LAB_EXPORT int lab_sample(int* tokens, const float* logits, long long ld, int rows, int vocab, const float* temperature,
                          const uint32_t* seeds, const int* positions, cudaStream_t stream) {
  if (rows <= 0) return 0;
  sample_kernel<<<rows, 1024, 0, stream>>>(tokens, logits, ld, vocab, temperature, seeds, positions);
  LAB_LAUNCH_CHECK();
}
