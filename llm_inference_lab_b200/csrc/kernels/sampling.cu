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

constexpr int CHUNK = 4096;   // vocabulary entries per block (the reference's argmax tile, kernels.rs:1489-1518)
constexpr int THREADS = 256;
static_assert(CHUNK % (THREADS * 4) == 0, "a thread takes whole groups of four entries");

// One block per (chunk of the vocabulary, row).  Each block leaves the best candidate of its
// chunk in `part_val/part_idx`; the block that finishes last for a row (counted in
// `counters`, which it sets back to zero) reduces the row's candidates and writes the token.
__global__ void __launch_bounds__(THREADS) sample_kernel(int* __restrict__ tokens, const float* __restrict__ logits,
                                                         long long ld, int vocab, const float* __restrict__ temperature,
                                                         const uint32_t* __restrict__ seeds,
                                                         const int* __restrict__ positions, float* __restrict__ part_val,
                                                         int* __restrict__ part_idx, int* __restrict__ counters) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ int is_last;
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.y, chunk = blockIdx.x, n_chunks = gridDim.x;
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
  const int end = min(vocab, (chunk + 1) * CHUNK);
  auto consider = [&](float v, int i) {
    if (temp > 0.f) {
      const uint32_t h = mix32(key + (uint32_t)i * 0x85EBCA6Bu);
      const float u = ((float)(h >> 9) + 0.5f) * (1.f / 8388608.f);
      v = v * inv_temp - logf(-logf(u));
    }
    if (better(v, i, bv, bi)) { bv = v; bi = i; }  // a NaN compares false and never wins
  };
  if ((ld & 3) == 0 && (((uintptr_t)logits) & 15) == 0) {
    // rows of 16-byte multiples: four entries a load, the chunk's four loads of a thread in flight together
    constexpr int ROUNDS = CHUNK / (THREADS * 4);
    float4 q[ROUNDS];
#pragma unroll
    for (int it = 0; it < ROUNDS; ++it) {
      const int i = chunk * CHUNK + (it * THREADS + (int)threadIdx.x) * 4;
      q[it] = i + 3 < end ? *reinterpret_cast<const float4*>(lr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int it = 0; it < ROUNDS; ++it) {
      const int i = chunk * CHUNK + (it * THREADS + (int)threadIdx.x) * 4;
      if (i + 3 < end) {
        consider(q[it].x, i);
        consider(q[it].y, i + 1);
        consider(q[it].z, i + 2);
        consider(q[it].w, i + 3);
      } else {
        for (int j = i; j < end; ++j) consider(lr[j], j);
      }
    }
  } else {
    for (int i = chunk * CHUNK + threadIdx.x; i < end; i += THREADS) consider(lr[i], i);
  }
  auto block_best = [&]() {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      bv = lane < THREADS / 32 ? sv[lane] : -INFINITY;
      bi = lane < THREADS / 32 ? si[lane] : INT_MAX;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
      }
    }
  };
  block_best();
  if (n_chunks == 1) {
    if (threadIdx.x == 0) tokens[row] = bi;
    return;
  }
  if (threadIdx.x == 0) {
    part_val[(size_t)row * n_chunks + chunk] = bv;
    part_idx[(size_t)row * n_chunks + chunk] = bi;
    __threadfence();
    is_last = atomicAdd(&counters[row], 1) == n_chunks - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  bv = -INFINITY;
  bi = INT_MAX;
  for (int c = threadIdx.x; c < n_chunks; c += THREADS) {
    const float v = part_val[(size_t)row * n_chunks + c];
    const int i = part_idx[(size_t)row * n_chunks + c];
    if (better(v, i, bv, bi)) { bv = v; bi = i; }
  }
  block_best();
  if (threadIdx.x == 0) {
    tokens[row] = bi;
    counters[row] = 0;   // ready for the next call
  }
}
}  // namespace

LAB_EXPORT int lab_sample_chunks(int vocab) { return (vocab + CHUNK - 1) / CHUNK; }

// temperature, seeds, positions: per row; temperature == nullptr or 0 means greedy.
// scratch: rows * chunks floats (part_val), rows * chunks ints (part_idx), rows ints (counters, zero
// before the first call; the kernel leaves them zero).  May be null when the vocabulary fits one chunk.
LAB_EXPORT int lab_sample(int* tokens, const float* logits, long long ld, int rows, int vocab, const float* temperature,
                          const uint32_t* seeds, const int* positions, float* part_val, int* part_idx, int* counters,
                          cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int chunks = (vocab + CHUNK - 1) / CHUNK;
  if (chunks > 1 && (!part_val || !part_idx || !counters)) return (int)cudaErrorInvalidValue;
  return (int)lab_launch(sample_kernel, dim3(chunks, rows), dim3(THREADS), 0, stream, tokens, logits, ld, vocab,
                         temperature, seeds, positions, part_val, part_idx, counters);
}
