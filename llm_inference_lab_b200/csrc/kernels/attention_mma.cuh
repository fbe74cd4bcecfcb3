// Pieces of the mma.sync attention kernels, shared by the files that walk the paged cache with
// them: asynchronous copies of key and value rows through a block table, and one tile of
// scores, masked online softmax and P V for 16 query rows held by a warp.  Built for one head
// size (-DLAB_HEAD_DIM=d, a multiple of 16 up to 128).
// Formulas: rust/engine/src/runner/model/qwen2/kernels.rs:946-1124 (tile loop).
#pragma once
#include "common.cuh"

#ifndef LAB_HEAD_DIM
#error "build with -DLAB_HEAD_DIM=<head size>"
#endif

constexpr int D = LAB_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 128, "head size must be a multiple of 16 up to 128");
constexpr int ROW_BYTES = D * 2 + 16;  // padded shared-memory row
constexpr int CPR = D / 8;             // 16-byte chunks per row
constexpr int KSTEPS = D / 16;         // k-steps of q . k
constexpr int DTILES = D / 8;          // 8-wide column tiles of the output
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the destination is filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Where key `j` of a request lies: element offset of its row in the cache, -1 if its page was
// given back, -2 if the block table names a page outside the pool (reported by the caller).
__device__ __forceinline__ long long key_offset(const int* __restrict__ bt, int j, int kvh, int n_kv, int page_size,
                                                int num_pages) {
  const int blk = j / page_size;
  const int page = bt[blk];
  if (page < 0) return -1;
  if (page >= num_pages) return -2;
  return (((long long)page * n_kv + kvh) * page_size + (j - blk * page_size)) * D;
}

// One tile of BN keys for 16 query rows held by a warp: scores, masked online softmax, PV.
//   qf: the rows' q fragments; ks/vs: shared-memory tiles [BN][ROW_BYTES];
//   rows of this thread: lane/4 (index 0) and lane/4 + 8 (index 1); a key j is visible to row i
//   iff lo[i] <= j <= hi[i].  m, l, o carry the running max (log2 units), sum and accumulator.
template <int BN>
__device__ __forceinline__ void tile_step(const uint32_t (&qf)[KSTEPS][4], uint32_t ks, uint32_t vs,
                                          float (&o)[DTILES][4], float (&m)[2], float (&l)[2], int key0,
                                          const int (&lo)[2], const int (&hi)[2], float scale_log2, int lane,
                                          bool all_visible = false) {
  float s[BN / 8][4];
#pragma unroll
  for (int j = 0; j < BN / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
  // S = Q K^T
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
#pragma unroll
    for (int jp = 0; jp < BN / 16; ++jp) {
      uint32_t b[4];
      const int key = jp * 16 + (lane & 7) + 8 * (lane >> 4);
      const int dcol = k * 16 + 8 * ((lane >> 3) & 1);
      ldmatrix_x4(b, ks + key * ROW_BYTES + dcol * 2);
      mma_bf16(s[2 * jp], qf[k], b[0], b[1]);
      mma_bf16(s[2 * jp + 1], qf[k], b[2], b[3]);
    }
  }
  // mask, scale, running max
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < BN / 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + j * 8 + 2 * (lane & 3) + (e & 1);
      const int r = e >> 1;
      const bool ok = all_visible || (key >= lo[r] && key <= hi[r]);
      s[j][e] = ok ? s[j][e] * scale_log2 : -INFINITY;
      mx[r] = fmaxf(mx[r], s[j][e]);
    }
  float corr[2], base[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(m[r], mx[r]);
    base[r] = (m_new == -INFINITY) ? 0.f : m_new;
    corr[r] = (m[r] == -INFINITY) ? 0.f : fast_exp2(m[r] - base[r]);
    m[r] = m_new;
  }
  float sum[2] = {0.f, 0.f};
  uint32_t pf[BN / 16][4];
#pragma unroll
  for (int j = 0; j < BN / 8; ++j) {
    float p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      p[e] = fast_exp2(s[j][e] - base[e >> 1]);  // exp2(-inf) = 0 for masked keys
      sum[e >> 1] += p[e];
    }
    pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
    pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) l[r] = l[r] * corr[r] + sum[r];  // quad-reduced at the very end
#pragma unroll
  for (int t = 0; t < DTILES; ++t) {
    o[t][0] *= corr[0];
    o[t][1] *= corr[0];
    o[t][2] *= corr[1];
    o[t][3] *= corr[1];
  }
  // O += P V
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
    for (int tp = 0; tp < DTILES / 2; ++tp) {
      uint32_t b[4];
      const int key = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
      const int dcol = tp * 16 + 8 * (lane >> 4);
      ldmatrix_x4_trans(b, vs + key * ROW_BYTES + dcol * 2);
      mma_bf16(o[2 * tp], pf[kk], b[0], b[1]);
      mma_bf16(o[2 * tp + 1], pf[kk], b[2], b[3]);
    }
  }
}

// R consecutive keys (R <= 32) and their values copied by one warp: lane r < R looks up the page
// of key0 + r once, then the lanes share the row offsets by shuffle, so that a tile costs one
// page lookup per lane and no 64-bit arithmetic per 16-byte chunk.  Keys outside
// [first_key, kv_len) and keys whose page was given back become rows of zeros (they are masked).
template <int R>
__device__ __forceinline__ void load_kv_rows_warp(uint32_t dst_k, uint32_t dst_v,
                                                  const __nv_bfloat16* __restrict__ cache_k,
                                                  const __nv_bfloat16* __restrict__ cache_v,
                                                  const int* __restrict__ bt, int key0, int first_key, int kv_len,
                                                  int kvh, int n_kv, int page_size, int num_pages, int lane) {
  const int j = key0 + lane;
  long long mine = -1;
  if (lane < R && j >= first_key && j < kv_len) mine = key_offset(bt, j, kvh, n_kv, page_size, num_pages);
  if (mine == -2) lab_set_error(LAB_ERR_PAGE_RANGE);
  constexpr int CHUNKS = R * CPR;
  constexpr int PASSES = (CHUNKS + 31) / 32;
#pragma unroll
  for (int i = 0; i < PASSES; ++i) {
    const int idx = i * 32 + lane;
    const int row = idx / CPR, col = idx - row * CPR;
    const long long off = __shfl_sync(0xffffffffu, mine, row & 31);
    if (idx >= CHUNKS) continue;
    const long long o = off < 0 ? 0 : off;
    cp_async16(dst_k + row * ROW_BYTES + col * 16, cache_k + o + col * 8, off >= 0);
    cp_async16(dst_v + row * ROW_BYTES + col * 16, cache_v + o + col * 8, off >= 0);
  }
}

