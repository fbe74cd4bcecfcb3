// Causal prefill attention over the paged cache on the 5th-generation tensor cores, for heads
// of 64 and of 128 (-DLAB_HEAD_DIM) and page sizes of 8, 16, 32, 64 or 128 tokens.
//
// One CTA serves 128 query rows of one head of one request and walks the keys in tiles of 128:
//   S = Q K^T        tcgen05.mma, Q and K tiles in 128-byte-swizzled shared memory (TMA; K is
//                    gathered page by page through the block table; a head of 128 is two swizzled
//                    tiles of 64 columns side by side), S in tensor memory
//   P = softmax(S)   four warps, one query row per thread: tcgen05.ld of the row, scale and
//                    causal/window mask, running max and sum in 32-bit, exp2, P rounded to
//                    bfloat16 and written back to tensor memory (tcgen05.st, two keys per column)
//   O_j = P V        tcgen05.mma with P as the A operand from tensor memory and V as the N-major
//                    B operand from shared memory (V rows lie [key][d] as cached), 64 output
//                    columns per instruction
// Tensor memory holds two S buffers, so that the scores of tile j+1 are formed beside the softmax of
// tile j, and one O of D columns that accumulates over all tiles.  P overwrites the scores it came
// from (the next scores for that buffer are issued after the product that reads P).  A row's O is
// rescaled in place only when its maximum has grown by more than a factor of 256 since the reference
// it is held against, and divided by the sum at the end.  (Measured slower: for heads of 64 an
// accumulator in registers, rescaled every tile from two O buffers, by 10 %; two CTAs per SM with one
// S buffer each, by 70 % at 2,048 tokens and 6 % at 8,192.  No faster: two groups of four softmax warps
// that share the key tiles, even and odd, each with an S buffer, an O and running maxima of its own,
// merged at the end; 2.96 ms a 2,048-token prefill of 24 layers either way.  In-kernel clocks of the
// CTA with the most keys showed why: a warp's 128 ex2 of a tile take about 1,000 cycles of the one
// special-function unit of its SM sub-partition, which two groups can only share; a group that has
// handed over P waits about 1,500 cycles for its next scores (wake the MMA warp, issue P V, issue S,
// the MMAs, wake the group), which the other group's exponentials fill but do not shorten; the first
// scores of a CTA arrive 5,000 cycles after its start and the masked tile on the diagonal takes twice
// the time of a full one.)
// Formulas as the reference's tensor-core prefill attention
// (rust/engine/src/runner/model/qwen2/kernels.rs:946-1124, 1295-1452): scores scaled by 1/sqrt(d)
// (folded into the exp2 argument), key <= query, p rounded to T before PV, o = acc / sum.
//
// Warp 0 loads (TMA; the page that holds a request's last keys is copied by hand with rows
// beyond the length set to zero, and the rows of V of pages that are not fetched at all are set to
// zero, because a masked NaN would still poison P V), warp 1 issues the MMAs (the whole warp walks
// the loop, one elected lane issues) and owns tensor memory, warps 2-5 do the softmax.  Every wait
// is bounded.
#include "tcgen05.cuh"

#ifndef LAB_HEAD_DIM
#error "build with -DLAB_HEAD_DIM=64 or 128"
#endif

namespace {

constexpr int D = LAB_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 attention kernel is built for heads of 64 and of 128");
constexpr int BM = 128;        // query rows per CTA
constexpr int BN = 128;        // keys per tile
constexpr int THREADS = 192;
constexpr int ROW = 128;       // bytes of a swizzled row: 64 bf16
constexpr int HALVES = D / 64; // a head's row is cut into 64-wide halves, each a swizzled tile of its own
constexpr int HALF_BYTES = 128 * ROW;        // 128 rows (queries or keys) of one half
constexpr int KV_STAGES = D == 64 ? 4 : 2;
constexpr int Q_BYTES = HALVES * HALF_BYTES;
constexpr int KV_TILE = HALVES * HALF_BYTES;  // one K or V tile
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + Q_BYTES;
constexpr int OFF_V = OFF_K + KV_STAGES * KV_TILE;
constexpr int OFF_BAR = OFF_V + KV_STAGES * KV_TILE;
constexpr int SMEM = OFF_BAR + 256 + 1024;
// tensor memory columns: two S buffers (32-bit scores), then one O of D columns.  P (bfloat16 pairs:
// 128 keys in 64 columns) lies in the first 64 columns of the S buffer it came from.
constexpr int TM_S = 0, TM_O = 2 * BN, TMEM_COLS = 512;
static_assert(TM_O + D <= TMEM_COLS, "tensor memory holds S and O");
constexpr float LOG2E = 1.4426950408889634f;

// bf16 x bf16 -> f32, M = 128, N = n; b_n_major: the B operand is N-major (V as cached) instead of K-major.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_n_major) { return umma_instr_desc(BM, n, b_n_major); }

struct Barriers {
  uint64_t q_full;
  uint64_t kv_full[KV_STAGES], kv_empty[KV_STAGES];
  uint64_t s_full[2], s_empty[2], p_full[2], o_full;
  uint32_t tmem_slot;
  int abort_flag;
};

__global__ void __launch_bounds__(THREADS) attention_prefill_tc05_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, int out_stride,
    const __nv_bfloat16* __restrict__ cache_k, const __nv_bfloat16* __restrict__ cache_v,
    const int* __restrict__ q_start, const int* __restrict__ kv_len_arr, const int* __restrict__ pos0_arr,
    const int* __restrict__ block_table, int max_blocks, int n_q, int n_kv, int page_size, int num_pages, int window,
    float scale_log2, int min_q_len) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Barriers* bar = reinterpret_cast<Barriers*>(smem + OFF_BAR);
  volatile int* abort_flag = &bar->abort_flag;
  pdl_trigger();
  // Until pdl_wait() below only the step's metadata is read (no kernel of the step writes it): the
  // set-up of the CTA runs while the kernel before this one finishes.
  // Blocks are numbered with the head fastest and the tiles of the latest rows first: the CTAs
  // that walk the most keys all start in the first wave.
  const int b = blockIdx.z, h = blockIdx.x;
  const int qs = q_start[b], ql = q_start[b + 1] - qs;
  const int r0 = (gridDim.y - 1 - blockIdx.y) * BM;
  if (ql < min_q_len || r0 >= ql) {
    pdl_wait();  // this kernel ends only after the one before it: what follows may count on both
    return;
  }
  const int kvh = h / (n_q / n_kv);
  const int p0 = pos0_arr[b], kvl = kv_len_arr[b];
  const int* bt = block_table + (size_t)b * max_blocks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int last_row = min(r0 + BM, ql) - 1;
  const int hi_all = p0 + last_row;                                    // last key any row sees
  const int lo_all = window > 0 ? max(0, p0 + r0 - window + 1) : 0;    // first key any row sees
  const int t_first = lo_all / BN, t_last = hi_all / BN;
  const int n_tiles = t_last - t_first + 1;

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bar->kv_full[s], 2);  // the expect_tx arrival and the arrival after hand copies
      mbar_init(&bar->kv_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->s_full[i], 1);
      mbar_init(&bar->s_empty[i], 4);
      mbar_init(&bar->p_full[i], 4);
    }
    mbar_init(&bar->o_full, 1);
    bar->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(&bar->tmem_slot, TMEM_COLS);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = bar->tmem_slot;
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0) {
    // ---------------- loader ----------------
    if (lane == 0) {
      mbar_expect_tx(&bar->q_full, Q_BYTES);
      for (int hf = 0; hf < HALVES; ++hf)
        tma_load_2d(smem_base + OFF_Q + hf * HALF_BYTES, &map_q, &bar->q_full, h * D + hf * 64, qs + r0);
    }
    const int pages_per_tile = BN / page_size;  // at most 16: one lane looks up each page of a tile
    const int page_bytes = page_size * ROW;
    bool alive = true;
    // Lane pg classifies page pg of a tile and reads its number from the block table:
    // 0 nothing to fetch (beyond the length, or wholly before the window), 1 whole page (TMA),
    // 2 the page that holds the request's last keys (copied by hand, rows past the length zeroed).
    // The lookup for tile j + 1 is issued before tile j's copies, so its latency hides behind them.
    auto classify = [&](int j, int& kind, int& page) {
      kind = 0;
      page = -1;
      if (j < n_tiles && lane < pages_per_tile) {
        const int k_lo = (t_first + j) * BN + lane * page_size;
        if (k_lo < kvl && k_lo + page_size > lo_all) {
          kind = k_lo + page_size > kvl ? 2 : 1;
          page = bt[k_lo / page_size];
        }
      }
    };
    int next_kind, next_page;
    classify(0, next_kind, next_page);
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int s = j % KV_STAGES;
      const uint32_t ph = (j / KV_STAGES) & 1;
      const int key0 = (t_first + j) * BN;
      int kind = next_kind, page = next_page;
      classify(j + 1, next_kind, next_page);
      if (kind != 0 && (page < 0 || page >= num_pages)) {  // a page inside the length and the window must exist
        lab_set_error(LAB_ERR_PAGE_RANGE);
        kind = 0;
      }
      const uint32_t tma_lanes = __ballot_sync(0xffffffffu, kind == 1);
      const uint32_t tail_lanes = __ballot_sync(0xffffffffu, kind == 2);
      uint32_t skip_lanes = __ballot_sync(0xffffffffu, kind == 0 && lane < pages_per_tile);
      if (lane == 0) alive = mbar_wait(&bar->kv_empty[s], ph ^ 1, abort_flag);
      alive = __shfl_sync(0xffffffffu, alive, 0);
      if (!alive) break;
      const uint32_t k_dst = smem_base + OFF_K + s * KV_TILE, v_dst = smem_base + OFF_V + s * KV_TILE;
      // Lane 0 announces the bytes (one of the barrier's two arrivals); then every lane fetches its
      // own page, so the copies of a tile are issued side by side.  The phase cannot end before the
      // second arrival below, whatever the order in which bytes are announced and land.
      if (lane == 0) mbar_expect_tx(&bar->kv_full[s], 2 * HALVES * __popc(tma_lanes) * page_bytes);
      __syncwarp();
      if (kind == 1) {
        const int row = (page * n_kv + kvh) * page_size;
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
          tma_load_2d(k_dst + hf * HALF_BYTES + lane * page_bytes, &map_k, &bar->kv_full[s], hf * 64, row);
          tma_load_2d(v_dst + hf * HALF_BYTES + lane * page_bytes, &map_v, &bar->kv_full[s], hf * 64, row);
        }
      }
      if (tail_lanes) {
        // The page with the request's last keys: rows below the length are copied, the rest set to
        // zero, in the swizzled layout (16-byte chunk c of row r lies at chunk c ^ (r % 8)).
        const int tail_slot = __ffs(tail_lanes) - 1;
        const int tail_page = __shfl_sync(0xffffffffu, page, tail_slot);
        const int k_lo = key0 + tail_slot * page_size;
        const size_t src0 = ((size_t)tail_page * n_kv + kvh) * page_size * D;
        for (int c = lane; c < page_size * (D / 8); c += 32) {
          const int r = c / (D / 8), q16 = c - r * (D / 8), hf = q16 >> 3, q8 = q16 & 7;
          const int tile_row = tail_slot * page_size + r;
          uint4 kk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
          if (k_lo + r < kvl) {
            kk = *reinterpret_cast<const uint4*>(cache_k + src0 + (size_t)r * D + q16 * 8);
            vv = *reinterpret_cast<const uint4*>(cache_v + src0 + (size_t)r * D + q16 * 8);
          }
          const int off = hf * HALF_BYTES + tile_row * ROW + ((q8 ^ (tile_row & 7)) << 4);
          *reinterpret_cast<uint4*>(smem + OFF_K + s * KV_TILE + off) = kk;
          *reinterpret_cast<uint4*>(smem + OFF_V + s * KV_TILE + off) = vv;
        }
      }
      // Pages that are not fetched (beyond the length, before the window) leave stale rows in the
      // stage.  Their keys are masked, but p = 0 times a stale NaN would still poison P V: their
      // rows of V are set to zero.
      while (skip_lanes) {
        const int slot = __ffs(skip_lanes) - 1;
        skip_lanes &= skip_lanes - 1;
        for (int hf = 0; hf < HALVES; ++hf) {
          uint4* vz = reinterpret_cast<uint4*>(smem + OFF_V + s * KV_TILE + hf * HALF_BYTES + slot * page_bytes);
          for (int c = lane; c < page_bytes / 16; c += 32) vz[c] = make_uint4(0, 0, 0, 0);
        }
      }
      proxy_fence();  // the hand-written rows become visible to the tensor cores
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->kv_full[s]);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the loop with the same values, and one elected lane issues each MMA and
    // commit: the operands are uniform across the warp, as the instructions want them.
    {
      constexpr uint32_t idesc_s = instr_desc(BN, false);
      constexpr uint32_t idesc_o = instr_desc(64, true);   // P V in pieces of 64 output columns
      auto wait_all = [&](uint64_t* b, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(b, parity, abort_flag));
      };
      bool ok = wait_all(&bar->q_full, 0);
      auto issue_s = [&](int j) -> bool {
        const int s = j % KV_STAGES, sb = j & 1;
        if (!wait_all(&bar->kv_full[s], (j / KV_STAGES) & 1)) return false;
        if (!wait_all(&bar->s_empty[sb], ((j >> 1) & 1) ^ 1)) return false;
        tc_fence_after();
        // descriptors of the first 16 dimensions; each further 16 lie 32 bytes (two address units) on
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
          const uint64_t qd = smem_desc_sw128(smem_base + OFF_Q + hf * HALF_BYTES),
                         kd = smem_desc_sw128(smem_base + OFF_K + s * KV_TILE + hf * HALF_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + TM_S + sb * BN, qd + 2 * k, kd + 2 * k, idesc_s, (hf | k) > 0 ? 1u : 0u);
        }
        umma_commit(&bar->s_full[sb]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);  // the next tile's scores run beside this tile's softmax
        if (!ok) break;
        const int s = j % KV_STAGES, sb = j & 1;
        ok = wait_all(&bar->p_full[sb], (j >> 1) & 1);
        if (!ok) break;
        tc_fence_after();
        // V rows are keys: 16 keys lie 16 * 128 bytes (128 address units) on.  The product is formed in
        // pieces of 64 output columns and added to the one O of all tiles.
        const uint32_t o_at = tmem_base + TM_O;
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
          const uint64_t vd = smem_desc_sw128(smem_base + OFF_V + s * KV_TILE + hf * HALF_BYTES);
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            umma_bf16_tmem_a(o_at + hf * 64, tmem_base + TM_S + sb * BN + kk * 8,
                             vd + (uint64_t)(kk * 16 * ROW / 16), idesc_o,
                             (kk | j) > 0 ? 1u : 0u);
        }
        umma_commit(&bar->o_full);
        umma_commit(&bar->kv_empty[s]);  // both products of this stage have been issued
      }
    }
  } else {
    // ---------------- softmax: one query row per thread ----------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;            // row of the tile = lane of tensor memory
    const int pos = p0 + r0 + row;                  // absolute position of this row's query
    const bool row_valid = r0 + row < ql;
    const int hi = row_valid ? pos : -1;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    {
      // O accumulates in tensor memory over all tiles, relative to a reference maximum m_ref per row
      // (log2 units); l is the running sum relative to m_ref.  m_ref follows the true maximum lazily: only when a row's maximum has grown by more than RESCALE (a factor
      // of 256) is the row of O rescaled, so p = 2^(s - m_ref) stays below 256: exact in the exponent,
      // rounded to bfloat16 as ever, and O and l are 32-bit.  P overwrites the scores it came from.
      constexpr float RESCALE = 8.f;
      const uint32_t o_addr = lane_addr + TM_O;
      float m_ref = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; j < n_tiles; ++j) {
        const int sb = j & 1;
        ok = ok && mbar_wait(&bar->s_full[sb], (j >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sr[BN];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) tmem_ld32_issue(lane_addr + TM_S + sb * BN + c * 32, sr + c * 32);
        tmem_wait();
        const int key0 = (t_first + j) * BN;
        const bool all_visible = key0 >= lo && key0 + BN - 1 <= hi;
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (all_visible) {
#pragma unroll
          for (int c = 0; c < BN; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c]));
        } else {
#pragma unroll
          for (int c = 0; c < BN; ++c) {
            if (key0 + c < lo || key0 + c > hi) sr[c] = __float_as_uint(-INFINITY);
            mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c]));
          }
        }
        const float m_new = fmaxf(m_ref, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2);
        if (j == 0) {
          m_ref = m_new;
        } else if (__any_sync(0xffffffffu, m_new > m_ref + RESCALE || (m_ref == -INFINITY && m_new != -INFINITY))) {
          // Some row of this warp has outgrown its reference: every row of the warp moves to its true
          // maximum.  The product of the previous tile must have landed in O before O is rescaled.
          ok = ok && mbar_wait(&bar->o_full, (j - 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const float f = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);  // 1 for a row that has not grown
#pragma unroll
          for (int part = 0; part < D / 32; ++part) {
            uint32_t r[32];
            tmem_ld32_issue(o_addr + part * 32, r);
            tmem_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
            tmem_st32(o_addr + part * 32, r);
          }
          l *= f;
          m_ref = m_new;
        }
        const float base = (m_ref == -INFINITY) ? 0.f : m_ref;  // a row that has seen no key yet
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c32 = 0; c32 < BN / 64; ++c32) {
          uint32_t pk[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int c = c32 * 64 + 2 * i;
            const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c]), scale_log2, -base));  // 2^(-inf) = 0 for masked keys
            const float p1 = fast_exp2(fmaf(__uint_as_float(sr[c + 1]), scale_log2, -base));
            sum4[i & 1] += p0;
            sum4[2 + (i & 1)] += p1;
            pk[i] = pack_bf16(p0, p1);
          }
          tmem_st32(lane_addr + TM_S + sb * BN + c32 * 32, pk);
        }
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        tmem_st_wait();
        // The product of the tile before is awaited in every tile, before this warp's arrival lets
        // the product of this tile be issued: a parity names a phase only among the current one and
        // the one before, and at this point the barrier can only be in phase j - 1 or j.  (It has
        // long completed: that product ran beside this tile's softmax.)
        if (j > 0) {
          ok = mbar_wait(&bar->o_full, (j - 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        tc_fence_before();  // the loads of S and the stores of P (and of O) are ordered before the arrivals
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bar->s_empty[sb]);  // given free with P: the next scores for this buffer are
          mbar_arrive(&bar->p_full[sb]);   // issued after the product that reads P from it
        }
      }
      // The last product: the barrier is in phase n - 1 or has completed it.
      if (ok && n_tiles > 0) {
        ok = mbar_wait(&bar->o_full, (n_tiles - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = out + (size_t)(qs + r0 + row) * out_stride + (size_t)h * D;
#pragma unroll
        for (int part = 0; part < D / 32; ++part) {
          uint32_t r[32];
          tmem_ld32_issue(o_addr + part * 32, r);   // every lane takes part in the load
          tmem_wait();
          if (!row_valid || n_tiles == 0) continue;
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            const uint4 packed = make_uint4(
                pack_bf16(__uint_as_float(r[q8 * 8]) * inv, __uint_as_float(r[q8 * 8 + 1]) * inv),
                pack_bf16(__uint_as_float(r[q8 * 8 + 2]) * inv, __uint_as_float(r[q8 * 8 + 3]) * inv),
                pack_bf16(__uint_as_float(r[q8 * 8 + 4]) * inv, __uint_as_float(r[q8 * 8 + 5]) * inv),
                pack_bf16(__uint_as_float(r[q8 * 8 + 6]) * inv, __uint_as_float(r[q8 * 8 + 7]) * inv));
            __nv_bfloat16* d8 = dst + part * 32 + q8 * 8;
            if ((((uintptr_t)d8) & 15) == 0) {
              *reinterpret_cast<uint4*>(d8) = packed;
            } else {
              const __nv_bfloat16* hp = reinterpret_cast<const __nv_bfloat16*>(&packed);
              for (int e = 0; e < 8; ++e) d8[e] = hp[e];
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

LAB_EXPORT int lab_attention_tc05_head_dim() { return D; }

// 1 if the kernel takes this page size (pages are fetched as TMA boxes and must tile 128 keys
// with swizzle groups of 8 rows).
LAB_EXPORT int lab_attention_tc05_supports(int page_size) {
  return page_size >= 8 && page_size <= BN && (page_size & (page_size - 1)) == 0;
}

// Arguments as lab_attention_prefill; total_rows is the number of rows of q (for the TMA bounds).
LAB_EXPORT int lab_attention_prefill_tc05(void* out, int out_stride, const void* q, int q_stride, int total_rows,
                                          const void* cache_k, const void* cache_v, const int* q_start,
                                          const int* kv_len, const int* pos0, const int* block_table, int max_blocks,
                                          int requests, int max_q_len, int n_q, int n_kv, int page_size, int num_pages,
                                          int window, float scale, int min_q_len, cudaStream_t stream) {
  if (requests <= 0 || max_q_len <= 0) return 0;
  if (!lab_attention_tc05_supports(page_size) || n_q % n_kv || q_stride % 8 || (((uintptr_t)q) & 15) ||
      (((uintptr_t)cache_k) & 15) || (((uintptr_t)cache_v) & 15))
    return (int)cudaErrorInvalidValue;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = lab_make_map_bf16(&mq, q, total_rows, n_q * D, q_stride, BM))) return rc;
  const long long cache_rows = (long long)num_pages * n_kv * page_size;
  if ((rc = lab_make_map_bf16(&mk, cache_k, cache_rows, D, D, page_size))) return rc;
  if ((rc = lab_make_map_bf16(&mv, cache_v, cache_rows, D, D, page_size))) return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(attention_prefill_tc05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(n_q, (max_q_len + BM - 1) / BM, requests);
  return (int)lab_launch(attention_prefill_tc05_kernel, grid, dim3(THREADS), (size_t)SMEM, stream, mq, mk, mv,
                         (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)cache_k, (const __nv_bfloat16*)cache_v,
                         q_start, kv_len, pos0, block_table, max_blocks, n_q, n_kv, page_size, num_pages, window,
                         scale * LOG2E, min_q_len);
}
