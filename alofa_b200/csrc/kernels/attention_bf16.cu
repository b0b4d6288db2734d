// Causal grouped-query attention over the paged bfloat16 cache, for prefill
// portions and decode tokens in one launch.
//
// One CTA owns one (request, KV head, tile of 64 query rows).  A query row is a
// (token, head-of-the-group) pair: the g = heads / kv_heads query heads that
// share a KV head are packed along the row axis, so the K/V pages of that head
// are read once for all of them (for one decode token the tile holds its g
// heads).  Keys are streamed in blocks of 64 through shared memory with
// cp.async (double buffered), found through the request's block table row by
// row, so any page size works.  Scores and the output accumulate in fp32 with
// mma.sync m16n8k16 (bf16 operands); softmax is the streaming form in fp32:
// running maximum, exp2 with the scale folded in, rescaled sums.
// Visibility: key j is seen by the row at position P when j <= P and, with a
// window, j > P - window.
//
// Decode-only launches may split the keys of a request over several CTAs
// (split s owns keys [s * split_keys, (s + 1) * split_keys), a function of the
// key index alone); the partial (output, maximum, sum) triples are merged by
// attention_combine_kernel in split order.
//
// Prompt portions go to the tcgen05 kernel of attention_prefill_tc.cuh instead
// when the head size is 64 or 128 and a page holds whole 64-key blocks; decode
// tokens of small head groups to attention_decode_kernel below.
//
// HEAD_DIM is a compile-time constant (a multiple of 16 up to 128): the
// library is built per head size.  Formulas: src/alofa/kernels/cpu/scalar.mojo:392-470,
// paged addressing src/alofa/kernels/cpu/paged.mojo:249-336.
#include "common.cuh"
#include "tma.cuh"
#include "attention_core.cuh"

struct AttnParams {
  bf16* out;             // [T, nh, HD]
  const bf16* q;         // [T, nh, HD]
  const bf16* k_cache;   // [slots, nkv, HD]
  const bf16* v_cache;
  const int* q_start;    // [R + 1] first row of each request in this step
  const int* kv_len;     // [R] keys of each request after this step
  const int* block_table;  // [R, max_blocks]
  float* partial_o;      // split mode: [splits, T * nh, HD]
  float* partial_ml;     // split mode: [splits, T * nh, 2]
  int max_blocks, page_size, nh, nkv, window, split_keys, n_splits, n_rows_total, table_entries;
  float scale_log2;      // scale * log2(e)
  int* status;           // set to 2 when a wait on a bulk copy gave up (may be null)
};

#include "attention_prefill_tc.cuh"

// Copy keys [j0, j0 + 64) of one KV head, keys and values, into shared tiles
// [64][ROW]; rows past j_end (exclusive) or before j_begin are zero-filled.
// `table` is the shared copy of the request's block-table entries from entry
// `first_entry` on (a lookup in global memory here would stall every copy
// behind it).  When a page holds whole key blocks (page_size % 64 == 0) the
// block lies in one page and a row's address is the block's base plus a fixed
// stride; else every row looks its page up.
__device__ __forceinline__ void load_kv_tiles(bf16* k_tile, bf16* v_tile, const bf16* k_cache, const bf16* v_cache, const int* table,
                                              int first_entry, int page_size, bool block_in_page, int nkv, int kvh, int j0, int j_begin,
                                              int j_end) {
  if constexpr (128 % CHUNKS != 0) {
    // head sizes whose rows do not divide a round of 128 threads: one chunk at a time
    for (int idx = threadIdx.x; idx < BLOCK_N * CHUNKS; idx += 128) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      const int j = j0 + r;
      const bool ok = j >= j_begin && j < j_end;
      size_t offset = 0;
      if (ok) {
        const int e = j / page_size;
        const int slot = table[e - first_entry] * page_size + (j - e * page_size);
        offset = ((size_t)slot * nkv + kvh) * HD + c * 8;
      }
      cp_async16((uint32_t)__cvta_generic_to_shared(k_tile + r * ROW + c * 8), k_cache + offset, ok);
      cp_async16((uint32_t)__cvta_generic_to_shared(v_tile + r * ROW + c * 8), v_cache + offset, ok);
    }
    return;
  }
  const int r0 = threadIdx.x / CHUNKS, c = threadIdx.x % CHUNKS;
  const uint32_t k_dst = (uint32_t)__cvta_generic_to_shared(k_tile + r0 * ROW + c * 8);
  const uint32_t v_dst = (uint32_t)__cvta_generic_to_shared(v_tile + r0 * ROW + c * 8);
  constexpr int ROWS_PER_ROUND = (128 % CHUNKS == 0) ? 128 / CHUNKS : 1;
  if (block_in_page) {
    const int e = j0 / page_size;
    const size_t first_slot = (size_t)table[e - first_entry] * page_size + (j0 - e * page_size);
    const size_t base = ((first_slot + r0) * nkv + kvh) * HD + c * 8;
    const size_t step = (size_t)ROWS_PER_ROUND * nkv * HD;
#pragma unroll
    for (int it = 0; it < BLOCK_N / ROWS_PER_ROUND; ++it) {
      const int j = j0 + r0 + it * ROWS_PER_ROUND;
      const bool ok = j >= j_begin && j < j_end;
      const size_t offset = ok ? base + it * step : 0;
      cp_async16(k_dst + it * ROWS_PER_ROUND * ROW * 2, k_cache + offset, ok);
      cp_async16(v_dst + it * ROWS_PER_ROUND * ROW * 2, v_cache + offset, ok);
    }
    return;
  }
#pragma unroll
  for (int it = 0; it < BLOCK_N / ROWS_PER_ROUND; ++it) {
    const int j = j0 + r0 + it * ROWS_PER_ROUND;
    const bool ok = j >= j_begin && j < j_end;
    size_t offset = 0;
    if (ok) {
      const int e = j / page_size;
      const int slot = table[e - first_entry] * page_size + (j - e * page_size);
      offset = ((size_t)slot * nkv + kvh) * HD + c * 8;
    }
    cp_async16(k_dst + it * ROWS_PER_ROUND * ROW * 2, k_cache + offset, ok);
    cp_async16(v_dst + it * ROWS_PER_ROUND * ROW * 2, v_cache + offset, ok);
  }
}

// STAGES key blocks are in flight at a time; a decode split of up to
// STAGES * 64 keys is fetched in one go, so its latency is paid once.
template <bool SPLIT, int STAGES>
__global__ void __launch_bounds__(128) attention_bf16_kernel(const AttnParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);          // [64][ROW]
  bf16* k_tiles = q_tile + BLOCK_M * ROW;                    // [STAGES][64][ROW]
  bf16* v_tiles = k_tiles + STAGES * BLOCK_N * ROW;          // [STAGES][64][ROW]
  pdl_begin();

  const int seq = blockIdx.z, kvh = blockIdx.y;
  const int g = p.nh / p.nkv;
  const int row_begin = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - row_begin;
  const int kv_len = p.kv_len[seq];
  const int pos0 = kv_len - q_len;
  const int n_rows = q_len * g;
  // split mode: blockIdx.x = tile * n_splits + split (decode tokens have one tile)
  const int tile = SPLIT ? (int)blockIdx.x / p.n_splits : (int)blockIdx.x;
  const int split = SPLIT ? (int)blockIdx.x % p.n_splits : 0;
  const int row0 = tile * BLOCK_M;
  if (row0 >= n_rows) return;
  const int last_row = min(n_rows, row0 + BLOCK_M) - 1;
  const int t_first = row0 / g, t_last = last_row / g;
  int k_hi = pos0 + t_last;  // last visible key of the tile (inclusive)
  int k_lo = 0;
  if (p.window > 0) k_lo = max(0, pos0 + t_first - p.window + 1);
  if (SPLIT) {
    k_lo = max(k_lo, split * p.split_keys);
    k_hi = min(k_hi, (split + 1) * p.split_keys - 1);
    if (k_lo > k_hi) return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the block-table entries this CTA will use, copied to shared memory once
  int* table = reinterpret_cast<int*>(v_tiles + STAGES * BLOCK_N * ROW);
  const int first_entry = k_lo / p.page_size;
  const bool block_in_page = p.page_size % BLOCK_N == 0;
  {
    const int* src = p.block_table + (size_t)seq * p.max_blocks + first_entry;
    const int n_entries = k_hi / p.page_size - first_entry + 1;
    for (int e = threadIdx.x; e < n_entries; e += 128) table[e] = src[e];
    __syncthreads();
  }

  // ---- stage the query tile: row r = (token r / g, head kvh * g + r % g) ----
  for (int idx = threadIdx.x; idx < BLOCK_M * CHUNKS; idx += 128) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const int row = row0 + r;
    const bool ok = row < n_rows;
    const bf16* src = p.q;
    if (ok) src = p.q + ((size_t)(row_begin + row / g) * p.nh + kvh * g + row % g) * HD + c * 8;
    cp_async16((uint32_t)__cvta_generic_to_shared(q_tile + r * ROW + c * 8), src, ok);
  }
  const int nb_lo = k_lo / BLOCK_N, nb_hi = k_hi / BLOCK_N;
#pragma unroll
  for (int st = 0; st < STAGES; ++st) {  // one commit group per stage, empty past the last block
    if (nb_lo + st <= nb_hi) {
      load_kv_tiles(k_tiles + st * BLOCK_N * ROW, v_tiles + st * BLOCK_N * ROW, p.k_cache, p.v_cache, table, first_entry, p.page_size,
                    block_in_page, p.nkv, kvh, (nb_lo + st) * BLOCK_N, k_lo, k_hi + 1);
    }
    cp_async_commit();
  }

  // this thread's two rows of the warp's 16-row slab
  const int r_lo = row0 + warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const int pos_lo = pos0 + min(r_lo, n_rows - 1) / g, pos_hi = pos0 + min(r_hi, n_rows - 1) / g;
  const int warp_pos_min = pos0 + min(row0 + warp * 16, n_rows - 1) / g;
  const int warp_pos_max = pos0 + min(row0 + warp * 16 + 15, n_rows - 1) / g;

  uint32_t qf[KSTEPS][4];
  float o[DTILES][4];
#pragma unroll
  for (int d = 0; d < DTILES; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int nb = nb_lo; nb <= nb_hi; ++nb) {
    const int buf = (nb - nb_lo) % STAGES;
    cp_async_wait<STAGES - 1>();  // the group of this block (and the query tile) has landed
    __syncthreads();
    if (nb == nb_lo) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const bf16* src = q_tile + (warp * 16 + (lane & 15)) * ROW + ks * 16 + (lane >> 4) * 8;
        ldmatrix_x4(qf[ks], (uint32_t)__cvta_generic_to_shared(src));
      }
    }
    const bf16* kt = k_tiles + buf * BLOCK_N * ROW;
    const bf16* vt = v_tiles + buf * BLOCK_N * ROW;

    // ---- S = Q K^T : 16 rows x 64 keys per warp ---------------------------------
    float s[BLOCK_N / 8][4];
#pragma unroll
    for (int n = 0; n < BLOCK_N / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int n2 = 0; n2 < BLOCK_N / 16; ++n2) {
        // keys n2*16 .. +15, dims ks*16 .. +15: four 8x8 matrices
        uint32_t kf[4];
        const bf16* src = kt + (n2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * ROW + ks * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(kf, (uint32_t)__cvta_generic_to_shared(src));
        mma_16816(s[2 * n2], qf[ks], kf[0], kf[1]);
        mma_16816(s[2 * n2 + 1], qf[ks], kf[2], kf[3]);
      }
    }
    // ---- visibility -------------------------------------------------------------
    const int j0 = nb * BLOCK_N;
    const bool all_visible = (j0 + BLOCK_N - 1 <= min(warp_pos_min, k_hi)) && (j0 >= k_lo) &&
                             (p.window <= 0 || j0 > warp_pos_max - p.window);
    if (!all_visible) {
#pragma unroll
      for (int n = 0; n < BLOCK_N / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + n * 8 + (lane & 3) * 2 + (e & 1);
          const int pos = (e < 2) ? pos_lo : pos_hi;
          bool vis = j <= pos && j >= k_lo && j <= k_hi;
          if (p.window > 0) vis = vis && j > pos - p.window;
          if (!vis) s[n][e] = -INFINITY;
        }
      }
    }
    // ---- streaming softmax ----------------------------------------------------------
    float bm_lo = -INFINITY, bm_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < BLOCK_N / 8; ++n) {
      bm_lo = fmaxf(bm_lo, fmaxf(s[n][0], s[n][1]));
      bm_hi = fmaxf(bm_hi, fmaxf(s[n][2], s[n][3]));
    }
    bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 1));
    bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 2));
    bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 1));
    bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 2));
    const float mn_lo = fmaxf(m_lo, bm_lo), mn_hi = fmaxf(m_hi, bm_hi);
    const float base_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo * p.scale_log2;
    const float base_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi * p.scale_log2;
    const float corr_lo = (m_lo == -INFINITY) ? 0.f : fast_exp2(m_lo * p.scale_log2 - base_lo);
    const float corr_hi = (m_hi == -INFINITY) ? 0.f : fast_exp2(m_hi * p.scale_log2 - base_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pf[BLOCK_N / 16][4];
#pragma unroll
    for (int n = 0; n < BLOCK_N / 8; ++n) {
      const float p0 = fast_exp2(s[n][0] * p.scale_log2 - base_lo), p1 = fast_exp2(s[n][1] * p.scale_log2 - base_lo);
      const float p2 = fast_exp2(s[n][2] * p.scale_log2 - base_hi), p3 = fast_exp2(s[n][3] * p.scale_log2 - base_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      // the accumulator layout of two adjacent 8-key tiles is the A layout of one 16-key step
      pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l_lo = l_lo * corr_lo + sum_lo;
    l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
    for (int d = 0; d < DTILES; ++d) {
      o[d][0] *= corr_lo;
      o[d][1] *= corr_lo;
      o[d][2] *= corr_hi;
      o[d][3] *= corr_hi;
    }
    // ---- O += P V ---------------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
#pragma unroll
      for (int d2 = 0; d2 < HD / 16; ++d2) {
        // keys kk*16 .. +15 (k), dims d2*16 .. +15 (n): transposed 8x8 loads
        uint32_t vf[4];
        const bf16* src = vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROW + d2 * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vf, (uint32_t)__cvta_generic_to_shared(src));
        mma_16816(o[2 * d2], pf[kk], vf[0], vf[1]);
        mma_16816(o[2 * d2 + 1], pf[kk], vf[2], vf[3]);
      }
    }
    __syncthreads();  // everyone is done with this buffer before it is refilled
    if (nb + STAGES <= nb_hi) {
      load_kv_tiles(k_tiles + buf * BLOCK_N * ROW, v_tiles + buf * BLOCK_N * ROW, p.k_cache, p.v_cache, table, first_entry, p.page_size,
                    block_in_page, p.nkv, kvh, (nb + STAGES) * BLOCK_N, k_lo, k_hi + 1);
    }
    cp_async_commit();
  }
  // ---- finish ---------------------------------------------------------------------------
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? r_hi : r_lo;
    if (row >= n_rows) continue;
    const float l = half ? l_hi : l_lo, m = half ? m_hi : m_lo;
    const size_t out_row = (size_t)(row_begin + row / g) * p.nh + kvh * g + row % g;
    if (SPLIT) {
      float* po = p.partial_o + ((size_t)split * p.n_rows_total + out_row) * HD;
#pragma unroll
      for (int d = 0; d < DTILES; ++d)
        *reinterpret_cast<float2*>(po + d * 8 + (lane & 3) * 2) = make_float2(o[d][half * 2], o[d][half * 2 + 1]);
      if ((lane & 3) == 0) {
        float* ml = p.partial_ml + ((size_t)split * p.n_rows_total + out_row) * 2;
        ml[0] = (m == -INFINITY) ? -INFINITY : m * p.scale_log2;
        ml[1] = l;
      }
    } else {
      const float inv = 1.0f / l;
      bf16* po = p.out + out_row * HD;
#pragma unroll
      for (int d = 0; d < DTILES; ++d)
        *reinterpret_cast<uint32_t*>(po + d * 8 + (lane & 3) * 2) = pack_bf16(o[d][half * 2] * inv, o[d][half * 2 + 1] * inv);
    }
  }
}

// ---------------------------------------------------------------------------
// Decode tokens, keys spread over the warps.  One CTA owns one (request, KV
// head, split of split_keys keys); the split's 64-key blocks are dealt to its
// warps in turn (block b of the split to warp b % WARPS), all against the same
// 16 query rows (the g <= 16 heads of the group, padded), so that WARPS blocks
// are fetched and processed side by side.  A warp that has more than one block
// keeps one key tile and one value tile: the next block's keys are asked for as
// soon as the scores of this one are taken, its values as soon as this block's
// have been multiplied in, so the copies run behind the softmax and the
// products and the warps of an SM fall out of step with one another instead of
// all loading, then all computing.  The warps' (output, maximum, sum) triples
// are merged through shared memory in warp order, and the split's triple goes
// to the partial buffers for attention_combine_kernel (or, with a single
// split, straight to the output).
// ---------------------------------------------------------------------------
// With TMA (pages that hold whole 64-key blocks, head size 64 or 128) a block
// arrives by bulk tensor copies - keys and values, 128-byte swizzled, each on
// its own mbarrier of the warp - issued by one lane; else by 16-byte cp.async
// copies into padded tiles, one block after the other.
constexpr int TILE_BYTES_TMA = BLOCK_N * HD * 2;  // one dense tile

// LONG: splits of more than one block per warp; without it a warp's keys and values come on one
// barrier and nothing is refilled.
template <int WARPS, bool TMA, bool LONG>
__global__ void __launch_bounds__(WARPS * 32) attention_decode_kernel(const AttnParams p, const __grid_constant__ CUtensorMap map_k,
                                                                      const __grid_constant__ CUtensorMap map_v) {
  constexpr int THREADS = WARPS * 32;
  constexpr int TILE_ELEMS = TMA ? BLOCK_N * HD : BLOCK_N * ROW;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* aligned = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  bf16* k_tiles = reinterpret_cast<bf16*>(aligned);       // [WARPS] tiles of 64 keys
  bf16* v_tiles = k_tiles + WARPS * TILE_ELEMS;           // [WARPS] tiles of 64 keys
  bf16* q_tile = v_tiles + WARPS * TILE_ELEMS;            // [16][ROW]
  // the merge buffers reuse the key tiles once every warp is done with them
  float* merge_o = reinterpret_cast<float*>(k_tiles);     // [WARPS][16][MERGE_ROW]
  float* merge_ml = merge_o + WARPS * 16 * MERGE_ROW;     // [WARPS][16][2]
  __shared__ uint64_t k_bar[WARPS], v_bar[WARPS];
  __shared__ int abort_flag;
  if (TMA && (threadIdx.x & 31) == 0) {
    if (threadIdx.x == 0) abort_flag = 0;
    mbar_init(&k_bar[threadIdx.x >> 5], 1);
    mbar_init(&v_bar[threadIdx.x >> 5], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Lengths and block tables came with the step's metadata, before any kernel of the step ran,
  // so the split's key range is known ahead of the wait on the kernel before this one.
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int g = p.nh / p.nkv;
  const int pos = p.kv_len[seq] - 1;  // the one query position of this request
  int k_lo = 0;
  if (p.window > 0) k_lo = max(0, pos - p.window + 1);
  k_lo = max(k_lo, split * p.split_keys);
  const int k_hi = min(pos, (split + 1) * p.split_keys - 1);
  if (k_lo > k_hi) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // this warp's blocks of keys: first, first + WARPS, ... up to last (block numbers within the request)
  const int b_lo = k_lo / BLOCK_N, b_hi = k_hi / BLOCK_N;
  const int mine = split * (p.split_keys / BLOCK_N) + warp;
  const int first = mine >= b_lo ? mine : mine + (b_lo - mine + WARPS - 1) / WARPS * WARPS;
  const bool has_keys = first <= b_hi;
  const int last = !has_keys ? first - WARPS : LONG ? first + (b_hi - first) / WARPS * WARPS : first;
  bf16* kt = k_tiles + warp * TILE_ELEMS;
  bf16* vt = v_tiles + warp * TILE_ELEMS;
  // a block lies inside one page, its 64 rows are consecutive cache slots
  auto block_row = [&](int block) {
    const int j = block * BLOCK_N, e = j / p.page_size;
    return p.block_table[(size_t)seq * p.max_blocks + e] * p.page_size + (j - e * p.page_size);
  };
  auto fetch_keys = [&](int row) {  // one lane
    mbar_expect_tx(&k_bar[warp], TILE_BYTES_TMA);
#pragma unroll
    for (int sub = 0; sub < HD / 64; ++sub)
      tma_load_2d(reinterpret_cast<uint8_t*>(kt) + sub * BLOCK_N * 128, &map_k, &k_bar[warp], kvh * HD + sub * 64, row);
  };
  auto fetch_values = [&](int row) {  // one lane
    mbar_expect_tx(&v_bar[warp], TILE_BYTES_TMA);
#pragma unroll
    for (int sub = 0; sub < HD / 64; ++sub)
      tma_load_2d(reinterpret_cast<uint8_t*>(vt) + sub * BLOCK_N * 128, &map_v, &v_bar[warp], kvh * HD + sub * 64, row);
  };
  auto fetch_padded = [&](int block) {  // the whole warp
    const int* table = p.block_table + (size_t)seq * p.max_blocks;
    for (int idx = lane; idx < BLOCK_N * CHUNKS; idx += 32) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      const int j = block * BLOCK_N + r;
      const bool ok = j >= k_lo && j <= k_hi;
      size_t offset = 0;
      if (ok) {
        const int e = j / p.page_size;
        const int slot = table[e] * p.page_size + (j - e * p.page_size);
        offset = ((size_t)slot * p.nkv + kvh) * HD + c * 8;
      }
      cp_async16((uint32_t)__cvta_generic_to_shared(kt + r * ROW + c * 8), p.k_cache + offset, ok);
      cp_async16((uint32_t)__cvta_generic_to_shared(vt + r * ROW + c * 8), p.v_cache + offset, ok);
    }
  };
  auto fetch_first = [&](int row) {  // one lane
    if (LONG) {
      fetch_keys(row);
      fetch_values(row);
    } else {
      mbar_expect_tx(&k_bar[warp], 2 * TILE_BYTES_TMA);
#pragma unroll
      for (int sub = 0; sub < HD / 64; ++sub) {
        tma_load_2d(reinterpret_cast<uint8_t*>(kt) + sub * BLOCK_N * 128, &map_k, &k_bar[warp], kvh * HD + sub * 64, row);
        tma_load_2d(reinterpret_cast<uint8_t*>(vt) + sub * BLOCK_N * 128, &map_v, &k_bar[warp], kvh * HD + sub * 64, row);
      }
    }
  };
  int row_first = 0, row_next = 0;  // lane 0: cache rows of the first block and of the one after it
  if (TMA && has_keys && lane == 0) {
    row_first = block_row(first);
    if (LONG && first < last) row_next = block_row(first + WARPS);
  }
  const int token = p.q_start[seq];
  // A block that ends before the query's own position holds only keys of earlier steps: its copy
  // need not wait for the kernel that writes this step's key and may start at once.
  const bool early = TMA && has_keys && first * BLOCK_N + BLOCK_N - 1 < pos;
  if (early && lane == 0) fetch_first(row_first);
  pdl_wait();

  // the query rows: head kvh * g + r for r < g, zero rows above
  for (int idx = threadIdx.x; idx < 16 * CHUNKS; idx += THREADS) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool ok = r < g;
    const bf16* src = ok ? p.q + ((size_t)token * p.nh + kvh * g + r) * HD + c * 8 : p.q;
    cp_async16((uint32_t)__cvta_generic_to_shared(q_tile + r * ROW + c * 8), src, ok);
  }
  if (TMA) {
    if (lane == 0 && has_keys && !early) fetch_first(row_first);
  } else if (has_keys) {
    fetch_padded(first);
  }
  pdl_launch();
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();  // the query tile was copied by all threads (and the barriers are initialised)

  RowState st;
  st.m_lo = st.m_hi = -INFINITY;
  st.l_lo = st.l_hi = 0.f;
#pragma unroll
  for (int d = 0; d < DTILES; ++d) st.o[d][0] = st.o[d][1] = st.o[d][2] = st.o[d][3] = 0.f;
  if (has_keys) {
    uint32_t qf[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const bf16* src = q_tile + (lane & 15) * ROW + ks * 16 + (lane >> 4) * 8;
      ldmatrix_x4(qf[ks], (uint32_t)__cvta_generic_to_shared(src));
    }
    const uint32_t kt_s = (uint32_t)__cvta_generic_to_shared(kt), vt_s = (uint32_t)__cvta_generic_to_shared(vt);
    uint32_t parity = 0;
    for (int block = first; block <= last; block += WARPS, parity ^= 1) {
      const bool more = LONG && block < last;
      if (TMA) {
        if (!mbar_wait(&k_bar[warp], parity, &abort_flag)) break;
        const int row_more = row_next;
        int row_after = 0;  // looked up two blocks ahead, so that the copy does not wait for the table
        if (LONG && lane == 0 && block + 2 * WARPS <= last) row_after = block_row(block + 2 * WARPS);
        bool values_here = true;
        attend_block<true>(
            st, qf, kt_s, vt_s, block * BLOCK_N, lane, pos, k_lo, k_hi, p.window, p.scale_log2,
            [&] {
              if (more) {
                __syncwarp();  // every lane has taken its scores from the key tile
                if (lane == 0) fetch_keys(row_more);
              }
            },
            [&] {
              if (LONG) values_here = mbar_wait(&v_bar[warp], parity, &abort_flag);
            });
        if (!values_here) break;
        if (more) {
          __syncwarp();  // every lane has multiplied the value tile in
          if (lane == 0) fetch_values(row_more);
        }
        row_next = row_after;
      } else {
        attend_block<false>(st, qf, kt_s, vt_s, block * BLOCK_N, lane, pos, k_lo, k_hi, p.window, p.scale_log2);
        if (more) {
          __syncwarp();
          fetch_padded(block + WARPS);
          cp_async_commit();
          cp_async_wait<0>();
          __syncwarp();
        }
      }
    }
  }
  // ---- merge the warps in warp order ---------------------------------------------------
  __syncthreads();  // every warp is done with the key tiles the merge buffers overlay
  if (TMA && threadIdx.x == 0 && abort_flag && p.status) atomicExch(p.status, 2);
  st.l_lo += __shfl_xor_sync(0xffffffffu, st.l_lo, 1);
  st.l_lo += __shfl_xor_sync(0xffffffffu, st.l_lo, 2);
  st.l_hi += __shfl_xor_sync(0xffffffffu, st.l_hi, 1);
  st.l_hi += __shfl_xor_sync(0xffffffffu, st.l_hi, 2);
  {
    const int r = lane >> 2;
    float* mo = merge_o + (warp * 16) * MERGE_ROW;
#pragma unroll
    for (int d = 0; d < DTILES; ++d) {
      *reinterpret_cast<float2*>(mo + r * MERGE_ROW + d * 8 + (lane & 3) * 2) = make_float2(st.o[d][0], st.o[d][1]);
      *reinterpret_cast<float2*>(mo + (r + 8) * MERGE_ROW + d * 8 + (lane & 3) * 2) = make_float2(st.o[d][2], st.o[d][3]);
    }
    if ((lane & 3) == 0) {
      float* ml = merge_ml + warp * 32;
      ml[r * 2] = (st.m_lo == -INFINITY) ? -INFINITY : st.m_lo * p.scale_log2;
      ml[r * 2 + 1] = st.l_lo;
      ml[(r + 8) * 2] = (st.m_hi == -INFINITY) ? -INFINITY : st.m_hi * p.scale_log2;
      ml[(r + 8) * 2 + 1] = st.l_hi;
    }
  }
  __syncthreads();
  const bool single = gridDim.x == 1;
  for (int idx = threadIdx.x; idx < g * HD; idx += THREADS) {
    const int r = idx / HD, d = idx % HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, merge_ml[w * 32 + r * 2]);
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float mw = merge_ml[w * 32 + r * 2];
      const float scale = (mw == -INFINITY) ? 0.f : fast_exp2(mw - m);
      l += merge_ml[w * 32 + r * 2 + 1] * scale;
      acc += merge_o[(w * 16 + r) * MERGE_ROW + d] * scale;
    }
    const size_t out_row = (size_t)token * p.nh + kvh * g + r;
    if (single) {
      p.out[out_row * HD + d] = __float2bfloat16_rn(acc / l);
    } else {
      p.partial_o[((size_t)split * p.n_rows_total + out_row) * HD + d] = acc;
      if (d == 0) {
        float* ml = p.partial_ml + ((size_t)split * p.n_rows_total + out_row) * 2;
        ml[0] = m;
        ml[1] = l;
      }
    }
  }
}

static size_t decode_smem_bytes(int warps, bool tma) {
  const size_t tile = tma ? (size_t)BLOCK_N * HD * sizeof(bf16) : (size_t)BLOCK_N * ROW * sizeof(bf16);
  const size_t tiles = 2 * warps * tile;
  const size_t merge = (size_t)warps * 16 * MERGE_ROW * sizeof(float) + (size_t)warps * 32 * sizeof(float);
  return 1024 + (tiles > merge ? tiles : merge) + (size_t)16 * ROW * sizeof(bf16);
}

template <int WARPS, bool TMA, bool LONG>
static int launch_decode_as(const AttnParams& p, const CUtensorMap& map_k, const CUtensorMap& map_v, int n_splits, int nkv, int n_seqs,
                            cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_decode_kernel<WARPS, TMA, LONG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)decode_smem_bytes(WARPS, TMA)) != cudaSuccess)
      return ALOFA_ERR_LAUNCH;
    prefer_max_shared(attention_decode_kernel<WARPS, TMA, LONG>);
    configured = true;
  }
  launch_dep(attention_decode_kernel<WARPS, TMA, LONG>, dim3(n_splits, nkv, n_seqs), WARPS * 32, decode_smem_bytes(WARPS, TMA), stream, p, map_k,
             map_v);
  return cudaGetLastError() == cudaSuccess ? ALOFA_OK : ALOFA_ERR_LAUNCH;
}

template <int WARPS, bool TMA>
static int launch_decode(const AttnParams& p, const CUtensorMap& map_k, const CUtensorMap& map_v, int n_splits, int nkv, int n_seqs,
                         cudaStream_t stream) {
  if (p.split_keys > WARPS * BLOCK_N) return launch_decode_as<WARPS, TMA, true>(p, map_k, map_v, n_splits, nkv, n_seqs, stream);
  return launch_decode_as<WARPS, TMA, false>(p, map_k, map_v, n_splits, nkv, n_seqs, stream);
}

// Merge the splits of every (token, head) row in split order.  One block of HD
// threads per row; a row's splits are those its visible keys fall into.
__global__ void attention_combine_kernel(bf16* __restrict__ out, const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                         const int* __restrict__ positions, int nh, int window, int split_keys, int n_rows_total) {
  const int row = blockIdx.x;       // token * nh + head
  pdl_begin();
  const int P = positions[row / nh];
  int k_lo = 0;
  if (window > 0) k_lo = max(0, P - window + 1);
  const int s_lo = k_lo / split_keys, s_hi = P / split_keys;
  float m = -INFINITY;
  for (int s = s_lo; s <= s_hi; ++s) m = fmaxf(m, partial_ml[((size_t)s * n_rows_total + row) * 2]);
  float l = 0.f, acc = 0.f;
  const int d = threadIdx.x;
  for (int s = s_lo; s <= s_hi; ++s) {
    const float* ml = partial_ml + ((size_t)s * n_rows_total + row) * 2;
    const float w = (ml[0] == -INFINITY) ? 0.f : fast_exp2(ml[0] - m);
    l += ml[1] * w;
    acc += partial_o[((size_t)s * n_rows_total + row) * HD + d] * w;
  }
  out[(size_t)row * HD + d] = __float2bfloat16_rn(acc / l);
}

constexpr int PREFILL_STAGES = 2, SPLIT_STAGES = 4;
static size_t attention_smem_bytes(int stages, int table_entries) {
  return (size_t)(BLOCK_M + 2 * stages * BLOCK_N) * ROW * sizeof(bf16) + (size_t)table_entries * sizeof(int);
}

ALOFA_API int alofa_attention_head_dim() { return HD; }

// The decode kernel's wide form: one CTA per SM with as many warps as its shared memory holds
// key and value tiles for (16 KB a warp at head size 64, 32 KB at 128), on pages of whole key
// blocks.  Taken when a launch's splits are a multiple of WIDE_WARPS * 64 keys.
constexpr int WIDE_WARPS = HD == 64 ? 8 : HD == 128 ? 6 : 0;
ALOFA_API int alofa_attention_decode_wide_warps() { return WIDE_WARPS; }

// How many CTAs of the decode kernel with `warps` warps (4, or the wide form's) the device holds
// at a time: what a caller sizes the key splits by, so that a step's CTAs are resident together.
// 0 when that kernel does not exist here or the device cannot be asked.
ALOFA_API int alofa_attention_decode_slots(int page_size, int warps) {
  const bool tma = (HD == 64 || HD == 128) && page_size % BLOCK_N == 0;
  int device = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  cudaError_t rc;
  if (WIDE_WARPS > 0 && warps == WIDE_WARPS) {
    if (!tma) return 0;
    constexpr int W = WIDE_WARPS > 0 ? WIDE_WARPS : 4;
    const size_t smem = decode_smem_bytes(W, true);
    cudaFuncSetAttribute(attention_decode_kernel<W, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rc = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<W, true, true>, W * 32, smem);
  } else if (warps != 4) {
    return 0;
  } else if (tma) {
    const size_t smem = decode_smem_bytes(4, true);
    cudaFuncSetAttribute(attention_decode_kernel<4, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rc = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<4, true, true>, 128, smem);
  } else {
    const size_t smem = decode_smem_bytes(4, false);
    cudaFuncSetAttribute(attention_decode_kernel<4, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rc = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<4, false, true>, 128, smem);
  }
  if (rc != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return sms * per_sm;
}

// Merge the splits a launch with do_combine = 0 left behind: out [T, nh, HD] bf16.
ALOFA_API int alofa_attention_combine(void* out, const float* partial_o, const float* partial_ml, const int* positions, int n_tokens, int nh,
                                      int window, int split_keys, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (!partial_o || !partial_ml || !positions || split_keys <= 0) return ALOFA_ERR_ARGUMENT;
  launch_dep(attention_combine_kernel, n_tokens * nh, HD, 0, stream, (bf16*)out, partial_o, partial_ml, positions, nh, window, split_keys, n_tokens * nh);
  return launch_status();
}

// cache_slots: rows of k_cache / v_cache (token slots), for the tensor maps.
// do_combine = 0 (decode tokens in splits only): the splits are left in partial_o / partial_ml
// for the consumer to merge (alofa_attention_combine, or a product that merges them as it reads).
// max_kv_len: the most keys any request of this step has (sizes the shared copy of
// block-table entries).  tiles: query tiles of the longest request = ceil(max_q_len * g / 64).  n_splits > 0
// selects split mode: the keys of a request (decode tokens) or of every query tile
// (prompt portions) are spread over n_splits CTAs of split_keys keys each and merged by
// attention_combine_kernel; partial_o / partial_ml must then hold n_splits planes.
ALOFA_API int alofa_attention_bf16(void* out, const void* q, const void* k_cache, const void* v_cache, const int* q_start, const int* kv_len, const int* positions,
                                   const int* block_table, int max_blocks, int page_size, int n_seqs, int n_tokens, int tiles, int nh, int nkv,
                                   int window, float scale, int n_splits, int split_keys, float* partial_o, float* partial_ml,
                                   int max_kv_len, long long cache_slots, int* status, int do_combine, cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return ALOFA_OK;
  if (nkv <= 0 || nh % nkv != 0 || page_size <= 0 || tiles <= 0) return ALOFA_ERR_ARGUMENT;
  if (n_splits > 0 && (split_keys <= 0 || split_keys % BLOCK_N != 0 || !partial_o || !partial_ml || !positions)) return ALOFA_ERR_ARGUMENT;
  const bool decode_only = n_seqs == n_tokens;
  if (n_splits > 0 && decode_only && nh / nkv > BLOCK_M) return ALOFA_ERR_ARGUMENT;
  AttnParams p;
  p.out = (bf16*)out;
  p.q = (const bf16*)q;
  p.status = status;
  p.k_cache = (const bf16*)k_cache;
  p.v_cache = (const bf16*)v_cache;
  p.q_start = q_start;
  p.kv_len = kv_len;
  p.block_table = block_table;
  p.partial_o = partial_o;
  p.partial_ml = partial_ml;
  p.max_blocks = max_blocks;
  p.page_size = page_size;
  p.nh = nh;
  p.nkv = nkv;
  p.window = window;
  p.split_keys = split_keys;
  p.n_splits = n_splits > 0 ? n_splits : 1;
  p.n_rows_total = n_tokens * nh;
  p.scale_log2 = scale * 1.4426950408889634f;
  // entries of a block table one CTA may touch: a split's keys, or up to the longest request
  const int reach = n_splits > 0 ? split_keys : max_kv_len;
  p.table_entries = reach / page_size + 2;
  const size_t smem = attention_smem_bytes((n_splits > 0 && decode_only) ? SPLIT_STAGES : PREFILL_STAGES, p.table_entries);
  if (smem > 200 * 1024) return ALOFA_ERR_ARGUMENT;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_bf16_kernel<false, PREFILL_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(attention_bf16_kernel<true, SPLIT_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(attention_bf16_kernel<true, PREFILL_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024) != cudaSuccess)
      return ALOFA_ERR_LAUNCH;
    prefer_max_shared(attention_bf16_kernel<false, PREFILL_STAGES>);
    prefer_max_shared(attention_bf16_kernel<true, SPLIT_STAGES>);
    prefer_max_shared(attention_bf16_kernel<true, PREFILL_STAGES>);
    prefer_max_shared(attention_combine_kernel);
    configured = true;
  }
  if (n_splits > 0 && decode_only && nh / nkv <= 16 &&
      (split_keys % (4 * BLOCK_N) == 0 || split_keys == 2 * BLOCK_N || (WIDE_WARPS > 0 && split_keys % ((WIDE_WARPS > 0 ? WIDE_WARPS : 4) * BLOCK_N) == 0))) {
    // decode tokens of small head groups: the key blocks of a split side by side on the warps
    // pages that hold whole key blocks and rows of 128 or 256 bytes: bulk tensor copies
    CUtensorMap map_k, map_v;
    bool tma = (HD == 64 || HD == 128) && page_size % BLOCK_N == 0 && cache_slots > 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0;
    if (tma)
      tma = make_tensor_map_bf16(&map_k, k_cache, (uint64_t)cache_slots, (uint64_t)nkv * HD, BLOCK_N, 64) &&
            make_tensor_map_bf16(&map_v, v_cache, (uint64_t)cache_slots, (uint64_t)nkv * HD, BLOCK_N, 64);
    if (!tma) {
      memset(&map_k, 0, sizeof(map_k));
      memset(&map_v, 0, sizeof(map_v));
    }
    int rc;
    if (tma && WIDE_WARPS > 0 && split_keys % ((WIDE_WARPS > 0 ? WIDE_WARPS : 4) * BLOCK_N) == 0)
      // splits of a multiple of the wide form's keys: one CTA per SM (see alofa_attention_decode_slots)
      rc = launch_decode<(WIDE_WARPS > 0 ? WIDE_WARPS : 4), true>(p, map_k, map_v, n_splits, nkv, n_seqs, stream);
    else if (split_keys % (4 * BLOCK_N) == 0)
      rc = tma ? launch_decode<4, true>(p, map_k, map_v, n_splits, nkv, n_seqs, stream) : launch_decode<4, false>(p, map_k, map_v, n_splits, nkv, n_seqs, stream);
    else
      rc = tma ? launch_decode<2, true>(p, map_k, map_v, n_splits, nkv, n_seqs, stream) : launch_decode<2, false>(p, map_k, map_v, n_splits, nkv, n_seqs, stream);
    if (rc != ALOFA_OK) return rc;
    if (n_splits > 1 && do_combine)
      launch_dep(attention_combine_kernel, n_tokens * nh, HD, 0, stream, (bf16*)out, partial_o, partial_ml, positions, nh, window, split_keys, p.n_rows_total);
  } else if (n_splits > 0 && !decode_only) {
    // prompt portions: every query tile's keys split over n_splits CTAs, so that the tiles
    // at the end of a long prompt do not set the pace
    launch_dep(attention_bf16_kernel<true, PREFILL_STAGES>, dim3(tiles * n_splits, nkv, n_seqs), 128, smem, stream, p);
    if (cudaGetLastError() != cudaSuccess) return ALOFA_ERR_LAUNCH;
    launch_dep(attention_combine_kernel, n_tokens * nh, HD, 0, stream, (bf16*)out, partial_o, partial_ml, positions, nh, window, split_keys, p.n_rows_total);
  } else if (n_splits > 0) {
    launch_dep(attention_bf16_kernel<true, SPLIT_STAGES>, dim3(n_splits, nkv, n_seqs), 128, smem, stream, p);
    if (cudaGetLastError() != cudaSuccess) return ALOFA_ERR_LAUNCH;
    launch_dep(attention_combine_kernel, n_tokens * nh, HD, 0, stream, (bf16*)out, partial_o, partial_ml, positions, nh, window, split_keys, p.n_rows_total);
  } else {
    // prompt portions: the tcgen05 kernel where the head size and the pages are its own
    // (ALOFA_ATTENTION_TC=0 keeps the mma.sync kernel), else mma.sync
    static int use_tc = -1;
    if (use_tc < 0) {
      const char* env = getenv("ALOFA_ATTENTION_TC");
      use_tc = (env && env[0] == '0') ? 0 : 1;
    }
    int rc = ALOFA_OK;
    if (use_tc && !decode_only && launch_prefill_tc(p, k_cache, v_cache, cache_slots, tiles, nkv, n_seqs, max_kv_len, stream, &rc)) return rc;
    launch_dep(attention_bf16_kernel<false, PREFILL_STAGES>, dim3(tiles, nkv, n_seqs), 128, smem, stream, p);
  }
  return launch_status();
}
