// Causal grouped-query attention of prompt portions on the fifth-generation
// tensor cores (tcgen05), for head sizes 64 and 128 and pages that hold whole
// 64-key blocks.  Included by attention_bf16.cu, which owns AttnParams.
//
// One CTA owns 128 query rows of one (request, KV head): a row is a (token,
// head of the group) pair, as in the mma.sync kernel.  Keys go by in blocks of
// 128.  Ten warps:
//   warp 0   one lane issues the bulk tensor copies of the key and value
//            blocks (two 64-key boxes per 64-wide panel of the head, found
//            through the block table) into a ring of stages;
//   warp 1   one lane issues the MMAs: S = Q K^T (M 128, N 128, accumulator in
//            tensor memory, two S buffers in turn) and O += P V (N = head
//            size; V is used as it lies in the cache, as an MN-major operand);
//   warps 2-9  the softmax, two threads per query row (64 key columns each):
//            the row of S comes out of tensor memory, is masked (causal,
//            window), scaled and exponentiated in fp32, and written back
//            over it as bfloat16 pairs: P, the second MMA's operand from
//            tensor memory.
// The running maximum is kept lazily: P is scaled by 2^-m for a maximum m that
// is only raised (and O and the running sum rescaled, in tensor memory) when a
// row's scores outgrow it by more than 2^8, so most blocks leave O alone; the
// result is O / sum either way.  While the softmax of block j runs, the tensor
// core computes S of block j + 1 and finishes O of block j - 1.
// Every wait is bounded; a wait that runs out sets the status word to 2.
// Formulas: src/alofa/kernels/cpu/scalar.mojo:392-470.
#pragma once
#include "attention_core.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

constexpr int TC_BM = 128;                       // query rows per CTA
constexpr int TC_BN = 128;                       // keys per block
constexpr int TC_PANELS = HD / 64;               // 64-wide panels of a head
constexpr int TC_PANEL_BYTES = 128 * 128;        // 128 rows of 128 bytes
constexpr int TC_KV_BYTES = TC_PANELS * TC_PANEL_BYTES;  // one key (or value) block
constexpr int TC_Q_BYTES = TC_PANELS * TC_PANEL_BYTES;
constexpr int TC_STAGES = HD <= 64 ? 4 : 2;
constexpr int TC_THREADS = 320;  // a warp of copies, a warp of MMAs, eight of softmax
constexpr float TC_RESCALE_ABOVE = 8.0f;         // log2 units a row's maximum may outgrow the one in use

__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(addr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void umma_bf16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Descriptor of an MN-major operand with 128-byte swizzle: rows (depth index)
// of 128 bytes, 8-row groups 1024 bytes apart, 64-wide panels `panel_bytes` apart.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t panel_bytes) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(panel_bytes >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

static size_t prefill_tc_smem_bytes(int table_entries) {
  return 1024 + (size_t)TC_Q_BYTES + (size_t)TC_STAGES * 2 * TC_KV_BYTES + (size_t)table_entries * sizeof(int);
}

__global__ void __launch_bounds__(TC_THREADS, 1) attention_prefill_tc_kernel(const AttnParams p, const __grid_constant__ CUtensorMap map_k,
                                                                             const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* q_tile = smem;                                   // [panel][128 rows][128 B], K-major
  uint8_t* kv_ring = q_tile + TC_Q_BYTES;                   // [stage][K | V][panel][128 keys][128 B]
  int* table = reinterpret_cast<int*>(kv_ring + TC_STAGES * 2 * TC_KV_BYTES);  // the request's block-table entries from the first block on
  __shared__ uint64_t kv_full[TC_STAGES], kv_free[TC_STAGES], s_full[2], q_ready, p_full, pv_done, pair_bar[4];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;
  __shared__ float row_max[2][2][TC_BM];  // [block parity][column half][row]: what the two threads of a row tell each other

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.z, kvh = blockIdx.y;
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;  // the long tiles at the end of a prompt first
  const int g = p.nh / p.nkv;
  const int row_begin = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - row_begin;
  const int kv_len = p.kv_len[seq];
  const int pos0 = kv_len - q_len;
  const int n_rows = q_len * g;
  const int row0 = tile * TC_BM;
  if (row0 >= n_rows) return;
  const int last_row = min(n_rows, row0 + TC_BM) - 1;
  const int t_first = row0 / g, t_last = last_row / g;
  const int k_hi = pos0 + t_last;  // last visible key of the tile
  const int k_lo = p.window > 0 ? max(0, pos0 + t_first - p.window + 1) : 0;
  const int jb0 = k_lo / TC_BN, nblk = k_hi / TC_BN - jb0 + 1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_free[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
    }
    mbar_init(&q_ready, 256);
    mbar_init(&p_full, 256);
    mbar_init(&pv_done, 1);
    for (int b = 0; b < 4; ++b) mbar_init(&pair_bar[b], 64);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) tmem_alloc(&tmem_base_smem, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_smem;
  const uint32_t tmem_o = tmem + 256;  // S buffers at columns 0 and 128, O behind them
  pdl_begin();

  if (warp == 0) {
    // ---- the key and value blocks ------------------------------------------------------
    const int first_entry = (jb0 * TC_BN) / p.page_size;
    const int n_entries = k_hi / p.page_size - first_entry + 1;
    for (int e = lane; e < n_entries; e += 32) table[e] = p.block_table[(size_t)seq * p.max_blocks + first_entry + e];
    __syncwarp();
    if (lane == 0) {
      for (int i = 0; i < nblk; ++i) {
        const int s = i % TC_STAGES;
        if (i >= TC_STAGES && !mbar_wait(&kv_free[s], ((i / TC_STAGES) - 1) & 1, &abort_flag)) break;
        uint8_t* k_stage = kv_ring + (size_t)s * 2 * TC_KV_BYTES;
        uint8_t* v_stage = k_stage + TC_KV_BYTES;
        mbar_expect_tx(&kv_full[s], 2 * TC_KV_BYTES);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          int j = (jb0 + i) * TC_BN + half * 64;
          if (j > k_hi) j -= 64;  // nothing there: the first half again, every key of it masked
          const int e = j / p.page_size;
          const int slot0 = table[e - first_entry] * p.page_size + (j - e * p.page_size);
#pragma unroll
          for (int pn = 0; pn < TC_PANELS; ++pn) {
            tma_load_2d(k_stage + pn * TC_PANEL_BYTES + half * 8192, &map_k, &kv_full[s], kvh * HD + pn * 64, slot0);
            tma_load_2d(v_stage + pn * TC_PANEL_BYTES + half * 8192, &map_v, &kv_full[s], kvh * HD + pn * 64, slot0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- the MMAs ------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      const uint32_t q_addr = smem_u32(q_tile);
      auto issue_qk = [&](int i) -> bool {  // S[i & 1] = Q K_i^T
        const int s = i % TC_STAGES;
        if (!mbar_wait(&kv_full[s], (i / TC_STAGES) & 1, &abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(kv_ring + (size_t)s * 2 * TC_KV_BYTES);
#pragma unroll
        for (int k = 0; k < HD / UMMA_K; ++k) {
          const uint32_t off = (k >> 2) * TC_PANEL_BYTES + (k & 3) * 32;
          umma_bf16(tmem + (i & 1) * TC_BN, smem_desc_sw128(q_addr + off), smem_desc_sw128(k_addr + off), IDESC_QK, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[i & 1]);
        return true;
      };
      bool ok = mbar_wait(&q_ready, 0, &abort_flag);
      if (ok) {
        tc_fence_after();
        ok = issue_qk(0);
      }
      for (int i = 0; i < nblk && ok; ++i) {
        if (i + 1 < nblk) ok = issue_qk(i + 1);
        if (!ok || !mbar_wait(&p_full, i & 1, &abort_flag)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(kv_ring + (size_t)(i % TC_STAGES) * 2 * TC_KV_BYTES + TC_KV_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BN / UMMA_K; ++k) {  // O += P V_i, sixteen keys (eight packed columns of P) at a time
          const uint64_t desc_v = smem_desc_mn_sw128(v_addr + k * 2048, TC_PANEL_BYTES);
          umma_bf16_tmem_a(tmem_o, tmem + (i & 1) * TC_BN + k * 8, desc_v, IDESC_PV, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&kv_free[i % TC_STAGES]);  // both products of block i have read its stage
        umma_commit(&pv_done);
      }
    }
  } else {
    // ---- the softmax, two threads per query row -----------------------------------------
    // Warps 2-5 take key columns 0-63 of a block, warps 6-9 columns 64-127; a warp reads the
    // tensor-memory lanes of its quadrant (warp index modulo 4).  The two threads of a row
    // exchange their maxima through shared memory and keep separate partial sums.
    const int q4 = warp & 3, half = (warp - 2) >> 2;
    const int r = q4 * 32 + lane;           // row of the tile = lane of tensor memory
    const int R = row0 + r;
    const bool row_ok = R < n_rows;
    const int my_pos = pos0 + (row_ok ? R / g : 0);
    const int my_lo = p.window > 0 ? max(0, my_pos - p.window + 1) : 0;
    uint32_t pair_phase = 0;
    auto pair_sync = [&]() -> bool {  // the two warps of a quadrant meet (bounded, like every wait here)
      mbar_arrive(&pair_bar[q4]);
      const bool met = mbar_wait(&pair_bar[q4], pair_phase, &abort_flag);
      pair_phase ^= 1u;
      return met;
    };
    {
      // the query rows into their tile (128-byte swizzle: chunk c of row r at c ^ (r & 7)), half a row per thread
      const bf16* src = row_ok ? p.q + ((size_t)(row_begin + R / g) * p.nh + kvh * g + R % g) * HD : p.q;
#pragma unroll
      for (int cc = 0; cc < HD / 16; ++cc) {
        const int c = half * (HD / 16) + cc;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row_ok) v = *reinterpret_cast<const uint4*>(src + c * 8);
        *reinterpret_cast<uint4*>(q_tile + (c >> 3) * TC_PANEL_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(&q_ready);
    }
    constexpr int COLS = TC_BN / 2;  // key columns per thread
    constexpr int OCOLS = HD / 2;    // output columns per thread
    const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
    float m_used = -INFINITY;  // the maximum (log2 units) that P, O and the sums are scaled by
    float l = 0.f;             // this thread's share of the row's sum
    bool ok = true;
    for (int i = 0; i < nblk && ok; ++i) {
      ok = mbar_wait(&s_full[i & 1], (i >> 1) & 1, &abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float s[COLS];
#pragma unroll
      for (int c0 = 0; c0 < COLS; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(tmem + lane_addr + (i & 1) * TC_BN + half * COLS + c0, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) s[c0 + j] = __uint_as_float(v[j]);
      }
      tmem_ld_wait();
      const int j0 = (jb0 + i) * TC_BN + half * COLS;
      const bool all_visible = row_ok && j0 + COLS - 1 <= my_pos && j0 >= my_lo;
      if (!all_visible) {
#pragma unroll
        for (int j = 0; j < COLS; ++j) {
          const int kj = j0 + j;
          if (!row_ok || kj > my_pos || kj < my_lo) s[j] = -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains, not one of 64
#pragma unroll
      for (int j = 0; j < COLS; j += 4) {
        mx4[0] = fmaxf(mx4[0], s[j]);
        mx4[1] = fmaxf(mx4[1], s[j + 1]);
        mx4[2] = fmaxf(mx4[2], s[j + 2]);
        mx4[3] = fmaxf(mx4[3], s[j + 3]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      row_max[i & 1][half][r] = mx;
      ok = pair_sync();
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      mx = fmaxf(mx, row_max[i & 1][half ^ 1][r]) * p.scale_log2;  // -inf stays -inf (the scale is positive)
      // raise the maximum in use only when this row outgrows it by a margin (or has none yet)
      float corr = 1.f;
      const bool raise = mx > m_used + TC_RESCALE_ABOVE || (m_used == -INFINITY && mx != -INFINITY);
      if (raise) {
        corr = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - mx);
        m_used = mx;
        l *= corr;
      }
      const float base = (m_used == -INFINITY) ? 0.f : m_used;
      uint32_t packed[COLS / 2];
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < COLS; j += 4) {
        const float p0 = fast_exp2(fmaf(s[j], p.scale_log2, -base)), p1 = fast_exp2(fmaf(s[j + 1], p.scale_log2, -base));
        const float p2 = fast_exp2(fmaf(s[j + 2], p.scale_log2, -base)), p3 = fast_exp2(fmaf(s[j + 3], p.scale_log2, -base));
        sum4[0] += p0;
        sum4[1] += p1;
        sum4[2] += p2;
        sum4[3] += p3;
        packed[j >> 1] = pack_bf16(p0, p1);
        packed[(j >> 1) + 1] = pack_bf16(p2, p3);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // O belongs to the MMA until the product of the block before is complete.  Every block
      // waits for it, although only a raised maximum needs O: a wait by parity must see every
      // phase of its barrier, or it takes an older phase for the one it wants.
      if (i > 0) {
        ok = mbar_wait(&pv_done, (i - 1) & 1, &abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, raise)) {  // a warp-wide instruction: rows that stay are scaled by one
#pragma unroll
          for (int c0 = 0; c0 < OCOLS; c0 += 16) {
            uint32_t v[16];
            tmem_ld16(tmem_o + lane_addr + half * OCOLS + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
            tmem_st16(tmem_o + lane_addr + half * OCOLS + c0, v);
          }
        }
      }
      // P over the S it came from: bfloat16 pairs, two keys to a column, this thread's 64 keys in 32 columns
      // (its partner has read the S columns they replace: the two met after reading)
#pragma unroll
      for (int c0 = 0; c0 < COLS / 2; c0 += 16) {
        uint32_t v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = packed[c0 + j];
        tmem_st16(tmem + lane_addr + (i & 1) * TC_BN + half * (COLS / 2) + c0, v);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    if (ok) {
      ok = mbar_wait(&pv_done, (nblk - 1) & 1, &abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    // the two partial sums of a row
    row_max[0][half][r] = l;
    if (ok) {
      ok = pair_sync();
      ok = __all_sync(0xffffffffu, ok);
    }
    l += row_max[0][half ^ 1][r];
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      bf16* dst = p.out + ((size_t)(row_begin + (row_ok ? R / g : 0)) * p.nh + kvh * g + (row_ok ? R % g : 0)) * HD + half * OCOLS;
#pragma unroll
      for (int c0 = 0; c0 < OCOLS; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(tmem_o + lane_addr + half * OCOLS + c0, v);
        tmem_ld_wait();
        if (row_ok) {
          uint32_t o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = pack_bf16(__uint_as_float(v[2 * j]) * inv, __uint_as_float(v[2 * j + 1]) * inv);
          *reinterpret_cast<uint4*>(dst + c0) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(dst + c0 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && p.status) atomicExch(p.status, 2);
  if (warp == 2) tmem_dealloc(tmem, 512);
}

// Launch for a step with prompt portions; false when the shapes are not the kernel's.
static bool launch_prefill_tc(const AttnParams& p, const void* k_cache, const void* v_cache, long long cache_slots, int tiles64, int nkv, int n_seqs,
                              int max_kv_len, cudaStream_t stream, int* rc) {
  if (!(HD == 64 || HD == 128) || p.page_size % 64 != 0 || cache_slots <= 0) return false;
  if (((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)p.q & 15) || ((uintptr_t)p.out & 15)) return false;
  const int entries = max_kv_len / p.page_size + 2;
  const size_t smem = prefill_tc_smem_bytes(entries);
  if (smem > 220 * 1024) return false;
  CUtensorMap map_k, map_v;
  if (!make_tensor_map_bf16(&map_k, k_cache, (uint64_t)cache_slots, (uint64_t)nkv * HD, 64, 64) ||
      !make_tensor_map_bf16(&map_v, v_cache, (uint64_t)cache_slots, (uint64_t)nkv * HD, 64, 64))
    return false;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess) {
      *rc = ALOFA_ERR_LAUNCH;
      return true;
    }
    prefer_max_shared(attention_prefill_tc_kernel);
    configured = true;
  }
  launch_dep(attention_prefill_tc_kernel, dim3((tiles64 + 1) / 2, nkv, n_seqs), TC_THREADS, smem, stream, p, map_k, map_v);
  *rc = cudaGetLastError() == cudaSuccess ? ALOFA_OK : ALOFA_ERR_LAUNCH;
  return true;
}
