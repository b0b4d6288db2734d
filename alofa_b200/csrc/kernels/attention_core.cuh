// Device code shared by the attention kernels: the tile constants for one head
// size, the asynchronous-copy / ldmatrix / mma.sync wrappers, and attend_block,
// which runs 16 query rows against one 64-key block held in shared memory with
// the streaming softmax in fp32 (running maximum, exp2 with the scale folded
// in, rescaled sums).  HEAD_DIM is a compile-time constant (a multiple of 16 up
// to 128).  Formulas: src/alofa/kernels/cpu/scalar.mojo:392-470.
#pragma once
#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

constexpr int HD = HEAD_DIM;
constexpr int BLOCK_M = 64;   // query rows per CTA (4 warps x 16)
constexpr int BLOCK_N = 64;   // keys per block
constexpr int ROW = HD + 8;   // shared-memory row in elements: 16 bytes of padding keep ldmatrix conflict-free
constexpr int KSTEPS = HD / 16;
constexpr int DTILES = HD / 8;
constexpr int CHUNKS = HD / 8;  // 16-byte chunks per row
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head_dim must be a multiple of 16 between 16 and 128");

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* gptr, bool pred) {
  const int bytes = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem), "l"(gptr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 2^x by the hardware approximation (2 ulp); 2^-inf = 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Running state of 16 query rows held by one warp: maxima, sums and output tiles.
struct RowState {
  float m_lo, m_hi, l_lo, l_hi;
  float o[DTILES][4];
};

// Shared-memory address of the 16-byte chunk at (row, col) of a 64-key tile.
// Padded layout: rows of ROW elements (the cp.async path).  Swizzled layout (what a
// TMA load with 128-byte swizzle leaves): sub-tiles of 64 dims, rows of 128 bytes,
// the chunk index XOR-ed with the low bits of the row.
template <bool SWIZZLED>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int col) {
  if (SWIZZLED) {
    const int sub = col >> 6, chunk = (col & 63) >> 3;
    return base + sub * (BLOCK_N * 128) + row * 128 + ((chunk ^ (row & 7)) << 4);
  }
  return base + (row * ROW + col) * 2;
}

// One warp: 16 query rows against the 64 keys of one block held in shared tiles.
// keys_done() runs when the key tile has been read for the last time (it may be
// refilled), values_wanted() just before the value tile is read for the first time.
template <bool SWIZZLED, class KeysDone, class ValuesWanted>
__device__ __forceinline__ void attend_block(RowState& st, const uint32_t (&qf)[KSTEPS][4], uint32_t kt, uint32_t vt, int j0, int lane,
                                             int pos, int k_lo, int k_hi, int window, float scale_log2, KeysDone keys_done,
                                             ValuesWanted values_wanted) {
  float s[BLOCK_N / 8][4];
#pragma unroll
  for (int n = 0; n < BLOCK_N / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
    for (int n2 = 0; n2 < BLOCK_N / 16; ++n2) {
      uint32_t kf[4];
      ldmatrix_x4(kf, tile_addr<SWIZZLED>(kt, n2 * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 16 + ((lane >> 3) & 1) * 8));
      mma_16816(s[2 * n2], qf[ks], kf[0], kf[1]);
      mma_16816(s[2 * n2 + 1], qf[ks], kf[2], kf[3]);
    }
  }
  keys_done();
  const bool all_visible = j0 >= k_lo && j0 + BLOCK_N - 1 <= k_hi && (window <= 0 || j0 > pos - window);
  if (!all_visible) {
#pragma unroll
    for (int n = 0; n < BLOCK_N / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + n * 8 + (lane & 3) * 2 + (e & 1);
        bool vis = j <= pos && j >= k_lo && j <= k_hi;
        if (window > 0) vis = vis && j > pos - window;
        if (!vis) s[n][e] = -INFINITY;
      }
  }
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
  const float mn_lo = fmaxf(st.m_lo, bm_lo), mn_hi = fmaxf(st.m_hi, bm_hi);
  const float base_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo * scale_log2;
  const float base_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi * scale_log2;
  const float corr_lo = (st.m_lo == -INFINITY) ? 0.f : fast_exp2(st.m_lo * scale_log2 - base_lo);
  const float corr_hi = (st.m_hi == -INFINITY) ? 0.f : fast_exp2(st.m_hi * scale_log2 - base_hi);
  st.m_lo = mn_lo;
  st.m_hi = mn_hi;
  float sum_lo = 0.f, sum_hi = 0.f;
  uint32_t pf[BLOCK_N / 16][4];
#pragma unroll
  for (int n = 0; n < BLOCK_N / 8; ++n) {
    const float p0 = fast_exp2(s[n][0] * scale_log2 - base_lo), p1 = fast_exp2(s[n][1] * scale_log2 - base_lo);
    const float p2 = fast_exp2(s[n][2] * scale_log2 - base_hi), p3 = fast_exp2(s[n][3] * scale_log2 - base_hi);
    sum_lo += p0 + p1;
    sum_hi += p2 + p3;
    pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
    pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
  }
  st.l_lo = st.l_lo * corr_lo + sum_lo;
  st.l_hi = st.l_hi * corr_hi + sum_hi;
#pragma unroll
  for (int d = 0; d < DTILES; ++d) {
    st.o[d][0] *= corr_lo;
    st.o[d][1] *= corr_lo;
    st.o[d][2] *= corr_hi;
    st.o[d][3] *= corr_hi;
  }
  values_wanted();
#pragma unroll
  for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
#pragma unroll
    for (int d2 = 0; d2 < HD / 16; ++d2) {
      uint32_t vf[4];
      ldmatrix_x4_trans(vf, tile_addr<SWIZZLED>(vt, kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, d2 * 16 + (lane >> 4) * 8));
      mma_16816(st.o[2 * d2], pf[kk], vf[0], vf[1]);
      mma_16816(st.o[2 * d2 + 1], pf[kk], vf[2], vf[3]);
    }
  }
}

template <bool SWIZZLED>
__device__ __forceinline__ void attend_block(RowState& st, const uint32_t (&qf)[KSTEPS][4], uint32_t kt, uint32_t vt, int j0, int lane,
                                             int pos, int k_lo, int k_hi, int window, float scale_log2) {
  attend_block<SWIZZLED>(st, qf, kt, vt, j0, lane, pos, k_lo, k_hi, window, scale_log2, [] {}, [] {});
}

constexpr int MERGE_ROW = HD + 4;  // floats per merged row in shared memory

