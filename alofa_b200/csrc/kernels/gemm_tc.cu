// bfloat16 matrix product on the 5th-generation tensor cores (sm_100a):
//   y[t, f] = sum_k x[t, k] * W[f, k]   (+ bias, fused epilogue)
// W [N, K] and x [T, K] are row-major (K contiguous), accumulation is fp32.
//
// The weight is the M operand: one CTA owns 128 output features and BN tokens,
// so the same kernel streams weights for a handful of decode tokens (BN = 16)
// and computes prompt portions (BN up to 256).  Per 64-deep k-slice a producer
// thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the
// weight tile [128 x 64] and the token tile [BN x 64] into a ring of shared
// memory stages; one thread issues tcgen05.mma (M = 128, N = BN, K = 16, four
// per slice) accumulating in tensor memory; four epilogue warps read the
// accumulator with tcgen05.ld (lane = feature) and write it out:
//   EPI_STORE    out[t, f] = acc + bias[f]                (bf16 or fp32)
//   EPI_RESIDUAL out[t, f] += acc + bias[f]               (fp32 residual stream)
//   EPI_GATED    W = [gate; up]: out[t, f] = silu(g) * u  (two accumulators)
//   EPI_PARTIAL  ws[z, t, f] = acc                        (split-K; see reduce)
//   EPI_ROPE     W = [q; k; v]: bias, NeoX rotation of q and k, q to its buffer,
//                k and v to their cache slots
// Formulas: the product with its bias src/alofa/kernels/cpu/scalar.mojo:132-205,
// silu(gate) * up scalar.mojo:208-231, the rotation scalar.mojo:283-344, the
// cache write through the block table src/alofa/kernels/cpu/paged.mojo:208-246.
// Split-K (grid.z > 1) spreads the k-slices of one tile over several CTAs so
// that a small token count still pulls weights through every SM; the partial
// sums are added in a fixed order by alofa_splitk_reduce.
//
// Decode steps of a few dozen tokens keep the residual stream as a base tensor plus a 64-bit
// fixed-point accumulator (units of 2^-32): residual products add their split sums into the
// accumulator with atomic integer adds - the sum does not depend on the order of arrival.  In
// steps of up to 16 tokens the product that reads the stream next (q/k/v, gate/up) makes its
// token operand from base + accumulator itself, with the RMSNorm folded in (B_NORMED): the
// operand is (base + acc) * gamma, the row's 1/sqrt(mean square + eps) is a per-token factor and
// is applied to the accumulator in the epilogue (src/alofa/kernels/cpu/scalar.mojo:93-129 for the
// norm).  No norm kernel, no split sums in memory.  In larger steps the norm kernel reads base +
// accumulator.
//
// Every wait on an mbarrier is bounded: after the limit the CTA raises the
// status word, skips its remaining work, frees its tensor memory and returns.
#include "common.cuh"
#include <string.h>

#include "tcgen05.cuh"
#include "tma.cuh"

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_GATED = 2, EPI_ROPE = 3 };  // EPI_ROPE: weights-on-M tiles of 16 tokens only
enum { B_ROWS = 0, B_MERGED_SPLITS = 1, B_NORMED = 2 };

constexpr int BM = 128;        // features per CTA (UMMA M)
constexpr int BK = 64;         // k-slice: 64 bf16 = one 128-byte swizzle row
constexpr int NUM_THREADS = 192;  // warp 0 producer, warp 1 MMA, warps 2-5 epilogue
// The kernels with the tokens on the M side have eight epilogue warps, two to each quarter of the
// accumulator's lanes (a warp reads the lanes 32 (w % 4) ... of tensor memory): each takes half of
// the columns and half of the rows' stores.  One warp per scheduler left the epilogue waiting on
// its own instructions' latency for most of its time.
constexpr int TOKENS_THREADS = 320;  // warp 0 producer, warp 1 MMA, warps 2-9 epilogue

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
struct GemmArgs {
  void* out;          // EPI_STORE/GATED: [T, N] bf16 or fp32; EPI_RESIDUAL: [T, N] fp32
  float* partial;     // split-K: [splits, n_acc, T, N] fp32
  const float* bias;  // [N] (GATED: [2N]) or null
  int T, N, K;        // tokens, output features (GATED: per half), depth
  int k_slices_per_split;
  int out_bf16;
  int pair;           // tokens on M: the wide product runs on pairs of CTAs (the weight map's box is then 128 rows)
  int few;            // tokens on M, persistent, up to 64 tokens: the token map's box is this many rows (32 or 64), else 0
  int* status;
  // The token operand of the weights-on-M kernel need not lie in memory as rows: the
  // epilogue warps, idle while the MMAs run, can make each k-slice of it in shared memory.
  int b_kind;               // B_ROWS: rows of x by TMA; B_MERGED_SPLITS: made from the key splits of decode attention
  const float* b_src;       // merged splits: partial outputs [splits, T * heads, head_dim]
  const float* b_ml;        // merged splits: (maximum, sum) [splits, T * heads, 2]
  const int* b_positions;   // merged splits: position of each token
  int b_heads, b_head_dim, b_window, b_split_keys;
  int cluster;              // the splits of a tile are a thread-block cluster and add their sums up themselves (MODE_CLUSTER)
  // EPI_RESIDUAL into a stream kept as base + accumulator: every CTA adds its sums (the first split
  // the bias too) into acc [T, N] with atomic 64-bit integer adds, in units of 2^-32
  long long* acc;
  // B_NORMED (cluster kernels of 16 tokens): the token operand is RMSNorm(base + n_acc) made by the
  // epilogue warps; the CTAs of the first feature tile also write base + n_acc to n_out (the
  // stream's new base) and zero n_zero (the accumulator the next residual product adds into)
  const float* n_base;       // [T, K] fp32
  const long long* n_acc;    // [T, K] or null
  const float* n_gamma;      // [K]
  float* n_out;              // [T, K]
  long long* n_zero;         // [T, K] or null
  float n_eps;
  // EPI_ROPE: the weight is [q heads | k heads | v heads] stacked; the epilogue adds the bias, rotates q and k
  // (NeoX halves, cos/sin from a table by position) and writes q to its buffer, k and v to their cache slots
  bf16* rope_q;             // [T, heads * head_dim]
  bf16* rope_k;             // cache [slots, kv_heads, head_dim]
  bf16* rope_v;
  const int* rope_slots;    // [T] cache slot of each token, negative: not written
  const int* rope_positions;
  const float* rope_table;  // [positions, head_dim / 2, 2]
  int rope_heads, rope_kv_heads, rope_head_dim;
};

// ---------------------------------------------------------------------------
// A token operand that is computed, not loaded: eight consecutive depth entries
// for token t from depth k0 on, as packed bfloat16.  All loads of a chunk are
// issued before any is used, so a chunk costs one trip to L2.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 packed;
  __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
  packed.x = *reinterpret_cast<uint32_t*>(&h0);
  packed.y = *reinterpret_cast<uint32_t*>(&h1);
  packed.z = *reinterpret_cast<uint32_t*>(&h2);
  packed.w = *reinterpret_cast<uint32_t*>(&h3);
  return packed;
}

// B_MERGED_SPLITS: the attention output of a decode token whose keys were split
// over CTAs - (output, maximum, sum) per split, merged in split order exactly as
// attention_combine_kernel does.  Up to MERGE_MAX splits.
constexpr int MERGE_MAX = 16;
__device__ __forceinline__ uint4 merged_splits8(const GemmArgs& a, int t, int k0, int P) {
  const int head = k0 / a.b_head_dim, d = k0 - head * a.b_head_dim;
  const int rows = a.T * a.b_heads, row = t * a.b_heads + head;
  const int k_lo = a.b_window > 0 ? max(0, P - a.b_window + 1) : 0;
  const int s_lo = k_lo / a.b_split_keys, n = P / a.b_split_keys - s_lo + 1;  // splits that hold keys of this token
  float2 ml[MERGE_MAX];
  float4 lo[MERGE_MAX / 2], hi[MERGE_MAX / 2];
#pragma unroll
  for (int i = 0; i < MERGE_MAX; ++i)
    ml[i] = i < n ? *reinterpret_cast<const float2*>(a.b_ml + ((size_t)(s_lo + i) * rows + row) * 2) : make_float2(-INFINITY, 0.f);
#pragma unroll
  for (int i = 0; i < MERGE_MAX / 2; ++i) {
    const float* src = a.b_src + ((size_t)(s_lo + (i < n ? i : 0)) * rows + row) * a.b_head_dim + d;
    lo[i] = *reinterpret_cast<const float4*>(src);
    hi[i] = *reinterpret_cast<const float4*>(src + 4);
  }
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < MERGE_MAX; ++i) m = fmaxf(m, ml[i].x);
  float l = 0.f, v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = 0.f;
  auto add = [&](float2 mls, float4 x, float4 y) {
    float w;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w) : "f"(mls.x - m));
    if (mls.x == -INFINITY) w = 0.f;
    l += mls.y * w;
    v[0] += x.x * w, v[1] += x.y * w, v[2] += x.z * w, v[3] += x.w * w;
    v[4] += y.x * w, v[5] += y.y * w, v[6] += y.z * w, v[7] += y.w * w;
  };
#pragma unroll
  for (int i = 0; i < MERGE_MAX / 2; ++i) add(ml[i], lo[i], hi[i]);
  if (n > MERGE_MAX / 2) {  // a second trip for the rest
#pragma unroll
    for (int i = 0; i < MERGE_MAX / 2; ++i) {
      const int s = MERGE_MAX / 2 + i;
      const float* src = a.b_src + ((size_t)(s_lo + (s < n ? s : 0)) * rows + row) * a.b_head_dim + d;
      lo[i] = *reinterpret_cast<const float4*>(src);
      hi[i] = *reinterpret_cast<const float4*>(src + 4);
    }
#pragma unroll
    for (int i = 0; i < MERGE_MAX / 2; ++i) add(ml[MERGE_MAX / 2 + i], lo[i], hi[i]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = v[j] / l;
  return pack8(v);
}

// Variants (kernels of their own, so that the plain one keeps its small register count and the
// next kernel's CTAs can become resident beside it under programmatic dependent launch):
// MODE_COMPUTED: the token operand is made by the epilogue warps (GemmArgs::b_kind).
// MODE_CLUSTER: the CTAs that split the depth of a tile form a thread-block cluster along z; the
// others push their accumulators into the shared memory of the first, which adds them in split
// order and runs the epilogue - no partial sums in global memory, no second kernel.
// MODE_NORMED: MODE_CLUSTER with the token operand made from the residual stream (B_NORMED).
enum { MODE_PLAIN = 0, MODE_COMPUTED = 1, MODE_CLUSTER = 2, MODE_NORMED = 3 };

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {  // every thread of every CTA of the cluster, exactly once
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void store_remote_f32(uint32_t local_smem_addr, uint32_t rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

template <int BN, int EPI, int MODE = MODE_PLAIN>
__global__ void __launch_bounds__(NUM_THREADS, MODE == MODE_COMPUTED ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmArgs args, const int stages) {
  constexpr int N_ACC = (EPI == EPI_GATED) ? 2 : 1;
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = N_ACC * A_BYTES + B_BYTES;
  constexpr int CHAINS = 1;
  constexpr int ACC_COLS = N_ACC * CHAINS * BN;
  constexpr uint32_t TMEM_COLS = (ACC_COLS <= 32) ? 32 : (ACC_COLS <= 64) ? 64 : (ACC_COLS <= 128) ? 128 : (ACC_COLS <= 256) ? 256 : 512;
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[12], empty_bar[12], acc_bar;
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = blockIdx.x * BM, t0 = blockIdx.y * BN;
  const int total_slices = (args.K + BK - 1) / BK;
  const int slice_begin = blockIdx.z * args.k_slices_per_split;
  const int slice_end = min(total_slices, slice_begin + args.k_slices_per_split);
  const int n_slices = slice_end - slice_begin;

  constexpr bool COMPUTED = MODE == MODE_COMPUTED, NORMED = MODE == MODE_NORMED, CLUSTER = MODE == MODE_CLUSTER || NORMED;
  constexpr bool computed_b = COMPUTED || NORMED;
  const uint32_t rank = CLUSTER ? cluster_rank() : 0;  // this CTA's split of the depth, within its cluster
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], computed_b ? 1 + 128 : 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) tmem_alloc(&tmem_base_smem, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  // the position of this thread's token, for a merged-splits operand: written with the step's
  // metadata before any kernel of the step ran, so it may be read ahead of the wait below
  int token_pos = 0;
  if (COMPUTED && args.b_kind == B_MERGED_SPLITS && warp >= 2) {
    const int t = t0 + ((threadIdx.x - 64) >> 3);
    if (t < args.T) token_pos = args.b_positions[t];
  }
  // Rotate-and-store: each epilogue thread's cosines and sines (one feature, 16 tokens) and the
  // tokens' cache slots.  Positions and slots came with the step's metadata and the table is a
  // constant of the model, so they too may be read ahead of the wait.
  float2 rope_cs[EPI == EPI_ROPE ? 16 : 1];
  int rope_slot[EPI == EPI_ROPE ? 16 : 1];
  float rope_bias = 0.f;  // the bias of this thread's feature: a constant of the model as well
  if constexpr (EPI == EPI_ROPE) {
    if (warp >= 2 && rank == 0) {
      const int row = ((warp & 3) << 5) + lane, hd = args.rope_head_dim, half = hd >> 1;
      if (args.bias && f0 + row < args.N) rope_bias = args.bias[f0 + row];
      const int d = row % hd, i = d < half ? d : d - half;
      const bool rotated = (f0 + row) / hd < args.rope_heads + args.rope_kv_heads;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int t = t0 + j;
        rope_cs[j] = make_float2(1.f, 0.f);
        rope_slot[j] = -1;
        if (t < args.T) {
          if (rotated) rope_cs[j] = *reinterpret_cast<const float2*>(args.rope_table + ((size_t)args.rope_positions[t] * half + i) * 2);
          if (args.rope_slots) rope_slot[j] = args.rope_slots[t];
        }
      }
    }
  }
  // B_NORMED: this thread's chunks of the norm's weight (a constant of the model), ahead of the wait
  constexpr int NORM_BATCH = 3;  // k-slices whose loads are in flight together (a batch is one trip to L2)
  float4 gamma_lo[NORMED ? NORM_BATCH : 1], gamma_hi[NORMED ? NORM_BATCH : 1];
  if constexpr (NORMED) {
    if (warp >= 2) {
      const int c = (threadIdx.x - 64) & 7;
#pragma unroll
      for (int b = 0; b < NORM_BATCH; ++b) {
        const int k = (slice_begin + b) * BK + c * 8;
        gamma_lo[b] = gamma_hi[b] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < n_slices && k < args.K) {
          gamma_lo[b] = *reinterpret_cast<const float4*>(args.n_gamma + k);
          gamma_hi[b] = *reinterpret_cast<const float4*>(args.n_gamma + k + 4);
        }
      }
    }
  }
  // The weights depend on no earlier kernel: the producer asks for the first ring of weight tiles
  // before it waits for the kernel before this one; only the token operand comes after the wait.
  // The kernel after this one is let in after the wait (see pdl_launch).
  int early_slices = 0;
  if (threadIdx.x == 0) {
    early_slices = min(stages, n_slices);
    for (int i = 0; i < early_slices; ++i) {
      uint8_t* stage = tiles + (size_t)i * STAGE_BYTES;
      mbar_expect_tx(&full_bar[i], computed_b ? N_ACC * A_BYTES : STAGE_BYTES);
      const int k = (slice_begin + i) * BK;
      tma_load_2d(stage, &map_w, &full_bar[i], k, f0);
      if (N_ACC == 2) tma_load_2d(stage + A_BYTES, &map_w, &full_bar[i], k, args.N + f0);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
  } else {
    pdl_wait();
    pdl_launch();
  }

  // The epilogue of the four epilogue warps: warp q reads lanes [32q, 32q + 32) of the accumulator.
  // with_remote (first CTA of a cluster): the other CTAs' accumulators, pushed into `pushed`
  // [rank - 1][accumulator][token][feature], are added in rank order first.
  bool epilogue_ok = false;
  float* pushed = reinterpret_cast<float*>(tiles + (size_t)stages * STAGE_BYTES);
  float* rope_xchg = pushed + (CLUSTER ? (size_t)(gridDim.z - 1) * N_ACC * BN * 128 : 0);  // EPI_ROPE: [16 tokens][128 features]
  float* row_ss = rope_xchg + (EPI == EPI_ROPE ? 16 * 128 : 0);  // MODE_NORMED: [8 ranks][16 tokens] sums of squares, then the 16 factors, in the first CTA
  auto epilogue = [&](bool with_remote) {
    const int q = warp & 3;
    const int f = f0 + q * 32 + lane;
    const bool f_ok = f < args.N;
    const bool split = gridDim.z > 1 && !CLUSTER;
    const bool push = CLUSTER && rank != 0;
    // MODE_NORMED: the accumulator holds sums over (base + acc) * gamma; the row's factor 1 / sqrt(mean
    // square + eps) comes from the sums of squares all CTAs of the cluster sent to the first
    float rstd[NORMED ? 16 : 1];
    if constexpr (NORMED) {
      if (!push) {
        // one thread per token adds the CTAs' sums up (in rank order) and takes the root; the others read the 16 factors
        // (every thread adding them up for itself cost 5 us: 16 x 7 dependent reads of shared memory)
        const int et = threadIdx.x - 64;
        if (et < 16) {
          float part[8];
#pragma unroll
          for (int z = 0; z < 8; ++z) part[z] = z < (int)gridDim.z ? row_ss[z * 16 + et] : 0.f;
          float ss = 0.f;
#pragma unroll
          for (int z = 0; z < 8; ++z) ss += part[z];
          row_ss[8 * 16 + et] = 1.0f / sqrtf(ss / (float)args.K + args.n_eps);
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");  // the four epilogue warps
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          const float4 f = *reinterpret_cast<const float4*>(row_ss + 8 * 16 + j);
          rstd[j] = f.x, rstd[j + 1] = f.y, rstd[j + 2] = f.z, rstd[j + 3] = f.w;
        }
      }
    }
    float bias0 = 0.f, bias1 = 0.f;
    if (EPI == EPI_ROPE) {
      bias0 = rope_bias;
    } else if (!split && !push && args.bias && f_ok) {
      bias0 = args.bias[f];
      if (N_ACC == 2) bias1 = args.bias[args.N + f];
    }
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
      if (t0 + c0 >= args.T) break;
      uint32_t r0[16], r1[16];
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
      if (n_slices > 0) {
        tmem_ld16(taddr, r0);
        if (N_ACC == 2) tmem_ld16(taddr + CHAINS * BN, r1);
        tmem_ld_wait();
#pragma unroll
        for (int c = 1; c < CHAINS; ++c) {
          uint32_t x0[16], x1[16];
          tmem_ld16(taddr + c * BN, x0);
          if (N_ACC == 2) tmem_ld16(taddr + (CHAINS + c) * BN, x1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            r0[j] = __float_as_uint(__uint_as_float(r0[j]) + __uint_as_float(x0[j]));
            if (N_ACC == 2) r1[j] = __float_as_uint(__uint_as_float(r1[j]) + __uint_as_float(x1[j]));
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r0[j] = r1[j] = 0u;
      }
      if constexpr (CLUSTER) {
        const int row = q * 32 + lane;
        const int live = min(16, args.T - (t0 + c0));  // tokens of this group that exist: the others are neither sent nor added
        if (push) {  // this CTA's sums into the first CTA's shared memory; nothing goes to global memory
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j < live) {
              store_remote_f32(smem_u32(pushed + (((rank - 1) * N_ACC + 0) * BN + c0 + j) * 128 + row), 0, __uint_as_float(r0[j]));
              if (N_ACC == 2) store_remote_f32(smem_u32(pushed + (((rank - 1) * N_ACC + 1) * BN + c0 + j) * 128 + row), 0, __uint_as_float(r1[j]));
            }
          }
          continue;
        }
        if (with_remote) {
          for (uint32_t z = 1; z < gridDim.z; ++z) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j < live) {
                r0[j] = __float_as_uint(__uint_as_float(r0[j]) + pushed[(((z - 1) * N_ACC + 0) * BN + c0 + j) * 128 + row]);
                if (N_ACC == 2) r1[j] = __float_as_uint(__uint_as_float(r1[j]) + pushed[(((z - 1) * N_ACC + 1) * BN + c0 + j) * 128 + row]);
              }
            }
          }
        }
      }
      if constexpr (NORMED) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          r0[j] = __float_as_uint(__uint_as_float(r0[j]) * rstd[j]);
          if (N_ACC == 2) r1[j] = __float_as_uint(__uint_as_float(r1[j]) * rstd[j]);
        }
      }
      if constexpr (EPI == EPI_ROPE) {
        // Rotate-and-store.  A thread holds one feature of 16 tokens; its rotation partner, half a
        // head away, is another thread of this CTA (a tile of 128 features holds whole heads): the
        // values change hands through shared memory, [token][feature] so that no bank is hit twice.
        const int row = q * 32 + lane, hd = args.rope_head_dim, half = hd >> 1;
        float v[16], pv[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          v[j] = __uint_as_float(r0[j]) + bias0;
          rope_xchg[j * 128 + row] = v[j];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        const int d = row % hd;  // tiles start at multiples of 128, which head_dim divides
        const int partner = d < half ? row + half : row - half;
#pragma unroll
        for (int j = 0; j < 16; ++j) pv[j] = rope_xchg[j * 128 + partner];
        if (!f_ok) continue;
        const int head = f / hd;
        const bool is_q = head < args.rope_heads, is_k = !is_q && head < args.rope_heads + args.rope_kv_heads;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = t0 + c0 + j;
          if (t >= args.T) break;
          const float2 cs = rope_cs[j];  // (1, 0) for the value heads
          const float y = d < half ? v[j] * cs.x - pv[j] * cs.y : v[j] * cs.x + pv[j] * cs.y;
          if (is_q) {
            args.rope_q[(size_t)t * args.rope_heads * hd + f] = __float2bfloat16_rn(y);
          } else {
            const int slot = rope_slot[j];
            if (slot < 0) continue;
            if (is_k) args.rope_k[((size_t)slot * args.rope_kv_heads + (head - args.rope_heads)) * hd + d] = __float2bfloat16_rn(y);
            else args.rope_v[((size_t)slot * args.rope_kv_heads + (head - args.rope_heads - args.rope_kv_heads)) * hd + d] = __float2bfloat16_rn(y);
          }
        }
        continue;
      }
      if (!f_ok) continue;
      const int t_base = t0 + c0;
      if (EPI == EPI_RESIDUAL && args.acc) {
        // the stream stands as base + accumulator: integer adds, whose sum does not depend on their order
        unsigned long long* a = reinterpret_cast<unsigned long long*>(args.acc) + (size_t)t_base * args.N + f;
        const float b = blockIdx.z == 0 && args.bias ? args.bias[f] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (t_base + j < args.T) atomicAdd(a + (size_t)j * args.N, (unsigned long long)__float2ll_rn((__uint_as_float(r0[j]) + b) * STREAM_SCALE));
        continue;
      }
      if (!split && EPI == EPI_RESIDUAL) {
        // read the 16 residual values first, then write: the loads overlap
        float* o = (float*)args.out + (size_t)t_base * args.N + f;
        float prev[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) prev[j] = (t_base + j < args.T) ? o[(size_t)j * args.N] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (t_base + j < args.T) o[(size_t)j * args.N] = prev[j] + (__uint_as_float(r0[j]) + bias0);
        continue;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int t = t_base + j;
        if (t >= args.T) break;
        const float a0 = __uint_as_float(r0[j]);
        if (split) {
          const size_t plane = (size_t)args.T * args.N;
          float* p = args.partial + (size_t)blockIdx.z * N_ACC * plane + (size_t)t * args.N + f;
          p[0] = a0;
          if (N_ACC == 2) p[plane] = __uint_as_float(r1[j]);
        } else if (EPI == EPI_GATED) {
          const float g = a0 + bias0, u = __uint_as_float(r1[j]) + bias1;
          const float y = silu_times(g, u);
          if (args.out_bf16) ((bf16*)args.out)[(size_t)t * args.N + f] = __float2bfloat16_rn(y);
          else ((float*)args.out)[(size_t)t * args.N + f] = y;
        } else {
          const float y = a0 + bias0;
          if (args.out_bf16) ((bf16*)args.out)[(size_t)t * args.N + f] = __float2bfloat16_rn(y);
          else ((float*)args.out)[(size_t)t * args.N + f] = y;
        }
      }
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: TMA loads into the ring --------------------------------
      for (int i = 0; i < n_slices; ++i) {
        const int s = i % stages;
        if (i >= stages && !mbar_wait(&empty_bar[s], ((i / stages) - 1) & 1, &abort_flag)) break;
        uint8_t* stage = tiles + (size_t)s * STAGE_BYTES;
        const int k = (slice_begin + i) * BK;
        if (i >= early_slices) {  // the first ring's weights were asked for ahead of the wait
          mbar_expect_tx(&full_bar[s], computed_b ? N_ACC * A_BYTES : STAGE_BYTES);
          tma_load_2d(stage, &map_w, &full_bar[s], k, f0);
          if (N_ACC == 2) tma_load_2d(stage + A_BYTES, &map_w, &full_bar[s], k, args.N + f0);
        }
        if (!computed_b) tma_load_2d(stage + N_ACC * A_BYTES, &map_x, &full_bar[s], k, t0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer --------------------------------------------------------
      bool ok = true;
      for (int i = 0; i < n_slices && ok; ++i) {
        const int s = i % stages;
        ok = mbar_wait(&full_bar[s], (i / stages) & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t stage = smem_u32(tiles + (size_t)s * STAGE_BYTES);
        const uint64_t desc_b = smem_desc_sw128(stage + N_ACC * A_BYTES);
#pragma unroll
        for (int a = 0; a < N_ACC; ++a) {
          const uint64_t desc_a = smem_desc_sw128(stage + a * A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_base + (a * CHAINS + k % CHAINS) * BN, desc_a + (uint64_t)(k * 2), desc_b + (uint64_t)(k * 2), IDESC,
                      (i > 0 || k >= CHAINS) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
      }
      umma_commit(&acc_bar);  // the accumulator is complete once all MMAs are done
    }
  } else {
    // ---- the four epilogue warps ------------------------------------------------
    if constexpr (COMPUTED) {
      // First the token operand, slice by slice: rows of 128 bytes, 16-byte chunk c of row r at
      // c ^ (r & 7).  The host allows this for tiles of 16 tokens only: one chunk per thread.
      const int tid = threadIdx.x - 64;
      const int r = tid >> 3, c = tid & 7, t = t0 + r;
      const uint32_t at = r * 128 + ((c ^ (r & 7)) << 4);
      for (int i = 0; i < n_slices; ++i) {
        const int s = i % stages;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (t < args.T && (slice_begin + i) * BK + c * 8 < args.K) v = merged_splits8(args, t, (slice_begin + i) * BK + c * 8, token_pos);
        if (i >= stages && !mbar_wait(&empty_bar[s], ((i / stages) - 1) & 1, &abort_flag)) break;
        *reinterpret_cast<uint4*>(tiles + (size_t)s * STAGE_BYTES + N_ACC * A_BYTES + at) = v;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(&full_bar[s]);
      }
    }
    if constexpr (NORMED) {
      // The token operand from the residual stream, a batch of k-slices per trip to L2: this thread's
      // eight values of token r are base + accumulator (rounded to fp32 once), times the norm's weight;
      // their squares are summed for the row's factor.  Rows of 128 bytes, chunk c of row r at c ^ (r & 7).
      const int tid = threadIdx.x - 64;
      const int r = tid >> 3, c = tid & 7, t = t0 + r;
      const uint32_t at = r * 128 + ((c ^ (r & 7)) << 4);
      const bool writes_stream = blockIdx.x == 0;  // one feature tile brings the stream's new base to memory
      float ss = 0.f;
      for (int i0 = 0; i0 < n_slices; i0 += NORM_BATCH) {
        float4 lo[NORM_BATCH], hi[NORM_BATCH];
        longlong2 a[NORM_BATCH][4];
#pragma unroll
        for (int b = 0; b < NORM_BATCH; ++b) {
          const int k = (slice_begin + i0 + b) * BK + c * 8;
          const bool live = i0 + b < n_slices && t < args.T && k < args.K;
          lo[b] = hi[b] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int q = 0; q < 4; ++q) a[b][q] = make_longlong2(0, 0);
          if (live) {
            const size_t e = (size_t)t * args.K + k;
            lo[b] = *reinterpret_cast<const float4*>(args.n_base + e);
            hi[b] = *reinterpret_cast<const float4*>(args.n_base + e + 4);
            if (args.n_acc) {
              const longlong2* p = reinterpret_cast<const longlong2*>(args.n_acc + e);
#pragma unroll
              for (int q = 0; q < 4; ++q) a[b][q] = p[q];
            }
            if (i0 > 0) {  // the first batch's weights were read ahead of the wait
              gamma_lo[b] = *reinterpret_cast<const float4*>(args.n_gamma + k);
              gamma_hi[b] = *reinterpret_cast<const float4*>(args.n_gamma + k + 4);
            }
          }
        }
#pragma unroll
        for (int b = 0; b < NORM_BATCH; ++b) {
          const int i = i0 + b;
          if (i >= n_slices) break;
          const int s = i % stages;
          const int k = (slice_begin + i) * BK + c * 8;
          const bool live = t < args.T && k < args.K;
          float v[8] = {lo[b].x, lo[b].y, lo[b].z, lo[b].w, hi[b].x, hi[b].y, hi[b].z, hi[b].w};
          if (live && args.n_acc) {
            const long long w8[8] = {a[b][0].x, a[b][0].y, a[b][1].x, a[b][1].y, a[b][2].x, a[b][2].y, a[b][3].x, a[b][3].y};
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = stream_add(v[j], w8[j]);
          }
          if (live && writes_stream) {
            const size_t e = (size_t)t * args.K + k;
            *reinterpret_cast<float4*>(args.n_out + e) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(args.n_out + e + 4) = make_float4(v[4], v[5], v[6], v[7]);
            if (args.n_zero) {
              longlong2* z = reinterpret_cast<longlong2*>(args.n_zero + e);
#pragma unroll
              for (int q = 0; q < 4; ++q) z[q] = make_longlong2(0, 0);
            }
          }
          const float g[8] = {gamma_lo[b].x, gamma_lo[b].y, gamma_lo[b].z, gamma_lo[b].w, gamma_hi[b].x, gamma_hi[b].y, gamma_hi[b].z, gamma_hi[b].w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            ss = fmaf(v[j], v[j], ss);
            v[j] *= g[j];
          }
          if (i >= stages && !mbar_wait(&empty_bar[s], ((i / stages) - 1) & 1, &abort_flag)) break;
          *reinterpret_cast<uint4*>(tiles + (size_t)s * STAGE_BYTES + N_ACC * A_BYTES + at) = pack8(v);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_arrive(&full_bar[s]);
        }
      }
      // the row's sum of squares over this CTA's share of the depth, to the first CTA of the cluster
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 4);
      if (c == 0) store_remote_f32(smem_u32(row_ss + rank * 16 + r), 0, ss);
    }
    bool ok = n_slices > 0 ? mbar_wait(&acc_bar, 0, &abort_flag) : true;
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    epilogue_ok = ok;
    if (ok && !(CLUSTER && rank == 0)) epilogue(false);  // in a cluster the first CTA waits for the others' sums
  }
  if constexpr (CLUSTER) {
    cluster_sync_all();  // the pushed accumulators are in the first CTA's shared memory
    if (warp >= 2 && rank == 0 && epilogue_ok) epilogue(true);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag && args.status) atomicExch(args.status, 2);
}

// The epilogue of a 128-token tile whose width is a multiple of 4: warp q owns
// rows [32q, 32q + 32) of the accumulator at `tmem_acc`; `staging` holds
// 4 x 32 rows of 132 floats.  Two warps share a quarter: `half` (0 or 1) takes columns
// [64 half, 64 half + 64) of every 128 and rows [16 half, 16 half + 16) of the stores; they meet
// on the named barrier 8 + q.  `release` (optional, one arrival per warp) is signalled once the
// accumulator has been read out.
__device__ __forceinline__ void quarter_sync(int q) { asm volatile("bar.sync %0, 64;" ::"r"(8 + q) : "memory"); }
// All eight epilogue warps: true when every thread brought true (one verdict for all, so that they
// go on, or give up, together).
__device__ __forceinline__ bool epilogue_warps_agree(bool ok) {
  uint32_t any_bad;
  asm volatile(
      "{\n\t.reg .pred p, r;\n\t"
      "setp.eq.u32 p, %1, 0;\n\t"
      "bar.red.or.pred r, 1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, r;\n\t}"
      : "=r"(any_bad)
      : "r"((uint32_t)ok)
      : "memory");
  return any_bad == 0;
}

template <int BNF, int EPI>
__device__ __forceinline__ void tokens_epilogue_staged(const GemmArgs& args, uint32_t tmem_base, float* staging, int q, int half, int lane, int f0,
                                                       int t0, int n_splits, int split_index, uint64_t* release, uint32_t release_in_cluster = 0) {
  constexpr bool GATED = EPI == EPI_GATED;
  constexpr int FEATS = GATED ? BNF / 2 : BNF;
  // The accumulator rows go through shared memory so
  // that global memory is written a whole row of 128 features at a time:
  // each thread drops its row's values into a padded tile, then the warp
  // walks the 32 rows with one 16-byte access per lane.
  constexpr int PITCH = 132;  // floats per staged row: 128 + padding against bank conflicts
  float* stage = staging + (size_t)q * 32 * PITCH;
  const bool split = n_splits > 1;
  const int N = args.N;
  const size_t plane = (size_t)args.T * N;
#pragma unroll 1
  for (int cb = 0; cb < FEATS; cb += 128) {
    if (f0 + cb >= N) break;
#pragma unroll 1
    for (int c0 = half * 64; c0 < half * 64 + 64 && cb + c0 < FEATS; c0 += 16) {
      const int f = f0 + cb + c0;
      if (f >= N) break;
      uint32_t r0[16], r1[16];
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(cb + c0);
      tmem_ld16(taddr, r0);
      if (GATED) tmem_ld16(taddr + FEATS, r1);
      tmem_ld_wait();
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float a = __uint_as_float(r0[j]);
        if (!split && args.bias && f + j < N) a += args.bias[f + j];
        if (GATED) {
          float u = __uint_as_float(r1[j]);
          if (args.bias && f + j < N) u += args.bias[N + f + j];
          a = silu_times(a, u);
        }
        v[j] = a;
      }
#pragma unroll
      for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(stage + lane * PITCH + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
    const bool read_out = (release || release_in_cluster) && (cb + 128 >= FEATS || f0 + cb + 128 >= N);
    if (read_out) tc_fence_before();  // the accumulator is read out: the next tile but one may have it
    __syncwarp();
    if (read_out && lane == 0) {  // one arrival per warp: arrivals at a barrier of the other CTA are dear
      if (release_in_cluster) mbar_arrive_in_cluster(release_in_cluster);
      else mbar_arrive(release);
    }
    quarter_sync(q);  // both halves of the columns are staged
    const int f = f0 + cb + lane * 4;  // this lane's four features of every row
    const bool f_ok = f < N && cb + lane * 4 < FEATS;  // N % 4 == 0: a group is inside or outside as a whole
    const int r_lo = half * 16;
    const int rows = min(r_lo + 16, args.T - (t0 + q * 32));  // this warp stores rows [r_lo, rows)
    if (f_ok) {
      if (split) {
        float* p = args.partial + (size_t)split_index * plane + (size_t)(t0 + q * 32) * N + f;
#pragma unroll 4
        for (int r = r_lo; r < rows; ++r) *reinterpret_cast<float4*>(p + (size_t)r * N) = *reinterpret_cast<const float4*>(stage + r * PITCH + lane * 4);
      } else if (EPI == EPI_RESIDUAL) {
        float* o = (float*)args.out + (size_t)(t0 + q * 32) * N + f;
        {  // sixteen rows: all their loads in flight, then the stores
          const int rb = r_lo;
          float4 b[16];
#pragma unroll
          for (int r = 0; r < 16; ++r)
            if (rb + r < rows) b[r] = *reinterpret_cast<float4*>(o + (size_t)(rb + r) * N);
#pragma unroll
          for (int r = 0; r < 16; ++r)
            if (rb + r < rows) {
              const float4 a = *reinterpret_cast<const float4*>(stage + (rb + r) * PITCH + lane * 4);
              *reinterpret_cast<float4*>(o + (size_t)(rb + r) * N) = make_float4(b[r].x + a.x, b[r].y + a.y, b[r].z + a.z, b[r].w + a.w);
            }
        }
      } else if (args.out_bf16) {
        bf16* o = (bf16*)args.out + (size_t)(t0 + q * 32) * N + f;
#pragma unroll 4
        for (int r = r_lo; r < rows; ++r) {
          const float4 a = *reinterpret_cast<const float4*>(stage + r * PITCH + lane * 4);
          __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
          *reinterpret_cast<uint2*>(o + (size_t)r * N) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
      } else {
        float* o = (float*)args.out + (size_t)(t0 + q * 32) * N + f;
#pragma unroll 4
        for (int r = r_lo; r < rows; ++r) *reinterpret_cast<float4*>(o + (size_t)r * N) = *reinterpret_cast<const float4*>(stage + r * PITCH + lane * 4);
      }
    }
    quarter_sync(q);  // the staged rows are stored: the next 128 columns, or the next tile, may overwrite them
  }
}

// ---------------------------------------------------------------------------
// The same product with the tokens as the M operand, for prompt portions:
// one CTA owns 128 tokens and BNF weight rows (features; for EPI_GATED the
// first half of the tile's rows are gate rows, the second half the matching up
// rows, loaded by two TMA boxes into one shared-memory tile).  A tcgen05.mma of
// M = 128 takes the same time for any N up to 256, so wide feature tiles are
// what brings the tensor cores near their rate.  The accumulator has one lane
// per token and one column per feature: each epilogue thread owns a token row
// and writes runs of 16 consecutive features with 16-byte stores.
// ---------------------------------------------------------------------------
template <int BNF, int EPI>
__global__ void __launch_bounds__(TOKENS_THREADS, 2)
gemm_tc_tokens_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmArgs args, const int stages) {
  constexpr bool GATED = EPI == EPI_GATED;
  constexpr int FEATS = GATED ? BNF / 2 : BNF;  // output features per CTA
  constexpr uint32_t A_BYTES = 128 * BK * 2;    // token tile
  constexpr uint32_t B_BYTES = BNF * BK * 2;    // weight tile
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = BNF <= 32 ? 32 : BNF <= 64 ? 64 : BNF <= 128 ? 128 : 256;
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BNF >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[12], empty_bar[12], acc_bar;
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = blockIdx.x * FEATS, t0 = blockIdx.y * 128;
  const int total_slices = (args.K + BK - 1) / BK;
  const int slice_begin = blockIdx.z * args.k_slices_per_split;
  const int n_slices = min(total_slices, slice_begin + args.k_slices_per_split) - slice_begin;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) tmem_alloc(&tmem_base_smem, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  auto load_weights = [&](int i) {  // the weight tile of slice i into its stage
    const int s = i % stages;
    uint8_t* stage = tiles + (size_t)s * STAGE_BYTES;
    const int k = (slice_begin + i) * BK;
    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
    if (GATED) {
      tma_load_2d(stage + A_BYTES, &map_w, &full_bar[s], k, f0);
      tma_load_2d(stage + A_BYTES + B_BYTES / 2, &map_w, &full_bar[s], k, args.N + f0);
    } else {
      tma_load_2d(stage + A_BYTES, &map_w, &full_bar[s], k, f0);
    }
  };
  // the weights depend on no earlier kernel: the first ring of them is asked for ahead of the wait
  int early_slices = 0;
  if (threadIdx.x == 0) {
    asm volatile("griddepcontrol.launch_dependents;");
    early_slices = min(stages, n_slices);
    for (int i = 0; i < early_slices; ++i) load_weights(i);
    asm volatile("griddepcontrol.wait;" ::: "memory");
  } else {
    pdl_begin();  // set-up above overlaps the previous kernel; its results are read from here on
  }

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < n_slices; ++i) {
        const int s = i % stages;
        if (i >= stages && !mbar_wait(&empty_bar[s], ((i / stages) - 1) & 1, &abort_flag)) break;
        if (i >= early_slices) load_weights(i);
        tma_load_2d(tiles + (size_t)s * STAGE_BYTES, &map_x, &full_bar[s], (slice_begin + i) * BK, t0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int i = 0; i < n_slices; ++i) {
        const int s = i % stages;
        if (!mbar_wait(&full_bar[s], (i / stages) & 1, &abort_flag)) break;
        tc_fence_after();
        const uint32_t stage = smem_u32(tiles + (size_t)s * STAGE_BYTES);
        const uint64_t desc_a = smem_desc_sw128(stage), desc_b = smem_desc_sw128(stage + A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16(tmem_base, desc_a + (uint64_t)(k * 2), desc_b + (uint64_t)(k * 2), IDESC, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      umma_commit(&acc_bar);
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int t = t0 + q * 32 + lane;
    bool ok = mbar_wait(&acc_bar, 0, &abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    ok = epilogue_warps_agree(ok);  // the quarter's other warp must not be left waiting for this one
    tc_fence_after();
    const bool staged = (args.N & 3) == 0 && !(GATED && gridDim.z > 1);
    if (ok && staged && t0 + q * 32 < args.T) {
      tokens_epilogue_staged<BNF, EPI>(args, tmem_base, reinterpret_cast<float*>(tiles), q, half, lane, f0, t0, (int)gridDim.z, (int)blockIdx.z, nullptr);
    } else if (ok && t0 + q * 32 < args.T) {
      // widths that are no multiple of 4 (or gated partial sums): element-wise, straight from the registers
      const bool split = gridDim.z > 1;
      const bool t_ok = t < args.T;
      const int N = args.N;
      const size_t plane = (size_t)args.T * N;
#pragma unroll 1
      for (int c0 = half * 16; c0 < FEATS; c0 += 32) {  // the quarter's two warps take the runs of 16 columns in turn
        const int f = f0 + c0;
        if (f >= N) break;
        uint32_t r0[16], r1[16];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        tmem_ld16(taddr, r0);
        if (GATED) tmem_ld16(taddr + FEATS, r1);
        tmem_ld_wait();
        if (!t_ok) continue;
        float v[16], u[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          v[j] = __uint_as_float(r0[j]);
          u[j] = GATED ? __uint_as_float(r1[j]) : 0.f;
        }
        const bool whole = f + 16 <= N;
        if (split) {
          float* p = args.partial + (size_t)blockIdx.z * (GATED ? 2 : 1) * plane + (size_t)t * N + f;
          if (whole && (N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
              *reinterpret_cast<float4*>(p + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              if (GATED) *reinterpret_cast<float4*>(p + plane + j) = make_float4(u[j], u[j + 1], u[j + 2], u[j + 3]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (f + j < N) {
                p[j] = v[j];
                if (GATED) p[plane + j] = u[j];
              }
          }
          continue;
        }
        if (args.bias) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (f + j < N) {
              v[j] += args.bias[f + j];
              if (GATED) u[j] += args.bias[N + f + j];
            }
        }
        if (GATED) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = silu_times(v[j], u[j]);
        }
        if (EPI == EPI_RESIDUAL) {
          float* o = (float*)args.out + (size_t)t * N + f;
          if (whole && (N & 3) == 0) {
            float4 prev[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) prev[j] = reinterpret_cast<float4*>(o)[j];
#pragma unroll
            for (int j = 0; j < 4; ++j)
              reinterpret_cast<float4*>(o)[j] = make_float4(prev[j].x + v[4 * j], prev[j].y + v[4 * j + 1], prev[j].z + v[4 * j + 2], prev[j].w + v[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (f + j < N) o[j] += v[j];
          }
        } else if (args.out_bf16) {
          bf16* o = (bf16*)args.out + (size_t)t * N + f;
          if (whole && (N & 7) == 0) {
            uint32_t packed[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
              packed[j] = *reinterpret_cast<uint32_t*>(&h2);
            }
            reinterpret_cast<uint4*>(o)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            reinterpret_cast<uint4*>(o)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (f + j < N) o[j] = __float2bfloat16_rn(v[j]);
          }
        } else {
          float* o = (float*)args.out + (size_t)t * N + f;
          if (whole && (N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (f + j < N) o[j] = v[j];
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag && args.status) atomicExch(args.status, 2);
}

// ---------------------------------------------------------------------------
// The same, persistent: one CTA per SM works through the tiles of a wide
// product (tile = 128 tokens x 256 weight rows; width a multiple of 4, depth
// unsplit).  The ring of stages runs on across tiles, and the accumulator has
// two homes in tensor memory that the MMA warp fills in turn, so the epilogue
// of one tile (tensor memory -> registers -> shared memory -> global) runs
// beside the MMAs of the next.  Tiles are taken feature-tile first, so CTAs
// that run side by side read the same tokens and neighbouring weights.
// ---------------------------------------------------------------------------
constexpr int STAGING_BYTES = 4 * 32 * 132 * 4;  // the epilogue's padded rows
// ROWS (32 or 64 instead of 128: an output head in a decode step of up to that many tokens): only
// ROWS rows of the token tile are fetched - the MMA reads 128, the rest from whatever follows in
// shared memory, and their accumulator rows are never read - and only ROWS / 32 quarters of the
// epilogue have rows, so a stage is 36 or 40 KB instead of 48 and the ring five or four deep
// instead of three: more weight bytes in flight per SM.
template <int ROWS>
struct PersistentRing {
  static constexpr int STAGES = ROWS == 32 ? 5 : ROWS == 64 ? 4 : 3;
  static constexpr uint32_t A_BYTES = ROWS * BK * 2;
  static constexpr uint32_t STAGING = STAGING_BYTES / 128 * ROWS;
};

template <int EPI, int ROWS>
__global__ void __launch_bounds__(TOKENS_THREADS, 1)
gemm_tc_tokens_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmArgs args) {
  constexpr int BNF = 256;
  constexpr bool GATED = EPI == EPI_GATED;
  constexpr int FEATS = GATED ? BNF / 2 : BNF;
  constexpr int PERSISTENT_STAGES = PersistentRing<ROWS>::STAGES;
  constexpr uint32_t A_BYTES = PersistentRing<ROWS>::A_BYTES;
  constexpr uint32_t B_BYTES = BNF * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BNF >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* staging = reinterpret_cast<float*>(tiles + (size_t)PERSISTENT_STAGES * STAGE_BYTES);
  __shared__ uint64_t full_bar[PERSISTENT_STAGES], empty_bar[PERSISTENT_STAGES], acc_full[2], acc_free[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_ftiles = (args.N + FEATS - 1) / FEATS, n_ttiles = (args.T + 127) / 128;
  const int n_tiles = n_ftiles * n_ttiles;
  const int n_slices = (args.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < PERSISTENT_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_free[b], 8);  // the epilogue warps
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) tmem_alloc(&tmem_base_smem, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  auto load_weights = [&](int it, int i, int f0) {  // the weight tile of slice i of a tile into the stage of ring position it
    const int s = it % PERSISTENT_STAGES;
    uint8_t* stage = tiles + (size_t)s * STAGE_BYTES;
    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
    if (GATED) {
      tma_load_2d(stage + A_BYTES, &map_w, &full_bar[s], i * BK, f0);
      tma_load_2d(stage + A_BYTES + B_BYTES / 2, &map_w, &full_bar[s], i * BK, args.N + f0);
    } else {
      tma_load_2d(stage + A_BYTES, &map_w, &full_bar[s], i * BK, f0);
    }
  };
  // the weights depend on no earlier kernel: those of the first tile's first ring go ahead of the wait
  int early_slices = 0;
  if (threadIdx.x == 0) {
    asm volatile("griddepcontrol.launch_dependents;");
    if ((int)blockIdx.x < n_tiles) {
      early_slices = min(PERSISTENT_STAGES, n_slices);
      for (int i = 0; i < early_slices; ++i) load_weights(i, i, ((int)blockIdx.x % n_ftiles) * FEATS);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
  } else {
    pdl_begin();
  }

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;  // slices asked for so far, over all tiles
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int f0 = (tile % n_ftiles) * FEATS, t0 = (tile / n_ftiles) * 128;
        for (int i = 0; i < n_slices; ++i, ++it) {
          const int s = it % PERSISTENT_STAGES;
          if (it >= PERSISTENT_STAGES && !mbar_wait(&empty_bar[s], ((it / PERSISTENT_STAGES) - 1) & 1, &abort_flag)) break;
          if (it >= early_slices) load_weights(it, i, f0);
          tma_load_2d(tiles + (size_t)s * STAGE_BYTES, &map_x, &full_bar[s], i * BK, t0);
        }
        if (abort_flag) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, j = 0;  // slices consumed; tiles of this CTA so far
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++j) {
        const int buf = j & 1;
        if (j >= 2) ok = mbar_wait(&acc_free[buf], ((j >> 1) - 1) & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int i = 0; i < n_slices; ++i, ++it) {
          const int s = it % PERSISTENT_STAGES;
          ok = mbar_wait(&full_bar[s], (it / PERSISTENT_STAGES) & 1, &abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t stage = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t desc_a = smem_desc_sw128(stage), desc_b = smem_desc_sw128(stage + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_base + buf * BNF, desc_a + (uint64_t)(k * 2), desc_b + (uint64_t)(k * 2), IDESC, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    int j = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++j) {
      const int buf = j & 1;
      const int f0 = (tile % n_ftiles) * FEATS, t0 = (tile / n_ftiles) * 128;
      bool ok = mbar_wait(&acc_full[buf], (j >> 1) & 1, &abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!epilogue_warps_agree(ok)) break;
      tc_fence_after();
      if (t0 + q * 32 < args.T) {
        tokens_epilogue_staged<BNF, EPI>(args, tmem_base + buf * BNF, staging, q, half, lane, f0, t0, 1, 0, &acc_free[buf]);
      } else {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_free[buf]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && abort_flag && args.status) atomicExch(args.status, 2);
}

// ---------------------------------------------------------------------------
// The same, on pairs of CTAs (a cluster of two, one CTA per SM): a pair works
// through tiles of 256 tokens x 256 weight rows with MMAs of M = 256 that the
// first CTA issues for both.  Each CTA fetches its own 128 tokens and its own
// half of the weight rows (for EPI_GATED the first CTA the gate rows, the
// second the matching up rows), 32 KB per k-slice where the single CTA fetches
// 48 KB for the same MMA time: the product is no longer bound by what an SM can
// pull out of L2, and the ring is four stages deep.  The first CTA's full
// barrier counts the bytes of both CTAs' copies; the MMAs' completion is
// signalled on the barriers of both; both CTAs' epilogue warps free an
// accumulator on the first CTA's barrier.
// ---------------------------------------------------------------------------
constexpr int PAIR_STAGES = 4;

template <int EPI>
__global__ void __launch_bounds__(TOKENS_THREADS, 1)
gemm_tc_tokens_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmArgs args) {
  constexpr int BNF = 256;
  constexpr bool GATED = EPI == EPI_GATED;
  constexpr int FEATS = GATED ? BNF / 2 : BNF;
  constexpr uint32_t A_BYTES = 128 * BK * 2;
  constexpr uint32_t B_BYTES = (BNF / 2) * BK * 2;  // this CTA's half of the weight rows
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BNF >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* staging = reinterpret_cast<float*>(tiles + (size_t)PAIR_STAGES * STAGE_BYTES);
  __shared__ uint64_t full_bar[PAIR_STAGES], empty_bar[PAIR_STAGES], acc_full[2], acc_free[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool first = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int n_ftiles = (args.N + FEATS - 1) / FEATS, n_ttiles = (args.T + 255) / 256;
  const int n_tiles = n_ftiles * n_ttiles;
  const int n_slices = (args.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_free[b], 16);  // the epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) tmem_alloc_pair(&tmem_base_smem, 512);
  tc_fence_before();
  cluster_sync_all();  // both CTAs' barriers stand before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  // this CTA's weight rows of a tile that starts at feature f0
  auto weight_row = [&](int f0) { return GATED ? (first ? f0 : args.N + f0) : f0 + (int)rank * (BNF / 2); };
  auto load_weights = [&](int it, int i, int f0) {  // the weight tile of slice i of a tile into the stage of ring position it
    const int s = it % PAIR_STAGES;
    if (first) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
    tma_load_2d_pair(tiles + (size_t)s * STAGE_BYTES + A_BYTES, &map_w, in_cluster_cta(&full_bar[s], 0), i * BK, weight_row(f0));
  };
  // the weights depend on no earlier kernel: those of the first tile's first ring go ahead of the wait
  int early_slices = 0;
  if (threadIdx.x == 0) {
    asm volatile("griddepcontrol.launch_dependents;");
    if (pair < n_tiles) {
      early_slices = min(PAIR_STAGES, n_slices);
      for (int i = 0; i < early_slices; ++i) load_weights(i, i, (pair % n_ftiles) * FEATS);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
  } else {
    pdl_begin();
  }

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;  // slices asked for so far, over all tiles
      for (int tile = pair; tile < n_tiles; tile += n_pairs) {
        const int f0 = (tile % n_ftiles) * FEATS, t0 = (tile / n_ftiles) * 256 + (int)rank * 128;
        for (int i = 0; i < n_slices; ++i, ++it) {
          const int s = it % PAIR_STAGES;
          if (it >= PAIR_STAGES && !mbar_wait(&empty_bar[s], ((it / PAIR_STAGES) - 1) & 1, &abort_flag)) break;
          if (it >= early_slices) load_weights(it, i, f0);
          tma_load_2d_pair(tiles + (size_t)s * STAGE_BYTES, &map_x, in_cluster_cta(&full_bar[s], 0), i * BK, t0);
        }
        if (abort_flag) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && first) {
      int it = 0, j = 0;  // slices consumed; tiles of this pair so far
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++j) {
        const int buf = j & 1;
        if (j >= 2) ok = mbar_wait(&acc_free[buf], ((j >> 1) - 1) & 1, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int i = 0; i < n_slices; ++i, ++it) {
          const int s = it % PAIR_STAGES;
          ok = mbar_wait(&full_bar[s], (it / PAIR_STAGES) & 1, &abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t stage = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t desc_a = smem_desc_sw128(stage), desc_b = smem_desc_sw128(stage + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_pair(tmem_base + buf * BNF, desc_a + (uint64_t)(k * 2), desc_b + (uint64_t)(k * 2), IDESC, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[s], 3);
        }
        if (ok) umma_commit_pair(&acc_full[buf], 3);
      }
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    int j = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++j) {
      const int buf = j & 1;
      const int f0 = (tile % n_ftiles) * FEATS, t0 = (tile / n_ftiles) * 256 + (int)rank * 128;
      bool ok = mbar_wait(&acc_full[buf], (j >> 1) & 1, &abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!epilogue_warps_agree(ok)) break;
      tc_fence_after();
      const uint32_t free_bar = in_cluster_cta(&acc_free[buf], 0);
      if (t0 + q * 32 < args.T) {
        tokens_epilogue_staged<BNF, EPI>(args, tmem_base + buf * BNF, staging, q, half, lane, f0, t0, 1, 0, nullptr, free_bar);
      } else {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_in_cluster(free_bar);
      }
    }
  }
  tc_fence_before();
  cluster_sync_all();  // neither CTA leaves, or frees tensor memory, while the other may still signal or read it
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
  if (threadIdx.x == 0 && abort_flag && args.status) atomicExch(args.status, 2);
}

// ---------------------------------------------------------------------------
// Second stage of split-K: add the partial sums in split order, then the
// epilogue.  partial [splits, n_acc, T, N].
// ---------------------------------------------------------------------------
template <int EPI>
__global__ void splitk_reduce_kernel(void* __restrict__ out, const float* __restrict__ partial, const float* __restrict__ bias, int T, int N,
                                     int splits, int out_bf16) {
  constexpr int N_ACC = (EPI == EPI_GATED) ? 2 : 1;
  const size_t plane = (size_t)T * N;
  pdl_begin();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= plane) return;
  const int f = (int)(idx % N);
  float a0 = 0.f, a1 = 0.f;
  for (int z0 = 0; z0 < splits; z0 += 8) {  // eight splits in flight, added in split order
    float x0[8], x1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool ok = z0 + i < splits;
      x0[i] = ok ? partial[(size_t)(z0 + i) * N_ACC * plane + idx] : 0.f;
      x1[i] = (ok && N_ACC == 2) ? partial[(size_t)(z0 + i) * N_ACC * plane + plane + idx] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a0 += x0[i];
      a1 += x1[i];
    }
  }
  if (bias) {
    a0 += bias[f];
    if (N_ACC == 2) a1 += bias[N + f];
  }
  float y = a0;
  if (EPI == EPI_GATED) y = silu_times(a0, a1);
  if (EPI == EPI_RESIDUAL) {
    ((float*)out)[idx] += y;
  } else if (out_bf16) {
    ((bf16*)out)[idx] = __float2bfloat16_rn(y);
  } else {
    ((float*)out)[idx] = y;
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// A [rows, K] bf16 row-major matrix seen as boxes of [box_rows, 64] with 128-byte swizzle.
static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  return make_tensor_map_bf16(map, base, rows, K, box_rows, BK);
}

template <int BN, int EPI>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& args, int splits, cudaStream_t stream) {
  constexpr int N_ACC = (EPI == EPI_GATED) ? 2 : 1;
  constexpr size_t STAGE = (size_t)N_ACC * BM * BK * 2 + (size_t)BN * BK * 2;
  constexpr size_t XCHG = (EPI == EPI_ROPE) ? 16 * 128 * sizeof(float) : 0;  // where rotation partners swap values
  int stages = (int)((200 * 1024 - XCHG) / STAGE);
  if (stages > 12) stages = 12;
  if (stages < 2) return ALOFA_ERR_ARGUMENT;
  // (The ring is not cut down to the k-slices a CTA has: with a small footprint the next kernel's
  // CTAs become resident beside this kernel's and their weight fetches take bandwidth from it;
  // measured 1.03 ms against 0.95 ms per decode step at batch 8.)
  const size_t smem = STAGE * stages + XCHG + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048) != cudaSuccess)
      return ALOFA_ERR_LAUNCH;
    prefer_max_shared(gemm_tc_kernel<BN, EPI>);
    prefer_max_shared(splitk_reduce_kernel<EPI>);
    configured = true;
  }
  dim3 grid((args.N + BM - 1) / BM, (args.T + BN - 1) / BN, splits);
  if (args.b_kind == B_MERGED_SPLITS) {
    if constexpr (BN == 16 && EPI == EPI_RESIDUAL) {
      static bool configured_c = false;
      if (!configured_c) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, MODE_COMPUTED>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048) != cudaSuccess)
          return ALOFA_ERR_LAUNCH;
        prefer_max_shared(gemm_tc_kernel<BN, EPI, MODE_COMPUTED>);
        configured_c = true;
      }
      launch_dep(gemm_tc_kernel<BN, EPI, MODE_COMPUTED>, grid, NUM_THREADS, smem, stream, mw, mx, args, stages);
      return launch_status();
    } else {
      return ALOFA_ERR_ARGUMENT;  // a computed operand feeds residual products of up to 16 tokens
    }
  }
  if (args.cluster || args.b_kind == B_NORMED) {
    if constexpr (((BN == 16 || BN == 32) && EPI == EPI_GATED) || (BN == 16 && EPI == EPI_ROPE)) {
      const bool normed = args.b_kind == B_NORMED;
      if (normed && (BN != 16 || grid.y != 1 || splits > 8)) return ALOFA_ERR_ARGUMENT;
      // room behind the ring for the accumulators the other CTAs of a cluster push, and the rows' sums of squares
      const size_t pushed = (size_t)(splits - 1) * N_ACC * BN * 128 * sizeof(float) + XCHG + (normed ? 9 * 16 * sizeof(float) : 0);
      int cstages = (int)((200 * 1024 - pushed) / STAGE);
      if (cstages > 12) cstages = 12;
      if (cstages < 2) return ALOFA_ERR_ARGUMENT;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(NUM_THREADS);
      cfg.dynamicSmemBytes = STAGE * cstages + pushed + 1024;
      cfg.stream = stream;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
      attr[1].id = cudaLaunchAttributeClusterDimension;
      attr[1].val.clusterDim.x = 1;
      attr[1].val.clusterDim.y = 1;
      attr[1].val.clusterDim.z = (unsigned)splits;
      cfg.attrs = attr;
      cfg.numAttrs = 2;
      if (normed) {
        if constexpr (BN == 16) {
          static bool configured_n = false;
          if (!configured_n) {
            if (cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, MODE_NORMED>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048) != cudaSuccess)
              return ALOFA_ERR_LAUNCH;
            prefer_max_shared(gemm_tc_kernel<BN, EPI, MODE_NORMED>);
            configured_n = true;
          }
          cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, EPI, MODE_NORMED>, mw, mx, args, cstages);
        }
        return launch_status();
      }
      static bool configured_k = false;
      if (!configured_k) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, MODE_CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048) != cudaSuccess)
          return ALOFA_ERR_LAUNCH;
        prefer_max_shared(gemm_tc_kernel<BN, EPI, MODE_CLUSTER>);
        configured_k = true;
      }
      cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, EPI, MODE_CLUSTER>, mw, mx, args, cstages);
      return launch_status();
    } else {
      return ALOFA_ERR_ARGUMENT;
    }
  }
  launch_dep(gemm_tc_kernel<BN, EPI>, grid, NUM_THREADS, smem, stream, mw, mx, args, stages);
  return launch_status();
}

// Whether a tokens-on-M product runs on pairs of CTAs: a wide product over at least two token
// tiles with more tiles than SMs, and deep (ALOFA_GEMM_PAIR=0 keeps one CTA per tile).  Measured
// on 2,048 tokens: depth 3,584 x 37,888 weight rows 477 against 540 us, 18,944 x 3,584 233 against
// 238 us, depth 1,536 x 17,920 rows 85 against 92 us; at depth 896 the pair's epilogue is not
// hidden behind its shorter MMA phase and one CTA per tile is as fast or faster (32.7 against
// 33.9 us for 9,728 weight rows), so shallow products stay there.
constexpr int PAIR_MIN_DEPTH = 1024;
static bool pair_product(int bnf, int splits, int T, int N, int K, int epi) {
  static int sms = 0, allowed = -1;
  if (allowed < 0) {
    const char* env = getenv("ALOFA_GEMM_PAIR");
    allowed = (env && env[0] == '0') ? 0 : 1;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 0;
  }
  if (!allowed || sms < 2 || bnf != 256 || splits != 1 || (N & 3) || T <= 128 || K < PAIR_MIN_DEPTH) return false;
  const int feats = epi == EPI_GATED ? 128 : 256;
  return (long long)((N + feats - 1) / feats) * ((T + 127) / 128) > sms;
}

template <int EPI, int ROWS>
static int launch_persistent(int sms, const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& args, cudaStream_t stream) {
  static bool configured = false;
  constexpr size_t SMEM = (size_t)PersistentRing<ROWS>::STAGES * (PersistentRing<ROWS>::A_BYTES + (size_t)256 * BK * 2) + PersistentRing<ROWS>::STAGING + 1024;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_tokens_persistent_kernel<EPI, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return ALOFA_ERR_LAUNCH;
    prefer_max_shared(gemm_tc_tokens_persistent_kernel<EPI, ROWS>);
    configured = true;
  }
  launch_dep(gemm_tc_tokens_persistent_kernel<EPI, ROWS>, dim3(sms), TOKENS_THREADS, SMEM, stream, mw, mx, args);
  return launch_status();
}

// How many token rows (32 or 64) the persistent kernel's few-token form fetches for a tokens-on-M
// product of up to 64 tokens, 0 when the product does not run on it
// (the same conditions as launch_tokens has for the persistent kernel; ALOFA_GEMM_PERSISTENT=0
// turns both off).
static int few_tokens_product(int bnf, int splits, int T, int N, int K, int epi) {
  static int sms = 0, allowed = -1;
  if (allowed < 0) {
    const char* env = getenv("ALOFA_GEMM_PERSISTENT");
    allowed = (env && env[0] == '0') ? 0 : 1;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 0;
  }
  if (!allowed || sms <= 0 || bnf != 256 || splits != 1 || (N & 3) || K > 2048 || T > 64) return 0;
  const int feats = epi == EPI_GATED ? 128 : 256;
  if ((N + feats - 1) / feats <= sms) return 0;  // one token tile: the feature tiles alone must be more than the SMs
  return T <= 32 ? 32 : 64;
}

template <int BNF, int EPI>
static int launch_tokens(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& args, int splits, cudaStream_t stream) {
  constexpr size_t STAGE = (size_t)128 * BK * 2 + (size_t)BNF * BK * 2;
  constexpr int FEATS = (EPI == EPI_GATED) ? BNF / 2 : BNF;
  // Many token tiles: two CTAs share an SM (shared memory and the 512
  // tensor-memory columns allow it), so that while one runs its epilogue the
  // other keeps the tensor cores busy.  One token tile (decode): the CTAs are
  // few and each streams its weights once, so the ring is made as deep as
  // shared memory allows to keep many loads in flight.
  static int sm_count = 0;
  if (!sm_count) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sm_count = 1;
  }
  dim3 grid((args.N + FEATS - 1) / FEATS, (args.T + 127) / 128, splits);
  // A grid that does not fill the GPU once (the narrow q/k/v and output products of a prompt portion) has an SM
  // to each CTA anyway: the deep ring then, or the CTA waits on the latency of three stages in flight.
  const bool one_wave = (long long)grid.x * grid.y * grid.z <= sm_count;
  const size_t budget = (args.T > 128 && !one_wave) ? 108 * 1024 : 200 * 1024;
  int stages = (int)(budget / STAGE);
  if (stages > 12) stages = 12;
  if (stages < 2) stages = 2;
  const size_t smem = STAGE * stages + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_tokens_kernel<BNF, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048) != cudaSuccess)
      return ALOFA_ERR_LAUNCH;
    prefer_max_shared(gemm_tc_tokens_kernel<BNF, EPI>);
    configured = true;
  }
  if (BNF == 256 && splits == 1 && (args.N & 3) == 0 && (args.K <= 2048 || args.pair)) {
    // More tiles than SMs and a shallow depth, where a tile's epilogue is a large share of its
    // time: one resident CTA per SM works through the tiles, epilogues beside MMAs.  (Deep
    // products measured faster as two CTAs per SM, which keep four stages in flight per SM.)
    static int sms = 0, persistent = -1;
    if (persistent < 0) {
      const char* env = getenv("ALOFA_GEMM_PERSISTENT");
      persistent = (env && env[0] == '0') ? 0 : 1;
      int device = 0;
      if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sms = 0;
    }
    const int n_tiles = (int)(grid.x * grid.y);
    if (args.pair) {
      static bool configured_2 = false;
      constexpr size_t SMEM_2 = (size_t)PAIR_STAGES * ((size_t)128 * BK * 2 + (size_t)128 * BK * 2) + STAGING_BYTES + 1024;
      if (!configured_2) {
        if (cudaFuncSetAttribute(gemm_tc_tokens_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_2) != cudaSuccess)
          return ALOFA_ERR_LAUNCH;
        prefer_max_shared(gemm_tc_tokens_pair_kernel<EPI>);
        configured_2 = true;
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(sms / 2 * 2);
      cfg.blockDim = dim3(TOKENS_THREADS);
      cfg.dynamicSmemBytes = SMEM_2;
      cfg.stream = stream;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
      attr[1].id = cudaLaunchAttributeClusterDimension;
      attr[1].val.clusterDim.x = 2;
      attr[1].val.clusterDim.y = 1;
      attr[1].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 2;
      cudaLaunchKernelEx(&cfg, gemm_tc_tokens_pair_kernel<EPI>, mw, mx, args);
      return launch_status();
    }
    if (persistent && sms > 0 && n_tiles > sms && args.few == 32) return launch_persistent<EPI, 32>(sms, mw, mx, args, stream);
    if (persistent && sms > 0 && n_tiles > sms && args.few == 64) return launch_persistent<EPI, 64>(sms, mw, mx, args, stream);
    if (persistent && sms > 0 && n_tiles > sms) return launch_persistent<EPI, 128>(sms, mw, mx, args, stream);
  }
  if (args.few || args.pair) return ALOFA_ERR_ARGUMENT;  // their maps have other boxes than this kernel's
  launch_dep(gemm_tc_tokens_kernel<BNF, EPI>, grid, TOKENS_THREADS, smem, stream, mw, mx, args, stages);
  return launch_status();
}

template <int EPI>
static int dispatch_tokens(int bnf, const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& args, int splits, cudaStream_t stream) {
  switch (bnf) {
    case 64: return launch_tokens<64, EPI>(mw, mx, args, splits, stream);
    case 128: return launch_tokens<128, EPI>(mw, mx, args, splits, stream);
    case 256: return launch_tokens<256, EPI>(mw, mx, args, splits, stream);
    default: return ALOFA_ERR_ARGUMENT;
  }
}

template <int EPI>
static int dispatch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& args, int splits, cudaStream_t stream) {
  switch (bn) {
    case 16: return launch_tc<16, EPI>(mw, mx, args, splits, stream);
    case 32: return launch_tc<32, EPI>(mw, mx, args, splits, stream);
    case 64: return launch_tc<64, EPI>(mw, mx, args, splits, stream);
    case 128: return launch_tc<128, EPI>(mw, mx, args, splits, stream);
    case 256: return launch_tc<256, EPI>(mw, mx, args, splits, stream);
    default: return ALOFA_ERR_ARGUMENT;
  }
}

// out = x W^T with the epilogue `epi`.  x [T, K] bf16, w [N (GATED: 2N), K] bf16.
// bn: tokens per CTA (16..256).  splits > 1 needs `partial` of
// splits * (GATED ? 2 : 1) * T * N floats and, when do_reduce is set, runs the
// reduce kernel after (else the caller's next kernel adds the partials up).
// Returns ALOFA_ERR_ARGUMENT for sizes this kernel does not take (K % 8 != 0,
// pointers not 16-byte aligned).
// Whether a product with these settings adds its split sums up inside a thread-block cluster
// (no partial sums in global memory, no second kernel): gated products of up to 16 tokens
// split two to eight ways, of up to 32 tokens split two to four ways (the pushed sums must fit
// in shared memory beside the ring).
ALOFA_API int alofa_gemm_tc_reduces_in_cluster(int epi, int bn, int splits) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* env = getenv("ALOFA_GEMM_CLUSTER");
    enabled = (env && env[0] == '0') ? 0 : 1;
  }
  return enabled && epi == EPI_GATED && (bn == 16 || (bn == 32 && splits <= 4)) && splits >= 2 && splits <= 8;
}

// b_kind = B_MERGED_SPLITS (residual products of up to 16 tokens only): x is ignored and the
// token operand is computed in the kernel from the attention output of decode tokens still in
// key splits (b_src partial outputs, b_ml maxima and sums, b_positions; heads * head_dim == K).
// acc (EPI_RESIDUAL, weights on M): the product's sums go into this fixed-point accumulator
// [T, N] with atomic adds instead of into `out` or `partial` (see GemmArgs::acc).
// b_kind = B_NORMED (gated products of up to 16 tokens, split up to 8 ways over a cluster): the token
// operand is RMSNorm(b_src + n_acc) with weight n_gamma, made in the kernel; b_src + n_acc is also
// written to n_out and n_zero is zeroed (GemmArgs::n_*).
ALOFA_API int alofa_gemm_tc(void* out, const void* x, const void* w, const float* bias, float* partial, int T, int N, int K, int epi, int out_bf16,
                            int bn, int splits, int do_reduce, int* status, int b_kind, const float* b_src, const float* b_ml,
                            const int* b_positions, int b_heads, int b_head_dim, int b_window, int b_split_keys, long long* acc,
                            const long long* n_acc, const float* n_gamma, float n_eps, float* n_out, long long* n_zero, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return ALOFA_OK;
  if (acc && (epi != EPI_RESIDUAL || bn <= 0)) return ALOFA_ERR_ARGUMENT;
  if (b_kind == B_NORMED) {
    if (bn != 16 || T > 16 || epi != EPI_GATED || !b_src || !n_gamma || !n_out || n_out == b_src || (K % 8) != 0 || !do_reduce) return ALOFA_ERR_ARGUMENT;
    if (((uintptr_t)b_src & 15) || ((uintptr_t)n_gamma & 15) || ((uintptr_t)n_out & 15) || ((uintptr_t)n_acc & 15) || ((uintptr_t)n_zero & 15)) return ALOFA_ERR_ARGUMENT;
    if (splits > 8) splits = 8;
    x = w;  // any mapped address: the map of x is made but never used
  } else if (b_kind != B_ROWS) {
    if (bn <= 0 || !b_src || ((uintptr_t)b_src & 15) || (K % 8) != 0) return ALOFA_ERR_ARGUMENT;
    if (b_kind != B_MERGED_SPLITS || !b_ml || !b_positions || b_heads * b_head_dim != K || b_head_dim % 8 || b_split_keys <= 0) return ALOFA_ERR_ARGUMENT;
    if (bn != 16 || epi != EPI_RESIDUAL) return ALOFA_ERR_ARGUMENT;  // one 16-byte chunk of a k-slice per epilogue thread
    x = w;  // any mapped address: the map of x is made but never used
  }
  if (K <= 0 || (K % 8) != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return ALOFA_ERR_ARGUMENT;
  if (epi == EPI_RESIDUAL && out_bf16) return ALOFA_ERR_ARGUMENT;
  const int total_slices = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > total_slices) splits = total_slices;
  if (splits > 1 && !partial && !acc && b_kind != B_NORMED) return ALOFA_ERR_ARGUMENT;
  const int w_rows = (epi == EPI_GATED) ? 2 * N : N;
  // bn > 0: weights on the M side, bn tokens per CTA.  bn < 0: tokens on the M
  // side (128 per CTA), -bn weight rows per MMA (for GATED half gate, half up).
  const bool tokens_on_m = bn < 0;
  const int bnf = -bn;
  CUtensorMap mw, mx;
  const bool pair = tokens_on_m && pair_product(bnf, splits, T, N, K, epi);
  const int few = (tokens_on_m && !pair) ? few_tokens_product(bnf, splits, T, N, K, epi) : 0;
  if (tokens_on_m) {
    const int w_box = (epi == EPI_GATED || pair) ? bnf / 2 : bnf;
    if (!make_map(&mw, w, w_rows, K, w_box) || !make_map(&mx, x, T, K, few ? few : 128)) return ALOFA_ERR_ARGUMENT;
  } else if (!make_map(&mw, w, w_rows, K, BM) || !make_map(&mx, x, T, K, bn)) {
    return ALOFA_ERR_ARGUMENT;
  }
  GemmArgs args;
  memset(&args, 0, sizeof(args));
  args.out = out;
  args.partial = partial;
  args.bias = bias;
  args.T = T;
  args.N = N;
  args.K = K;
  args.k_slices_per_split = (total_slices + splits - 1) / splits;
  splits = (total_slices + args.k_slices_per_split - 1) / args.k_slices_per_split;  // no empty split
  args.out_bf16 = out_bf16;
  args.pair = pair ? 1 : 0;
  args.few = few;
  args.status = status;
  args.b_kind = b_kind;
  args.b_src = b_src;
  args.b_ml = b_ml;
  args.b_positions = b_positions;
  args.b_heads = b_heads;
  args.b_head_dim = b_head_dim;
  args.b_window = b_window;
  args.b_split_keys = b_split_keys;
  args.cluster = (alofa_gemm_tc_reduces_in_cluster(epi, bn, splits) && do_reduce && b_kind == B_ROWS) || b_kind == B_NORMED;
  args.acc = acc;
  args.n_base = b_kind == B_NORMED ? b_src : nullptr;
  args.n_acc = n_acc;
  args.n_gamma = n_gamma;
  args.n_eps = n_eps;
  args.n_out = n_out;
  args.n_zero = n_zero;
  int rc;
  if (tokens_on_m) {
    if (epi == EPI_STORE) rc = dispatch_tokens<EPI_STORE>(bnf, mw, mx, args, splits, stream);
    else if (epi == EPI_RESIDUAL) rc = dispatch_tokens<EPI_RESIDUAL>(bnf, mw, mx, args, splits, stream);
    else if (epi == EPI_GATED) rc = dispatch_tokens<EPI_GATED>(bnf, mw, mx, args, splits, stream);
    else return ALOFA_ERR_ARGUMENT;
  } else if (epi == EPI_STORE) rc = dispatch_bn<EPI_STORE>(bn, mw, mx, args, splits, stream);
  else if (epi == EPI_RESIDUAL) rc = dispatch_bn<EPI_RESIDUAL>(bn, mw, mx, args, splits, stream);
  else if (epi == EPI_GATED) rc = dispatch_bn<EPI_GATED>(bn, mw, mx, args, splits, stream);
  else return ALOFA_ERR_ARGUMENT;
  if (rc != ALOFA_OK || splits == 1 || !do_reduce || args.cluster || acc) return rc;
  const size_t plane = (size_t)T * N;
  const int threads = 256;
  const unsigned blocks = (unsigned)((plane + threads - 1) / threads);
  if (epi == EPI_STORE) launch_dep(splitk_reduce_kernel<EPI_STORE>, blocks, threads, 0, stream, out, partial, bias, T, N, splits, out_bf16);
  else if (epi == EPI_RESIDUAL) launch_dep(splitk_reduce_kernel<EPI_RESIDUAL>, blocks, threads, 0, stream, out, partial, bias, T, N, splits, out_bf16);
  else launch_dep(splitk_reduce_kernel<EPI_GATED>, blocks, threads, 0, stream, out, partial, bias, T, N, splits, out_bf16);
  return launch_status();
}

// The second stage alone: out (op)= bias + sum_z partial[z], for partial sums a
// deferred product left behind.
ALOFA_API int alofa_splitk_reduce(void* out, const float* partial, const float* bias, int T, int N, int splits, int epi, int out_bf16,
                                  cudaStream_t stream) {
  if (T <= 0 || N <= 0) return ALOFA_OK;
  if (epi == EPI_RESIDUAL && out_bf16) return ALOFA_ERR_ARGUMENT;
  const size_t plane = (size_t)T * N;
  const int threads = 256;
  const unsigned blocks = (unsigned)((plane + threads - 1) / threads);
  if (epi == EPI_STORE) launch_dep(splitk_reduce_kernel<EPI_STORE>, blocks, threads, 0, stream, out, partial, bias, T, N, splits, out_bf16);
  else if (epi == EPI_RESIDUAL) launch_dep(splitk_reduce_kernel<EPI_RESIDUAL>, blocks, threads, 0, stream, out, partial, bias, T, N, splits, out_bf16);
  else if (epi == EPI_GATED) launch_dep(splitk_reduce_kernel<EPI_GATED>, blocks, threads, 0, stream, out, partial, bias, T, N, splits, out_bf16);
  else return ALOFA_ERR_ARGUMENT;
  return launch_status();
}

// q/k/v of up to 16 tokens in one kernel: x [T, K] bf16 times the stacked weight w
// [(heads + 2 kv_heads) * head_dim, K] (heads * head_dim rows when the layer reads another
// layer's cache: kv_heads = 0), bias, NeoX rotation of q and k by `table`
// [positions, head_dim / 2, 2] at `positions`, q to q_out [T, heads * head_dim], k and v to
// their cache slots.  The depth is split over a cluster of up to 8 CTAs that add their sums up
// themselves.  head_dim must divide 128 (a tile of 128 weight rows then holds whole heads).
// With n_base the token operand is not x but RMSNorm(n_base + n_acc) with weight n_gamma, made in
// the kernel (B_NORMED); n_base + n_acc is written to n_out and n_zero is zeroed.
ALOFA_API int alofa_gemm_tc_rope(const void* x, const void* w, const float* bias, int T, int K, void* q_out, void* k_cache, void* v_cache,
                                 const int* slots, const int* positions, const float* table, int heads, int kv_heads, int head_dim,
                                 int splits, int* status, const float* n_base, const long long* n_acc, const float* n_gamma, float n_eps,
                                 float* n_out, long long* n_zero, cudaStream_t stream) {
  if (T <= 0) return ALOFA_OK;
  if (n_base) {
    if (!n_gamma || !n_out || n_out == n_base) return ALOFA_ERR_ARGUMENT;
    if (((uintptr_t)n_base & 15) || ((uintptr_t)n_gamma & 15) || ((uintptr_t)n_out & 15) || ((uintptr_t)n_acc & 15) || ((uintptr_t)n_zero & 15)) return ALOFA_ERR_ARGUMENT;
    x = w;  // the map of x is made but never used
  }
  const int N = (heads + 2 * kv_heads) * head_dim;
  if (T > 16 || K <= 0 || (K % 8) != 0 || head_dim <= 0 || 128 % head_dim || head_dim % 2 || heads <= 0) return ALOFA_ERR_ARGUMENT;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || !q_out || !positions || !table || (kv_heads > 0 && (!k_cache || !v_cache || !slots))) return ALOFA_ERR_ARGUMENT;
  const int total_slices = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > 8) splits = 8;
  if (splits > total_slices) splits = total_slices;
  CUtensorMap mw, mx;
  if (!make_map(&mw, w, N, K, BM) || !make_map(&mx, x, T, K, 16)) return ALOFA_ERR_ARGUMENT;
  GemmArgs args;
  memset(&args, 0, sizeof(args));
  args.bias = bias;
  args.T = T;
  args.N = N;
  args.K = K;
  args.k_slices_per_split = (total_slices + splits - 1) / splits;
  splits = (total_slices + args.k_slices_per_split - 1) / args.k_slices_per_split;
  args.status = status;
  args.b_kind = n_base ? B_NORMED : B_ROWS;
  args.cluster = splits > 1 || n_base;
  args.n_base = n_base;
  args.n_acc = n_acc;
  args.n_gamma = n_gamma;
  args.n_eps = n_eps;
  args.n_out = n_out;
  args.n_zero = n_zero;
  args.rope_q = (bf16*)q_out;
  args.rope_k = (bf16*)k_cache;
  args.rope_v = (bf16*)v_cache;
  args.rope_slots = slots;
  args.rope_positions = positions;
  args.rope_table = table;
  args.rope_heads = heads;
  args.rope_kv_heads = kv_heads;
  args.rope_head_dim = head_dim;
  return launch_tc<16, EPI_ROPE>(mw, mx, args, splits, stream);
}

// How many clusters of `splits` CTAs of the q/k/v kernel (16 tokens, depth split over a cluster
// along z; `normed`: with the norm folded in) the device holds at a time - a GPC places only whole
// clusters, so eight-CTA clusters may leave SMs idle that six-CTA clusters fill.  A caller keeps all
// of a product's clusters in one wave by it.  0 when the device cannot be asked.
template <int MODE>
static int resident_rope_clusters(int splits) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_kernel<16, EPI_ROPE, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 2048) != cudaSuccess) return 0;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, 1, (unsigned)splits);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = 200 * 1024 + 1024;  // what a launch asks for at most: the ring and the pushed accumulators
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)splits;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<16, EPI_ROPE, MODE>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
ALOFA_API int alofa_gemm_tc_rope_resident_clusters(int splits, int normed) {
  if (splits < 1 || splits > 8) return 0;
  return normed ? resident_rope_clusters<MODE_NORMED>(splits) : resident_rope_clusters<MODE_CLUSTER>(splits);
}

// How many splits alofa_gemm_tc will really use (it never leaves one empty).
ALOFA_API int alofa_gemm_tc_splits(int K, int splits) {
  const int total = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > total) splits = total;
  const int per = (total + splits - 1) / splits;
  return (total + per - 1) / per;
}
