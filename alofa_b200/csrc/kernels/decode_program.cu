// A decode step of a few tokens as ONE resident kernel that runs a list of phases.
//
// With a handful of tokens every product of a layer moves a few megabytes of
// weights and takes a microsecond or two; launched one kernel after the other,
// a step spends most of its time between kernels.  Here the step is a program:
// an array of phase descriptors in device memory (embedding, products with
// their epilogues, attention over the paged cache, the merge of its splits),
// run by one cooperative launch of one CTA per SM.  All CTAs work through the
// same list; a barrier over the grid separates two phases, so a phase may read
// whatever an earlier phase wrote.  The descriptors are plain data made by the
// parts of the model; the kernel knows nothing of the model they come from.
//
// Products (tokens <= 16): out[t, n] = sum_k A[t, k] * W[n, k].  The tokens
// are the 16 rows of an mma.sync m16n8k16 tile, eight weight rows its columns.
// The operand A is put into shared memory once per phase and CTA - either
// bfloat16 rows as they are, or rows of the fp32 residual stream normalised on
// the way (RMSNorm: sum of squares in fp32, x * rsqrt * gamma rounded to
// bfloat16) - and every warp streams its share of the weights straight from
// global memory into registers, 16 bytes per lane and row, many loads in
// flight.  An item is one or two 8-row weight tiles; `wpi` warps share an item
// by splitting the depth and their partial tiles are added in warp order in
// shared memory, so a result does not depend on timing.  Epilogues: store
// (bfloat16 or fp32), add into the fp32 residual stream, silu(gate) * up for a
// stacked [gate; up] weight, and rotate-and-store for a stacked [q; k; v]
// weight (bias, NeoX rotation from a cos/sin table, q to a buffer, k and v to
// their cache slots).
//
// Attention: an item is (request, KV head, split of 256 keys), run by a group
// of four warps, one 64-key block each, fetched by bulk tensor copies
// (128-byte swizzle) and awaited on an mbarrier with a bound; the groups'
// partial (output, maximum, sum) triples are merged, in split order, by whichever
// group delivers the last split of a (request, KV head).  Pages must hold whole 64-key blocks and the head size must be 64 or
// 128; the host refuses other shapes and the caller launches kernels instead.
//
// Data that one phase writes and a later one reads is read past the L1 cache
// (ld.global.cg, cp.async.cg, bulk copies), which the barrier does not clean.
//
// Every wait is bounded: a barrier or a copy that does not complete within
// the limit sets the status word to 2 and the kernel returns.
// Formulas: src/alofa/kernels/cpu/scalar.mojo:10-18 (product), 93-129 (norm),
// 132-193 (rotation), 208-231 (gated), 392-470 (attention).
#include <string.h>

#include "attention_core.cuh"
#include "common.cuh"
#include "tma.cuh"

#ifndef PROGRAM_THREADS_N
#define PROGRAM_THREADS_N 512
#endif
constexpr int PROGRAM_THREADS = PROGRAM_THREADS_N;
constexpr int PROGRAM_WARPS = PROGRAM_THREADS / 32;
constexpr int GROUP_WARPS = 4;                      // warps of an attention group: 256 keys per item
constexpr int SPLIT_KEYS = GROUP_WARPS * BLOCK_N;
constexpr int TILE_BYTES = BLOCK_N * HD * 2;        // one dense 64-key tile
constexpr int ATTN_GROUPS = (HD <= 64) ? 2 : 1;     // attention items a CTA works on at a time
constexpr int GROUP_BYTES = 2 * GROUP_WARPS * TILE_BYTES;
constexpr int Q_TILE_BYTES = 16 * ROW * 2;
constexpr int MAX_SMEM = 220 * 1024;

enum PhaseOp { OP_EMBED = 0, OP_LINEAR = 1, OP_ATTENTION = 2 };
enum OperandKind { A_BF16 = 0, A_NORMED = 1 };
enum Epilogue { E_STORE_BF16 = 0, E_STORE_F32 = 1, E_RESIDUAL = 2, E_GATED = 3, E_ROPE_STORE = 4 };

struct alignas(128) Phase {
  CUtensorMap map_k, map_v;  // attention: the layer's key and value caches as [slots, kv_heads * head_dim]
  int op, a_kind, epi, T;    // T: tokens of the step (one per request)
  int N, K, wpi, items;      // N: weight rows an item may touch (clamp); K: depth; wpi: warps per item
  int tiles, a_stride, out_cols, hidden;  // tiles per item (1 or 2); bytes between operand rows in shared memory
  int nh, nkv, window, page_size;
  int max_blocks, n_splits, writes, vocab;
  int ring_offset, ring_threads, depth, phase_index;  // the weight feed's ring: where it starts, threads that use it, units in flight
  float eps, scale_log2;
  const void* a;             // operand rows (bf16 [T, K]) or the fp32 stream [T, K]
  const float* gamma;        // norm weight [K] when the operand is normalised
  const bf16* w;             // weight [rows, K]
  const float* bias;         // [rows] or null
  void* out;                 // store / residual / gated target
  bf16* q;                   // rotate-and-store: q [T, nh, HD]; attention reads it
  bf16* k_cache;
  bf16* v_cache;
  const int* slot_map;       // [T] cache slot of each token's key
  const int* positions;      // [T]
  const int* block_table;    // [T, max_blocks]
  const int* kv_len;         // [T]
  const int* ids;            // [T] token ids (embedding)
  const int* token_src;      // [T] or null: -1 takes ids[t], r >= 0 takes fed[r]
  const int* fed;            // tokens the step before sampled
  const float* rope_table;   // [max_pos, HD / 2, 2]
  float* partial_o;          // [n_splits, T * nh, HD]
  float* partial_ml;         // [n_splits, T * nh, 2]
  int* counters;             // [T * nkv] splits that have delivered, zero between steps
};

// ---------------------------------------------------------------------------
// Barrier over the grid.  `target` counts the arrivals expected so far; the
// counter is zeroed by the host before the launch.  Returns false when the
// wait ran out or another CTA gave up.
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned& target, int* status, int* shared_ok) {
  __syncthreads();
  target += gridDim.x;
  if (threadIdx.x == 0) {
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
    int ok = 0;
    for (unsigned i = 0; i < (1u << 22); ++i) {
      if (ld_acquire_u32(counter) >= target) {
        ok = 1;
        break;
      }
      if ((i & 255u) == 255u && *reinterpret_cast<volatile int*>(status) == 2) break;
    }
    if (!ok) atomicExch(status, 2);
    *shared_ok = ok;
  }
  __syncthreads();
  return *shared_ok != 0;
}

__device__ __forceinline__ uint4 load_weights(const bf16* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_tile(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------
// Embedding: h[t] = table[ids[t]] widened to fp32; ids outside the vocabulary
// set the status word to 1 and give a zero row.
// ---------------------------------------------------------------------------
__device__ void embed_phase(const Phase& ph, int* status) {
  float* h = reinterpret_cast<float*>(ph.out);
  const bf16* table = reinterpret_cast<const bf16*>(ph.w);
  for (int t = blockIdx.x; t < ph.T; t += gridDim.x) {
    int id = ph.ids[t];
    if (ph.token_src && ph.token_src[t] >= 0) id = ph.fed[ph.token_src[t]];
    const bool ok = id >= 0 && id < ph.vocab;
    if (!ok && threadIdx.x == 0) atomicCAS(status, 0, 1);
    const bf16* row = table + (size_t)(ok ? id : 0) * ph.hidden;
    for (int c = threadIdx.x; c < ph.hidden; c += PROGRAM_THREADS) h[(size_t)t * ph.hidden + c] = ok ? __bfloat162float(row[c]) : 0.f;
  }
}

// ---------------------------------------------------------------------------
// Products
// ---------------------------------------------------------------------------
// The operand into shared memory: rows of a_stride bytes.
__device__ void stage_operand(const Phase& ph, uint8_t* a_tile) {
  const int K = ph.K, T = ph.T;
  if (ph.a_kind == A_BF16) {
    const int per_row = K >> 3;  // 16-byte chunks
    const uint4* src = reinterpret_cast<const uint4*>(ph.a);
    for (int idx = threadIdx.x; idx < T * per_row; idx += PROGRAM_THREADS) {
      const int t = idx / per_row, ch = idx - t * per_row;
      *reinterpret_cast<uint4*>(a_tile + (size_t)t * ph.a_stride + ch * 16) = __ldcg(src + idx);
    }
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n4 = K >> 2;
  const float4* gamma = reinterpret_cast<const float4*>(ph.gamma);
  constexpr int HELD = 8;  // float4 a lane can keep: rows up to 1024 wide are read once
  if (n4 <= 32 * HELD) {
    for (int t = warp; t < T; t += PROGRAM_WARPS) {
      const float4* row = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ph.a) + (size_t)t * K);
      float4 v[HELD];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < HELD; ++i) {
        const int ch = lane + 32 * i;
        v[i] = ch < n4 ? __ldcg(row + ch) : make_float4(0.f, 0.f, 0.f, 0.f);
        // the norm weight on its way to L1 meanwhile
        if (ch < n4 && (lane & 7) == 0) asm volatile("prefetch.global.L1 [%0];" ::"l"(gamma + ch));
      }
#pragma unroll
      for (int i = 0; i < HELD; ++i) {
        ss = fmaf(v[i].x, v[i].x, ss);
        ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss);
        ss = fmaf(v[i].w, v[i].w, ss);
      }
      ss = warp_sum(ss);
      const float scale = 1.0f / sqrtf(ss / (float)K + ph.eps);
#pragma unroll
      for (int i = 0; i < HELD; ++i) {
        const int ch = lane + 32 * i;
        if (ch < n4) {
          const float4 g = __ldg(gamma + ch);
          __nv_bfloat162 lo = __floats2bfloat162_rn(v[i].x * scale * g.x, v[i].y * scale * g.y);
          __nv_bfloat162 hi = __floats2bfloat162_rn(v[i].z * scale * g.z, v[i].w * scale * g.w);
          *reinterpret_cast<uint2*>(a_tile + (size_t)t * ph.a_stride + ch * 8) =
              make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
      }
    }
    return;
  }
  for (int t = warp; t < T; t += PROGRAM_WARPS) {
    const float4* row = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ph.a) + (size_t)t * K);
    float ss = 0.f;
    for (int ch = lane; ch < n4; ch += 32) {
      const float4 v = __ldcg(row + ch);
      ss = fmaf(v.x, v.x, ss);
      ss = fmaf(v.y, v.y, ss);
      ss = fmaf(v.z, v.z, ss);
      ss = fmaf(v.w, v.w, ss);
    }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)K + ph.eps);
    for (int ch = lane; ch < n4; ch += 32) {
      const float4 v = __ldcg(row + ch);
      const float4 g = gamma[ch];
      __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * scale * g.x, v.y * scale * g.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * scale * g.z, v.w * scale * g.w);
      *reinterpret_cast<uint2*>(a_tile + (size_t)t * ph.a_stride + ch * 8) =
          make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}

// First weight rows of an item's tiles.
__device__ __forceinline__ void item_rows(const Phase& ph, int item, int& row_a, int& row_b) {
  if (ph.epi == E_GATED) {
    row_a = item * 8;
    row_b = ph.out_cols + item * 8;
  } else if (ph.epi == E_ROPE_STORE) {
    const int per_head = HD / 16;
    const int head = item / per_head, j = item - head * per_head;
    if (head < ph.nh + ph.nkv) {
      row_a = head * HD + 8 * j;
      row_b = row_a + HD / 2;
    } else {
      row_a = head * HD + 16 * j;
      row_b = row_a + 8;
    }
  } else {
    row_a = item * 8 * ph.tiles;
    row_b = row_a + 8;
  }
}

// What an output element needs from memory besides its sums: fetched before
// the products run, so that the epilogue does not wait for it.
struct Fetched {
  float b0, b1;  // bias of the two rows
  float x0, x1;  // residual: the old values; rotation: cosine and sine
  int slot;      // rotate-and-store: the token's cache slot
  int pos;       // rotate-and-store: the token's position
};

__device__ __forceinline__ void epilogue_fetch(const Phase& ph, int item, int t, int n, Fetched& f) {
  int row_a, row_b;
  item_rows(ph, item, row_a, row_b);
  const bool has_a = row_a + n < ph.N, has_b = ph.tiles == 2 && row_b + n < ph.N;
  f.b0 = f.b1 = f.x0 = f.x1 = 0.f;
  f.slot = f.pos = 0;
  if (ph.bias) {
    if (has_a) f.b0 = __ldg(ph.bias + row_a + n);
    if (has_b) f.b1 = __ldg(ph.bias + row_b + n);
  }
  if (ph.epi == E_RESIDUAL) {
    const float* out = reinterpret_cast<const float*>(ph.out) + (size_t)t * ph.out_cols;
    if (has_a) f.x0 = __ldcg(out + row_a + n);
    if (has_b) f.x1 = __ldcg(out + row_b + n);
  } else if (ph.epi == E_ROPE_STORE) {
    const int head = item / (HD / 16);
    if (head >= ph.nh) f.slot = ph.slot_map[t];
    f.pos = ph.positions[t];
  }
}

// The second step of the fetch, for what is found through a fetched value.
__device__ __forceinline__ void epilogue_fetch_more(const Phase& ph, int item, int n, Fetched& f) {
  if (ph.epi != E_ROPE_STORE) return;
  const int per_head = HD / 16;
  const int head = item / per_head, j = item - head * per_head;
  if (head < ph.nh + ph.nkv) {
    const float2 cs = __ldg(reinterpret_cast<const float2*>(ph.rope_table + ((size_t)f.pos * (HD / 2) + 8 * j + n) * 2));
    f.x0 = cs.x;
    f.x1 = cs.y;
  }
}

// One finished element pair (token t, column n of the item's two tiles).
__device__ __forceinline__ void epilogue(const Phase& ph, int item, int t, int n, float v0, float v1, const Fetched& f) {
  int row_a, row_b;
  item_rows(ph, item, row_a, row_b);
  const bool has_a = row_a + n < ph.N, has_b = ph.tiles == 2 && row_b + n < ph.N;
  v0 += f.b0;
  v1 += f.b1;
  switch (ph.epi) {
    case E_STORE_BF16: {
      bf16* out = reinterpret_cast<bf16*>(ph.out) + (size_t)t * ph.out_cols;
      if (has_a) out[row_a + n] = __float2bfloat16_rn(v0);
      if (has_b) out[row_b + n] = __float2bfloat16_rn(v1);
      break;
    }
    case E_STORE_F32: {
      float* out = reinterpret_cast<float*>(ph.out) + (size_t)t * ph.out_cols;
      if (has_a) out[row_a + n] = v0;
      if (has_b) out[row_b + n] = v1;
      break;
    }
    case E_RESIDUAL: {
      float* out = reinterpret_cast<float*>(ph.out) + (size_t)t * ph.out_cols;
      if (has_a) out[row_a + n] = f.x0 + v0;
      if (has_b) out[row_b + n] = f.x1 + v1;
      break;
    }
    case E_GATED: {
      bf16* out = reinterpret_cast<bf16*>(ph.out) + (size_t)t * ph.out_cols;
      if (has_a) out[row_a + n] = __float2bfloat16_rn(v0 / (1.0f + __expf(-v0)) * v1);
      break;
    }
    case E_ROPE_STORE: {
      const int per_head = HD / 16;
      const int head = item / per_head, j = item - head * per_head;
      if (head >= ph.nh && f.slot < 0) return;
      if (head < ph.nh + ph.nkv) {
        const int d = 8 * j + n;
        const float ya = v0 * f.x0 - v1 * f.x1, yb = v1 * f.x0 + v0 * f.x1;
        bf16* dst = head < ph.nh ? ph.q + ((size_t)t * ph.nh + head) * HD : ph.k_cache + ((size_t)f.slot * ph.nkv + (head - ph.nh)) * HD;
        dst[d] = __float2bfloat16_rn(ya);
        dst[d + HD / 2] = __float2bfloat16_rn(yb);
      } else {
        bf16* dst = ph.v_cache + ((size_t)f.slot * ph.nkv + (head - ph.nh - ph.nkv)) * HD + 16 * j;
        dst[n] = __float2bfloat16_rn(v0);
        dst[8 + n] = __float2bfloat16_rn(v1);
      }
      break;
    }
  }
}

#ifdef ALOFA_PROGRAM_TIMING
// A build for measuring: CTA 0 notes the clock after each phase's work and after its barrier.
__device__ long long g_stamps[4096];
ALOFA_API int alofa_program_stamps(long long* host, int n) {
  return cudaMemcpyFromSymbol(host, g_stamps, sizeof(long long) * n) == cudaSuccess ? ALOFA_OK : ALOFA_ERR_LAUNCH;
}
#define STAMP(i)                                                              \
  do {                                                                        \
    if (blockIdx.x == 0 && threadIdx.x == 0 && (i) < 4096) g_stamps[i] = clock64(); \
  } while (0)
#else
#define STAMP(i)
#endif

// ---------------------------------------------------------------------------
// The weight feed.  A thread's weights come through a ring in shared memory
// that only this thread touches: cp.async copies 16 bytes per lane and tile
// into the thread's own slots, `depth` units ahead of the products that read
// them back, so no registers are held by loads in flight and no thread waits
// for another.  A unit is what one step of a warp consumes: for paired tiles
// one 32-deep chunk of both tiles, for single tiles two 32-deep chunks.  The
// feed runs ahead across rounds, and its first units are asked for before the
// barrier that precedes the product: weights depend on no earlier phase.
// ---------------------------------------------------------------------------
constexpr int PRE_ISSUE = 4;   // units asked for before the barrier that precedes a product; the rest follow the operand's loads
constexpr int MAX_DEPTH = 16;  // the ring's depth is a power of two up to this, set per phase by the host

__device__ __forceinline__ void cp_async_wait_dyn(int pending) {  // the count must be an immediate
  switch (pending) {
    case 0: cp_async_wait<0>(); break;
    case 1: cp_async_wait<1>(); break;
    case 3: cp_async_wait<3>(); break;
    case 7: cp_async_wait<7>(); break;
    default: cp_async_wait<15>(); break;
  }
}

struct Feed {
  int q, total;          // next unit to ask for; units of this warp in the phase
  int round, k, upw;     // its round and place in the round; units per warp and round
  int ch0, ch1;          // this warp's 32-deep chunks of the depth
  int local, per_iter, rounds;
  const bf16 *w_a, *w_b; // rows of the tiles of the round being asked for (null: no item)
};

__device__ __forceinline__ void feed_rows(Feed& f, const Phase& ph) {
  const int lane = threadIdx.x & 31;
  const int item = (f.round * f.per_iter + f.local) * gridDim.x + blockIdx.x;
  f.w_a = f.w_b = nullptr;
  if (f.round < f.rounds && item < ph.items) {
    int row_a, row_b;
    item_rows(ph, item, row_a, row_b);
    f.w_a = ph.w + (size_t)min(row_a + (lane >> 2), ph.N - 1) * ph.K + (lane & 3) * 8;
    f.w_b = ph.w + (size_t)min(row_b + (lane >> 2), ph.N - 1) * ph.K + (lane & 3) * 8;
  }
}

__device__ __forceinline__ void feed_begin(Feed& f, const Phase& ph) {
  const int warp = threadIdx.x >> 5;
  const int wpi = ph.wpi, chunks = ph.K >> 5;
  f.per_iter = PROGRAM_WARPS / wpi;
  int cpw = (chunks + wpi - 1) / wpi;
  if (ph.tiles == 1) cpw = (cpw + 1) & ~1;  // whole units
  f.local = warp / wpi;
  const int part = warp - f.local * wpi;
  f.ch0 = part * cpw;
  f.ch1 = min(chunks, f.ch0 + cpw);
  f.upw = ph.tiles == 2 ? cpw : cpw >> 1;
  f.rounds = (ph.items + f.per_iter * gridDim.x - 1) / (f.per_iter * gridDim.x);
  f.total = f.rounds * f.upw;
  f.q = f.round = f.k = 0;
  feed_rows(f, ph);
}

// Ask for the next unit (if any is left) and close a copy group either way.
__device__ __forceinline__ void feed_issue(Feed& f, const Phase& ph, uint8_t* smem) {
  if (f.q < f.total) {
    const int half = ph.ring_threads * 16;
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem + ph.ring_offset + (size_t)(f.q & (ph.depth - 1)) * 2 * half + threadIdx.x * 16);
    if (f.w_a) {
      if (ph.tiles == 2) {
        const int ch = f.ch0 + f.k;
        if (ch < f.ch1) {
          cp_async16(dst, f.w_a + ch * 32, true);
          cp_async16(dst + half, f.w_b + ch * 32, true);
        }
      } else {
        const int ch = f.ch0 + 2 * f.k;
        if (ch < f.ch1) cp_async16(dst, f.w_a + ch * 32, true);
        if (ch + 1 < f.ch1) cp_async16(dst + half, f.w_a + (ch + 1) * 32, true);
      }
    }
    ++f.q;
    if (++f.k == f.upw) {
      f.k = 0;
      ++f.round;
      feed_rows(f, ph);
    }
  }
  cp_async_commit();
}

// The products of one phase.  TILES weight tiles per item; ROWS16: the step has more than 8 tokens.
template <int TILES, bool ROWS16>
__device__ void linear_run(const Phase& ph, Feed& f, uint8_t* smem) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  const int rows = ROWS16 ? 16 : 8;
  float* red = reinterpret_cast<float*>(smem + (size_t)rows * ph.a_stride);
  const uint8_t* a_lo = smem + (size_t)g * ph.a_stride + c * 16;
  const uint8_t* a_hi = a_lo + (size_t)8 * ph.a_stride;
  const int wpi = ph.wpi, per_iter = f.per_iter, upw = f.upw, total = f.total, ch0 = f.ch0, ch1 = f.ch1, local = f.local;
  STAMP(2048 + 4 * ph.phase_index);
  constexpr int EPT = 128 * PROGRAM_WARPS / PROGRAM_THREADS;  // output elements a thread may own in a round
  const bool fetches = ph.bias != nullptr || ph.epi == E_RESIDUAL || ph.epi == E_ROPE_STORE;
  Fetched fetched[EPT];
#pragma unroll
  for (int i = 0; i < EPT; ++i) fetched[i].b0 = fetched[i].b1 = fetched[i].x0 = fetched[i].x1 = 0.f, fetched[i].slot = fetched[i].pos = 0;
  auto fetch_round = [&](int rnd, bool more) {
    if (!fetches) return;
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int e = threadIdx.x + i * PROGRAM_THREADS;
      const int li = e >> 7, t = (e & 127) >> 3, n = e & 7;
      const int it = (rnd * per_iter + li) * gridDim.x + blockIdx.x;
      if (e < per_iter * 128 && it < ph.items && t < ph.T) {
        if (more)
          epilogue_fetch_more(ph, it, n, fetched[i]);
        else
          epilogue_fetch(ph, it, t, n, fetched[i]);
      }
    }
  };
  fetch_round(0, false);
  stage_operand(ph, smem);
  for (int i = PRE_ISSUE; i < ph.depth; ++i) feed_issue(f, ph, smem);  // the rest of the ring, behind the operand's loads
  fetch_round(0, true);
  __syncthreads();
  STAMP(2048 + 4 * ph.phase_index + 1);
  float acc[TILES][4];
#pragma unroll
  for (int i = 0; i < TILES; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  int round = 0, k = 0;
  const int half = ph.ring_threads * 16, depth = ph.depth;
  const uint8_t* ring = smem + ph.ring_offset + threadIdx.x * 16;
  for (int q = 0; q < total; ++q) {
    cp_async_wait_dyn(depth - 1);
    const int item = (round * per_iter + local) * gridDim.x + blockIdx.x;
    const uint8_t* slot = ring + (size_t)(q & (depth - 1)) * 2 * half;
    if (item < ph.items) {
      if (TILES == 2) {
        const int ch = ch0 + k;
        if (ch < ch1) {
          const uint4 wa = *reinterpret_cast<const uint4*>(slot), wb = *reinterpret_cast<const uint4*>(slot + half);
          const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + ch * 64);
          uint4 hi = make_uint4(0u, 0u, 0u, 0u);
          if (ROWS16) hi = *reinterpret_cast<const uint4*>(a_hi + ch * 64);
          mma_tile(acc[0], lo.x, hi.x, lo.y, hi.y, wa.x, wa.y);
          mma_tile(acc[0], lo.z, hi.z, lo.w, hi.w, wa.z, wa.w);
          mma_tile(acc[TILES - 1], lo.x, hi.x, lo.y, hi.y, wb.x, wb.y);
          mma_tile(acc[TILES - 1], lo.z, hi.z, lo.w, hi.w, wb.z, wb.w);
        }
      } else {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int ch = ch0 + 2 * k + hf;
          if (ch < ch1) {
            const uint4 wa = *reinterpret_cast<const uint4*>(slot + hf * half);
            const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + ch * 64);
            uint4 hi = make_uint4(0u, 0u, 0u, 0u);
            if (ROWS16) hi = *reinterpret_cast<const uint4*>(a_hi + ch * 64);
            mma_tile(acc[0], lo.x, hi.x, lo.y, hi.y, wa.x, wa.y);
            mma_tile(acc[0], lo.z, hi.z, lo.w, hi.w, wa.z, wa.w);
          }
        }
      }
    }
    feed_issue(f, ph, smem);  // refills the slot just read
    if (++k == upw) {
      STAMP(2048 + 4 * ph.phase_index + 2);
      // the round is complete: add the warps' partial tiles in warp order, run the epilogue
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl) {
        float* r = red + ((warp * 2 + tl) * 16) * 8;  // red[warp][tile][row][8]
        *reinterpret_cast<float2*>(r + g * 8 + c * 2) = make_float2(acc[tl][0], acc[tl][1]);
        if (ROWS16) *reinterpret_cast<float2*>(r + (g + 8) * 8 + c * 2) = make_float2(acc[tl][2], acc[tl][3]);
        acc[tl][0] = acc[tl][1] = acc[tl][2] = acc[tl][3] = 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < EPT; ++i) {
        const int e = threadIdx.x + i * PROGRAM_THREADS;
        const int li = e >> 7, t = (e & 127) >> 3, n = e & 7;
        const int it = (round * per_iter + li) * gridDim.x + blockIdx.x;
        if (e < per_iter * 128 && it < ph.items && t < ph.T) {
          float v0 = 0.f, v1 = 0.f;
          for (int p = 0; p < wpi; ++p) {
            const float* r = red + (((li * wpi + p) * 2) * 16) * 8 + t * 8 + n;
            v0 += r[0];
            if (TILES == 2) v1 += r[128];
          }
          epilogue(ph, it, t, n, v0, v1, fetched[i]);
        }
      }
      if (round + 1 < f.rounds) {
        fetch_round(round + 1, false);
        fetch_round(round + 1, true);
      }
      __syncthreads();
      k = 0;
      ++round;
    }
  }
  cp_async_wait<0>();
}

__device__ void linear_phase(const Phase& ph, Feed& f, uint8_t* smem) {
  if (ph.T <= 8) {
    if (ph.tiles == 2)
      linear_run<2, false>(ph, f, smem);
    else
      linear_run<1, false>(ph, f, smem);
  } else {
    if (ph.tiles == 2)
      linear_run<2, true>(ph, f, smem);
    else
      linear_run<1, true>(ph, f, smem);
  }
}

// ---------------------------------------------------------------------------
// Attention over the cache, one token per request
// ---------------------------------------------------------------------------
__device__ void attention_phase(const Phase& ph, const Phase* ph_global, uint8_t* smem, uint64_t* tile_bar, uint32_t& parity, int* abort_flag,
                                int* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = warp / GROUP_WARPS, w = warp % GROUP_WARPS, gtid = threadIdx.x - grp * GROUP_WARPS * 32;
  const bool in_group = grp < ATTN_GROUPS;
  uint8_t* group_base = smem + (size_t)(in_group ? grp : 0) * GROUP_BYTES;
  uint8_t* kt = group_base + w * TILE_BYTES;
  uint8_t* vt = group_base + (GROUP_WARPS + w) * TILE_BYTES;
  bf16* q_tile = reinterpret_cast<bf16*>(smem + ATTN_GROUPS * GROUP_BYTES + (in_group ? grp : 0) * Q_TILE_BYTES);
  float* merge_o = reinterpret_cast<float*>(group_base);          // [GROUP_WARPS][16][MERGE_ROW], over the key tiles
  float* merge_ml = merge_o + GROUP_WARPS * 16 * MERGE_ROW;       // [GROUP_WARPS][16][2]
  const int g = ph.nh / ph.nkv;
  const int n_rows_total = ph.T * ph.nh;
  const int per_split = ph.T * ph.nkv;
  const int items = per_split * ph.n_splits;
  const int rounds = (items + ATTN_GROUPS * gridDim.x - 1) / (ATTN_GROUPS * gridDim.x);
  __shared__ int group_last[ATTN_GROUPS];
  fence_async_shared();
  __syncthreads();
  for (int round = 0; round < rounds; ++round) {
    const int item = (round * ATTN_GROUPS + grp) * gridDim.x + blockIdx.x;
    bool active = in_group && item < items;
    int split = 0, seq = 0, kvh = 0, pos = 0, k_lo = 0, k_hi = -1;
    if (active) {
      split = item / per_split;
      const int rest = item - split * per_split;
      seq = rest / ph.nkv;
      kvh = rest - seq * ph.nkv;
      pos = ph.kv_len[seq] - 1;
      if (ph.window > 0) k_lo = max(0, pos - ph.window + 1);
      k_lo = max(k_lo, split * SPLIT_KEYS);
      k_hi = min(pos, (split + 1) * SPLIT_KEYS - 1);
      active = k_lo <= k_hi;
    }
    const int j0 = (split * GROUP_WARPS + w) * BLOCK_N;
    const bool has_keys = active && j0 <= k_hi && j0 + BLOCK_N - 1 >= k_lo;
    if (active) {
      for (int idx = gtid; idx < 16 * CHUNKS; idx += GROUP_WARPS * 32) {
        const int r = idx / CHUNKS, ch = idx % CHUNKS;
        const bool ok = r < g;
        const bf16* src = ok ? ph.q + ((size_t)seq * ph.nh + kvh * g + r) * HD + ch * 8 : ph.q;
        cp_async16((uint32_t)__cvta_generic_to_shared(q_tile + r * ROW + ch * 8), src, ok);
      }
      if (has_keys && lane == 0) {
        const int e = j0 / ph.page_size;
        const int row0 = ph.block_table[(size_t)seq * ph.max_blocks + e] * ph.page_size + (j0 - e * ph.page_size);
        mbar_expect_tx(&tile_bar[warp], 2 * TILE_BYTES);
#pragma unroll
        for (int sub = 0; sub < HD / 64; ++sub) {
          tma_load_2d(kt + sub * BLOCK_N * 128, &ph_global->map_k, &tile_bar[warp], kvh * HD + sub * 64, row0);
          tma_load_2d(vt + sub * BLOCK_N * 128, &ph_global->map_v, &tile_bar[warp], kvh * HD + sub * 64, row0);
        }
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();  // the query tiles are in place
    RowState st;
    st.m_lo = st.m_hi = -INFINITY;
    st.l_lo = st.l_hi = 0.f;
#pragma unroll
    for (int d = 0; d < DTILES; ++d) st.o[d][0] = st.o[d][1] = st.o[d][2] = st.o[d][3] = 0.f;
    if (has_keys) {
      const bool arrived = mbar_wait(&tile_bar[warp], parity, abort_flag);
      parity ^= 1u;
      if (arrived) {
        uint32_t qf[KSTEPS][4];
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
          const bf16* src = q_tile + (lane & 15) * ROW + ks * 16 + (lane >> 4) * 8;
          ldmatrix_x4(qf[ks], (uint32_t)__cvta_generic_to_shared(src));
        }
        attend_block<true>(st, qf, (uint32_t)__cvta_generic_to_shared(kt), (uint32_t)__cvta_generic_to_shared(vt), j0, lane, pos, k_lo, k_hi,
                           ph.window, ph.scale_log2);
      }
    }
    __syncthreads();  // every warp is done with the tiles the merge buffers lie over
    if (active) {
      st.l_lo += __shfl_xor_sync(0xffffffffu, st.l_lo, 1);
      st.l_lo += __shfl_xor_sync(0xffffffffu, st.l_lo, 2);
      st.l_hi += __shfl_xor_sync(0xffffffffu, st.l_hi, 1);
      st.l_hi += __shfl_xor_sync(0xffffffffu, st.l_hi, 2);
      const int r = lane >> 2;
      float* mo = merge_o + (w * 16) * MERGE_ROW;
#pragma unroll
      for (int d = 0; d < DTILES; ++d) {
        *reinterpret_cast<float2*>(mo + r * MERGE_ROW + d * 8 + (lane & 3) * 2) = make_float2(st.o[d][0], st.o[d][1]);
        *reinterpret_cast<float2*>(mo + (r + 8) * MERGE_ROW + d * 8 + (lane & 3) * 2) = make_float2(st.o[d][2], st.o[d][3]);
      }
      if ((lane & 3) == 0) {
        float* ml = merge_ml + w * 32;
        ml[r * 2] = (st.m_lo == -INFINITY) ? -INFINITY : st.m_lo * ph.scale_log2;
        ml[r * 2 + 1] = st.l_lo;
        ml[(r + 8) * 2] = (st.m_hi == -INFINITY) ? -INFINITY : st.m_hi * ph.scale_log2;
        ml[(r + 8) * 2 + 1] = st.l_hi;
      }
    }
    __syncthreads();
    if (active) {
      for (int idx = gtid; idx < g * HD; idx += GROUP_WARPS * 32) {
        const int r = idx / HD, d = idx % HD;
        float m = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < GROUP_WARPS; ++ww) m = fmaxf(m, merge_ml[ww * 32 + r * 2]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int ww = 0; ww < GROUP_WARPS; ++ww) {
          const float mw = merge_ml[ww * 32 + r * 2];
          const float scale = (mw == -INFINITY) ? 0.f : fast_exp2(mw - m);
          l += merge_ml[ww * 32 + r * 2 + 1] * scale;
          acc += merge_o[(ww * 16 + r) * MERGE_ROW + d] * scale;
        }
        const size_t out_row = (size_t)seq * ph.nh + kvh * g + r;
        ph.partial_o[((size_t)split * n_rows_total + out_row) * HD + d] = acc;
        if (d == 0) {
          float* ml = ph.partial_ml + ((size_t)split * n_rows_total + out_row) * 2;
          ml[0] = m;
          ml[1] = l;
        }
      }
    }
    // the group whose split is the last of its (request, KV head) to deliver merges them all
    __syncthreads();
    if (active && gtid == 0) {
      const int s_lo = (ph.window > 0 ? max(0, pos - ph.window + 1) : 0) / SPLIT_KEYS, s_hi = pos / SPLIT_KEYS;
      __threadfence();
      int* counter = ph.counters + seq * ph.nkv + kvh;
      const int last = atomicAdd(counter, 1) == s_hi - s_lo;
      if (last) {
        *counter = 0;  // for the next step
        __threadfence();
      }
      group_last[grp] = last;
    }
    __syncthreads();
    if (active && group_last[grp]) {
      const int s_lo = (ph.window > 0 ? max(0, pos - ph.window + 1) : 0) / SPLIT_KEYS, s_hi = pos / SPLIT_KEYS;
      bf16* out = reinterpret_cast<bf16*>(ph.out);
      for (int idx = gtid; idx < g * HD; idx += GROUP_WARPS * 32) {
        const int r = idx / HD, d = idx % HD;
        const size_t row = (size_t)seq * ph.nh + kvh * g + r;
        // four splits' values in flight at a time; the sums run in split order
        float m = -INFINITY;
        for (int s0 = s_lo; s0 <= s_hi; s0 += 4) {
          float ms[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) ms[i] = s0 + i <= s_hi ? __ldcg(ph.partial_ml + ((size_t)(s0 + i) * n_rows_total + row) * 2) : -INFINITY;
#pragma unroll
          for (int i = 0; i < 4; ++i) m = fmaxf(m, ms[i]);
        }
        float l = 0.f, acc = 0.f;
        for (int s0 = s_lo; s0 <= s_hi; s0 += 4) {
          float ms[4], ls[4], os[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const bool in = s0 + i <= s_hi;
            const float* ml = ph.partial_ml + ((size_t)(s0 + i) * n_rows_total + row) * 2;
            ms[i] = in ? __ldcg(ml) : -INFINITY;
            ls[i] = in ? __ldcg(ml + 1) : 0.f;
            os[i] = in ? __ldcg(ph.partial_o + ((size_t)(s0 + i) * n_rows_total + row) * HD + d) : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float wgt = (ms[i] == -INFINITY) ? 0.f : fast_exp2(ms[i] - m);
            l += ls[i] * wgt;
            acc += os[i] * wgt;
          }
        }
        out[row * HD + d] = __float2bfloat16_rn(acc / l);
      }
    }
    fence_async_shared();
    __syncthreads();  // the merge buffers are read; the next round's copies may land on them
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(status, 2);
}

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------

__global__ void __launch_bounds__(PROGRAM_THREADS, 1) decode_program_kernel(const Phase* __restrict__ phases, int n_phases, unsigned* sync_counter,
                                                                            int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ Phase ring[3];  // this phase's descriptor, the next one's, and the one after being fetched
  __shared__ uint64_t tile_bar[PROGRAM_WARPS];
  __shared__ int abort_flag, barrier_ok;
  if ((threadIdx.x & 31) == 0) {
    if (threadIdx.x == 0) abort_flag = 0;
    mbar_init(&tile_bar[threadIdx.x >> 5], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  uint32_t parity = 0;
  unsigned target = 0;
  constexpr int WORDS = (int)(sizeof(Phase) / 16);
  for (int i = threadIdx.x; i < 2 * WORDS; i += PROGRAM_THREADS)
    if (i / WORDS < n_phases) reinterpret_cast<int4*>(ring)[i] = reinterpret_cast<const int4*>(phases)[i];
  __syncthreads();
  STAMP(0);
  Feed feed;
  if (ring[0].op == OP_LINEAR) {
    feed_begin(feed, ring[0]);
    for (int i = 0; i < min(PRE_ISSUE, ring[0].depth); ++i) feed_issue(feed, ring[0], smem);
  }
  for (int p = 0; p < n_phases; ++p) {
    const Phase& ph = ring[p % 3];
#ifdef ALOFA_PROGRAM_TIMING
    if (threadIdx.x == 0) ring[p % 3].phase_index = p;
#endif
    if (p + 2 < n_phases && threadIdx.x < WORDS)  // in place by the time the barrier after this phase is passed
      reinterpret_cast<int4*>(&ring[(p + 2) % 3])[threadIdx.x] = reinterpret_cast<const int4*>(phases + p + 2)[threadIdx.x];
    switch (ph.op) {
      case OP_EMBED: embed_phase(ph, status); break;
      case OP_LINEAR: linear_phase(ph, feed, smem); break;
      case OP_ATTENTION: attention_phase(ph, phases + p, smem, tile_bar, parity, &abort_flag, status); break;
    }
    if (p + 1 < n_phases && ring[(p + 1) % 3].op == OP_LINEAR) {  // the next product's first weights, ahead of the barrier
      const Phase& next = ring[(p + 1) % 3];
      feed_begin(feed, next);
      for (int i = 0; i < min(PRE_ISSUE, next.depth); ++i) feed_issue(feed, next, smem);
    }
    STAMP(2 * p + 1);
    if (p + 1 < n_phases && !grid_barrier(sync_counter, target, status, &barrier_ok)) return;
    STAMP(2 * p + 2);
  }
}

// ---------------------------------------------------------------------------
// Host side: descriptors are filled in host memory by these functions, copied
// to the device by the caller, and run by alofa_program_run.
// ---------------------------------------------------------------------------
ALOFA_API int alofa_program_head_dim() { return HD; }
ALOFA_API int alofa_program_phase_bytes() { return (int)sizeof(Phase); }
ALOFA_API int alofa_program_max_tokens() { return 16; }

static int operand_stride(int K) {
  // rows 64 bytes apart modulo 128: the eight rows of a fragment load fall on different banks
  const int bytes = K * 2;
  return bytes + ((64 - bytes % 128) + 128) % 128;
}

// Shared memory one phase needs.
static size_t phase_smem(const Phase& ph) {
  if (ph.op == OP_LINEAR) return (size_t)ph.ring_offset + (size_t)ph.depth * ph.ring_threads * 32;
  if (ph.op == OP_ATTENTION) return (size_t)ATTN_GROUPS * (GROUP_BYTES + Q_TILE_BYTES);
  return 0;
}

ALOFA_API long long alofa_program_smem_bytes(const void* phases, int n) {
  const Phase* ph = reinterpret_cast<const Phase*>(phases);
  size_t most = 0;
  for (int i = 0; i < n; ++i) most = phase_smem(ph[i]) > most ? phase_smem(ph[i]) : most;
  return (long long)(most + 1024);
}

ALOFA_API int alofa_program_embed(void* phase, void* h, const void* table, const int* ids, const int* token_src, const int* fed, int T,
                                  int hidden, int vocab) {
  if (T <= 0 || T > 16) return ALOFA_ERR_ARGUMENT;
  Phase ph;
  memset(&ph, 0, sizeof(ph));
  ph.op = OP_EMBED;
  ph.T = T;
  ph.hidden = hidden;
  ph.vocab = vocab;
  ph.out = h;
  ph.w = (const bf16*)table;
  ph.ids = ids;
  ph.token_src = token_src;
  ph.fed = fed;
  memcpy(phase, &ph, sizeof(ph));
  return ALOFA_OK;
}

// out_cols: columns of a row of `out` (features of the product; the intermediate
// size for a gated weight).  n_rows: rows of the weight.  warps_total: warps of
// the whole grid, to choose how many warps share an item.  tiles: 8-row weight
// tiles per item (1, 2, or 0 to let this function choose).
ALOFA_API int alofa_program_linear(void* phase, int a_kind, const void* a, const float* gamma, float eps, const void* w, const float* bias,
                                   void* out, int epi, int T, int n_rows, int K, int out_cols, int tiles, void* q, void* k_cache,
                                   void* v_cache, const int* slot_map, const int* positions, const float* rope_table, int nh, int nkv,
                                   int writes, int grid) {
  if (T <= 0 || T > 16 || K <= 0 || K % 32 || n_rows <= 0 || grid <= 0) return ALOFA_ERR_ARGUMENT;
  if (((uintptr_t)w & 15) || ((uintptr_t)a & 15) || (gamma && ((uintptr_t)gamma & 15))) return ALOFA_ERR_ARGUMENT;
  Phase ph;
  memset(&ph, 0, sizeof(ph));
  ph.op = OP_LINEAR;
  ph.a_kind = a_kind;
  ph.epi = epi;
  ph.T = T;
  ph.K = K;
  ph.N = n_rows;
  ph.out_cols = out_cols;
  ph.tiles = tiles;
  ph.eps = eps;
  ph.a = a;
  ph.gamma = gamma;
  ph.w = (const bf16*)w;
  ph.bias = bias;
  ph.out = out;
  ph.a_stride = operand_stride(K);
  if (epi == E_GATED) {
    if (n_rows != 2 * out_cols || out_cols % 8) return ALOFA_ERR_ARGUMENT;
    ph.tiles = 2;
    ph.items = out_cols / 8;
  } else if (epi == E_ROPE_STORE) {
    if (HD % 16) return ALOFA_ERR_ARGUMENT;
    const int heads = nh + (writes ? 2 * nkv : 0);
    if (n_rows != heads * HD) return ALOFA_ERR_ARGUMENT;
    ph.tiles = 2;
    ph.items = heads * (HD / 16);
    ph.q = (bf16*)q;
    ph.k_cache = (bf16*)k_cache;
    ph.v_cache = (bf16*)v_cache;
    ph.slot_map = slot_map;
    ph.positions = positions;
    ph.rope_table = rope_table;
    ph.nh = nh;
    ph.nkv = writes ? nkv : 0;
    ph.writes = writes;
  } else {
    // single tiles while one round of the grid covers them (more CTAs pull on the weights), else pairs
    if (tiles == 0) tiles = (n_rows + 7) / 8 <= grid * PROGRAM_WARPS ? 1 : 2;
    if (tiles != 1 && tiles != 2) return ALOFA_ERR_ARGUMENT;
    ph.tiles = tiles;
    ph.items = (n_rows + 8 * tiles - 1) / (8 * tiles);
  }
  // the most warps per item that still finish all items in one round
  const int chunks = K / 32;
  int wpi = 1;
  for (int cand = PROGRAM_WARPS; cand > 1; cand >>= 1) {
    if (cand > chunks) continue;
    const long long per_iter = (long long)(PROGRAM_WARPS / cand) * grid;
    if (ph.items <= per_iter) {
      wpi = cand;
      break;
    }
  }
  ph.wpi = wpi;
  // the ring of the weight feed takes the shared memory above the operand and the partial tiles,
  // shared among the warps that have an item: the fewer they are, the deeper each one's ring
  const size_t area = (size_t)(T <= 8 ? 8 : 16) * ph.a_stride + (size_t)PROGRAM_WARPS * 2 * 16 * 8 * sizeof(float);
  ph.ring_offset = (int)((area + 127) & ~(size_t)127);
  const int per_cta = (ph.items + grid - 1) / grid;
  int active = per_cta * wpi < PROGRAM_WARPS ? per_cta * wpi : PROGRAM_WARPS;
  ph.ring_threads = active * 32;
  const long long room = (long long)MAX_SMEM - 1024 - ph.ring_offset;
  int depth = MAX_DEPTH;
  while (depth >= 1 && (long long)depth * ph.ring_threads * 32 > room) depth >>= 1;
  if (depth < 1) return ALOFA_ERR_ARGUMENT;
  ph.depth = depth;
  memcpy(phase, &ph, sizeof(ph));
  return ALOFA_OK;
}

// out [T, nh, HD]; partial_o [splits, T * nh, HD], partial_ml [splits, T * nh, 2] and counters [T * nkv]
// (zero before the first run) are scratch, splits = alofa_program_splits(max_context).
ALOFA_API int alofa_program_attention(void* phase, void* out, void* q, void* k_cache, void* v_cache, long long cache_slots, const int* kv_len,
                                      const int* block_table, int max_blocks, int page_size, int T, int nh, int nkv, int window, float scale,
                                      int max_context, float* partial_o, float* partial_ml, int* counters) {
  if (T <= 0 || T > 16 || nkv <= 0 || nh % nkv || nh / nkv > 16) return ALOFA_ERR_ARGUMENT;
  if ((HD != 64 && HD != 128) || page_size % BLOCK_N || cache_slots <= 0) return ALOFA_ERR_ARGUMENT;
  if (((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)q & 15)) return ALOFA_ERR_ARGUMENT;
  Phase ph;
  memset(&ph, 0, sizeof(ph));
  ph.op = OP_ATTENTION;
  ph.T = T;
  ph.nh = nh;
  ph.nkv = nkv;
  ph.window = window;
  ph.page_size = page_size;
  ph.max_blocks = max_blocks;
  ph.n_splits = (max_context + SPLIT_KEYS - 1) / SPLIT_KEYS;
  ph.scale_log2 = scale * 1.4426950408889634f;
  ph.q = (bf16*)q;
  ph.k_cache = (bf16*)k_cache;
  ph.v_cache = (bf16*)v_cache;
  ph.kv_len = kv_len;
  ph.block_table = block_table;
  ph.partial_o = partial_o;
  ph.partial_ml = partial_ml;
  ph.counters = counters;
  ph.out = out;
  if (!make_tensor_map_bf16(&ph.map_k, k_cache, (uint64_t)cache_slots, (uint64_t)nkv * HD, BLOCK_N, 64)) return ALOFA_ERR_ARGUMENT;
  if (!make_tensor_map_bf16(&ph.map_v, v_cache, (uint64_t)cache_slots, (uint64_t)nkv * HD, BLOCK_N, 64)) return ALOFA_ERR_ARGUMENT;
  memcpy(phase, &ph, sizeof(ph));
  return ALOFA_OK;
}

ALOFA_API int alofa_program_splits(int max_context) { return (max_context + SPLIT_KEYS - 1) / SPLIT_KEYS; }

// CTAs of the grid: one per SM, all resident at once.
ALOFA_API int alofa_program_grid() {
  static int grid = -1;
  if (grid < 0) {
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    grid = sms;
  }
  return grid;
}

// Run a program of n phases (device memory).  `sync_counter` is one word of
// device memory that this call zeroes; `smem_bytes` comes from
// alofa_program_smem_bytes.  The launch is cooperative: every CTA is resident,
// so the barriers between phases cannot starve.
ALOFA_API int alofa_program_run(const void* phases, int n_phases, void* sync_counter, int* status, long long smem_bytes, cudaStream_t stream) {
  if (n_phases <= 0) return ALOFA_OK;
  if (smem_bytes > MAX_SMEM) return ALOFA_ERR_ARGUMENT;
  static long long configured = -1;
  if (smem_bytes > configured) {
    if (cudaFuncSetAttribute(decode_program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) != cudaSuccess)
      return ALOFA_ERR_LAUNCH;
    configured = smem_bytes;
  }
  const int grid = alofa_program_grid();
  if (grid <= 0) return ALOFA_ERR_LAUNCH;
  if (cudaMemsetAsync(sync_counter, 0, sizeof(unsigned), stream) != cudaSuccess) return ALOFA_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(PROGRAM_THREADS);
  cfg.dynamicSmemBytes = (size_t)configured;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const Phase* list = reinterpret_cast<const Phase*>(phases);
  unsigned* counter = reinterpret_cast<unsigned*>(sync_counter);
  if (cudaLaunchKernelEx(&cfg, decode_program_kernel, list, n_phases, counter, status) != cudaSuccess) {
    cudaGetLastError();
    return ALOFA_ERR_LAUNCH;
  }
  return ALOFA_OK;
}
