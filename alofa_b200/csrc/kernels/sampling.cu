// Sampling on the device: from rows of fp32 logits to one token id per row.
//
// alofa_sample        temperature only: argmax (ties to the lowest index) when
//                     the temperature is 0, else softmax(x / T) and the inverse
//                     CDF at a given uniform number.
// alofa_sample_chain  the reference's whole chain in its order
//                     (src/alofa/runtime/sampler.mojo:308-481): logit bias,
//                     repetition penalty, frequency and presence penalties,
//                     temperature, top-k (ties at the k-th value survive),
//                     top-p (smallest prefix in descending order, ties by
//                     lower index, reaching top_p), min-p, softmax, inverse CDF.
//
// One block of 1024 threads per row.  Every sum is taken in an order fixed by
// the vocabulary size, so a row's draw does not depend on the batch around it.
// The reference accumulates probabilities in f64; here they are fp32, so a
// cumulative weight within fp32 rounding of a threshold may fall on the other
// side of it.
#include "common.cuh"
#include "no_alloc.h"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned sort_key(float x) {
  const unsigned u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

// Largest value of x[0..n), ties to the lowest index.  All threads get it.
__device__ ArgMax block_argmax(const float* x, int n, float* sval, int* sidx) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = tid; i < n; i += blockDim.x) best = better(best, ArgMax{x[i], i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  __syncthreads();
  if (lane == 0) {
    sval[warp] = best.v;
    sidx[warp] = best.i;
  }
  __syncthreads();
  ArgMax out{sval[0], sidx[0]};
  for (int w = 1; w < nwarp; ++w) out = better(out, ArgMax{sval[w], sidx[w]});
  if (out.i == 0x7fffffff) out.i = 0;  // a row of -inf or NaN: fall back to index 0
  return out;
}

// Inclusive scan of one value per thread across the block (blockDim.x values).
// Returns this thread's inclusive prefix; *total gets the block's sum.
__device__ __forceinline__ float block_scan(float v, float* swarp, float* total) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
  float scan = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, scan, o);
    if (lane >= o) scan += n;
  }
  __syncthreads();
  if (lane == 31) swarp[warp] = scan;
  __syncthreads();
  float before = 0.f, all = 0.f;
  for (int w = 0; w < nwarp; ++w) {
    if (w < warp) before += swarp[w];
    all += swarp[w];
  }
  *total = all;
  return before + scan;
}

// First index whose running sum of p exceeds `target`, or -1.  p(i) is given by
// a functor so that callers need no probability array.
template <typename F>
__device__ int inverse_cdf(F p_of, int n, float target, float* swarp, int* chosen) {
  const int tid = threadIdx.x;
  if (tid == 0) *chosen = 0x7fffffff;
  float running = 0.f;
  __syncthreads();
  for (int c0 = 0; c0 < n; c0 += blockDim.x) {
    const int i = c0 + tid;
    const float p = i < n ? p_of(i) : 0.f;
    float total;
    const float cum = running + block_scan(p, swarp, &total);
    if (i < n && p > 0.f && target < cum) atomicMin(chosen, i);
    __syncthreads();
    if (*chosen != 0x7fffffff) break;
    running += total;
  }
  __syncthreads();
  return *chosen == 0x7fffffff ? -1 : *chosen;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(int* __restrict__ tokens, const float* __restrict__ logits,
                                                                const float* __restrict__ temperature,
                                                                const float* __restrict__ uniform, int vocab) {
  __shared__ float scratch[32];
  __shared__ float sval[32];
  __shared__ int sidx[32];
  __shared__ int chosen;
  const int r = blockIdx.x, tid = threadIdx.x;
  pdl_begin();
  const float* x = logits + (size_t)r * vocab;
  const ArgMax top = block_argmax(x, vocab, sval, sidx);
  const float temp = temperature ? temperature[r] : 0.f;
  if (!(temp > 0.f)) {
    if (tid == 0) tokens[r] = top.i;
    return;
  }
  const float xmax = top.v;
  float part = 0.f;
  for (int i = tid; i < vocab; i += blockDim.x) part += expf((x[i] - xmax) / temp);
  const float total = block_sum(part, scratch);
  auto p_of = [&](int i) { return expf((x[i] - xmax) / temp); };
  const int pick = inverse_cdf(p_of, vocab, uniform[r] * total, scratch, &chosen);
  if (tid == 0) tokens[r] = pick >= 0 ? pick : top.i;
}

// Greedy rows in two stages, so that a few rows still use many SMs: stage 1
// finds the best entry of each of ARGMAX_PARTS slices of a row, stage 2 the
// best of those (ties to the lowest index in both).  Rows whose temperature is
// positive are left to sample_kernel.
#define ARGMAX_PARTS 32

__global__ void __launch_bounds__(256) argmax_parts_kernel(float* __restrict__ part_val, int* __restrict__ part_idx,
                                                           const float* __restrict__ logits, int vocab) {
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const int r = blockIdx.y, part = blockIdx.x;
  pdl_begin();
  const int per = (vocab + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
  const int lo = part * per, hi = min(vocab, lo + per);
  const float* x = logits + (size_t)r * vocab;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = lo + tid; i < hi; i += blockDim.x) best = better(best, ArgMax{x[i], i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (lane == 0) {
    sval[warp] = best.v;
    sidx[warp] = best.i;
  }
  __syncthreads();
  if (tid == 0) {
    ArgMax out{sval[0], sidx[0]};
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) out = better(out, ArgMax{sval[w], sidx[w]});
    part_val[r * ARGMAX_PARTS + part] = out.v;
    part_idx[r * ARGMAX_PARTS + part] = out.i;
  }
}

__global__ void argmax_final_kernel(int* __restrict__ tokens, const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                    const float* __restrict__ temperature) {
  const int r = blockIdx.x, lane = threadIdx.x;  // one warp per row
  pdl_begin();
  // every row gets its largest logit; rows with a positive temperature are overwritten by
  // sample_hot_kernel when it runs, and keep the largest logit when the caller promised no such row
  ArgMax best{part_val[r * ARGMAX_PARTS + lane], part_idx[r * ARGMAX_PARTS + lane]};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (lane == 0) tokens[r] = best.i == 0x7fffffff ? 0 : best.i;
}

// Rows with a positive temperature only (greedy rows return at once).
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_hot_kernel(int* __restrict__ tokens, const float* __restrict__ logits,
                                                                    const float* __restrict__ temperature,
                                                                    const float* __restrict__ uniform, int vocab) {
  __shared__ float scratch[32];
  __shared__ float sval[32];
  __shared__ int sidx[32];
  __shared__ int chosen;
  const int r = blockIdx.x, tid = threadIdx.x;
  pdl_begin();
  const float temp = temperature[r];
  if (!(temp > 0.f)) return;
  const float* x = logits + (size_t)r * vocab;
  const ArgMax top = block_argmax(x, vocab, sval, sidx);
  const float xmax = top.v;
  float part = 0.f;
  for (int i = tid; i < vocab; i += blockDim.x) part += expf((x[i] - xmax) / temp);
  const float total = block_sum(part, scratch);
  auto p_of = [&](int i) { return expf((x[i] - xmax) / temp); };
  const int pick = inverse_cdf(p_of, vocab, uniform[r] * total, scratch, &chosen);
  if (tid == 0) tokens[r] = pick >= 0 ? pick : top.i;
}

// scratch: n_rows * ARGMAX_PARTS floats followed by as many ints, or null (then
// one block per row does everything).  any_hot: some row has temperature > 0.
ALOFA_API int alofa_sample(int* tokens, const float* logits, const float* temperature, const float* uniform, int n_rows,
                           int vocab, void* scratch, int any_hot, cudaStream_t stream) {
  if (n_rows <= 0) return ALOFA_OK;
  ALOFA_PREFER_MAX_SHARED(sample_kernel);
  if (!scratch) {
    launch_dep(sample_kernel, n_rows, SAMPLE_THREADS, 0, stream, tokens, logits, temperature, uniform, vocab);
    return launch_status();
  }
  if (any_hot && temperature && !uniform) return ALOFA_ERR_ARGUMENT;  // a draw needs its uniform number
  float* part_val = (float*)scratch;
  int* part_idx = (int*)(part_val + (size_t)n_rows * ARGMAX_PARTS);
  ALOFA_PREFER_MAX_SHARED(argmax_parts_kernel);
  ALOFA_PREFER_MAX_SHARED(argmax_final_kernel);
  ALOFA_PREFER_MAX_SHARED(sample_hot_kernel);
  launch_dep(argmax_parts_kernel, dim3(ARGMAX_PARTS, n_rows), 256, 0, stream, part_val, part_idx, logits, vocab);
  launch_dep(argmax_final_kernel, n_rows, 32, 0, stream, tokens, part_val, part_idx, temperature);
  if (any_hot && temperature && uniform) launch_dep(sample_hot_kernel, n_rows, SAMPLE_THREADS, 0, stream, tokens, logits, temperature, uniform, vocab);
  return launch_status();
}

// ---------------------------------------------------------------------------
// The same without a caller-provided scratch buffer (see no_alloc.h): the
// stage-1 results live in an array that is part of the library image.
// ---------------------------------------------------------------------------
static __device__ __align__(256) float g_noalloc_scratch[2 * ALOFA_NOALLOC_MAX_ROWS * ARGMAX_PARTS];

// Device address of g_noalloc_scratch on the current device, looked up once per
// device.  In host code the array's name is only a handle for this lookup; it
// is not an address a kernel could use.  Two host threads that make their first
// call on a device at the same moment both look the address up and both store
// the same value: harmless, and not guarded.
static float* noalloc_scratch_address() {
  static float* address[64] = {nullptr};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
  if (!address[device]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) {
      cudaGetLastError();  // leave no sticky error behind
      return nullptr;
    }
    address[device] = static_cast<float*>(ptr);
  }
  return address[device];
}

ALOFA_API int alofa_sample_noalloc_max_rows(void) { return ALOFA_NOALLOC_MAX_ROWS; }

ALOFA_API int alofa_sample_noalloc(int* tokens, const float* logits, const float* temperature, const float* uniform, int n_rows, int vocab,
                                   int any_hot, cudaStream_t stream) {
  if (n_rows <= 0) return ALOFA_OK;
  if (n_rows > ALOFA_NOALLOC_MAX_ROWS) return ALOFA_NOALLOC_TOO_MANY_ROWS;
  if (!tokens || !logits || vocab <= 0) return ALOFA_ERR_ARGUMENT;
  if (any_hot && temperature && !uniform) return ALOFA_ERR_ARGUMENT;  // a draw needs its uniform number
  float* scratch = noalloc_scratch_address();
  if (!scratch) return ALOFA_ERR_LAUNCH;
  float* part_val = scratch;
  int* part_idx = reinterpret_cast<int*>(scratch + (size_t)n_rows * ARGMAX_PARTS);
  argmax_parts_kernel<<<dim3(ARGMAX_PARTS, n_rows), 256, 0, stream>>>(part_val, part_idx, logits, vocab);
  argmax_final_kernel<<<n_rows, 32, 0, stream>>>(tokens, part_val, part_idx, temperature);
  if (any_hot && temperature && uniform) sample_hot_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(tokens, logits, temperature, uniform, vocab);
  return launch_status();
}

// ---------------------------------------------------------------------------
// The whole chain.
// ---------------------------------------------------------------------------
struct ChainShared {
  float scratch[32];
  float sval[32];
  int sidx[32];
  int hist[256];
  int chosen;
  unsigned prefix;
  int remaining;
};

__device__ int block_count(int v, ChainShared& sh) {
  // integer sum over the block, exact
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) sh.sidx[warp] = v;
  __syncthreads();
  int total = 0;
  for (int w = 0; w < nwarp; ++w) total += sh.sidx[w];
  return total;
}

// Key of the n-th largest value (1-based) of vals[0..V): radix select, 8 bits a
// pass, with exact integer histograms.
__device__ unsigned nth_largest_key(const float* vals, int V, int n, ChainShared& sh) {
  const int tid = threadIdx.x;
  unsigned prefix = 0, mask = 0;
  int remaining = n;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = tid; b < 256; b += blockDim.x) sh.hist[b] = 0;
    __syncthreads();
    for (int i = tid; i < V; i += blockDim.x) {
      const unsigned k = sort_key(vals[i]);
      if ((k & mask) == prefix) atomicAdd(&sh.hist[(k >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int left = remaining;
      int b = 255;
      for (; b > 0; --b) {
        if (sh.hist[b] >= left) break;
        left -= sh.hist[b];
      }
      sh.prefix = prefix | ((unsigned)b << shift);
      sh.remaining = left;
    }
    __syncthreads();
    prefix = sh.prefix;
    remaining = sh.remaining;
    mask |= 255u << shift;
    __syncthreads();
  }
  return prefix;
}

// Keep the first n entries in descending order of value, ties by lower index;
// everything else becomes -inf.
__device__ void keep_first_n(float* vals, int V, int n, ChainShared& sh) {
  if (n >= V) return;
  const int tid = threadIdx.x;
  const unsigned t = nth_largest_key(vals, V, n, sh);
  int above = 0;
  for (int i = tid; i < V; i += blockDim.x) above += sort_key(vals[i]) > t ? 1 : 0;
  above = block_count(above, sh);
  const int ties_kept = n - above;
  int running = 0;
  for (int c0 = 0; c0 < V; c0 += blockDim.x) {
    const int i = c0 + tid;
    const unsigned k = i < V ? sort_key(vals[i]) : 0u;
    const bool tie = i < V && k == t;
    float total;
    const float incl = block_scan(tie ? 1.f : 0.f, sh.scratch, &total);  // counts below 2^24 are exact in fp32
    const int rank = running + (int)incl - 1;
    if (i < V && (k < t || (tie && rank >= ties_kept))) vals[i] = -INFINITY;
    running += (int)total;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_chain_kernel(
    int* __restrict__ tokens, const float* __restrict__ logits, float* __restrict__ work, int vocab,
    const float* __restrict__ fparams,  // [rows, 8]: temperature, top_p, min_p, repetition, frequency, presence, uniform, -
    const int* __restrict__ iparams,    // [rows, 4]: top_k, min_tokens_to_keep, -, -
    const int* __restrict__ bias_start, const int* __restrict__ bias_index, const float* __restrict__ bias_value,
    const int* __restrict__ hist_start, const int* __restrict__ hist_token, const int* __restrict__ hist_count) {
  __shared__ ChainShared sh;
  pdl_begin();
  const int r = blockIdx.x, tid = threadIdx.x, V = vocab;
  const float* x = logits + (size_t)r * V;
  float* vals = work + (size_t)r * V;
  const float temp = fparams[r * 8 + 0], top_p = fparams[r * 8 + 1], min_p = fparams[r * 8 + 2];
  const float rep = fparams[r * 8 + 3], freq = fparams[r * 8 + 4], pres = fparams[r * 8 + 5], u = fparams[r * 8 + 6];
  const int top_k = iparams[r * 4 + 0];
  int keep = iparams[r * 4 + 1];
  if (keep < 1) keep = 1;

  for (int i = tid; i < V; i += blockDim.x) vals[i] = x[i];
  __syncthreads();
  for (int j = bias_start[r] + tid; j < bias_start[r + 1]; j += blockDim.x) {
    const int t = bias_index[j];
    if (t >= 0 && t < V) vals[t] += bias_value[j];
  }
  __syncthreads();
  for (int j = hist_start[r] + tid; j < hist_start[r + 1]; j += blockDim.x) {
    const int t = hist_token[j];
    if (t < 0 || t >= V) continue;
    float v = vals[t];
    if (rep != 1.0f) v = v < 0.f ? v * rep : v / rep;
    v -= freq * (float)hist_count[j];
    v -= pres;
    vals[t] = v;
  }
  __syncthreads();
  if (!(temp > 0.f)) {
    const ArgMax top = block_argmax(vals, V, sh.sval, sh.sidx);
    if (tid == 0) tokens[r] = top.i;
    return;
  }
  if (temp != 1.0f) {
    for (int i = tid; i < V; i += blockDim.x) vals[i] = vals[i] / temp;
    __syncthreads();
  }
  if (top_k > 0 && top_k < V) {
    const unsigned kth = nth_largest_key(vals, V, top_k, sh);
    for (int i = tid; i < V; i += blockDim.x)
      if (sort_key(vals[i]) < kth) vals[i] = -INFINITY;
    __syncthreads();
  }
  if (top_p < 1.0f) {
    const ArgMax top = block_argmax(vals, V, sh.sval, sh.sidx);
    float part = 0.f;
    for (int i = tid; i < V; i += blockDim.x) part += expf(vals[i] - top.v);
    const float total = block_sum(part, sh.scratch);
    const float target = top_p * total;
    // largest key t with mass(key >= t) >= target, by bisection over the key bits
    unsigned t = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned cand = t | (1u << bit);
      float m = 0.f;
      for (int i = tid; i < V; i += blockDim.x)
        if (sort_key(vals[i]) >= cand) m += expf(vals[i] - top.v);
      m = block_sum(m, sh.scratch);
      if (m >= target) t = cand;
    }
    float above_mass = 0.f, tie_p = 0.f;
    int above = 0, ties = 0;
    for (int i = tid; i < V; i += blockDim.x) {
      const unsigned k = sort_key(vals[i]);
      if (k > t) {
        above_mass += expf(vals[i] - top.v);
        above++;
      } else if (k == t) {
        ties++;
        tie_p = expf(vals[i] - top.v);
      }
    }
    above_mass = block_sum(above_mass, sh.scratch);
    tie_p = block_max(tie_p, sh.scratch);
    above = block_count(above, sh);
    ties = block_count(ties, sh);
    int c = ties;
    if (tie_p > 0.f) {
      c = (int)ceilf((target - above_mass) / tie_p);
      if (c < 1) c = 1;
      if (c > ties) c = ties;
    }
    int taken = above + c;
    if (taken < keep) taken = keep;
    keep_first_n(vals, V, taken, sh);
  }
  if (min_p > 0.0f) {
    const ArgMax top = block_argmax(vals, V, sh.sval, sh.sidx);
    if (keep <= 1) {
      // p_i / p_max = exp(v_i - v_max); the maximum itself always stays
      for (int i = tid; i < V; i += blockDim.x)
        if (expf(vals[i] - top.v) < min_p) vals[i] = -INFINITY;
    } else {
      // the first `keep` entries in sorted order are protected
      const int n = keep < V ? keep : V;
      const unsigned t = nth_largest_key(vals, V, n, sh);
      int above = 0;
      for (int i = tid; i < V; i += blockDim.x) above += sort_key(vals[i]) > t ? 1 : 0;
      above = block_count(above, sh);
      const int ties_kept = n - above;
      int running = 0;
      for (int c0 = 0; c0 < V; c0 += blockDim.x) {
        const int i = c0 + tid;
        const unsigned k = i < V ? sort_key(vals[i]) : 0u;
        const bool tie = i < V && k == t;
        float total;
        const float incl = block_scan(tie ? 1.f : 0.f, sh.scratch, &total);
        const int rank = running + (int)incl - 1;
        const bool guarded = i < V && (k > t || (tie && rank < ties_kept));
        if (i < V && !guarded && expf(vals[i] - top.v) < min_p) vals[i] = -INFINITY;
        running += (int)total;
      }
    }
    __syncthreads();
  }
  const ArgMax top = block_argmax(vals, V, sh.sval, sh.sidx);
  float part = 0.f;
  for (int i = tid; i < V; i += blockDim.x) part += expf(vals[i] - top.v);
  const float total = block_sum(part, sh.scratch);
  auto p_of = [&](int i) { return expf(vals[i] - top.v); };
  const int pick = inverse_cdf(p_of, V, u * total, sh.scratch, &sh.chosen);
  if (tid == 0) tokens[r] = pick >= 0 ? pick : top.i;
}

// work: fp32 [n_rows, vocab] scratch.  Lists are CSR: *_start has n_rows + 1 entries.
ALOFA_API int alofa_sample_chain(int* tokens, const float* logits, float* work, int n_rows, int vocab, const float* fparams,
                                 const int* iparams, const int* bias_start, const int* bias_index, const float* bias_value,
                                 const int* hist_start, const int* hist_token, const int* hist_count, cudaStream_t stream) {
  if (n_rows <= 0) return ALOFA_OK;
  if (vocab >= (1 << 24)) return ALOFA_ERR_ARGUMENT;
  launch_dep(sample_chain_kernel, n_rows, SAMPLE_THREADS, 0, stream, tokens, logits, work, vocab, fparams, iparams, bias_start,
                                                             bias_index, bias_value, hist_start, hist_token, hist_count);
  return launch_status();
}
