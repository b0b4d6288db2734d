// Kernels that take every size: the true 32-bit path of the whole model, and
// the place the bfloat16 path falls back to for shapes its fast kernels refuse.
//
// Everything accumulates in fp32 with plain FMA (no tensor cores, no TF32, no
// approximate intrinsics; this file is compiled without fast-math).  For every
// output element the order of additions is fixed by the problem sizes alone,
// never by which other rows share the launch, so a row's result does not
// depend on how a batch was put together.
//
// Arithmetic follows the reference's scalar kernels
// (src/alofa/kernels/cpu/scalar.mojo:93-470, paged.mojo:208-336,
// segments.mojo:48-130) with fp32 instead of f64 accumulators.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = table[ids[t], :] widened to fp32.
// An id outside [0, vocab) writes zeros and raises the status flag.
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_gather_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                    const int* __restrict__ ids, const int* __restrict__ src, const int* __restrict__ fed,
                                    int hidden, int vocab, int* status) {
  pdl_begin();
  const int t = blockIdx.x;
  int id = ids[t];
  if (src && src[t] >= 0) id = fed[src[t]];  // the token an earlier step sampled, still on the device
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0 && status) atomicExch(status, 1);
  const TW* row = table + (size_t)(ok ? id : 0) * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) out[(size_t)t * hidden + c] = ok ? to_f(row[c]) : 0.f;
}

// src (optional): per token, -1 to take ids[t], else the row of `fed` (tokens
// sampled by the step before, on the device) that holds the id.
ALOFA_API int alofa_embed_gather(void* out, const void* table, const int* ids, const int* src, const int* fed, int n_tokens, int hidden,
                                 int vocab, int table_bf16, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  ALOFA_PREFER_MAX_SHARED(embed_gather_kernel<bf16>);
  ALOFA_PREFER_MAX_SHARED(embed_gather_kernel<float>);
  if (table_bf16)
    launch_dep(embed_gather_kernel<bf16>, n_tokens, 256, 0, stream, (float*)out, (const bf16*)table, ids, src, fed, hidden, vocab, status);
  else
    launch_dep(embed_gather_kernel<float>, n_tokens, 256, 0, stream, (float*)out, (const float*)table, ids, src, fed, hidden, vocab, status);
  return launch_status();
}

// ---------------------------------------------------------------------------
// RMSNorm: y = x * (1/sqrt(mean(x^2) + eps)) * w, one block per output row.
// `rows` (optional) picks the input row of each output row.
// ---------------------------------------------------------------------------
template <typename TO>
__global__ void rmsnorm_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                               const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float v = xr[c];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) out[(size_t)r * hidden + c] = from_f<TO>(xr[c] * scale * w[c]);
}

ALOFA_API int alofa_rmsnorm(void* out, const void* x, const void* w, const int* rows, int n_rows, int hidden, float eps,
                            int out_bf16, cudaStream_t stream) {
  if (n_rows <= 0) return ALOFA_OK;
  if (out_bf16)
    rmsnorm_kernel<bf16><<<n_rows, 256, 0, stream>>>((bf16*)out, (const float*)x, (const float*)w, rows, hidden, eps);
  else
    rmsnorm_kernel<float><<<n_rows, 256, 0, stream>>>((float*)out, (const float*)x, (const float*)w, rows, hidden, eps);
  return launch_status();
}

// ---------------------------------------------------------------------------
// Matrix product y = x W^T (+ bias), W row-major [N, K].
//   EPI_STORE    out[m, n] = acc
//   EPI_RESIDUAL out[m, n] += acc        (out is the fp32 residual stream)
//   EPI_GATED    W holds [gate; up] (2N rows): out[m, n] = silu(gate) * up
// 64x64 tile, 16-deep slices, 256 threads with 4x4 outputs each; every output
// is summed by one thread over k ascending.
// ---------------------------------------------------------------------------
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_GATED = 2 };

template <typename TA, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256) gemm_generic_kernel(TO* __restrict__ out, const TA* __restrict__ x,
                                                           const TW* __restrict__ w, const float* __restrict__ bias, int M,
                                                           int N, int K) {
  constexpr int BM = 64, BN = 64, BK = 16;
  constexpr int NW = (EPI == EPI_GATED) ? 2 : 1;
  __shared__ float xs[BK][BM + 1];
  __shared__ float ws[NW][BK][BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[NW][4][4];
#pragma unroll
  for (int a = 0; a < NW; ++a)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[a][i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + 256 * i;
      const int r = e >> 4, k = e & 15;
      const int gm = m0 + r, gk = k0 + k;
      xs[k][r] = (gm < M && gk < K) ? to_f(x[(size_t)gm * K + gk]) : 0.f;
      const int gn = n0 + r;
#pragma unroll
      for (int a = 0; a < NW; ++a)
        ws[a][k][r] = (gn < N && gk < K) ? to_f(w[((size_t)a * N + gn) * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float xv[4], wv[NW][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = xs[k][ty + 16 * i];
#pragma unroll
      for (int a = 0; a < NW; ++a)
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[a][j] = ws[a][k][tx + 16 * j];
#pragma unroll
      for (int a = 0; a < NW; ++a)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[a][i][j] = fmaf(xv[i], wv[a][j], acc[a][i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty + 16 * i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx + 16 * j;
      if (gn >= N) continue;
      const size_t o = (size_t)gm * N + gn;
      if (EPI == EPI_GATED) {
        float g = acc[0][i][j], u = acc[NW - 1][i][j];
        if (bias) {
          g += bias[gn];
          u += bias[N + gn];
        }
        out[o] = from_f<TO>(g / (1.0f + expf(-g)) * u);
      } else {
        float v = acc[0][i][j];
        if (bias) v += bias[gn];
        if (EPI == EPI_RESIDUAL)
          out[o] = from_f<TO>(to_f(out[o]) + v);
        else
          out[o] = from_f<TO>(v);
      }
    }
  }
}

template <typename TA, typename TW, typename TO>
static int gemm_generic_launch(void* out, const void* x, const void* w, const float* bias, int M, int N, int K, int epi,
                               cudaStream_t stream) {
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  if (epi == EPI_STORE)
    gemm_generic_kernel<TA, TW, TO, EPI_STORE><<<grid, 256, 0, stream>>>((TO*)out, (const TA*)x, (const TW*)w, bias, M, N, K);
  else if (epi == EPI_RESIDUAL)
    gemm_generic_kernel<TA, TW, TO, EPI_RESIDUAL><<<grid, 256, 0, stream>>>((TO*)out, (const TA*)x, (const TW*)w, bias, M, N, K);
  else if (epi == EPI_GATED)
    gemm_generic_kernel<TA, TW, TO, EPI_GATED><<<grid, 256, 0, stream>>>((TO*)out, (const TA*)x, (const TW*)w, bias, M, N, K);
  else
    return ALOFA_ERR_ARGUMENT;
  return launch_status();
}

// dtype flags: 0 = fp32, 1 = bf16.  N is the number of output columns (for
// EPI_GATED the weight has 2N rows).  EPI_RESIDUAL requires an fp32 output.
ALOFA_API int alofa_gemm_generic(void* out, const void* x, const void* w, const void* bias, int M, int N, int K, int epi,
                                 int x_bf16, int w_bf16, int out_bf16, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return ALOFA_OK;
  if (K <= 0) return ALOFA_ERR_ARGUMENT;
  if (epi == EPI_RESIDUAL && out_bf16) return ALOFA_ERR_ARGUMENT;
  const float* b = (const float*)bias;
  const int key = (x_bf16 ? 4 : 0) | (w_bf16 ? 2 : 0) | (out_bf16 ? 1 : 0);
  switch (key) {
    case 0: return gemm_generic_launch<float, float, float>(out, x, w, b, M, N, K, epi, stream);
    case 1: return gemm_generic_launch<float, float, bf16>(out, x, w, b, M, N, K, epi, stream);
    case 2: return gemm_generic_launch<float, bf16, float>(out, x, w, b, M, N, K, epi, stream);
    case 3: return gemm_generic_launch<float, bf16, bf16>(out, x, w, b, M, N, K, epi, stream);
    case 4: return gemm_generic_launch<bf16, float, float>(out, x, w, b, M, N, K, epi, stream);
    case 5: return gemm_generic_launch<bf16, float, bf16>(out, x, w, b, M, N, K, epi, stream);
    case 6: return gemm_generic_launch<bf16, bf16, float>(out, x, w, b, M, N, K, epi, stream);
    default: return gemm_generic_launch<bf16, bf16, bf16>(out, x, w, b, M, N, K, epi, stream);
  }
}

// ---------------------------------------------------------------------------
// Rotary position encoding (NeoX halves) on q and k, and the cache write.
//   qkv     [T, (nh + 2 nkv) * hd]  q heads, then k heads, then v heads
//   q_out   [T, nh * hd]            rotated queries
//   k_cache, v_cache [slots, nkv, hd]; slot_map[t] is the physical slot of
//   token t (page * page_size + offset), or < 0 to write nothing.
//   cos_sin [max_pos, rot/2, 2] fp32 (cos, sin).  rot == 0: no rotation.
// y[d] = a cos - b sin, y[d + rot/2] = b cos + a sin, a = x[d], b = x[d + rot/2];
// dims >= rot pass through.  The products are fp32.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  const T* __restrict__ qkv, const float* __restrict__ cos_sin,
                                  const int* __restrict__ positions, const int* __restrict__ slot_map, int nh, int nkv,
                                  int hd, int rot, int write_cache) {
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // 0..nh-1 q, nh..nh+nkv-1 k, then v
  const int pos = positions[t];
  const int half = rot >> 1;
  const T* src = qkv + ((size_t)t * (nh + 2 * nkv) + head) * hd;
  T* dst;
  bool rotate = true;
  if (head < nh) {
    dst = q_out + ((size_t)t * nh + head) * hd;
  } else {
    if (!write_cache) return;
    const int slot = slot_map[t];
    if (slot < 0) return;
    if (head < nh + nkv) {
      dst = k_cache + ((size_t)slot * nkv + (head - nh)) * hd;
    } else {
      dst = v_cache + ((size_t)slot * nkv + (head - nh - nkv)) * hd;
      rotate = false;
    }
  }
  const float* cs = cos_sin + (size_t)pos * rot;  // rot/2 pairs
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float y;
    if (rotate && d < rot) {
      const int i = d < half ? d : d - half;
      const float c = cs[2 * i], s = cs[2 * i + 1];
      const float a = to_f(src[i]), b = to_f(src[i + half]);
      y = d < half ? (a * c - b * s) : (b * c + a * s);
    } else {
      y = to_f(src[d]);
    }
    dst[d] = from_f<T>(y);
  }
}

ALOFA_API int alofa_rope_store(void* q_out, void* k_cache, void* v_cache, const void* qkv, const float* cos_sin,
                               const int* positions, const int* slot_map, int n_tokens, int nh, int nkv, int hd, int rot,
                               int write_cache, int is_bf16, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (rot < 0 || rot > hd || (rot & 1)) return ALOFA_ERR_ARGUMENT;
  dim3 grid(n_tokens, nh + 2 * nkv);
  const int threads = hd <= 32 ? 32 : (hd <= 64 ? 64 : 128);
  if (is_bf16)
    rope_store_kernel<bf16><<<grid, threads, 0, stream>>>((bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, (const bf16*)qkv,
                                                           cos_sin, positions, slot_map, nh, nkv, hd, rot, write_cache);
  else
    rope_store_kernel<float><<<grid, threads, 0, stream>>>((float*)q_out, (float*)k_cache, (float*)v_cache,
                                                            (const float*)qkv, cos_sin, positions, slot_map, nh, nkv, hd,
                                                            rot, write_cache);
  return launch_status();
}

// ---------------------------------------------------------------------------
// Causal grouped-query attention over the paged cache, one block per
// (token, query head).  The query at position P of request r sees the keys
// max(0, P - window + 1) .. P (window <= 0: all), found through
// block_table[r][j / page_size].  Keys are taken in chunks of 128 whose
// boundaries depend on the key index only; within a chunk each thread scores
// one key, the block takes max and sum in a fixed order, and the value sum is
// rescaled as in streaming softmax.  score = dot * scale, all in fp32.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) paged_attention_generic_kernel(
    T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
    int max_blocks, int page_size, int nh, int nkv, int hd, int window, float scale) {
  extern __shared__ float smem[];
  float* qs = smem;          // hd
  float* ps = smem + hd;     // 128
  __shared__ float scratch[32];
  __shared__ int pages[128];
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int kvh = h / (nh / nkv);
  const int P = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * max_blocks;
  for (int d = tid; d < hd; d += 128) qs[d] = to_f(q[((size_t)t * nh + h) * hd + d]);
  int first = 0;
  if (window > 0 && P - window + 1 > 0) first = P - window + 1;
  float m = -INFINITY, l = 0.f;
  float acc0 = 0.f, acc1 = 0.f;  // dims tid and tid + 128
  __syncthreads();
  for (int c0 = (first / 128) * 128; c0 <= P; c0 += 128) {
    const int j = c0 + tid;
    const bool visible = j >= first && j <= P;
    float s = -INFINITY;
    int slot = -1;
    if (visible) {
      const int page = table[j / page_size];
      slot = page * page_size + (j % page_size);
      const T* kr = k_cache + ((size_t)slot * nkv + kvh) * hd;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_f(kr[d]), dot);
      s = dot * scale;
    }
    pages[tid] = slot;
    const float cmax = block_max(s, scratch);
    const float m_new = fmaxf(m, cmax);
    const float p = visible ? expf(s - m_new) : 0.f;
    ps[tid] = p;
    const float csum = block_sum(p, scratch);  // also orders the writes of ps / pages
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + csum;
    acc0 *= corr;
    acc1 *= corr;
    const int n_in = min(128, P - c0 + 1);
    for (int i = 0; i < n_in; ++i) {
      const int sl = pages[i];
      if (sl < 0) continue;
      const T* vr = v_cache + ((size_t)sl * nkv + kvh) * hd;
      const float pi = ps[i];
      if (tid < hd) acc0 = fmaf(pi, to_f(vr[tid]), acc0);
      if (tid + 128 < hd) acc1 = fmaf(pi, to_f(vr[tid + 128]), acc1);
    }
    m = m_new;
    __syncthreads();
  }
  T* o = out + ((size_t)t * nh + h) * hd;
  if (tid < hd) o[tid] = from_f<T>(acc0 / l);
  if (tid + 128 < hd) o[tid + 128] = from_f<T>(acc1 / l);
}

ALOFA_API int alofa_paged_attention_generic(void* out, const void* q, const void* k_cache, const void* v_cache,
                                            const int* positions, const int* seq_of_token, const int* block_table,
                                            int max_blocks, int page_size, int n_tokens, int nh, int nkv, int hd,
                                            int window, float scale, int is_bf16, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (hd <= 0 || hd > 256 || nkv <= 0 || nh % nkv != 0 || page_size <= 0) return ALOFA_ERR_ARGUMENT;
  dim3 grid(n_tokens, nh);
  const size_t smem = (size_t)(hd + 128) * sizeof(float);
  if (is_bf16)
    paged_attention_generic_kernel<bf16><<<grid, 128, smem, stream>>>(
        (bf16*)out, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, positions, seq_of_token, block_table,
        max_blocks, page_size, nh, nkv, hd, window, scale);
  else
    paged_attention_generic_kernel<float><<<grid, 128, smem, stream>>>(
        (float*)out, (const float*)q, (const float*)k_cache, (const float*)v_cache, positions, seq_of_token, block_table,
        max_blocks, page_size, nh, nkv, hd, window, scale);
  return launch_status();
}
