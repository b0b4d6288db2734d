// Memory-bound kernels of the bfloat16 path, vectorised, with the second stage
// of split-K folded in: where a matrix product left partial sums
// [splits, T, N] (fp32), the consumer adds them up in split order while it
// reads, so the sum never makes a round trip through memory of its own.
//
//   alofa_norm_fused        h += bias + sum_z partial[z]  (optional), then
//                           x = h / sqrt(mean(h^2) + eps) * w      (RMSNorm,
//                           src/alofa/kernels/cpu/scalar.mojo:93-129)
//   alofa_stream_settle     h = base + accumulator: the residual stream of a small decode
//                           step brought back to one fp32 tensor (see STREAM_SCALE)
//   alofa_rope_store_fused  qkv = bias + sum_z partial[z] (or a bf16 tensor),
//                           NeoX rotation of q and k, k and v written to
//                           their cache slots (scalar.mojo:283-344,
//                           paged.mojo:208-246)
#include "common.cuh"

// ---------------------------------------------------------------------------
// RMSNorm with optional split-K reduction into the residual stream.
// One block per output row; hidden % 4 == 0.
// ---------------------------------------------------------------------------
// B partial sums of one group of four values: their loads in flight together, added in split order.
template <int B>
__device__ __forceinline__ void add_splits(float4& v, const float4* p, int z0, int splits, size_t plane4) {
  float4 a[B];
#pragma unroll
  for (int i = 0; i < B; ++i) a[i] = (z0 + i < splits) ? p[(size_t)(z0 + i) * plane4] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < B; ++i) {
    v.x += a[i].x;
    v.y += a[i].y;
    v.z += a[i].z;
    v.w += a[i].w;
  }
}

// The residual stream of a decode step of a few tokens may stand as a base tensor plus a
// 64-bit fixed-point accumulator (units of 2^-32) into which the products that add to the
// stream sent their split sums with atomic adds: integer addition does not depend on the
// order of arrival, so the sum is the same every run; base + accumulator is taken in fp32
// (stream_add in common.cuh), here or in the product that reads the stream next (gemm_tc.cu,
// B_NORMED).
__device__ __forceinline__ float4 stream_value(float4 v, const longlong2* acc2) {
  const longlong2 a = acc2[0], b = acc2[1];
  v.x = stream_add(v.x, a.x);
  v.y = stream_add(v.y, a.y);
  v.z = stream_add(v.z, b.x);
  v.w = stream_add(v.w, b.y);
  return v;
}

// h[t] = base[t] + acc[t] for every row, and both accumulators left zero.
__global__ void stream_settle_kernel(float* __restrict__ h, const float* __restrict__ base, long long* __restrict__ acc,
                                     long long* __restrict__ other, int count4) {
  pdl_begin();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count4) return;
  float4 v = reinterpret_cast<const float4*>(base)[i];
  longlong2* a2 = reinterpret_cast<longlong2*>(acc) + 2 * (size_t)i;
  v = stream_value(v, a2);
  reinterpret_cast<float4*>(h)[i] = v;
  a2[0] = a2[1] = make_longlong2(0, 0);
  if (other) {
    longlong2* o2 = reinterpret_cast<longlong2*>(other) + 2 * (size_t)i;
    o2[0] = o2[1] = make_longlong2(0, 0);
  }
}

template <typename TO>
__global__ void __launch_bounds__(256) norm_fused_kernel(TO* __restrict__ out, float* __restrict__ h, const float* __restrict__ w,
                                                         const float* __restrict__ partial, const float* __restrict__ bias,
                                                         const int* __restrict__ rows, int n_tokens, int hidden, int splits, float eps,
                                                         const float* __restrict__ base, long long* __restrict__ acc,
                                                         long long* __restrict__ other) {
  extern __shared__ float row_buf[];  // hidden floats
  __shared__ float scratch[32];
  const int n4 = hidden >> 2;
  // the norm's weight is a constant of the model: this thread's first group of it is read ahead of the wait
  float4 g_first = make_float4(0.f, 0.f, 0.f, 0.f);
  if ((int)threadIdx.x < n4) g_first = reinterpret_cast<const float4*>(w)[threadIdx.x];
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float4* hr = reinterpret_cast<float4*>(h + (size_t)src * hidden);
  const float4* br = base ? reinterpret_cast<const float4*>(base + (size_t)src * hidden) : hr;
  const size_t plane4 = ((size_t)n_tokens * hidden) >> 2;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n4; c += blockDim.x) {
    float4 v = br[c];
    if (acc) {
      // the stream stands as base + accumulator: this row is brought back to one tensor and its
      // share of both accumulators left zero (rows == nullptr here: every row has its block)
      longlong2* a2 = reinterpret_cast<longlong2*>(acc + (size_t)src * hidden) + 2 * c;
      v = stream_value(v, a2);
      a2[0] = a2[1] = make_longlong2(0, 0);
      if (other) {
        longlong2* o2 = reinterpret_cast<longlong2*>(other + (size_t)src * hidden) + 2 * c;
        o2[0] = o2[1] = make_longlong2(0, 0);
      }
      if (!partial) hr[c] = v;
    } else if (base && !partial) {
      hr[c] = v;
    }
    if (partial) {
      // up to 24 splits in one round of loads (a round is a trip to L2), more in rounds of 8
      const float4* p = reinterpret_cast<const float4*>(partial) + (size_t)src * n4 + c;
      if (splits <= 8) {
        add_splits<8>(v, p, 0, splits, plane4);
      } else {
        add_splits<24>(v, p, 0, splits, plane4);
        for (int z0 = 24; z0 < splits; z0 += 8) add_splits<8>(v, p, z0, splits, plane4);
      }
      if (bias) {
        const float4 b = reinterpret_cast<const float4*>(bias)[c];
        v.x += b.x;
        v.y += b.y;
        v.z += b.z;
        v.w += b.w;
      }
      hr[c] = v;
    }
    reinterpret_cast<float4*>(row_buf)[c] = v;
    ss = fmaf(v.x, v.x, ss);
    ss = fmaf(v.y, v.y, ss);
    ss = fmaf(v.z, v.z, ss);
    ss = fmaf(v.w, v.w, ss);
  }
  pdl_launch();
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int c = threadIdx.x; c < n4; c += blockDim.x) {
    const float4 v = reinterpret_cast<float4*>(row_buf)[c];
    const float4 g = c == (int)threadIdx.x ? g_first : reinterpret_cast<const float4*>(w)[c];
    const float y0 = v.x * scale * g.x, y1 = v.y * scale * g.y, y2 = v.z * scale * g.z, y3 = v.w * scale * g.w;
    if (sizeof(TO) == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
      uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      reinterpret_cast<uint2*>(out + (size_t)r * hidden)[c] = packed;
    } else {
      reinterpret_cast<float4*>(out + (size_t)r * hidden)[c] = make_float4(y0, y1, y2, y3);
    }
  }
}

// The same with one warp per row (eight rows per block): for the many rows of a
// prompt portion, where a block per row leaves most of a block idle.  A lane keeps
// its CHUNKS groups of four values in registers (all their loads in flight at
// once, the row read once); sums stay within the warp.  hidden <= CHUNKS * 128.
template <typename TO, int CHUNKS>
__global__ void __launch_bounds__(256) norm_rows_kernel(TO* __restrict__ out, float* __restrict__ h, const float* __restrict__ w,
                                                        const float* __restrict__ partial, const float* __restrict__ bias,
                                                        const int* __restrict__ rows, int n_rows, int n_tokens, int hidden, int splits,
                                                        float eps) {
  pdl_begin();
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= n_rows) return;
  const int src = rows ? rows[r] : r;
  float4* hr = reinterpret_cast<float4*>(h + (size_t)src * hidden);
  const int n4 = hidden >> 2;
  const size_t plane4 = ((size_t)n_tokens * hidden) >> 2;
  float4 v[CHUNKS];
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = lane + i * 32;
    v[i] = c < n4 ? hr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (partial) {
    const float4* p = reinterpret_cast<const float4*>(partial) + (size_t)src * n4;
    for (int z = 0; z < splits; ++z) {  // added in split order
#pragma unroll
      for (int i = 0; i < CHUNKS; ++i) {
        const int c = lane + i * 32;
        if (c < n4) {
          const float4 a = p[(size_t)z * plane4 + c];
          v[i].x += a.x, v[i].y += a.y, v[i].z += a.z, v[i].w += a.w;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const int c = lane + i * 32;
      if (c < n4) {
        if (bias) {
          const float4 b = reinterpret_cast<const float4*>(bias)[c];
          v[i].x += b.x, v[i].y += b.y, v[i].z += b.z, v[i].w += b.w;
        }
        hr[c] = v[i];
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    ss = fmaf(v[i].x, v[i].x, ss);
    ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss);
    ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = lane + i * 32;
    if (c >= n4) break;
    const float4 g = reinterpret_cast<const float4*>(w)[c];
    const float y0 = v[i].x * scale * g.x, y1 = v[i].y * scale * g.y, y2 = v[i].z * scale * g.z, y3 = v[i].w * scale * g.w;
    if (sizeof(TO) == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
      reinterpret_cast<uint2*>(out + (size_t)r * hidden)[c] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else {
      reinterpret_cast<float4*>(out + (size_t)r * hidden)[c] = make_float4(y0, y1, y2, y3);
    }
  }
}

template <typename TO, int CHUNKS>
static void launch_norm_rows(TO* out, float* h, const float* w, const float* partial, const float* bias, const int* rows, int n_rows,
                             int n_tokens, int hidden, int splits, float eps, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    prefer_max_shared(norm_rows_kernel<TO, CHUNKS>);
    configured = true;
  }
  launch_dep(norm_rows_kernel<TO, CHUNKS>, (unsigned)((n_rows + 7) / 8), 256, 0, stream, out, h, w, partial, bias, rows, n_rows, n_tokens, hidden, splits, eps);
}
template <typename TO>
static void dispatch_norm_rows(TO* out, float* h, const float* w, const float* partial, const float* bias, const int* rows, int n_rows,
                               int n_tokens, int hidden, int splits, float eps, cudaStream_t stream) {
  if (hidden <= 1024) launch_norm_rows<TO, 8>(out, h, w, partial, bias, rows, n_rows, n_tokens, hidden, splits, eps, stream);
  else if (hidden <= 2048) launch_norm_rows<TO, 16>(out, h, w, partial, bias, rows, n_rows, n_tokens, hidden, splits, eps, stream);
  else launch_norm_rows<TO, 32>(out, h, w, partial, bias, rows, n_rows, n_tokens, hidden, splits, eps, stream);
}

// base (optional): the rows are read from `base` instead of h (h is written, complete).  acc
// (optional, with rows == nullptr only): a fixed-point accumulator [n_tokens, hidden] added on
// top and left zero, as is `other`.
ALOFA_API int alofa_norm_fused(void* out, void* h, const float* w, const float* partial, const float* bias, const int* rows, int n_rows,
                               int n_tokens, int hidden, int splits, float eps, int out_bf16, const float* base, long long* acc,
                               long long* other, cudaStream_t stream) {
  if (n_rows <= 0) return ALOFA_OK;
  if (hidden % 4 != 0 || hidden > 12288) return ALOFA_ERR_ARGUMENT;
  if ((acc || base) && (rows || n_rows != n_tokens)) return ALOFA_ERR_ARGUMENT;
  if (n_rows >= 256 && hidden <= 4096 && !acc && !base) {  // many rows: a warp each, the row in registers
    if (out_bf16)
      dispatch_norm_rows<bf16>((bf16*)out, (float*)h, w, partial, bias, rows, n_rows, n_tokens, hidden, splits, eps, stream);
    else
      dispatch_norm_rows<float>((float*)out, (float*)h, w, partial, bias, rows, n_rows, n_tokens, hidden, splits, eps, stream);
    return launch_status();
  }
  const size_t smem = (size_t)hidden * sizeof(float);
  ALOFA_PREFER_MAX_SHARED(norm_fused_kernel<bf16>);
  ALOFA_PREFER_MAX_SHARED(norm_fused_kernel<float>);
  if (out_bf16)
    launch_dep(norm_fused_kernel<bf16>, n_rows, 256, smem, stream, (bf16*)out, (float*)h, w, partial, bias, rows, n_tokens, hidden, splits, eps, base, acc, other);
  else
    launch_dep(norm_fused_kernel<float>, n_rows, 256, smem, stream, (float*)out, (float*)h, w, partial, bias, rows, n_tokens, hidden, splits, eps, base, acc, other);
  return launch_status();
}

// h = base + acc for all `count` values (a multiple of 4), both accumulators left zero.
ALOFA_API int alofa_stream_settle(float* h, const float* base, long long* acc, long long* other, int count, cudaStream_t stream) {
  if (count <= 0) return ALOFA_OK;
  if ((count & 3) || !h || !base || !acc) return ALOFA_ERR_ARGUMENT;
  const int count4 = count >> 2;
  launch_dep(stream_settle_kernel, (count4 + 255) / 256, 256, 0, stream, h, base, acc, other, count4);
  return launch_status();
}

// ---------------------------------------------------------------------------
// Rotation of q and k and the cache write, 8 + 8 elements per thread.
// Source: bf16 qkv [T, C] or fp32 partials [splits, T, C] (+ bias [C]),
// C = (nh + 2 nkv) * hd.  Requires rot == hd and hd % 16 == 0.
// ---------------------------------------------------------------------------
struct Vec8 {
  float v[8];
};

__device__ __forceinline__ Vec8 load8(const bf16* src) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
  Vec8 o;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    o.v[2 * i] = f.x;
    o.v[2 * i + 1] = f.y;
  }
  return o;
}
__device__ __forceinline__ Vec8 load8_partial(const float* partial, const float* bias, size_t offset, int col, size_t plane, int splits) {
  Vec8 o;
#pragma unroll
  for (int i = 0; i < 8; ++i) o.v[i] = bias ? bias[col + i] : 0.f;
  for (int z0 = 0; z0 < splits; z0 += 4) {  // four splits in flight, added in split order
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool ok = z0 + i < splits;
      a[i] = ok ? *reinterpret_cast<const float4*>(partial + (size_t)(z0 + i) * plane + offset) : make_float4(0.f, 0.f, 0.f, 0.f);
      b[i] = ok ? *reinterpret_cast<const float4*>(partial + (size_t)(z0 + i) * plane + offset + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o.v[0] += a[i].x; o.v[1] += a[i].y; o.v[2] += a[i].z; o.v[3] += a[i].w;
      o.v[4] += b[i].x; o.v[5] += b[i].y; o.v[6] += b[i].z; o.v[7] += b[i].w;
    }
  }
  return o;
}
__device__ __forceinline__ void store8(bf16* dst, const Vec8& x) {
  __nv_bfloat162 p[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(x.v[2 * i], x.v[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(p);
}

__global__ void rope_store_fused_kernel(bf16* __restrict__ q_out, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                        const bf16* __restrict__ qkv, const float* __restrict__ partial, const float* __restrict__ bias,
                                        const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                        const int* __restrict__ slot_map, int n_tokens, int nh, int nkv, int hd, int splits, int write_cache) {
  const int chunks = hd >> 4;  // pairs of 8-element chunks per head
  const int heads = nh + 2 * nkv;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)n_tokens * heads * chunks) return;
  const int c = (int)(idx % chunks);
  const int head = (int)((idx / chunks) % heads);
  const int t = (int)(idx / ((size_t)chunks * heads));
  const int half = hd >> 1;
  const int C = heads * hd;
  const int col = head * hd + c * 8;
  // Where the values go and what they are rotated by: slots and positions came with the step's
  // metadata, before any kernel of the step ran, and the table is a constant of the model, so all
  // of it is read ahead of the wait for the kernel that makes the values.
  bf16* dst;
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
  float4 cs[4];  // (cos, sin) of eight elements
  if (rotate) {
    const float4* src = reinterpret_cast<const float4*>(cos_sin + ((size_t)positions[t] * half + c * 8) * 2);
#pragma unroll
    for (int i = 0; i < 4; ++i) cs[i] = src[i];
  }
  pdl_begin();
  Vec8 a, b;
  if (partial) {
    const size_t plane = (size_t)n_tokens * C;
    a = load8_partial(partial, bias, (size_t)t * C + col, col, plane, splits);
    b = load8_partial(partial, bias, (size_t)t * C + col + half, col + half, plane, splits);
  } else {
    a = load8(qkv + (size_t)t * C + col);
    b = load8(qkv + (size_t)t * C + col + half);
  }
  if (rotate) {
    Vec8 ya, yb;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ya.v[2 * i] = a.v[2 * i] * cs[i].x - b.v[2 * i] * cs[i].y;
      yb.v[2 * i] = b.v[2 * i] * cs[i].x + a.v[2 * i] * cs[i].y;
      ya.v[2 * i + 1] = a.v[2 * i + 1] * cs[i].z - b.v[2 * i + 1] * cs[i].w;
      yb.v[2 * i + 1] = b.v[2 * i + 1] * cs[i].z + a.v[2 * i + 1] * cs[i].w;
    }
    a = ya;
    b = yb;
  }
  store8(dst + c * 8, a);
  store8(dst + c * 8 + half, b);
}

// The same from split-K partial sums, 4 + 4 elements per thread so that even a
// handful of tokens spreads over many threads, eight splits in flight.
__global__ void rope_store_partial_kernel(bf16* __restrict__ q_out, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                          const float* __restrict__ partial, const float* __restrict__ bias,
                                          const float* __restrict__ cos_sin, const int* __restrict__ positions,
                                          const int* __restrict__ slot_map, int n_tokens, int nh, int nkv, int hd, int splits, int write_cache) {
  const int chunks = hd >> 3;  // pairs of 4-element chunks per head
  pdl_begin();
  const int heads = nh + 2 * nkv;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)n_tokens * heads * chunks) return;
  const int c = (int)(idx % chunks);
  const int head = (int)((idx / chunks) % heads);
  const int t = (int)(idx / ((size_t)chunks * heads));
  const int half = hd >> 1;
  const int C = heads * hd;
  const int col = head * hd + c * 4;
  bf16* dst;
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
  const size_t plane = (size_t)n_tokens * C;
  const float* pa = partial + (size_t)t * C + col;
  float4 a = bias ? *reinterpret_cast<const float4*>(bias + col) : make_float4(0.f, 0.f, 0.f, 0.f);
  float4 b = bias ? *reinterpret_cast<const float4*>(bias + col + half) : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int z0 = 0; z0 < splits; z0 += 8) {
    float4 xa[8], xb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool ok = z0 + i < splits;
      xa[i] = ok ? *reinterpret_cast<const float4*>(pa + (size_t)(z0 + i) * plane) : make_float4(0.f, 0.f, 0.f, 0.f);
      xb[i] = ok ? *reinterpret_cast<const float4*>(pa + (size_t)(z0 + i) * plane + half) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a.x += xa[i].x; a.y += xa[i].y; a.z += xa[i].z; a.w += xa[i].w;
      b.x += xb[i].x; b.y += xb[i].y; b.z += xb[i].z; b.w += xb[i].w;
    }
  }
  float va[4] = {a.x, a.y, a.z, a.w}, vb[4] = {b.x, b.y, b.z, b.w};
  if (rotate) {
    const float* cs = cos_sin + ((size_t)positions[t] * half + c * 4) * 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float co = cs[2 * i], si = cs[2 * i + 1];
      const float ya = va[i] * co - vb[i] * si, yb = vb[i] * co + va[i] * si;
      va[i] = ya;
      vb[i] = yb;
    }
  }
  __nv_bfloat162 lo0 = __floats2bfloat162_rn(va[0], va[1]), lo1 = __floats2bfloat162_rn(va[2], va[3]);
  __nv_bfloat162 hi0 = __floats2bfloat162_rn(vb[0], vb[1]), hi1 = __floats2bfloat162_rn(vb[2], vb[3]);
  *reinterpret_cast<uint2*>(dst + c * 4) = make_uint2(*reinterpret_cast<uint32_t*>(&lo0), *reinterpret_cast<uint32_t*>(&lo1));
  *reinterpret_cast<uint2*>(dst + c * 4 + half) = make_uint2(*reinterpret_cast<uint32_t*>(&hi0), *reinterpret_cast<uint32_t*>(&hi1));
}

ALOFA_API int alofa_rope_store_fused(void* q_out, void* k_cache, void* v_cache, const void* qkv, const float* partial, const float* bias,
                                     const float* cos_sin, const int* positions, const int* slot_map, int n_tokens, int nh, int nkv, int hd,
                                     int splits, int write_cache, cudaStream_t stream) {
  if (n_tokens <= 0) return ALOFA_OK;
  if (hd % 16 != 0 || (!qkv && !partial)) return ALOFA_ERR_ARGUMENT;
  const int threads = 128;
  if (partial) {
    const size_t n = (size_t)n_tokens * (nh + 2 * nkv) * (hd >> 3);
    ALOFA_PREFER_MAX_SHARED(rope_store_partial_kernel);
    launch_dep(rope_store_partial_kernel, (unsigned)((n + threads - 1) / threads), threads, 0, stream, 
        (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, partial, bias, cos_sin, positions, slot_map, n_tokens, nh, nkv, hd, splits, write_cache);
    return launch_status();
  }
  const size_t total = (size_t)n_tokens * (nh + 2 * nkv) * (hd >> 4);
  ALOFA_PREFER_MAX_SHARED(rope_store_fused_kernel);
  launch_dep(rope_store_fused_kernel, (unsigned)((total + threads - 1) / threads), threads, 0, stream, 
      (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, (const bf16*)qkv, partial, bias, cos_sin, positions, slot_map, n_tokens, nh, nkv, hd, splits,
      write_cache);
  return launch_status();
}
