// Shared device helpers: element conversion, block reductions with a fixed
// order, and the launch-error check used by every exported function.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define ALOFA_API extern "C" __attribute__((visibility("default")))

// Return codes of the exported launch functions.
#define ALOFA_OK 0
#define ALOFA_ERR_ARGUMENT 1   // a size the kernel does not take
#define ALOFA_ERR_LAUNCH 2     // the CUDA runtime refused the launch

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16_rn(x); }

// The residual stream of a small decode step may stand as an fp32 base plus a 64-bit fixed-point
// accumulator in units of 2^-32 (products add their split sums into it with atomic integer adds, whose
// result does not depend on their order).  base + acc in fp32: the accumulator is split into the
// nearest whole number (exact in fp32 below 2^24) and a signed fraction in [-1/2, 1/2); the whole part
// is added to the base first, the fraction after.  While the accumulator is below 1/2 in size (the
// usual case) the whole part is zero and the sum is rounded once, up to the fraction's own 2^-26;
// otherwise twice, which keeps it within two units in the last place of max(1, |sum|).  The result
// is the same for the same inputs wherever it is computed.  (Double arithmetic would round once, but
// 64-bit conversions and adds run at a few per clock per SM here and cost the product that reads
// the stream 0.3 us per k-slice.)
constexpr float STREAM_SCALE = 4294967296.0f;  // 2^32
__device__ __forceinline__ float stream_add(float base, long long acc) {
  const int whole = (int)((acc + 0x80000000ll) >> 32);
  const int fraction = (int)(unsigned)(acc & 0xffffffffll);  // acc == whole * 2^32 + fraction
  return (base + (float)whole) + (float)fraction * (1.0f / 4294967296.0f);
}

// silu(g) * u = g / (1 + e^-g) * u in the bfloat16 kernels: the exponential and the reciprocal by
// the hardware approximations (2 ulp and 1 ulp), denormals flushed.  One function for every kernel
// that has a gated epilogue, so that a token's value does not depend on which of them ran; the
// library forms (__expf, a division) cost the prompt kernels' epilogue a fifth of its time.
// (src/alofa/kernels/cpu/scalar.mojo:208-232 for the formula.)
__device__ __forceinline__ float silu_times(float g, float u) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return g * r * u;
}

// Sum over a warp in a fixed butterfly order; every lane gets the result.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum / max; `scratch` holds 32 floats.  All threads get the result.
// The order of additions depends only on the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nwarp; ++w) total += scratch[w];
  return total;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float m = scratch[0];
  for (int w = 1; w < nwarp; ++w) m = fmaxf(m, scratch[w]);
  return m;
}

// Ask for the largest shared-memory carve-out for a kernel, once.  Kernels that
// follow one another in a step then all run under the same L1/shared split;
// a change of the split between two launches costs a drain of the SMs.
template <typename K>
static inline void prefer_max_shared(K kernel) {
  cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
}
#define ALOFA_PREFER_MAX_SHARED(kernel)  \
  do {                                   \
    static bool done_ = false;           \
    if (!done_) {                        \
      prefer_max_shared(kernel);         \
      done_ = true;                      \
    }                                    \
  } while (0)

// Programmatic dependent launch.  A kernel launched with launch_dep may become
// resident while the kernel before it in the stream is still running; it must
// call pdl_begin() before it touches global memory: that lets the kernel after
// it start launching in turn, then waits until everything the stream ran
// before has completed and is visible.  Launch latency and per-CTA set-up
// (barrier initialisation, tensor-memory allocation) thus overlap the tail of
// the previous kernel.  Under an ordinary launch pdl_begin() does nothing.
// ALOFA_PDL=0 in the environment turns the attribute off.
__device__ __forceinline__ void pdl_begin() {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// The two halves, for the kernels of a decode step, where the order is the other way round:
// pdl_wait() first, then pdl_launch() (the norm and decode attention call it once their own loads
// are on their way).  The kernel after this one then becomes resident while
// this kernel's body runs, not while the kernel before it still does: two steps ahead its CTAs
// only took shared memory and bandwidth from kernels that still had work to do (measured
// 0.852 -> 0.830 ms per decode step at batch 8; the same order in the prompt-step kernels
// measured slower, so they keep pdl_begin()).
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

static inline bool pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* env = getenv("ALOFA_PDL");
    enabled = (env && env[0] == '0') ? 0 : 1;
  }
  return enabled == 1;
}

template <typename... KArgs, typename... Args>
static inline void launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int launch_status() { return cudaGetLastError() == cudaSuccess ? ALOFA_OK : ALOFA_ERR_LAUNCH; }
