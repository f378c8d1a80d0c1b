// Shared helpers of the sm_100a kernels: element conversion, reductions, error reporting.
//
// Every exported function is `extern "C"`, takes raw device pointers and a stream, launches on
// that stream, allocates nothing, and returns 0 or a negative code whose text `erb_last_error()`
// gives.  Each source is compiled twice, into one library per element type (float for the 32-bit
// path, bfloat16 for serving), so a run builds and loads only the type it uses.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

// Each source is compiled once per element type: -DERB_ELEM=0 (float) or 1 (bfloat16).
#ifndef ERB_ELEM
#error "compile with -DERB_ELEM=0 (float) or -DERB_ELEM=1 (bfloat16)"
#endif
#if ERB_ELEM == 0
typedef float elem_t;
#else
typedef __nv_bfloat16 elem_t;
#endif

#define ERB_OK 0
#define ERB_ERR_ARG -1
#define ERB_ERR_CUDA -2
#define ERB_ERR_UNSUPPORTED -3

namespace erb {

// One message buffer per library; written by the host wrappers only.
inline char* error_buffer() {
  static thread_local char buf[512];
  return buf;
}

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(ERB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return ERB_OK;
}

// Streaming multiprocessors of the current device (asked once per device).
inline int sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (!counts[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    counts[dev] = n;
  }
  return counts[dev];
}

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// Loads `N` consecutive elements (N * sizeof(T) must be 16 bytes, pointer 16-byte aligned) as floats.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* out) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load4(const float* p, float* out) {
  float4 raw = *reinterpret_cast<const float4*>(p);
  out[0] = raw.x; out[1] = raw.y; out[2] = raw.z; out[3] = raw.w;
}

// silu(g) * u in float.  Where the result is rounded to 16 bits (ERB_ELEM == 1) the exponential and the
// division are the fast forms (relative error about 2^-21, far below that rounding); the 32-bit path keeps
// the exact ones.  Every kernel that gates (the gate kernel, the gated epilogues of the products for few
// rows) calls this, so that they agree to the bit.
__device__ __forceinline__ float silu_mul(float g, float u) {
#if ERB_ELEM == 1
  return __fdividef(g, 1.f + __expf(-g)) * u;
#else
  return g / (1.f + expf(-g)) * u;
#endif
}

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

// Sum over the block in a fixed order (warp trees, then the first warp over the warp sums);
// every thread gets the result.  `scratch` holds 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// One rotary pair (x[j], x[j + half]) turned by the angle whose cosine and sine are given.  Written
// with explicit roundings so that every kernel that rotates gives the same bits.
__device__ __forceinline__ void rotate_pair(float a, float b, float cs, float sn, float& lo, float& hi) {
  lo = __fmaf_rn(a, cs, -__fmul_rn(b, sn));
  hi = __fmaf_rn(b, cs, __fmul_rn(a, sn));
}

// Chained launches.  Kernels that run back to back in the decode step are launched with
// programmatic stream serialization: the next kernel's blocks may be scheduled while the previous
// kernel drains, which hides the launch latency between the many short kernels of a step.  Every
// such kernel calls chain_wait() before it touches memory, which blocks until the previous kernel
// has completed and its writes are visible; so the data flow is that of ordinary stream order.
// EDGERAG_B200_NO_CHAIN=1 in the environment turns the attribute off.
__device__ __forceinline__ void chain_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline bool chain_enabled() {
  static const bool on = [] {
    const char* v = getenv("EDGERAG_B200_NO_CHAIN");
    return !(v && v[0] == '1');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline void launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chain_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface in check_launch()
}

}  // namespace erb

#define ERB_EXPORT extern "C" __attribute__((visibility("default")))

// Each library exports its own copy under a library-specific name via this macro.
#define ERB_DEFINE_LAST_ERROR(name) \
  ERB_EXPORT const char* name() { return erb::error_buffer(); }
