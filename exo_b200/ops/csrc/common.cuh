// Shared device helpers for the sm_100a kernel library.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define EXO_API extern "C" __attribute__((visibility("default")))

// dtype codes used by every launcher
enum { EXO_BF16 = 0, EXO_F32 = 1 };

// Built with -DEXO_KERNEL_CHECKS=1 (EXO_KERNEL_CHECKS=1 python -m exo_b200.build) every launcher waits for its kernel
// and reports an execution error as ITS return code, so a fault is attributed to the launch that made it instead
// of surfacing at some later call; launchers of vectorised kernels also refuse pointers that are not 16-byte
// aligned.  (Not for graph capture: the synchronisation is illegal there.)
#ifdef EXO_KERNEL_CHECKS
#define EXO_CHECK_LAUNCH()                                                        \
  do {                                                                            \
    cudaError_t e__ = cudaGetLastError();                                         \
    if (e__ != cudaSuccess) return (int)e__;                                      \
    cudaStreamCaptureStatus cs__ = cudaStreamCaptureStatusNone;                   \
    if (cudaStreamIsCapturing(0, &cs__) == cudaSuccess && cs__ == cudaStreamCaptureStatusNone) { \
      e__ = cudaDeviceSynchronize();                                              \
      if (e__ != cudaSuccess) return (int)e__;                                    \
    }                                                                             \
  } while (0)
#define EXO_REQUIRE_ALIGNED16(p)                                                  \
  do {                                                                            \
    if ((p) && (reinterpret_cast<uintptr_t>(p) & 15)) return -8;                  \
  } while (0)
#else
#define EXO_CHECK_LAUNCH()                         \
  do {                                             \
    cudaError_t e__ = cudaGetLastError();          \
    if (e__ != cudaSuccess) return (int)e__;       \
  } while (0)
#define EXO_REQUIRE_ALIGNED16(p) do { } while (0)
#endif

template <typename T> struct Cvt;
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

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

// block-wide sum through shared memory; red must hold >= 32 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// 16-byte vector of 8 bf16 -> 8 floats
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// streaming (no L1 allocate) 16-byte load for weights that are read exactly once
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

// ---- programmatic dependent launch (PDL) -------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while its
// predecessor in the stream is still running; it must execute pdl_wait() before it touches
// anything the predecessor wrote.  pdl_trigger() lets the successor begin launching early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifdef __CUDACC__
// Launch helper: kernel<<<grid, block, smem, stream>>> with the PDL attribute set.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif
