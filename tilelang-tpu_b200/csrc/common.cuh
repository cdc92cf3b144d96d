// Shared host/device helpers for the sm_100a kernel library.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <atomic>

#include "tl_b200.h"

namespace tl {

// ---- host-side error reporting ------------------------------------------------
// Thread-local message buffer behind tl_b200_last_error(); mirrors the static
// error_buf of the reference's CUDA host wrappers (tilelang/jit/adapter/wrapper.py:22-42).
char* error_buffer();
int fail(int code, const char* fmt, ...);
void count_launch(int n = 1);

#define TL_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return ::tl::fail(TL_B200_EINVAL, __VA_ARGS__); \
  } while (0)

#define TL_CUDA(expr)                                                                      \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return ::tl::fail(TL_B200_ECUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                        __FILE__, __LINE__);                                               \
  } while (0)

// Call after every kernel launch: catches launch-configuration errors without synchronising.
#define TL_LAUNCH_CHECK(name)                                                              \
  do {                                                                                     \
    cudaError_t _e = cudaGetLastError();                                                   \
    if (_e != cudaSuccess)                                                                 \
      return ::tl::fail(TL_B200_ECUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
    ::tl::count_launch();                                                                  \
  } while (0)

// Programmatic dependent launch.  A kernel launched through launch_overlapped() may be scheduled
// while the kernel before it in the stream still runs; it calls dependency_wait() before it touches
// global memory (returns once that whole grid has finished and its writes are visible; returns at
// once when the predecessor was launched normally), so dependent chains stay correct and what
// overlaps is launch latency and CTA ramp-up.  dependency_release() lets the successor start.
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                     Args... args) {
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int dtype_bytes(int dtype) {
  switch (dtype) {
    case TL_F32: case TL_I32: case TL_U32: return 4;
    case TL_F16: case TL_BF16: return 2;
    case TL_E4M3: return 1;
    default: return 0;
  }
}

int sm_count();

// ---- device-side scalar conversions --------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

// Round-to-nearest-even, the rounding the reference's casts use (RM_HALF_TO_EVEN,
// src/target/codegen_ppl.cc:1138-1151).
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// A 16-byte vector of elements of type T.
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  union {
    uint4 raw;
    T e[N];
  };
};

// Streaming 16-byte global accesses: data touched once, so keep it out of L1.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// 32-byte (256-bit) global accesses, available from sm_100: half the instructions per byte and
// twice the bytes in flight per thread.  Addresses must be 32-byte aligned.
template <typename T> struct Vec32 {
  static constexpr int N = 32 / sizeof(T);
  union {
    uint32_t w[8];
    T e[N];
  };
};
template <typename T> __device__ __forceinline__ Vec32<T> ld_stream32(const void* p) {
  Vec32<T> v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                 "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p));
  return v;
}
template <typename T> __device__ __forceinline__ Vec32<T> ld_cached32(const void* p) {
  Vec32<T> v;
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                 "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p));
  return v;
}
template <typename T> __device__ __forceinline__ void st_stream32(void* p, const Vec32<T>& v) {
  asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.w[0]),
               "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7])
               : "memory");
}
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

// 16-byte load for data that is re-read by other CTAs (tables, weights): default caching.
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
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

}  // namespace tl
