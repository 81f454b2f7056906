// Shared host/device helpers for the flaggems_b200 kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/flaggems_b200.h"

namespace fg {

// ---- error reporting -------------------------------------------------------
char* last_error_buf();  // thread-local, 512 bytes
int fail(int code, const char* fmt, ...);
extern std::atomic<int64_t> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

#define FG_REQUIRE(cond, ...)                                  \
  do {                                                         \
    if (!(cond)) return ::fg::fail(FG_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define FG_CUDA_OK(expr)                                                          \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess)                                                        \
      return ::fg::fail(FG_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

// Check the launch that was just issued (configuration errors only; no sync).
#define FG_CHECK_LAUNCH(name)                                                        \
  do {                                                                               \
    cudaError_t _e = cudaGetLastError();                                             \
    if (_e != cudaSuccess)                                                           \
      return ::fg::fail(FG_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
    ::fg::count_launch();                                                            \
  } while (0)

inline int num_sms() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != cached_dev) {
    cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    cached_dev = dev;
  }
  return cached > 0 ? cached : 148;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int dtype_size(int dtype) { return dtype == FG_F32 ? 4 : 2; }

// ---- device-side dtype traits ---------------------------------------------
template <typename T>
struct Cvt;
template <>
struct Cvt<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <>
struct Cvt<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <>
struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};

// A 16-byte packet of T (4 floats or 8 halves).
template <typename T>
struct alignas(16) Pack16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__device__ __forceinline__ Pack16<T> ld16(const T* p) {
  Pack16<T> r;
  *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
  return r;
}
// Streaming (evict-first) 16-byte load for data touched exactly once.
template <typename T>
__device__ __forceinline__ Pack16<T> ld16_stream(const T* p) {
  Pack16<T> r;
  uint4 u;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
               : "l"(p));
  *reinterpret_cast<uint4*>(&r) = u;
  return r;
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const Pack16<T>& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
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

// Dispatch a lambda-like macro body over the three floating dtypes.
#define FG_DISPATCH_FLOAT(dtype, T, ...)                        \
  switch (dtype) {                                              \
    case FG_F32: {                                              \
      using T = float;                                          \
      __VA_ARGS__;                                              \
    } break;                                                    \
    case FG_F16: {                                              \
      using T = __half;                                         \
      __VA_ARGS__;                                              \
    } break;                                                    \
    case FG_BF16: {                                             \
      using T = __nv_bfloat16;                                  \
      __VA_ARGS__;                                              \
    } break;                                                    \
    default:                                                    \
      return ::fg::fail(FG_ERR_INVALID, "unknown dtype code %d", (int)(dtype)); \
  }

}  // namespace fg
