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

// Host-visible copy of the device status word (core.cu): non-zero after a kernel of this
// library gave up a bounded wait on the current device.  Reading it costs a load from pinned
// host memory, no synchronisation; every launching entry point refuses to launch while it is set.
int drained_code();
int fail_drained(const char* what, int code);
#define FG_REQUIRE_HEALTHY(what)                              \
  do {                                                        \
    const int _dc = ::fg::drained_code();                     \
    if (_dc != 0) return ::fg::fail_drained(what, _dc);       \
  } while (0)
// While one of these lives on a thread, device_status_ptr() does not perform the one-time
// set-up of the host-visible copy (a cudaHostRegister): for entry points that promise to make
// no allocating or registering call.
struct MirrorSetupGuard {
  MirrorSetupGuard();
  ~MirrorSetupGuard();
  bool saved_;
};

// Check the launch that was just issued (configuration errors only; no sync).
#define FG_CHECK_LAUNCH(name)                                                        \
  do {                                                                               \
    cudaError_t _e = cudaGetLastError();                                             \
    if (_e != cudaSuccess)                                                           \
      return ::fg::fail(FG_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
    ::fg::count_launch();                                                            \
  } while (0)

// Batch of independent GEMMs of one shape (bmm): element strides between consecutive
// problems; batch == 1 is the plain GEMM.
struct GemmBatch {
  int64_t batch = 1;
  int64_t a_bs = 0, b_bs = 0, c_bs = 0, bias_bs = 0;
};

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

// SMs the persistent kernels may occupy (fg_set_num_sms); the rest is left to kernels
// that run beside them, e.g. NCCL's copy kernels.
int sm_budget();

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

// Pair conversions on packed 32-bit words (two 16-bit values, or one float in .x).
// They cost one integer op per element on the way in and one cvt per pair on the way
// out, half of what element-wise conversion takes -- the memory-bound kernels are
// close to instruction-issue bound without them.
template <typename T>
struct Pair;
template <>
struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <>
struct Pair<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// 16 bytes of T as fp32 values and back (4 floats, or 8 halves through Pair<T>).
template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[N]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = Pair<T>::unpack(w[i]);
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[N]) {
    return make_uint4(Pair<T>::pack(f[0], f[1]), Pair<T>::pack(f[2], f[3]), Pair<T>::pack(f[4], f[5]),
                      Pair<T>::pack(f[6], f[7]));
  }
};
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[4]) {
    f[0] = __uint_as_float(u.x);
    f[1] = __uint_as_float(u.y);
    f[2] = __uint_as_float(u.z);
    f[3] = __uint_as_float(u.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};
__device__ __forceinline__ uint4 ldg16_stream(const void* p) {
  uint4 u;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
               : "l"(p));
  return u;
}
__device__ __forceinline__ uint4 ldg16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void stg16(void* p, const uint4& u) { *reinterpret_cast<uint4*>(p) = u; }

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
