// RMS normalisation kernels (HBM-bound): fused residual-add + RMSNorm (in place)
// and plain RMSNorm.  One CTA per row.  The fast kernel keeps the whole row in
// registers (one pass over HBM: read x, read residual, write residual, write x);
// the generic kernel handles any length/alignment with a second, cache-resident
// read of the row.
#include "common.cuh"

namespace fg {

__device__ __forceinline__ float block_sum(float v, float* smem) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? smem[lane] : 0.f;
  t = warp_sum(t);
  return t;  // every thread of every warp holds the total
}

// Row held in registers: thread t owns packets t, t+blockDim, ... (VPT of them).  All
// loads of the row are issued before the first use; conversions work on packed pairs.
template <typename T, int VPT, bool HAS_RES>
__global__ void __launch_bounds__(VPT >= 8 ? 512 : 1024)
rms_norm_row_kernel(T* x, T* res, const T* __restrict__ w,
                    T* out, int64_t N, int64_t x_stride, int64_t r_stride,
                    int64_t o_stride, float eps) {
  constexpr int E = Vec16<T>::N;
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  T* xr = x + row * x_stride;
  T* rr = HAS_RES ? res + row * r_stride : nullptr;
  T* orow = out + row * o_stride;
  const int npacks = (int)(N / E);

  uint4 xa[VPT], ra[VPT], wa[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int p = threadIdx.x + i * blockDim.x;
    if (p < npacks) {
      xa[i] = ldg16_stream(xr + (int64_t)p * E);
      if (HAS_RES) ra[i] = ldg16_stream(rr + (int64_t)p * E);
      wa[i] = ldg16(w + (int64_t)p * E);  // issued with the row so that it is not a second round trip
    }
  }
  float s[VPT][E];
  float sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int p = threadIdx.x + i * blockDim.x;
    if (p < npacks) {
      Vec16<T>::unpack(xa[i], s[i]);
      if (HAS_RES) {
        float rv[E];
        Vec16<T>::unpack(ra[i], rv);
#pragma unroll
        for (int e = 0; e < E; ++e) s[i][e] += rv[e];
        stg16(rr + (int64_t)p * E, Vec16<T>::pack(s[i]));  // residual: the sum rounded to T
      }
#pragma unroll
      for (int e = 0; e < E; ++e) sumsq = fmaf(s[i][e], s[i][e], sumsq);
    }
  }
  const float total = block_sum(sumsq, red);
  const float rrms = 1.0f / sqrtf(total / (float)N + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int p = threadIdx.x + i * blockDim.x;
    if (p < npacks) {
      float wv[E];
      Vec16<T>::unpack(wa[i], wv);
#pragma unroll
      for (int e = 0; e < E; ++e) s[i][e] = s[i][e] * rrms * wv[e];
      stg16(orow + (int64_t)p * E, Vec16<T>::pack(s[i]));
    }
  }
}

// Any N, any alignment.  Pass 1 accumulates the sum of squares, pass 2 re-reads
// the row (L1/L2 resident) and writes both outputs; each thread reads an element
// before it overwrites it, so the in-place update is safe.
template <typename T, bool HAS_RES>
__global__ void __launch_bounds__(1024)
rms_norm_generic_kernel(T* x, T* res, const T* __restrict__ w,
                        T* out, int64_t N, int64_t x_stride, int64_t r_stride,
                        int64_t o_stride, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  T* xr = x + row * x_stride;
  T* rr = HAS_RES ? res + row * r_stride : nullptr;
  T* orow = out + row * o_stride;
  float sumsq = 0.f;
  for (int64_t c = threadIdx.x; c < N; c += blockDim.x) {
    float v = Cvt<T>::to_f32(xr[c]);
    if (HAS_RES) v += Cvt<T>::to_f32(rr[c]);
    sumsq = fmaf(v, v, sumsq);
  }
  const float total = block_sum(sumsq, red);
  const float rrms = 1.0f / sqrtf(total / (float)N + eps);
  for (int64_t c = threadIdx.x; c < N; c += blockDim.x) {
    float v = Cvt<T>::to_f32(xr[c]);
    if (HAS_RES) {
      v += Cvt<T>::to_f32(rr[c]);
      rr[c] = Cvt<T>::from_f32(v);
    }
    orow[c] = Cvt<T>::from_f32(v * rrms * Cvt<T>::to_f32(w[c]));
  }
}

template <typename T, bool HAS_RES>
static int launch_norm(T* x, T* res, const T* w, T* out, int64_t M, int64_t N, int64_t xs,
                       int64_t rs, int64_t os, float eps, cudaStream_t st) {
  constexpr int E = Pack16<T>::N;
  const bool vec_ok = (N % E == 0) && aligned16(x) && aligned16(w) && aligned16(out) &&
                      (xs % E == 0) && (os % E == 0) &&
                      (!HAS_RES || (aligned16(res) && rs % E == 0));
  const int64_t npacks = N / E;
  if (M == 0 || N == 0) return FG_OK;
  if (M > 2147483647LL) return fail(FG_ERR_TOO_LARGE, "rms_norm: more than 2^31-1 rows");
  dim3 grid((unsigned)M);
  if (vec_ok && npacks <= 4096) {
    // Threads per row: aim for 2 packs per thread once the row is long enough that
    // a 1-pack mapping would need more than 256 threads.
    int vpt = 1;
    if (npacks > 256) vpt = 2;
    if (npacks > 1024) vpt = 4;
    if (npacks > 2048) vpt = 8;  // block = 512 (N up to 32768 halves)
    int threads = (int)((npacks + vpt - 1) / vpt);
    threads = ((threads + 31) / 32) * 32;
    if (threads > 1024) threads = 1024;
#define FG_NORM_CASE(V)                                                                      \
  case V:                                                                                    \
    rms_norm_row_kernel<T, V, HAS_RES><<<grid, threads, 0, st>>>(x, res, w, out, N, xs, rs, os, eps); \
    break;
    switch (vpt) {
      FG_NORM_CASE(1)
      FG_NORM_CASE(2)
      FG_NORM_CASE(4)
      FG_NORM_CASE(8)
    }
#undef FG_NORM_CASE
    FG_CHECK_LAUNCH("rms_norm_row_kernel");
  } else {
    int threads = (int)((N + 31) / 32 * 32);
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    rms_norm_generic_kernel<T, HAS_RES><<<grid, threads, 0, st>>>(x, res, w, out, N, xs, rs, os, eps);
    FG_CHECK_LAUNCH("rms_norm_generic_kernel");
  }
  return FG_OK;
}

}  // namespace fg

extern "C" int fg_fused_add_rms_norm(void* x, void* residual, const void* weight, int64_t M,
                                     int64_t N, int64_t x_row_stride, int64_t r_row_stride,
                                     double eps, int dtype, void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("fused_add_rms_norm");
  FG_REQUIRE(M >= 0 && N >= 0, "fused_add_rms_norm: negative size");
  if (M == 0 || N == 0) return FG_OK;
  FG_REQUIRE(x && residual && weight, "fused_add_rms_norm: null pointer");
  FG_REQUIRE(x != residual, "fused_add_rms_norm: input and residual must not alias");
  FG_DISPATCH_FLOAT(dtype, T,
                    return (launch_norm<T, true>((T*)x, (T*)residual, (const T*)weight, (T*)x, M, N,
                                                 x_row_stride, r_row_stride, x_row_stride,
                                                 (float)eps, (cudaStream_t)stream)));
  return FG_OK;
}

extern "C" int fg_rms_norm(const void* x, const void* weight, void* out, int64_t M, int64_t N,
                           int64_t x_row_stride, int64_t o_row_stride, double eps, int dtype,
                           void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("rms_norm");
  FG_REQUIRE(M >= 0 && N >= 0, "rms_norm: negative size");
  if (M == 0 || N == 0) return FG_OK;
  FG_REQUIRE(x && out && weight, "rms_norm: null pointer");
  FG_DISPATCH_FLOAT(dtype, T,
                    return (launch_norm<T, false>((T*)x, (T*)nullptr, (const T*)weight, (T*)out, M,
                                                  N, x_row_stride, 0, o_row_stride, (float)eps,
                                                  (cudaStream_t)stream)));
  return FG_OK;
}
