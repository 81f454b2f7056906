// silu_and_mul / gelu_and_mul: out = act(fp32(a)) * b  (HBM-bound elementwise).
// Fast kernel: tensors viewed as [rows, cols] with unit column stride, 16-byte
// packets, two packets of each operand in flight per thread.  Generic kernel:
// up to 6 broadcast dimensions with arbitrary element strides.
#include "common.cuh"

namespace fg {

__device__ __forceinline__ float silu_mul_f32(float x, float y) {
  return x / (1.0f + __expf(-x)) * y;
}
// 16-bit outputs carry 8-11 significant bits: tanh.approx (relative error about 2^-11)
// is exact enough and keeps the kernel off the MUFU / instruction-issue limits.
__device__ __forceinline__ float silu_mul_fast(float x, float y) {
  // x * sigmoid(x) = 0.5 x (1 + tanh(x / 2)): one MUFU op per element instead of two
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  const float hx = 0.5f * x;
  return fmaf(hx, t, hx) * y;
}
// gelu(x) * y, exact (erf) and tanh forms, constants as in fused/gelu_and_mul.py:15-21,52-64
__device__ __forceinline__ float gelu_none_mul(float x, float y) {
  return 0.5f * x * (1.0f + erff(x * 0.7071067811f)) * y;
}
template <bool FAST>
__device__ __forceinline__ float gelu_tanh_mul(float x, float y) {
  const float u = x * 0.79788456f * (1.0f + 0.044715f * x * x);
  float t;
  if (FAST) {
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  } else {
    t = tanhf(u);
  }
  return 0.5f * x * (1.0f + t) * y;
}
// ACT: 0 silu, 1 gelu (erf), 2 gelu (tanh).  FAST (16-bit element types) takes the MUFU
// approximations; fp32 tensors and the strided fallback take the precise forms.
template <typename T, int ACT, bool FAST>
__device__ __forceinline__ float act_mul_t(float x, float y) {
  if (ACT == 1) return gelu_none_mul(x, y);
  if (ACT == 2) return gelu_tanh_mul<FAST && sizeof(T) != 4>(x, y);
  return (FAST && sizeof(T) != 4) ? silu_mul_fast(x, y) : silu_mul_f32(x, y);
}

// [rows, cols] view; IDX is uint32_t when the packet count allows it (one 32-bit
// division per packet instead of a 64-bit one).
template <typename T, int UNROLL, typename IDX, int ACT>
__global__ void __launch_bounds__(256)
silu_mul_rows_kernel(const T* a, const T* b, T* out,
                     int64_t total_packs, int packs_per_row, int64_t a_stride, int64_t b_stride,
                     int64_t o_stride) {
  constexpr int E = Vec16<T>::N;
  const IDX base = (IDX)blockIdx.x * (IDX)(UNROLL * 256) + threadIdx.x;
  uint4 pa[UNROLL], pb[UNROLL];
  int64_t ooff[UNROLL];
  bool ok[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const IDX idx = base + (IDX)(u * 256);
    ok[u] = (int64_t)idx < total_packs;
    if (ok[u]) {
      const IDX row = idx / (IDX)packs_per_row;
      const int64_t col = (int64_t)(idx - row * (IDX)packs_per_row) * E;
      pa[u] = ldg16_stream(a + (int64_t)row * a_stride + col);
      pb[u] = ldg16_stream(b + (int64_t)row * b_stride + col);
      ooff[u] = (int64_t)row * o_stride + col;
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    if (ok[u]) {
      float fa[E], fb[E];
      Vec16<T>::unpack(pa[u], fa);
      Vec16<T>::unpack(pb[u], fb);
#pragma unroll
      for (int e = 0; e < E; ++e) fa[e] = act_mul_t<T, ACT, true>(fa[e], fb[e]);
      stg16(out + ooff[u], Vec16<T>::pack(fa));
    }
  }
}

struct Strided6 {
  int64_t size[6];
  int64_t sa[6], sb[6], so[6];
  int ndim;
};

template <typename T, int ACT>
__global__ void __launch_bounds__(256)
silu_mul_strided_kernel(const T* a, const T* b, T* out,
                        int64_t total, Strided6 d) {
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = idx, oa = 0, ob = 0, oo = 0;
#pragma unroll
    for (int k = 5; k >= 0; --k) {
      if (k < d.ndim) {
        const int64_t q = rem / d.size[k];
        const int64_t r = rem - q * d.size[k];
        rem = q;
        oa += r * d.sa[k];
        ob += r * d.sb[k];
        oo += r * d.so[k];
      }
    }
    out[oo] = Cvt<T>::from_f32(act_mul_t<T, ACT, false>(Cvt<T>::to_f32(a[oa]), Cvt<T>::to_f32(b[ob])));
  }
}

template <typename T, int ACT>
static int launch_silu_mul(const T* a, const T* b, T* out, int ndim, const int64_t* sizes,
                           const int64_t* sa, const int64_t* sb, const int64_t* so,
                           cudaStream_t st) {
  constexpr int E = Pack16<T>::N;
  int64_t total = 1;
  for (int i = 0; i < ndim; ++i) total *= sizes[i];
  if (total == 0) return FG_OK;

  // Try to view the problem as [rows, cols]: the last dim has unit stride in all
  // three tensors and every leading dim folds into one uniform row stride.
  bool rows_ok = ndim >= 1 && sa[ndim - 1] == 1 && sb[ndim - 1] == 1 && so[ndim - 1] == 1;
  int64_t cols = ndim >= 1 ? sizes[ndim - 1] : 1, rows = 1;
  int64_t ras = 0, rbs = 0, ros = 0;
  if (rows_ok) {
    // fold dims ndim-2 .. 0: need stride[k] == stride[k+1]*size[k+1] for k < ndim-2
    bool first = true;
    for (int k = ndim - 2; k >= 0 && rows_ok; --k) {
      if (sizes[k] == 1) continue;
      if (first) {
        ras = sa[k]; rbs = sb[k]; ros = so[k];
        rows = sizes[k];
        first = false;
      } else {
        rows_ok = sa[k] == ras * rows && sb[k] == rbs * rows && so[k] == ros * rows;
        rows *= sizes[k];
      }
    }
    rows_ok = rows_ok && (cols % E == 0) && aligned16(a) && aligned16(b) && aligned16(out) &&
              (ras % E == 0) && (rbs % E == 0) && (ros % E == 0);
  }
  if (rows_ok && cols / E <= 2147483647LL) {
    constexpr int UNROLL = 4;
    const int64_t total_packs = total / E;
    const int64_t blocks = (total_packs + 256 * UNROLL - 1) / (256 * UNROLL);
    if (blocks > 2147483647LL) return fail(FG_ERR_TOO_LARGE, "silu_and_mul: tensor too large");
    if (total_packs + 256 * UNROLL < 4294967295LL)
      silu_mul_rows_kernel<T, UNROLL, uint32_t, ACT><<<(unsigned)blocks, 256, 0, st>>>(
          a, b, out, total_packs, (int)(cols / E), ras, rbs, ros);
    else
      silu_mul_rows_kernel<T, UNROLL, int64_t, ACT><<<(unsigned)blocks, 256, 0, st>>>(
          a, b, out, total_packs, (int)(cols / E), ras, rbs, ros);
    FG_CHECK_LAUNCH("silu_mul_rows_kernel");
    return FG_OK;
  }
  Strided6 d;
  d.ndim = ndim;
  for (int i = 0; i < 6; ++i) {
    d.size[i] = i < ndim ? sizes[i] : 1;
    d.sa[i] = i < ndim ? sa[i] : 0;
    d.sb[i] = i < ndim ? sb[i] : 0;
    d.so[i] = i < ndim ? so[i] : 0;
  }
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)num_sms() * 32;
  if (blocks > cap) blocks = cap;
  silu_mul_strided_kernel<T, ACT><<<(unsigned)blocks, 256, 0, st>>>(a, b, out, total, d);
  FG_CHECK_LAUNCH("silu_mul_strided_kernel");
  return FG_OK;
}

}  // namespace fg

namespace fg {
static int act_and_mul(const char* what, int act, const void* a, const void* b, void* out, int ndim,
                       const int64_t* sizes, const int64_t* a_strides, const int64_t* b_strides,
                       const int64_t* o_strides, int dtype, void* stream) {
  FG_REQUIRE_HEALTHY(what);
  FG_REQUIRE(ndim >= 0 && ndim <= 6, "%s: ndim %d not in [0, 6]", what, ndim);
  FG_REQUIRE(ndim == 0 || (sizes && a_strides && b_strides && o_strides), "%s: null shape/stride array", what);
  for (int i = 0; i < ndim; ++i) {
    FG_REQUIRE(sizes[i] >= 0, "%s: negative size", what);
    if (sizes[i] == 0) return FG_OK;
  }
  FG_REQUIRE(a && b && out, "%s: null pointer", what);
  FG_DISPATCH_FLOAT(dtype, T, {
    switch (act) {
      case 0: return (launch_silu_mul<T, 0>((const T*)a, (const T*)b, (T*)out, ndim, sizes, a_strides, b_strides,
                                            o_strides, (cudaStream_t)stream));
      case 1: return (launch_silu_mul<T, 1>((const T*)a, (const T*)b, (T*)out, ndim, sizes, a_strides, b_strides,
                                            o_strides, (cudaStream_t)stream));
      default: return (launch_silu_mul<T, 2>((const T*)a, (const T*)b, (T*)out, ndim, sizes, a_strides, b_strides,
                                             o_strides, (cudaStream_t)stream));
    }
  });
  return FG_OK;
}
}  // namespace fg

extern "C" int fg_silu_and_mul(const void* a, const void* b, void* out, int ndim,
                               const int64_t* sizes, const int64_t* a_strides,
                               const int64_t* b_strides, const int64_t* o_strides, int dtype,
                               void* stream) {
  return fg::act_and_mul("silu_and_mul", 0, a, b, out, ndim, sizes, a_strides, b_strides, o_strides, dtype, stream);
}

extern "C" int fg_gelu_and_mul(const void* a, const void* b, void* out, int ndim,
                               const int64_t* sizes, const int64_t* a_strides,
                               const int64_t* b_strides, const int64_t* o_strides, int approximate_tanh,
                               int dtype, void* stream) {
  return fg::act_and_mul("gelu_and_mul", approximate_tanh ? 2 : 1, a, b, out, ndim, sizes, a_strides, b_strides,
                         o_strides, dtype, stream);
}
