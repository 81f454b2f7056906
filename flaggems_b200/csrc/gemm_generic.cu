// Generic GEMM: any dtype (fp32 / fp16 / bf16), any strides, any shape, including
// K == 0.  Plain fp32 FMA on CUDA cores (fp32 inputs are never rounded to TF32,
// matching allow_tf32=False in the reference, src/flag_gems/ops/mm.py:107).  It serves what
// the tcgen05 kernel does not take: fp32 operands, unaligned bases or leading dimensions,
// tiny problems.  Two tile shapes: 128 x 128 with 8 x 8 outputs per thread and the next
// K slice fetched into registers while the current one is multiplied (problems that fill
// the GPU with such tiles), and 64 x 64 with 4 x 4 outputs per thread for the rest.
#include "common.cuh"

namespace fg {

int gemm_tcgen05(const fg_gemm_params* p, const GemmBatch& bt, cudaStream_t st);
bool gemm_tcgen05_eligible(const fg_gemm_params* p);

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct GArgs {
  const void *a, *b, *bias;
  void* c;
  int64_t M, N, K;
  int64_t as0, as1, bs0, bs1, cs0, cs1, zs0, zs1;
  float alpha, beta;
  int has_bias;
  const int* only_if;   // null, or a device flag: the launch does nothing while it is zero
};

template <typename T>
__global__ void __launch_bounds__(256) gemm_generic_kernel(GArgs g) {
  if (g.only_if != nullptr && *g.only_if == 0) return;
  __shared__ float sa[TK][TM + 4];
  __shared__ float sb[TK][TN + 4];
  const T* A = reinterpret_cast<const T*>(g.a);
  const T* B = reinterpret_cast<const T*>(g.b);
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4x4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int64_t k0 = 0; k0 < g.K; k0 += TK) {
    // 64x16 elements of A and 16x64 of B: 1024 each, 4 per thread.
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256;
      {
        const int kk = e & 15, mm = e >> 4;
        const int64_t m = m0 + mm, k = k0 + kk;
        sa[kk][mm] = (m < g.M && k < g.K) ? Cvt<T>::to_f32(A[m * g.as0 + k * g.as1]) : 0.f;
      }
      {
        const int nn = e & 63, kk = e >> 6;
        const int64_t n = n0 + nn, k = k0 + kk;
        sb[kk][nn] = (n < g.N && k < g.K) ? Cvt<T>::to_f32(B[k * g.bs0 + n * g.bs1]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  T* C = reinterpret_cast<T*>(g.c);
  const T* Z = reinterpret_cast<const T*>(g.bias);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      if (g.has_bias) v = v * g.alpha + Cvt<T>::to_f32(Z[m * g.zs0 + n * g.zs1]) * g.beta;
      C[m * g.cs0 + n * g.cs1] = Cvt<T>::from_f32(v);
    }
  }
}

// 128 x 128 x 16 tiles, 256 threads, 8 x 8 outputs per thread as four 4 x 4 blocks (rows ty*4 and
// 64 + ty*4, columns tx*4 and 64 + tx*4: the shared-memory reads of a warp are two broadcast
// float4 of A and two conflict-free float4 runs of B).  Global loads go through registers: the
// slice k0 + 16 is in flight while slice k0 is multiplied.
constexpr int BTM = 128, BTN = 128, BTK = 16;
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float unpack_lo(uint64_t v) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return lo;
}
__device__ __forceinline__ float unpack_hi(uint64_t v) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return hi;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
#ifndef FG_SIMT128_MIN_CTAS
#define FG_SIMT128_MIN_CTAS 2
#endif

template <typename T>
__global__ void __launch_bounds__(256, FG_SIMT128_MIN_CTAS) gemm_simt128_kernel(GArgs g) {
  if (g.only_if != nullptr && *g.only_if == 0) return;
  __shared__ __align__(16) float sa[BTK][BTM + 4];
  __shared__ __align__(16) float sb[BTK][BTN + 4];
  const T* A = reinterpret_cast<const T*>(g.a);
  const T* B = reinterpret_cast<const T*>(g.b);
  const int64_t m0 = (int64_t)blockIdx.y * BTM, n0 = (int64_t)blockIdx.x * BTN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  // Loader coordinates: 2048 elements of each operand slice, 8 per thread.  The fastest-moving
  // index of a warp follows the operand's unit-stride dimension, so the loads coalesce for
  // row- and column-major operands alike.
  const bool a_k_fast = g.as1 == 1 || g.as0 != 1;   // A [M, K]: K contiguous unless column-major
  const bool b_n_fast = g.bs1 == 1 || g.bs0 != 1;   // B [K, N]: N contiguous unless column-major
  float ra[8], rb[8];
  auto fetch = [&](int64_t k0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = tid + i * 256;
      const int kk = a_k_fast ? (e & 15) : (e >> 7), mm = a_k_fast ? (e >> 4) : (e & 127);
      const int64_t m = m0 + mm, k = k0 + kk;
      ra[i] = (m < g.M && k < g.K) ? Cvt<T>::to_f32(A[m * g.as0 + k * g.as1]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = tid + i * 256;
      const int nn = b_n_fast ? (e & 127) : (e >> 4), kk = b_n_fast ? (e >> 7) : (e & 15);
      const int64_t n = n0 + nn, k = k0 + kk;
      rb[i] = (n < g.N && k < g.K) ? Cvt<T>::to_f32(B[k * g.bs0 + n * g.bs1]) : 0.f;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = tid + i * 256;
      const int kk = a_k_fast ? (e & 15) : (e >> 7), mm = a_k_fast ? (e >> 4) : (e & 127);
      sa[kk][mm] = ra[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = tid + i * 256;
      const int nn = b_n_fast ? (e & 127) : (e >> 4), kk = b_n_fast ? (e >> 7) : (e & 15);
      sb[kk][nn] = rb[i];
    }
  };
  uint64_t acc2[8][4];   // acc2[i][j] = outputs (i, 2j) and (i, 2j + 1) as a packed pair of floats
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc2[i][j] = 0ull;

  if (g.K > 0) fetch(0);
  for (int64_t k0 = 0; k0 < g.K; k0 += BTK) {
    stash();
    __syncthreads();
    if (k0 + BTK < g.K) fetch(k0 + BTK);
#pragma unroll
    for (int kk = 0; kk < BTK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&sa[kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&sa[kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&sb[kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&sb[kk][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      // Two IEEE fused multiply-adds per instruction (fma.rn.f32x2 on a pair of adjacent outputs):
      // half the issue slots of scalar FFMA, the same results bit for bit.
      const uint64_t bp[4] = {pack2(b0.x, b0.y), pack2(b0.z, b0.w), pack2(b1.x, b1.y), pack2(b1.z, b1.w)};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint64_t aa = pack2(av[i], av[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc2[i][j] = fma2(aa, bp[j], acc2[i][j]);
      }
    }
    __syncthreads();
  }
  T* C = reinterpret_cast<T*>(g.c);
  const T* Z = reinterpret_cast<const T*>(g.bias);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t m = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t n = n0 + (j >> 2) * 64 + tx * 4 + (j & 3);
      if (n >= g.N) continue;
      float v = (j & 1) ? unpack_hi(acc2[i][j >> 1]) : unpack_lo(acc2[i][j >> 1]);
      if (g.has_bias) v = v * g.alpha + Cvt<T>::to_f32(Z[m * g.zs0 + n * g.zs1]) * g.beta;
      C[m * g.cs0 + n * g.cs1] = Cvt<T>::from_f32(v);
    }
  }
}

}  // namespace
}  // namespace fg

namespace fg {
int gemm_tile_plan(const fg_gemm_params* p, int64_t batch, int num_sms, fg_gemm_plan* out);
}
extern "C" int fg_gemm_tile_plan(const fg_gemm_params* p, int64_t batch, int num_sms, fg_gemm_plan* out) {
  return fg::gemm_tile_plan(p, batch, num_sms, out);
}

extern "C" int fg_gemm_uses_tcgen05(const fg_gemm_params* p) {
  return (p != nullptr && fg::gemm_tcgen05_eligible(p)) ? 1 : 0;
}

namespace fg {
static int gemm_one(const fg_gemm_params* p, cudaStream_t st, const int* only_if = nullptr) {
  GArgs g;
  g.only_if = only_if;
  g.a = p->a; g.b = p->b; g.bias = p->bias; g.c = p->c;
  g.M = p->M; g.N = p->N; g.K = p->K;
  g.as0 = p->a_stride0; g.as1 = p->a_stride1; g.bs0 = p->b_stride0; g.bs1 = p->b_stride1;
  g.cs0 = p->c_stride0; g.cs1 = p->c_stride1; g.zs0 = p->bias_stride0; g.zs1 = p->bias_stride1;
  g.alpha = (float)p->alpha; g.beta = (float)p->beta;
  g.has_bias = p->bias != nullptr;
  // the large tile when its grid still gives every SM a CTA
  const int64_t bx = (p->N + BTN - 1) / BTN, by = (p->M + BTM - 1) / BTM;
  if (p->K >= 64 && bx * by >= num_sms() && by <= 65535) {
    dim3 grid((unsigned)bx, (unsigned)by);
    FG_DISPATCH_FLOAT(p->dtype, T, gemm_simt128_kernel<T><<<grid, 256, 0, st>>>(g));
    FG_CHECK_LAUNCH("gemm_simt128_kernel");
    return FG_OK;
  }
  const int64_t gx = (p->N + TN - 1) / TN, gy = (p->M + TM - 1) / TM;
  if (gy > 65535) return fail(FG_ERR_TOO_LARGE, "gemm (generic path): M = %lld exceeds %d rows", (long long)p->M,
                              65535 * TM);
  dim3 grid((unsigned)gx, (unsigned)gy);
  FG_DISPATCH_FLOAT(p->dtype, T, gemm_generic_kernel<T><<<grid, 256, 0, st>>>(g));
  FG_CHECK_LAUNCH("gemm_generic_kernel");
  return FG_OK;
}

// The CUDA-core kernel for `p`, gated on a device flag: its CTAs return at once while the flag is zero.
int gemm_simt_gated(const fg_gemm_params* p, const int* only_if_nonzero, cudaStream_t st) {
  return gemm_one(p, st, only_if_nonzero);
}

static int gemm_checked(const char* what, const fg_gemm_params* p) {
  FG_REQUIRE(p != nullptr, "%s: null params", what);
  FG_REQUIRE(p->M >= 0 && p->N >= 0 && p->K >= 0, "%s: negative size", what);
  if (p->M == 0 || p->N == 0) return 1;  // nothing to do
  FG_REQUIRE(p->c != nullptr, "%s: null output", what);
  FG_REQUIRE(p->K == 0 || (p->a && p->b), "%s: null operand", what);
  return FG_OK;
}
}  // namespace fg

extern "C" int fg_gemm(const fg_gemm_params* p, void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("gemm");
  const int rc = gemm_checked("gemm", p);
  if (rc != FG_OK) return rc < 0 ? rc : FG_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (gemm_tcgen05_eligible(p)) return gemm_tcgen05(p, GemmBatch(), st);
  return gemm_one(p, st);
}

namespace fg {
int64_t gemm_f32_split_workspace_bytes(const fg_gemm_params* p);
int gemm_f32_split(const fg_gemm_params* p, void* workspace, int64_t workspace_bytes, cudaStream_t st);
}
extern "C" int64_t fg_gemm_f32_split_workspace_bytes(const fg_gemm_params* p) {
  return fg::gemm_f32_split_workspace_bytes(p);
}
extern "C" int fg_gemm_f32_split(const fg_gemm_params* p, void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("gemm_f32_split");
  const int rc = gemm_checked("gemm_f32_split", p);
  if (rc != FG_OK) return rc < 0 ? rc : FG_OK;
  return gemm_f32_split(p, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" int fg_gemm_batched(const fg_gemm_params* p, int64_t batch, int64_t a_batch_stride,
                               int64_t b_batch_stride, int64_t c_batch_stride, int64_t bias_batch_stride,
                               void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("gemm_batched");
  const int rc = gemm_checked("gemm_batched", p);
  if (rc != FG_OK) return rc < 0 ? rc : FG_OK;
  FG_REQUIRE(batch >= 0, "gemm_batched: negative batch");
  if (batch == 0) return FG_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // One launch when the tensor-core path takes the shape and the batch strides keep every
  // problem 16-byte aligned and fit a tensor map; else one generic launch per problem.
  const bool strides_ok = batch == 1 || (a_batch_stride % 8 == 0 && b_batch_stride % 8 == 0 && a_batch_stride > 0 &&
                                         b_batch_stride > 0 && batch <= 2147483647LL);
  if (gemm_tcgen05_eligible(p) && strides_ok) {
    GemmBatch bt;
    bt.batch = batch; bt.a_bs = a_batch_stride; bt.b_bs = b_batch_stride; bt.c_bs = c_batch_stride;
    bt.bias_bs = bias_batch_stride;
    return gemm_tcgen05(p, bt, st);
  }
  const int64_t es = p->dtype == FG_F32 ? 4 : 2;
  for (int64_t i = 0; i < batch; ++i) {
    fg_gemm_params q = *p;
    q.a = p->a ? (const char*)p->a + i * a_batch_stride * es : nullptr;
    q.b = p->b ? (const char*)p->b + i * b_batch_stride * es : nullptr;
    q.c = (char*)p->c + i * c_batch_stride * es;
    q.bias = p->bias ? (const char*)p->bias + i * bias_batch_stride * es : nullptr;
    const int r = gemm_tcgen05_eligible(&q) ? gemm_tcgen05(&q, GemmBatch(), st) : gemm_one(&q, st);
    if (r != FG_OK) return r;
  }
  return FG_OK;
}
