// Rotary position embedding (HBM-bound).  One CTA per token; each thread owns a
// (head, chunk) pair and rotates both members of every pair it loads, so each
// element of q/k is read once and written once.
//   NeoX layout   : pair (j, j + D/2)
//   interleaved   : pair (2j, 2j + 1)
//   y0 = x0*cos[j] - x1*sin[j] ;  y1 = x1*cos[j] + x0*sin[j]   (fp32, rounded once)
#include "common.cuh"

namespace fg {

struct RopeArgs {
  const void *q, *k;
  void *qo, *ko;
  const void *cos, *sin, *pos;
  int64_t T;
  int Hq, Hk, D;
  int64_t qs_t, qs_h, qs_d, ks_t, ks_h, ks_d;
  int64_t qos_t, qos_h, qos_d, kos_t, kos_h, kos_d;
  int64_t pos_stride, cos_stride, sin_stride, seq_len, max_pos;
  int pos_i64;
};

__device__ __forceinline__ int64_t rope_position(const RopeArgs& a, int64_t tok) {
  int64_t pos;
  if (a.pos == nullptr) {
    pos = tok % a.seq_len;
  } else if (a.pos_i64) {
    pos = reinterpret_cast<const int64_t*>(a.pos)[tok * a.pos_stride];
  } else {
    pos = reinterpret_cast<const int32_t*>(a.pos)[tok * a.pos_stride];
  }
  // An out-of-range position would read outside the cos/sin tables; clamp it so a
  // bad index can never fault the device (the reference leaves this undefined).
  if (pos < 0) pos = 0;
  if (pos >= a.max_pos) pos = a.max_pos - 1;
  return pos;
}

// N consecutive cos (or sin) values as fp32.  VEC: the row is 16-byte aligned and N
// values are a whole number of 16-byte packets.
template <typename CT, int N, bool VEC>
__device__ __forceinline__ void load_table(const CT* p, float (&f)[N]) {
  if constexpr (VEC) {
    constexpr int PE = Vec16<CT>::N;
#pragma unroll
    for (int i = 0; i < N / PE; ++i) {
      float t[PE];
      Vec16<CT>::unpack(ldg16(p + i * PE), t);
#pragma unroll
      for (int e = 0; e < PE; ++e) f[i * PE + e] = t[e];
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = Cvt<CT>::to_f32(p[i]);
  }
}

// Vector kernel: unit stride over D, 16-byte aligned rows.  One work item covers E
// rotation pairs: NeoX -> the packets at j0 and j0 + D/2; interleaved -> two adjacent
// packets.  Needs (D/2) % E == 0.  One CTA per token, one item per thread; the kernel is
// kept lean in registers (packed words are converted pair by pair) because the bytes in
// flight per SM are set by how many of these small CTAs are resident.
template <typename T, typename CT, bool INTERLEAVED, bool CSVEC>
__global__ void __launch_bounds__(512) rope_vec_kernel(RopeArgs a) {
  constexpr int E = Vec16<T>::N;
  const int64_t tok = blockIdx.x;
  const int64_t pos = rope_position(a, tok);
  const CT* cosr = reinterpret_cast<const CT*>(a.cos) + pos * a.cos_stride;
  const CT* sinr = reinterpret_cast<const CT*>(a.sin) + pos * a.sin_stride;
  const int half = a.D >> 1;
  const int cph = half / E;  // work items per head
  const int work = (a.Hq + a.Hk) * cph;
  for (int w = threadIdx.x; w < work; w += blockDim.x) {
    const int h = w / cph;
    const int c = w - h * cph;
    const bool is_q = h < a.Hq;
    const T* src = is_q ? reinterpret_cast<const T*>(a.q) + tok * a.qs_t + (int64_t)h * a.qs_h
                        : reinterpret_cast<const T*>(a.k) + tok * a.ks_t + (int64_t)(h - a.Hq) * a.ks_h;
    T* dst = is_q ? reinterpret_cast<T*>(a.qo) + tok * a.qos_t + (int64_t)h * a.qos_h
                  : reinterpret_cast<T*>(a.ko) + tok * a.kos_t + (int64_t)(h - a.Hq) * a.kos_h;
    const int j0 = c * E;                               // first rotation pair of this item
    const int o0 = INTERLEAVED ? 2 * j0 : j0;           // element offsets of the two packets
    const int o1 = INTERLEAVED ? 2 * j0 + E : j0 + half;
    const uint4 u0 = ldg16(src + o0);
    const uint4 u1 = ldg16(src + o1);
    float cs[E], sn[E];
    load_table<CT, E, CSVEC>(cosr + j0, cs);
    load_table<CT, E, CSVEC>(sinr + j0, sn);
    float x[E], y[E];
    Vec16<T>::unpack(u0, x);
    Vec16<T>::unpack(u1, y);
    if (!INTERLEAVED) {
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float r0 = x[e] * cs[e] - y[e] * sn[e];
        y[e] = y[e] * cs[e] + x[e] * sn[e];
        x[e] = r0;
      }
    } else {
      // packet 0 holds pairs j0 .. j0+E/2-1 as (even, odd) neighbours, packet 1 the rest
#pragma unroll
      for (int e = 0; e < E; e += 2) {
        const int j = e >> 1, k = E / 2 + j;
        const float a0 = x[e] * cs[j] - x[e + 1] * sn[j];
        x[e + 1] = x[e + 1] * cs[j] + x[e] * sn[j];
        x[e] = a0;
        const float b0 = y[e] * cs[k] - y[e + 1] * sn[k];
        y[e + 1] = y[e + 1] * cs[k] + y[e] * sn[k];
        y[e] = b0;
      }
    }
    stg16(dst + o0, Vec16<T>::pack(x));
    stg16(dst + o1, Vec16<T>::pack(y));
  }
}

// Scalar kernel: any strides, any even D.
template <typename T, typename CT, bool INTERLEAVED>
__global__ void __launch_bounds__(256) rope_scalar_kernel(RopeArgs a) {
  const int64_t tok = blockIdx.x;
  const int64_t pos = rope_position(a, tok);
  const CT* cosr = reinterpret_cast<const CT*>(a.cos) + pos * a.cos_stride;
  const CT* sinr = reinterpret_cast<const CT*>(a.sin) + pos * a.sin_stride;
  const int half = a.D >> 1;
  const int work = (a.Hq + a.Hk) * half;
  for (int w = threadIdx.x; w < work; w += blockDim.x) {
    const int h = w / half;
    const int j = w - h * half;
    const int i0 = INTERLEAVED ? 2 * j : j;
    const int i1 = INTERLEAVED ? 2 * j + 1 : j + half;
    const bool is_q = h < a.Hq;
    const int hh = is_q ? h : h - a.Hq;
    const int64_t sd = is_q ? a.qs_d : a.ks_d;
    const int64_t od = is_q ? a.qos_d : a.kos_d;
    const T* src = is_q ? reinterpret_cast<const T*>(a.q) + tok * a.qs_t + (int64_t)hh * a.qs_h
                        : reinterpret_cast<const T*>(a.k) + tok * a.ks_t + (int64_t)hh * a.ks_h;
    T* dst = is_q ? reinterpret_cast<T*>(a.qo) + tok * a.qos_t + (int64_t)hh * a.qos_h
                  : reinterpret_cast<T*>(a.ko) + tok * a.kos_t + (int64_t)hh * a.kos_h;
    const float cs = Cvt<CT>::to_f32(cosr[j]);
    const float sn = Cvt<CT>::to_f32(sinr[j]);
    const float x0 = Cvt<T>::to_f32(src[i0 * sd]);
    const float x1 = Cvt<T>::to_f32(src[i1 * sd]);
    dst[i0 * od] = Cvt<T>::from_f32(x0 * cs - x1 * sn);
    dst[i1 * od] = Cvt<T>::from_f32(x1 * cs + x0 * sn);
  }
}

template <typename T, typename CT>
static int launch_rope(const fg_rope_params* p, cudaStream_t st) {
  constexpr int E = Pack16<T>::N;
  RopeArgs a;
  a.q = p->q; a.k = p->k; a.qo = p->q_out; a.ko = p->k_out;
  a.cos = p->cos; a.sin = p->sin; a.pos = p->positions;
  a.T = p->num_tokens; a.Hq = (int)p->q_heads; a.Hk = (int)p->k_heads; a.D = (int)p->head_dim;
  a.qs_t = p->q_stride_t; a.qs_h = p->q_stride_h; a.qs_d = p->q_stride_d;
  a.ks_t = p->k_stride_t; a.ks_h = p->k_stride_h; a.ks_d = p->k_stride_d;
  a.qos_t = p->qo_stride_t; a.qos_h = p->qo_stride_h; a.qos_d = p->qo_stride_d;
  a.kos_t = p->ko_stride_t; a.kos_h = p->ko_stride_h; a.kos_d = p->ko_stride_d;
  a.pos_stride = p->pos_stride; a.cos_stride = p->cos_stride; a.sin_stride = p->sin_stride;
  a.seq_len = p->seq_len > 0 ? p->seq_len : 1;
  a.max_pos = p->max_positions;
  a.pos_i64 = p->pos_is_i64;

  const int half = a.D / 2;
  auto mult = [](int64_t v) { return v % E == 0; };
  bool vec = a.qs_d == 1 && a.ks_d == 1 && a.qos_d == 1 && a.kos_d == 1 &&
             aligned16(a.q) && aligned16(a.qo) && mult(a.qs_t) && mult(a.qs_h) && mult(a.qos_t) &&
             mult(a.qos_h);
  if (a.Hk > 0)
    vec = vec && aligned16(a.k) && aligned16(a.ko) && mult(a.ks_t) && mult(a.ks_h) &&
          mult(a.kos_t) && mult(a.kos_h);
  vec = vec && (half % E == 0);
  // cos/sin rows readable as 16-byte packets?
  constexpr int CE = 16 / (int)sizeof(CT);
  const bool csvec = aligned16(a.cos) && aligned16(a.sin) && a.cos_stride % CE == 0 && a.sin_stride % CE == 0 &&
                     (E % CE == 0);
  dim3 grid((unsigned)a.T);
  if (vec) {
    const int cph = half / E;
    int threads = (a.Hq + a.Hk) * cph;
    threads = (threads + 31) / 32 * 32;
    if (threads > 512) threads = 512;
    if (p->interleaved) {
      if (csvec) rope_vec_kernel<T, CT, true, true><<<grid, threads, 0, st>>>(a);
      else rope_vec_kernel<T, CT, true, false><<<grid, threads, 0, st>>>(a);
    } else {
      if (csvec) rope_vec_kernel<T, CT, false, true><<<grid, threads, 0, st>>>(a);
      else rope_vec_kernel<T, CT, false, false><<<grid, threads, 0, st>>>(a);
    }
    FG_CHECK_LAUNCH("rope_vec_kernel");
  } else {
    int threads = (a.Hq + a.Hk) * half;
    threads = (threads + 31) / 32 * 32;
    if (threads > 256) threads = 256;
    if (p->interleaved)
      rope_scalar_kernel<T, CT, true><<<grid, threads, 0, st>>>(a);
    else
      rope_scalar_kernel<T, CT, false><<<grid, threads, 0, st>>>(a);
    FG_CHECK_LAUNCH("rope_scalar_kernel");
  }
  return FG_OK;
}

}  // namespace fg

extern "C" int fg_rotary_embedding(const fg_rope_params* p, void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("rotary_embedding");
  FG_REQUIRE(p != nullptr, "rotary_embedding: null params");
  FG_REQUIRE(p->num_tokens >= 0 && p->q_heads >= 0 && p->k_heads >= 0, "rotary_embedding: negative size");
  FG_REQUIRE(p->head_dim > 0 && p->head_dim % 2 == 0, "rotary_embedding: head_dim %lld must be even and positive",
             (long long)p->head_dim);
  FG_REQUIRE(p->num_tokens <= 2147483647LL, "rotary_embedding: too many tokens");
  if (p->num_tokens == 0 || p->q_heads + p->k_heads == 0) return FG_OK;
  FG_REQUIRE(p->cos && p->sin, "rotary_embedding: null cos/sin");
  FG_REQUIRE(p->q_heads == 0 || (p->q && p->q_out), "rotary_embedding: null q");
  FG_REQUIRE(p->k_heads == 0 || (p->k && p->k_out), "rotary_embedding: null k");
  FG_REQUIRE(p->max_positions > 0, "rotary_embedding: empty cos/sin table");
  FG_REQUIRE(p->positions != nullptr || p->seq_len > 0, "rotary_embedding: seq_len required without positions");
  cudaStream_t st = (cudaStream_t)stream;
  FG_DISPATCH_FLOAT(p->dtype, T, {
    switch (p->cos_dtype) {
      case FG_F32: return launch_rope<T, float>(p, st);
      case FG_F16: return launch_rope<T, __half>(p, st);
      case FG_BF16: return launch_rope<T, __nv_bfloat16>(p, st);
      default: return fail(FG_ERR_INVALID, "rotary_embedding: unknown cos dtype %d", p->cos_dtype);
    }
  });
  return FG_OK;
}
