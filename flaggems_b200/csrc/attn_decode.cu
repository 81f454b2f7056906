// Single-query (decode) attention over a paged or contiguous KV store: HBM-bound.
//
// One CTA owns (sequence, KV head, KV chunk).  The `group` query heads that share a
// KV head are packed into the 16 rows of an m16n8k16 tile, so every K/V byte is read
// once per KV head.  The CTA streams 64-row K/V tiles through a 3-stage cp.async
// ring; inside a tile each of the 4 warps owns 16 KV rows and keeps its own online
// softmax state, merged through shared memory at the end (flash-decoding inside the
// CTA).  With more than one chunk per sequence the partial (O, log-sum-exp) pairs go
// to an fp32 workspace and a second kernel combines them.
#include "attn_common.cuh"
#include "mma_helpers.cuh"

namespace fg {
namespace {

constexpr int BN = 64, NTHREADS = 128;

template <typename T, int DP>
__device__ __forceinline__ void load_rows64(T* sdst, const T* gbase, int64_t row_off, bool row_valid, int d,
                                            int row, int part) {
  constexpr int LD = DP + 8;
  constexpr int PER = DP / 16;  // chunks per thread (2 threads per row)
  const int dchunks = d >> 3;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int ch = part * PER + i;
    const bool ok = row_valid && ch < dchunks;
    cp_async16(sdst + row * LD + ch * 8, ok ? (const void*)(gbase + row_off + ch * 8) : (const void*)gbase, ok);
  }
}

template <typename T, int DP, int STAGES>
__global__ void __launch_bounds__(NTHREADS) attn_decode_kernel(AttnArgs a, int chunk_tokens) {
  constexpr int LD = DP + 8;
  constexpr int STAGE_ELEMS = 2 * BN * LD;  // K tile then V tile
  extern __shared__ __align__(16) uint8_t smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);            // [16][LD]
  T* sKV = sQ + 16 * LD;                             // [STAGES][2][BN][LD]

  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const SeqInfo s = seq_info(a, b);
  if (s.q_len < 1) return;
  const int kv_begin = split * chunk_tokens;
  const int kv_end = min(s.k_len, kv_begin + chunk_tokens);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = a.group;
  const int64_t qtok = s.q_begin;  // the single query token of this sequence

  float* part_o = nullptr;
  float* part_lse = nullptr;
  if (a.num_splits > 1) {
    part_o = a.ws_o + ((int64_t)split * a.total_q + qtok) * a.H * a.D;
    part_lse = a.ws_lse + (int64_t)split * a.H * a.total_q;
  }

  if (kv_begin >= kv_end) {
    // Empty chunk: contributes nothing.  (Only reachable with splitting, or k_len == 0.)
    if (a.num_splits > 1) {
      if (tid < group) part_lse[(int64_t)(hk * group + tid) * a.total_q + qtok] = -INFINITY;
    } else {
      T* out = reinterpret_cast<T*>(a.out) + qtok * a.o_rs + (int64_t)hk * group * a.o_hs;
      for (int i = tid; i < group * a.D; i += NTHREADS) out[(i / a.D) * a.o_hs + (i % a.D)] = Cvt<T>::from_f32(0.f);
      if (a.lse && tid < group) a.lse[(int64_t)(hk * group + tid) * a.total_q + qtok] = INFINITY;
    }
    return;
  }

  const T* K = reinterpret_cast<const T*>(a.k) + (int64_t)hk * a.k_hs;
  const T* V = reinterpret_cast<const T*>(a.v) + (int64_t)hk * a.v_hs;
  const int32_t* bt_row = a.paged ? a.block_table + (int64_t)b * a.bt_stride : nullptr;
  const int lrow = tid >> 1, lpart = tid & 1;

  // Q rows: row r < group is query head hk*group + r; rows >= group are zero.
  if (lrow < 16) {
    const bool ok = lrow < group;
    const int64_t off = qtok * a.q_rs + (int64_t)(hk * group + (ok ? lrow : 0)) * a.q_hs;
    load_rows64<T, DP>(sQ, reinterpret_cast<const T*>(a.q), off, ok, a.D, lrow, lpart);
  }
  const int n_tiles = (kv_end - kv_begin + BN - 1) / BN;
  auto load_kv = [&](int t, int stage) {
    const int tok = kv_begin + t * BN + lrow;
    const bool ok = tok < kv_end;
    int64_t koff = 0, voff = 0;
    if (ok) {
      koff = kv_row_offset(a, bt_row, s.k_begin, tok, a.k_rs, a.k_bs);
      voff = kv_row_offset(a, bt_row, s.k_begin, tok, a.v_rs, a.v_bs);
    }
    T* st = sKV + stage * STAGE_ELEMS;
    load_rows64<T, DP>(st, K, koff, ok, a.D, lrow, lpart);
    load_rows64<T, DP>(st + BN * LD, V, voff, ok, a.D, lrow, lpart);
  };
#pragma unroll
  for (int t = 0; t < STAGES - 1; ++t) {
    if (t < n_tiles) load_kv(t, t);
    cp_async_commit();  // group t (the first one also carries Q)
  }

  uint32_t qf[DP / 16][4];
  float o[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t % STAGES;
    cp_async_wait<STAGES - 2>();  // tile t has landed
    __syncthreads();               // ... for every thread; and tile t-1 is fully consumed
    if (t + STAGES - 1 < n_tiles) load_kv(t + STAGES - 1, (t + STAGES - 1) % STAGES);
    cp_async_commit();
    if (t == 0) {
#pragma unroll
      for (int kk = 0; kk < DP / 16; ++kk)
        ldmatrix_x4(qf[kk], sQ + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
    }
    const T* sKs = sKV + stage * STAGE_ELEMS;
    const T* sVs = sKs + BN * LD;

    // S[16 q rows x 16 kv rows of this warp]
    float sacc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
      uint32_t bf[4];
      ldmatrix_x4(bf, sKs + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
      mma16816<T>(sacc[0], qf[kk], bf[0], bf[1]);
      mma16816<T>(sacc[1], qf[kk], bf[2], bf[3]);
    }
    const int j0 = kv_begin + t * BN + warp * 16;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = sacc[nt][e];
        if (a.has_softcap) v = tanhf(v * a.softcap_pre);
        v *= a.scale_log2;
        const int col = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        if (col >= kv_end) v = -INFINITY;
        sacc[nt][e] = v;
      }
    }
    float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      mx[0] = fmaxf(mx[0], fmaxf(sacc[nt][0], sacc[nt][1]));
      mx[1] = fmaxf(mx[1], fmaxf(sacc[nt][2], sacc[nt][3]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      msafe[r] = mx[r] == -INFINITY ? 0.f : mx[r];
      corr[r] = exp2f(m_run[r] - msafe[r]);
      m_run[r] = mx[r];
      l_run[r] *= corr[r];
    }
    if (corr[0] != 1.f || corr[1] != 1.f) {  // warp-uniform per quad is not required: plain scaling
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
    }
    uint32_t pf[4];
    {
      const float p00 = exp2f(sacc[0][0] - msafe[0]), p01 = exp2f(sacc[0][1] - msafe[0]);
      const float p02 = exp2f(sacc[0][2] - msafe[1]), p03 = exp2f(sacc[0][3] - msafe[1]);
      const float p10 = exp2f(sacc[1][0] - msafe[0]), p11 = exp2f(sacc[1][1] - msafe[0]);
      const float p12 = exp2f(sacc[1][2] - msafe[1]), p13 = exp2f(sacc[1][3] - msafe[1]);
      l_run[0] += p00 + p01 + p10 + p11;
      l_run[1] += p02 + p03 + p12 + p13;
      pf[0] = pack_pair<T>(p00, p01);
      pf[1] = pack_pair<T>(p02, p03);
      pf[2] = pack_pair<T>(p10, p11);
      pf[3] = pack_pair<T>(p12, p13);
    }
#pragma unroll
    for (int dp = 0; dp < DP / 16; ++dp) {
      uint32_t bf[4];
      ldmatrix_x4_trans(bf, sVs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dp * 16 + (lane >> 4) * 8);
      mma16816<T>(o[dp * 2], pf, bf[0], bf[1]);
      mma16816<T>(o[dp * 2 + 1], pf, bf[2], bf[3]);
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // the ring is free: reuse it for the cross-warp merge

  // ---- merge the 4 warps: each publishes (m, l, O) for its 16 rows -------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  float* sO = reinterpret_cast<float*>(sKV);        // [4 warps][16 rows][DP]
  float* sM = sO + 4 * 16 * DP;                      // [4][16]
  float* sL = sM + 4 * 16;                           // [4][16]
  {
    const int r0 = lane >> 2;
    if ((lane & 3) == 0) {
      sM[warp * 16 + r0] = m_run[0];
      sM[warp * 16 + r0 + 8] = m_run[1];
      sL[warp * 16 + r0] = l_run[0];
      sL[warp * 16 + r0 + 8] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      const int col = i * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(sO + (warp * 16 + r0) * DP + col) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(sO + (warp * 16 + r0 + 8) * DP + col) = make_float2(o[i][2], o[i][3]);
    }
  }
  __syncthreads();
  for (int idx = tid; idx < group * DP; idx += NTHREADS) {
    const int r = idx / DP, d = idx - r * DP;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, sM[w * 16 + r]);
    const float msafe = m == -INFINITY ? 0.f : m;
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float sc = exp2f(sM[w * 16 + r] - msafe);
      l += sL[w * 16 + r] * sc;
      acc += sO[(w * 16 + r) * DP + d] * sc;
    }
    const float val = l > 0.f ? acc / l : 0.f;
    const int h = hk * group + r;
    if (d < a.D) {
      if (a.num_splits > 1)
        part_o[(int64_t)h * a.D + d] = val;
      else
        reinterpret_cast<T*>(a.out)[qtok * a.o_rs + (int64_t)h * a.o_hs + d] = Cvt<T>::from_f32(val);
    }
    if (d == 0) {
      const float lse2 = l > 0.f ? m + log2f(l) : -INFINITY;  // log2 domain
      if (a.num_splits > 1)
        part_lse[(int64_t)h * a.total_q + qtok] = lse2;
      else if (a.lse)
        a.lse[(int64_t)h * a.total_q + qtok] = l > 0.f ? lse2 * 0.6931471805599453f : INFINITY;
    }
  }
}

// out[tok, h, :] = sum_s w_s * O_s / sum_s w_s,  w_s = 2^(lse_s - max lse).
// One warp per (token, head): the lanes first share the splits (maximum and sum of the weights by
// shuffles), then each lane owns four output columns per 128 and reads the partial outputs with
// 16-byte loads when the workspace is 16-byte aligned and D a multiple of 4 (else the scalar loop).
constexpr int kCombineWarps = 8;
template <typename T>
__global__ void __launch_bounds__(kCombineWarps * 32) attn_combine_kernel(AttnArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t pair = (int64_t)blockIdx.x * kCombineWarps + (threadIdx.x >> 5);   // (token, head), head fastest
  if (pair >= a.total_q * a.H) return;
  const int64_t tok = pair / a.H;
  const int h = (int)(pair - tok * a.H);
  const float* lse = a.ws_lse + (int64_t)h * a.total_q + tok;   // split s at lse[s * H * total_q]
  const int64_t lse_step = (int64_t)a.H * a.total_q;
  float m = -INFINITY;
  for (int s = lane; s < a.num_splits; s += 32) m = fmaxf(m, lse[s * lse_step]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float msafe = m == -INFINITY ? 0.f : m;
  float wsum = 0.f;
  for (int s = lane; s < a.num_splits; s += 32) wsum += exp2f(lse[s * lse_step] - msafe);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  const float* part = a.ws_o + (tok * a.H + h) * (int64_t)a.D;   // split s at part[s * total_q * H * D]
  const int64_t part_step = a.total_q * (int64_t)a.H * a.D;
  T* out = reinterpret_cast<T*>(a.out) + tok * a.o_rs + (int64_t)h * a.o_hs;
  if ((a.D & 3) == 0 && (reinterpret_cast<uintptr_t>(a.ws_o) & 15) == 0) {
    for (int d = lane * 4; d < a.D; d += 128) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < a.num_splits; ++s) {
        const float w = exp2f(lse[s * lse_step] - msafe);
        if (w > 0.f) {
          const float4 v = *reinterpret_cast<const float4*>(part + s * part_step + d);
          acc.x += w * v.x;
          acc.y += w * v.y;
          acc.z += w * v.z;
          acc.w += w * v.w;
        }
      }
      out[d] = Cvt<T>::from_f32(acc.x * inv);
      out[d + 1] = Cvt<T>::from_f32(acc.y * inv);
      out[d + 2] = Cvt<T>::from_f32(acc.z * inv);
      out[d + 3] = Cvt<T>::from_f32(acc.w * inv);
    }
  } else {
    for (int d = lane; d < a.D; d += 32) {
      float acc = 0.f;
      for (int s = 0; s < a.num_splits; ++s) {
        const float w = exp2f(lse[s * lse_step] - msafe);
        if (w > 0.f) acc += w * part[s * part_step + d];
      }
      out[d] = Cvt<T>::from_f32(acc * inv);
    }
  }
  if (a.lse && lane == 0)
    a.lse[(int64_t)h * a.total_q + tok] = wsum > 0.f ? (m + log2f(wsum)) * 0.6931471805599453f : INFINITY;
}

static inline unsigned combine_grid(const AttnArgs& a) {
  return (unsigned)((a.total_q * (int64_t)a.H + kCombineWarps - 1) / kCombineWarps);
}

template <typename T, int DP, int STAGES>
int launch_decode(const AttnArgs& a, int chunk_tokens, cudaStream_t st) {
  constexpr int LD = DP + 8;
  constexpr int ring = STAGES * 2 * BN * LD * (int)sizeof(T);
  constexpr int merge = (4 * 16 * DP + 2 * 4 * 16) * 4;
  constexpr int smem = 16 * LD * (int)sizeof(T) + (ring > merge ? ring : merge);
  static thread_local int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    FG_CUDA_OK(cudaFuncSetAttribute(attn_decode_kernel<T, DP, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    smem));
    attr_dev = dev;
  }
  dim3 grid(a.num_splits, a.Hk, a.batch);
  attn_decode_kernel<T, DP, STAGES><<<grid, NTHREADS, smem, st>>>(a, chunk_tokens);
  FG_CHECK_LAUNCH("attn_decode_kernel");
  if (a.num_splits > 1) {
    attn_combine_kernel<T><<<combine_grid(a), kCombineWarps * 32, 0, st>>>(a);
    FG_CHECK_LAUNCH("attn_combine_kernel");
  }
  return FG_OK;
}

}  // namespace

// Chunk length (tokens per CTA) and the number of chunks for a decode batch.  A pure
// function of the host-visible sizes so that the workspace query and the launch agree.
void decode_split_plan(int64_t batch, int64_t num_heads_k, int64_t max_seqlen_k, int forced_splits, int sms,
                       int* chunk_tokens, int* num_splits) {
  if (max_seqlen_k < 1) max_seqlen_k = 1;
  if (forced_splits >= 1) {
    int64_t c = (max_seqlen_k + forced_splits - 1) / forced_splits;
    c = (c + BN - 1) / BN * BN;
    *chunk_tokens = (int)c;
    *num_splits = (int)((max_seqlen_k + c - 1) / c);
    return;
  }
  // Enough CTAs to balance contexts of very different length over all SMs (two
  // resident CTAs each), but never chunks shorter than 256 tokens.
  const int64_t target = (int64_t)sms * 2 * 8;
  int64_t chunk = 1024;
  while (chunk > 256 && batch * num_heads_k * ((max_seqlen_k + chunk - 1) / chunk) < target) chunk >>= 1;
  if (max_seqlen_k <= chunk) {
    *chunk_tokens = (int)((max_seqlen_k + BN - 1) / BN * BN);
    *num_splits = 1;
    return;
  }
  *chunk_tokens = (int)chunk;
  *num_splits = (int)((max_seqlen_k + chunk - 1) / chunk);
}

bool attn_decode_tma_eligible(const AttnArgs& a);
int attn_decode_tma(const AttnArgs& a, int dtype, int chunk_tokens, cudaStream_t st);

// Combine pass shared by both decode kernels.
int launch_decode_combine(const AttnArgs& a, int dtype, cudaStream_t st) {
  if (dtype == FG_BF16)
    attn_combine_kernel<__nv_bfloat16><<<combine_grid(a), kCombineWarps * 32, 0, st>>>(a);
  else
    attn_combine_kernel<__half><<<combine_grid(a), kCombineWarps * 32, 0, st>>>(a);
  FG_CHECK_LAUNCH("attn_combine_kernel");
  return FG_OK;
}

int attn_decode(const AttnArgs& a, int dtype, int chunk_tokens, cudaStream_t st) {
  if (a.batch > 65535 || a.Hk > 65535) return fail(FG_ERR_TOO_LARGE, "flash_attn: batch or heads above 65535");
  // TMA-fed kernel whenever the cache geometry allows one box per page; the cp.async
  // kernel below covers the remaining block sizes.
  if (attn_decode_tma_eligible(a)) return attn_decode_tma(a, dtype, chunk_tokens, st);
  if (dtype == FG_BF16) {
    if (a.D <= 64) return launch_decode<__nv_bfloat16, 64, 3>(a, chunk_tokens, st);
    if (a.D <= 128) return launch_decode<__nv_bfloat16, 128, 3>(a, chunk_tokens, st);
    return launch_decode<__nv_bfloat16, 256, 2>(a, chunk_tokens, st);
  }
  if (a.D <= 64) return launch_decode<__half, 64, 3>(a, chunk_tokens, st);
  if (a.D <= 128) return launch_decode<__half, 128, 3>(a, chunk_tokens, st);
  return launch_decode<__half, 256, 2>(a, chunk_tokens, st);
}

}  // namespace fg
