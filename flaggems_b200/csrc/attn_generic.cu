// General FlashAttention-2 forward for variable-length sequences over a paged or
// contiguous KV store: any head dim <= 256 (multiple of 8), causal / sliding-window
// masks, ALiBi, soft-capping, fp16 / bf16.  Warp-level mma.sync (m16n8k16) with fp32
// accumulation; one CTA = 64 query rows of one (sequence, head), 4 warps x 16 rows,
// KV streamed in 64-row tiles through a two-stage cp.async ring.
//
// This is the feature-complete path.  Prefill at head dim 128 without ALiBi /
// soft-cap is taken by the tcgen05 kernel, single-token decode by the split-KV
// kernel; both fall back here for anything they do not cover.
#include "attn_common.cuh"
#include "mma_helpers.cuh"

namespace fg {
namespace {

constexpr int BM = 64, BN = 64, NTHREADS = 128;

// Load ROWS x DP elements into smem (row stride LD); 2 threads per row when ROWS == 64.
// row_off[r] < 0 marks a row to be zero-filled.
template <typename T, int DP>
__device__ __forceinline__ void load_rows(T* sdst, const T* gbase, int64_t row_off, bool row_valid, int d,
                                          int row, int part) {
  constexpr int LD = DP + 8;
  constexpr int CPR = DP / 8;        // 16-byte chunks per padded row
  constexpr int PER = CPR / 2;       // chunks per thread
  const int dchunks = d >> 3;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int ch = part * PER + i;
    const bool ok = row_valid && ch < dchunks;
    cp_async16(sdst + row * LD + ch * 8, ok ? (const void*)(gbase + row_off + ch * 8) : (const void*)gbase, ok);
  }
}

template <typename T, int DP>
__global__ void __launch_bounds__(NTHREADS) attn_fwd_generic_kernel(AttnArgs a) {
  constexpr int LD = DP + 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sK = sQ + BM * LD;            // [2][BN][LD]
  T* sV = sK + 2 * BN * LD;        // [2][BN][LD]

  const int num_mb = gridDim.x;
  const int m_block = num_mb - 1 - blockIdx.x;  // long (late) causal rows first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const SeqInfo s = seq_info(a, b);
  const int m0 = m_block * BM;
  if (m0 >= s.q_len) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hk = h / a.group;
  const int shift = s.k_len - s.q_len;  // bottom-right alignment of the mask
  const bool right_bound = a.causal || a.wr >= 0;
  const int wr = a.causal ? 0 : a.wr;

  int n_min = 0;
  if (a.wl >= 0) n_min = max(0, (m0 + shift - a.wl) / BN);
  int n_max = (s.k_len + BN - 1) / BN;
  if (right_bound) {
    const int lim = m0 + BM + shift + wr;  // exclusive bound on visible columns of this row block
    n_max = lim <= 0 ? 0 : min(n_max, (lim + BN - 1) / BN);
  }

  const T* Q = reinterpret_cast<const T*>(a.q);
  const T* K = reinterpret_cast<const T*>(a.k) + (int64_t)hk * a.k_hs;
  const T* V = reinterpret_cast<const T*>(a.v) + (int64_t)hk * a.v_hs;
  const int32_t* bt_row = a.paged ? a.block_table + (int64_t)b * a.bt_stride : nullptr;

  const int lrow = tid >> 1, lpart = tid & 1;  // loader mapping: 2 threads per tile row
  {
    const int qr = m0 + lrow;
    const bool ok = qr < s.q_len;
    const int64_t off = (int64_t)(s.q_begin + qr) * a.q_rs + (int64_t)h * a.q_hs;
    load_rows<T, DP>(sQ, Q, off, ok, a.D, lrow, lpart);
  }
  auto load_kv = [&](int n_block, int stage) {
    const int tok = n_block * BN + lrow;
    const bool ok = tok < s.k_len;
    int64_t koff = 0, voff = 0;
    if (ok) {
      koff = kv_row_offset(a, bt_row, s.k_begin, tok, a.k_rs, a.k_bs);
      voff = kv_row_offset(a, bt_row, s.k_begin, tok, a.v_rs, a.v_bs);
    }
    load_rows<T, DP>(sK + stage * BN * LD, K, koff, ok, a.D, lrow, lpart);
    load_rows<T, DP>(sV + stage * BN * LD, V, voff, ok, a.D, lrow, lpart);
  };
  if (n_min < n_max) load_kv(n_min, 0);
  cp_async_commit();

  float o[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  const int row_in_tile = warp * 16 + (lane >> 2);  // + 8 for the second row
  float slope2 = 0.f;
  if (a.has_alibi) slope2 = a.alibi[(int64_t)b * a.alibi_bs + h] * 1.4426950408889634f;

  for (int nb = n_min; nb < n_max; ++nb) {
    const int stage = (nb - n_min) & 1;
    // prefetch the next tile into the other stage (its previous reader finished at the
    // trailing __syncthreads of the last iteration)
    if (nb + 1 < n_max) load_kv(nb + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const T* sKs = sK + stage * BN * LD;
    const T* sVs = sV + stage * BN * LD;

    // ---- S = Q K^T (16 x 64 per warp) ----
    float sacc[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
      uint32_t af[4];
      ldmatrix_x4(af, sQ + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        uint32_t bf[4];
        ldmatrix_x4(bf, sKs + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
        mma16816<T>(sacc[np * 2], af, bf[0], bf[1]);
        mma16816<T>(sacc[np * 2 + 1], af, bf[2], bf[3]);
      }
    }

    // ---- scale / soft-cap / ALiBi / mask, all in the log2 domain ----
    const int j0 = nb * BN;
    const bool need_mask = (j0 + BN > s.k_len) || (right_bound && (j0 + BN - 1 > m0 + shift + wr)) ||
                           (a.wl >= 0 && (j0 < m0 + BM - 1 + shift - a.wl));
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = sacc[nt][e];
        if (a.has_softcap) v = tanhf(v * a.softcap_pre);
        v *= a.scale_log2;
        const int col = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        const int row = m0 + row_in_tile + (e >> 1) * 8;
        if (a.has_alibi) {
          if (a.causal)
            v += slope2 * (float)(col - s.k_len + 1);
          else
            v -= slope2 * fabsf((float)(col - shift - row));
        }
        if (need_mask) {
          bool dead = col >= s.k_len;
          if (right_bound) dead = dead || (col > row + shift + wr);
          if (a.wl >= 0) dead = dead || (col < row + shift - a.wl);
          if (dead) v = -INFINITY;
        }
        sacc[nt][e] = v;
      }
    }

    // ---- online softmax ----
    float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
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
      corr[r] = exp2f(m_run[r] - msafe[r]);  // m_run == -inf -> 0
      m_run[r] = mx[r];
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
    uint32_t pf[BN / 16][4];  // P as A fragments (k = kv index)
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      const float p0 = exp2f(sacc[nt][0] - msafe[0]);
      const float p1 = exp2f(sacc[nt][1] - msafe[0]);
      const float p2 = exp2f(sacc[nt][2] - msafe[1]);
      const float p3 = exp2f(sacc[nt][3] - msafe[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      // C-fragment of n-tiles (2k, 2k+1) == A-fragment of k-step k
      pf[nt >> 1][(nt & 1) * 2 + 0] = pack_pair<T>(p0, p1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = pack_pair<T>(p2, p3);
    }

    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
      for (int dp = 0; dp < DP / 16; ++dp) {
        uint32_t bf[4];
        ldmatrix_x4_trans(bf, sVs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dp * 16 + (lane >> 4) * 8);
        mma16816<T>(o[dp * 2], pf[kk], bf[0], bf[1]);
        mma16816<T>(o[dp * 2 + 1], pf[kk], bf[2], bf[3]);
      }
    }
    __syncthreads();  // everyone is done with this stage before it is refilled
  }
  cp_async_wait<0>();

  // ---- epilogue ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  float inv[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) inv[r] = (l_run[r] > 0.f) ? 1.f / l_run[r] : 1.f;

  __syncthreads();  // Q tile no longer needed by any warp: reuse it to stage O
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) {
    const int col = i * 8 + (lane & 3) * 2;
    *reinterpret_cast<uint32_t*>(sQ + row_in_tile * LD + col) = pack_pair<T>(o[i][0] * inv[0], o[i][1] * inv[0]);
    *reinterpret_cast<uint32_t*>(sQ + (row_in_tile + 8) * LD + col) = pack_pair<T>(o[i][2] * inv[1], o[i][3] * inv[1]);
  }
  __syncthreads();
  {
    constexpr int CPR = DP / 8, PER = CPR / 2;
    const int qr = m0 + lrow;
    if (qr < s.q_len) {
      T* orow = reinterpret_cast<T*>(a.out) + (int64_t)(s.q_begin + qr) * a.o_rs + (int64_t)h * a.o_hs;
      const int dchunks = a.D >> 3;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int ch = lpart * PER + i;
        if (ch < dchunks)
          *reinterpret_cast<uint4*>(orow + ch * 8) = *reinterpret_cast<const uint4*>(sQ + lrow * LD + ch * 8);
      }
    }
  }
  if (a.lse != nullptr && (lane & 3) == 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int qr = m0 + row_in_tile + r * 8;
      if (qr < s.q_len) {
        const float v = (l_run[r] > 0.f) ? m_run[r] * 0.6931471805599453f + logf(l_run[r]) : INFINITY;
        a.lse[(int64_t)h * a.total_q + s.q_begin + qr] = v;
      }
    }
  }
}

template <typename T, int DP>
int launch_generic(const AttnArgs& a, cudaStream_t st) {
  constexpr int LD = DP + 8;
  constexpr int smem = (BM + 4 * BN) * LD * (int)sizeof(T);
  static thread_local int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    FG_CUDA_OK(cudaFuncSetAttribute(attn_fwd_generic_kernel<T, DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_dev = dev;
  }
  dim3 grid((a.max_q + BM - 1) / BM, a.H, a.batch);
  attn_fwd_generic_kernel<T, DP><<<grid, NTHREADS, smem, st>>>(a);
  FG_CHECK_LAUNCH("attn_fwd_generic_kernel");
  return FG_OK;
}

}  // namespace

int attn_generic(const AttnArgs& a, int dtype, cudaStream_t st) {
  if (a.batch > 65535 || a.H > 65535) return fail(FG_ERR_TOO_LARGE, "flash_attn: batch or heads above 65535");
  if (dtype == FG_BF16) {
    if (a.D <= 64) return launch_generic<__nv_bfloat16, 64>(a, st);
    if (a.D <= 128) return launch_generic<__nv_bfloat16, 128>(a, st);
    return launch_generic<__nv_bfloat16, 256>(a, st);
  }
  if (a.D <= 64) return launch_generic<__half, 64>(a, st);
  if (a.D <= 128) return launch_generic<__half, 128>(a, st);
  return launch_generic<__half, 256>(a, st);
}

}  // namespace fg
