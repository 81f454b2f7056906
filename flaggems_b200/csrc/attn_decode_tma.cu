// Single-query (decode) attention, TMA-fed: the HBM-bound kernel of the paged decode step.
//
// CTA = (sequence, KV head, KV chunk), 5 warps:
//   warp 0     producer: looks up the pages of each 64-key tile in the block table and
//              issues one cp.async.bulk.tensor box per page and 64-column half for K and V
//              (4-D map over the paged cache; 3-D map over packed K/V) into a 128-byte-
//              swizzled shared-memory ring guarded by full/empty mbarriers
//   warps 1-4  consumers: each owns 16 keys of every tile; the `group` query heads that
//              share the KV head fill the 16 rows of an m16n8k16 tile (read straight from
//              global memory into A fragments), S = Q K^T and O += P V with mma.sync,
//              private online softmax per warp, merged through shared memory at the end
// Consumers issue no global loads in the loop, so the memory pipeline depth is set by the
// ring (3 stages x 32 KB at head dim 128, two CTAs per SM) and not by warp occupancy.
// Partial results of the chunks go to the fp32 workspace and attn_combine_kernel.
#include "attn_common.cuh"
#include "mma_helpers.cuh"
#include "sm100_common.cuh"

namespace fg {

int* device_status_ptr();
int launch_decode_combine(const AttnArgs& a, int dtype, cudaStream_t st);

namespace {

constexpr int BN = 64;
constexpr int NUM_THREADS = 160;
constexpr int HALF = BN * 128;  // bytes of one [64 keys x 64 columns] swizzled sub-tile

struct DecodeTmaArgs {
  AttnArgs a;
  int chunk_tokens;
  int page_rows;       // keys per TMA box
  int pages_per_tile;  // 64 / page_rows
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <typename T, int DP, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                       DecodeTmaArgs da) {
  using namespace sm100;
  constexpr int NH = DP / 64;                  // 64-column halves per row
  constexpr int KV_BYTES = NH * HALF;          // one K (or V) tile
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  const AttnArgs& a = da.a;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + STAGES);

  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const SeqInfo s = seq_info(a, b);
  if (s.q_len < 1) return;
  // drain after a timed-out wait on this device (one thread reads: CTA-uniform decision)
  __shared__ int s_drain;
  if (threadIdx.x == 0) s_drain = *reinterpret_cast<volatile int*>(a.status);
  __syncthreads();
  if (s_drain != 0) return;
  const int kv_begin = split * da.chunk_tokens;
  const int kv_end = min(s.k_len, kv_begin + da.chunk_tokens);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = a.group;
  const int64_t qtok = s.q_begin;

  float* part_o = nullptr;
  float* part_lse = nullptr;
  if (a.num_splits > 1) {
    part_o = a.ws_o + ((int64_t)split * a.total_q + qtok) * a.H * a.D;
    part_lse = a.ws_lse + (int64_t)split * a.H * a.total_q;
  }
  if (kv_begin >= kv_end) {  // empty chunk (or k_len == 0): contributes nothing
    if (a.num_splits > 1) {
      if (tid < group) part_lse[(int64_t)(hk * group + tid) * a.total_q + qtok] = -INFINITY;
    } else {
      T* out = reinterpret_cast<T*>(a.out) + qtok * a.o_rs + (int64_t)hk * group * a.o_hs;
      for (int i = tid; i < group * a.D; i += NUM_THREADS) out[(i / a.D) * a.o_hs + (i % a.D)] = Cvt<T>::from_f32(0.f);
      if (a.lse && tid < group) a.lse[(int64_t)(hk * group + tid) * a.total_q + qtok] = INFINITY;
    }
    return;
  }
  const int n_tiles = (kv_end - kv_begin + BN - 1) / BN;

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  __syncthreads();

  if (warp == 0) {
    // ================================ producer ====================================
    const int32_t* bt_row = a.paged ? a.block_table + (int64_t)b * a.bt_stride : nullptr;
    const int last_page = a.paged ? max(0, (s.k_len - 1) / a.block_size) : 0;
    auto lookup = [&](int t, int& page, int& row_off) {
      page = 0;
      row_off = 0;
      if (a.paged && lane < da.pages_per_tile && t < n_tiles) {
        const int tok = kv_begin + t * BN + lane * da.page_rows;
        int pg = tok / a.block_size;
        row_off = tok - pg * a.block_size;
        pg = min(pg, last_page);  // past the end of the sequence: any valid page (those keys are masked)
        page = max(0, min(bt_row[pg], a.num_blocks - 1));
      }
    };
    int page, row_off;
    lookup(0, page, row_off);
    for (int t = 0; t < n_tiles; ++t) {
      const int stg = t % STAGES;
      const uint32_t ph = (uint32_t)((t / STAGES) & 1);
      int npage, nrow;
      lookup(t + 1, npage, nrow);  // the table entry of the next tile is in flight while this one is issued
      if (!mbar_wait(&empty[stg], ph ^ 1, abort_flag, a.status, kStatusAttnTimeout)) break;
      if (lane == 0) mbar_expect_tx(&full[stg], STAGE_BYTES);
      __syncwarp();
      uint8_t* kdst = smem + stg * STAGE_BYTES;
      uint8_t* vdst = kdst + KV_BYTES;
      if (a.paged) {
        if (lane < da.pages_per_tile) {
          const int off = lane * da.page_rows * 128;
#pragma unroll
          for (int hf = 0; hf < NH; ++hf) {
            tma_load_4d(kdst + hf * HALF + off, &tmap_k, &full[stg], hf * 64, hk, row_off, page);
            tma_load_4d(vdst + hf * HALF + off, &tmap_v, &full[stg], hf * 64, hk, row_off, page);
          }
        }
      } else if (lane == 0) {
        const int row = s.k_begin + kv_begin + t * BN;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
          tma_load_3d(kdst + hf * HALF, &tmap_k, &full[stg], hf * 64, hk, row);
          tma_load_3d(vdst + hf * HALF, &tmap_v, &full[stg], hf * 64, hk, row);
        }
      }
      page = npage;
      row_off = nrow;
    }
  } else {
    // ================================ consumers ===================================
    const int w = warp - 1;
    const int g = lane >> 2, tq = lane & 3;
    // Q as A fragments, straight from global memory (rows >= group and columns >= D are zero)
    uint32_t qf[DP / 16][4];
    {
      const T* Q = reinterpret_cast<const T*>(a.q) + qtok * a.q_rs + (int64_t)hk * group * a.q_hs;
#pragma unroll
      for (int kk = 0; kk < DP / 16; ++kk) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = g + (i & 1) * 8;
          const int col = kk * 16 + tq * 2 + (i >> 1) * 8;
          qf[kk][i] = (row < group && col < a.D) ? *reinterpret_cast<const uint32_t*>(Q + (int64_t)row * a.q_hs + col) : 0u;
        }
      }
    }
    float o[DP / 8][4];
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    // per-lane pieces of the swizzled ldmatrix addresses
    const int k_row = w * 16 + (lane & 7) + (lane >> 4) * 8;          // K: n index
    const int k_chunk = (lane >> 3) & 1;                               // + kk*2
    const int v_row = w * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;     // V: key index
    const int v_chunk = lane >> 4;                                     // + dp*2
    const int sw = lane & 7;                                           // row & 7 for both
    bool ok = true;

    for (int t = 0; t < n_tiles; ++t) {
      const int stg = t % STAGES;
      const uint32_t ph = (uint32_t)((t / STAGES) & 1);
      if (!mbar_wait(&full[stg], ph, abort_flag, a.status, kStatusAttnTimeout)) {
        ok = false;
        break;
      }
      const uint8_t* sK = smem + stg * STAGE_BYTES;
      uint8_t* sV = smem + stg * STAGE_BYTES + KV_BYTES;

      float sacc[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DP / 16; ++kk) {
        const int ch = kk * 2 + k_chunk;
        uint32_t bf[4];
        ldmatrix_x4(bf, sK + (ch >> 3) * HALF + k_row * 128 + (((ch & 7) ^ sw) << 4));
        mma16816<T>(sacc[0], qf[kk], bf[0], bf[1]);
        mma16816<T>(sacc[1], qf[kk], bf[2], bf[3]);
      }
      const int j0 = kv_begin + t * BN + w * 16;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = sacc[nt][e];
          if (a.has_softcap) v = tanhf(v * a.softcap_pre);
          v *= a.scale_log2;
          const int col = j0 + nt * 8 + tq * 2 + (e & 1);
          if (col >= kv_end) v = -INFINITY;
          sacc[nt][e] = v;
        }
      }
      if (j0 + 16 > kv_end) {
        // keys of this warp past the end of the chunk: their V rows may hold anything
        // (the tail of a cache page); zero them so that 0 * garbage cannot give NaN
        const int first = max(0, kv_end - j0);
        for (int idx = lane; idx < (16 - first) * NH * 8; idx += 32) {
          const int r = w * 16 + first + idx / (NH * 8);
          const int c = idx % (NH * 8);
          *reinterpret_cast<uint4*>(sV + (c >> 3) * HALF + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
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
      if (corr[0] != 1.f || corr[1] != 1.f) {
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
        const int ch = dp * 2 + v_chunk;
        uint32_t bf[4];
        ldmatrix_x4_trans(bf, sV + (ch >> 3) * HALF + v_row * 128 + (((ch & 7) ^ sw) << 4));
        mma16816<T>(o[dp * 2], pf, bf[0], bf[1]);
        mma16816<T>(o[dp * 2 + 1], pf, bf[2], bf[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stg]);  // this warp is done with the stage
    }

    // ---- merge the 4 consumer warps (the ring is idle: every tile has been consumed) ----
    consumer_sync();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    float* sO = reinterpret_cast<float*>(smem);  // [4 warps][16 rows][DP]
    float* sM = sO + 4 * 16 * DP;                // [4][16]
    float* sL = sM + 4 * 16;                     // [4][16]
    if (ok) {
      if (tq == 0) {
        sM[w * 16 + g] = m_run[0];
        sM[w * 16 + g + 8] = m_run[1];
        sL[w * 16 + g] = l_run[0];
        sL[w * 16 + g + 8] = l_run[1];
      }
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        const int col = i * 8 + tq * 2;
        *reinterpret_cast<float2*>(sO + (w * 16 + g) * DP + col) = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2*>(sO + (w * 16 + g + 8) * DP + col) = make_float2(o[i][2], o[i][3]);
      }
    }
    consumer_sync();
    if (ok && !*abort_flag) {
      const int ctid = tid - 32;
      for (int idx = ctid; idx < group * DP; idx += 128) {
        const int r = idx / DP, d = idx - r * DP;
        float m = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < 4; ++ww) m = fmaxf(m, sM[ww * 16 + r]);
        const float msafe = m == -INFINITY ? 0.f : m;
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int ww = 0; ww < 4; ++ww) {
          const float sc = exp2f(sM[ww * 16 + r] - msafe);
          l += sL[ww * 16 + r] * sc;
          acc += sO[(ww * 16 + r) * DP + d] * sc;
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
          const float lse2 = l > 0.f ? m + log2f(l) : -INFINITY;
          if (a.num_splits > 1)
            part_lse[(int64_t)h * a.total_q + qtok] = lse2;
          else if (a.lse)
            a.lse[(int64_t)h * a.total_q + qtok] = l > 0.f ? lse2 * 0.6931471805599453f : INFINITY;
        }
      }
    }
  }
}

template <typename T, int DP, int STAGES>
int launch_decode_tma(const DecodeTmaArgs& da, const CUtensorMap& tk, const CUtensorMap& tv, int dtype,
                      cudaStream_t st) {
  constexpr int ring = STAGES * 2 * (DP / 64) * HALF;
  constexpr int merge = (4 * 16 * DP + 2 * 4 * 16) * 4;
  static_assert(merge <= ring, "merge buffers must fit in the ring");
  constexpr int smem = ring + 1024 + 128;
  static thread_local int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    FG_CUDA_OK(cudaFuncSetAttribute(attn_decode_tma_kernel<T, DP, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    smem));
    attr_dev = dev;
  }
  const AttnArgs& a = da.a;
  dim3 grid(a.num_splits, a.Hk, a.batch);
  attn_decode_tma_kernel<T, DP, STAGES><<<grid, NUM_THREADS, smem, st>>>(tk, tv, da);
  FG_CHECK_LAUNCH("attn_decode_tma_kernel");
  if (a.num_splits > 1) return launch_decode_combine(a, dtype, st);
  return FG_OK;
}

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace

bool attn_decode_tma_eligible(const AttnArgs& a) {
  if (a.batch > 65535 || a.Hk > 65535) return false;
  if (a.paged) {
    if (!is_pow2(a.block_size) || a.block_size < 8) return false;
  }
  return true;
}

int attn_decode_tma(const AttnArgs& a, int dtype, int chunk_tokens, cudaStream_t st) {
  DecodeTmaArgs da;
  da.a = a;
  da.chunk_tokens = chunk_tokens;
  da.page_rows = a.paged ? (a.block_size < BN ? a.block_size : BN) : BN;
  da.pages_per_tile = BN / da.page_rows;
  if (!da.a.status) return fail(FG_ERR_CUDA, "flash_attn_varlen: device status word unavailable");
  CUtensorMap tk, tv;
  if (a.paged) {
    uint64_t dims[4] = {(uint64_t)a.D, (uint64_t)a.Hk, (uint64_t)a.block_size, (uint64_t)a.num_blocks};
    uint32_t box[4] = {64, 1, (uint32_t)da.page_rows, 1};
    uint64_t ks[3] = {(uint64_t)a.k_hs * 2, (uint64_t)a.k_rs * 2, (uint64_t)a.k_bs * 2};
    uint64_t vs[3] = {(uint64_t)a.v_hs * 2, (uint64_t)a.v_rs * 2, (uint64_t)a.v_bs * 2};
    int rc = encode_tmap_16bit(&tk, a.k, 4, dims, ks, box);
    if (rc != FG_OK) return rc;
    rc = encode_tmap_16bit(&tv, a.v, 4, dims, vs, box);
    if (rc != FG_OK) return rc;
  } else {
    uint64_t dims[3] = {(uint64_t)a.D, (uint64_t)a.Hk, (uint64_t)(a.total_k > 0 ? a.total_k : 1)};
    uint32_t box[3] = {64, 1, 64};
    uint64_t ks[2] = {(uint64_t)a.k_hs * 2, (uint64_t)a.k_rs * 2};
    uint64_t vs[2] = {(uint64_t)a.v_hs * 2, (uint64_t)a.v_rs * 2};
    int rc = encode_tmap_16bit(&tk, a.k, 3, dims, ks, box);
    if (rc != FG_OK) return rc;
    rc = encode_tmap_16bit(&tv, a.v, 3, dims, vs, box);
    if (rc != FG_OK) return rc;
  }
  if (dtype == FG_BF16) {
    if (a.D <= 64) return launch_decode_tma<__nv_bfloat16, 64, 4>(da, tk, tv, dtype, st);
    if (a.D <= 128) return launch_decode_tma<__nv_bfloat16, 128, 3>(da, tk, tv, dtype, st);
    return launch_decode_tma<__nv_bfloat16, 256, 3>(da, tk, tv, dtype, st);
  }
  if (a.D <= 64) return launch_decode_tma<__half, 64, 4>(da, tk, tv, dtype, st);
  if (a.D <= 128) return launch_decode_tma<__half, 128, 3>(da, tk, tv, dtype, st);
  return launch_decode_tma<__half, 256, 3>(da, tk, tv, dtype, st);
}

}  // namespace fg
