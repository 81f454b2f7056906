// Prefill attention for head dim 128 on sm_100a tensor cores (tcgen05 + TMEM).
//
// One CTA = 128 query positions of one sequence x TWO query heads of the same KV
// group (one when the group size is odd): the two 128-row Q tiles share every K/V
// tile, which halves the K/V traffic and lets the tensor pipe work on one tile while
// the softmax warps work on the other.
//
//   warp 0       TMA producer: Q tiles once, then K and V tiles (128 keys x 128) through
//                two 2-stage rings; paged caches are fetched page by page with one
//                4-D box per page and 64-column half, so a tile lands as a dense,
//                128-byte-swizzled K-major tile
//   warp 1       issues tcgen05.mma from one thread: S_t = Q_t K^T as one SS group per 128
//                keys (M128 N128, 8 x K16 -- an SS instruction costs ~115 cycles whatever
//                its N, so N is kept at 128), and O_t += P_t V as TS MMAs (P read from TMEM
//                as the A operand, full rate) in two halves of 64 keys
//   warps 4-7    softmax of Q tile 0: one thread per row (TMEM lane = row), in two halves of
//   warps 8-11   64 keys: tcgen05.ld the scores, scale, mask, exp2, pack P to 16 bit and
//   (tile 1)     tcgen05.st it over the first 32 columns of that half; PV of the first half
//                runs while the second half is exponentiated.  The running max is only
//                raised when it grows by more than 8 (log2 units), so the O accumulator in
//                TMEM is rescaled rarely; the same warps write the normalised output
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P halves alias S halves.
//
// Covers: fp16/bf16, head dim 128, causal or full attention, paged (block size a
// power of two >= 8) or contiguous KV.  ALiBi, soft-cap, windows and other head dims
// take the general kernel.
#include "attn_common.cuh"
#include "sm100_common.cuh"

#ifdef FG_PREFILL_TRACE
// Debug build only: cycle stamps of one CTA's roles (never part of the shipped library).
__device__ long long g_fg_trace[8192];
#define FG_TRACE(slot, idx)                                                   \
  do {                                                                        \
    if (trace_on && (idx) < 64) g_fg_trace[(slot) * 64 + (idx)] = clock64(); \
  } while (0)
extern "C" __attribute__((visibility("default"))) int fg_debug_read_trace(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_fg_trace, sizeof(long long) * n);
}
#else
#define FG_TRACE(slot, idx) \
  do {                      \
  } while (0)
#endif

namespace fg {

int* device_status_ptr();

namespace {

constexpr int BM = 128, BN = 128, HD = 128;
constexpr int HALF_BYTES = 128 * 64 * 2;   // one [128 x 64] 128B-swizzled sub-tile
constexpr int TILE_BYTES = 2 * HALF_BYTES; // 32 KB
constexpr int NUM_THREADS = 384;
constexpr int SMEM_BYTES = 6 * TILE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct PrefillArgs {
  AttnArgs a;
  int tiles;            // query tiles per CTA (1 or 2)
  int page_rows;        // rows fetched per TMA box for K/V (min(block_size, 128)); 128 when contiguous
  int pages_per_tile;   // 128 / page_rows
  int is_bf16;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA pipe (the MUFU unit, 4 lanes per clock and scheduler, is what the two
// softmax warpgroups contend for): split x = n + f with a round-down add, evaluate a
// cubic for 2^f on [0,1) and add n to the exponent field.  Relative error about 1e-4,
// far below the 16-bit rounding of P.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -126.0f);
  const float magic = 12582912.0f;                 // 1.5 * 2^23
  const float xr = __fadd_rd(x, magic);            // integer part in the low mantissa bits
  const float f = x - (xr - magic);                // [0, 1)
  float p = fmaf(f, 0.077119873f, 0.227564394f);
  p = fmaf(p, f, 0.695146143f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + ((__float_as_int(xr) - 0x4B400000) << 23));
}
#ifndef FG_PREFILL_POLY_EVERY
#define FG_PREFILL_POLY_EVERY 0
#endif
// every kPolyEvery-th probability pair of a row takes ex2_poly (0 = never)
constexpr int kPolyEvery = FG_PREFILL_POLY_EVERY;
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, PrefillArgs pa) {
  using namespace sm100;
  const AttnArgs& a = pa.a;
  const int num_mb = gridDim.x;
  const int m_block = num_mb - 1 - blockIdx.x;
  const int b = blockIdx.z;
  const int NT = pa.tiles;
  const int h0 = blockIdx.y * NT;
  const SeqInfo s = seq_info(a, b);
  const int m0 = m_block * BM;
  if (m0 >= s.q_len) return;  // before any allocation
  // A wait that timed out anywhere on this device left the status word set: finish the
  // launch quickly instead of letting every remaining CTA run into the same timeout
  // (one thread reads it so that the whole CTA takes the same decision).
  __shared__ int s_drain;
  if (threadIdx.x == 0) s_drain = *reinterpret_cast<volatile int*>(a.status);
  __syncthreads();
  if (s_drain != 0) return;

  const int shift = s.k_len - s.q_len;
  int n_tiles = (s.k_len + BN - 1) / BN;
  if (a.causal) {
    const int lim = m0 + BM + shift;  // exclusive bound on visible keys of this row block
    n_tiles = lim <= 0 ? 0 : min(n_tiles, (lim + BN - 1) / BN);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef FG_PREFILL_TRACE
  const bool trace_on = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) && (lane == 0);
#endif

  if (n_tiles == 0) {
    // no visible key for any row of the block: zeros, lse = +inf
    for (int idx = threadIdx.x; idx < NT * BM * (HD / 8); idx += NUM_THREADS) {
      const int t = idx / (BM * (HD / 8));
      const int r = (idx / (HD / 8)) % BM;
      const int c = idx % (HD / 8);
      if (m0 + r < s.q_len) {
        uint4 z = make_uint4(0, 0, 0, 0);
        char* o = reinterpret_cast<char*>(a.out) +
                  ((int64_t)(s.q_begin + m0 + r) * a.o_rs + (int64_t)(h0 + t) * a.o_hs) * 2 + c * 16;
        *reinterpret_cast<uint4*>(o) = z;
      }
    }
    if (a.lse)
      for (int idx = threadIdx.x; idx < NT * BM; idx += NUM_THREADS) {
        const int t = idx / BM, r = idx % BM;
        if (m0 + r < s.q_len) a.lse[(int64_t)(h0 + t) * a.total_q + s.q_begin + m0 + r] = INFINITY;
      }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                       // [2 tiles][2 halves][128 x 64]
  uint8_t* sK = smem + 2 * TILE_BYTES;      // [2 stages]
  uint8_t* sV = smem + 4 * TILE_BYTES;      // [2 stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2] per tile
  uint64_t* p_ready = bars + 11;      // [2 tiles][2 halves]
  uint64_t* o_done = bars + 15;       // [2 tiles][2 halves]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&p_ready[i], 128);
      mbar_init(&o_done[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int hk = h0 / a.group;
  const int st_code = kStatusAttnTimeout;

  if (warp == 0) {
    // ================================ TMA producer ================================
    if (lane == 0) {
      mbar_expect_tx(q_full, NT * TILE_BYTES);
      for (int t = 0; t < NT; ++t)
        for (int hf = 0; hf < 2; ++hf)
          tma_load_3d(sQ + t * TILE_BYTES + hf * HALF_BYTES, &tmap_q, q_full, hf * 64, h0 + t, s.q_begin + m0);
    }
    const int32_t* bt_row = a.paged ? a.block_table + (int64_t)b * a.bt_stride : nullptr;
    const int last_page = a.paged ? max(0, (s.k_len - 1) / a.block_size) : 0;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int stg = j & 1;
      const uint32_t ph = (uint32_t)((j >> 1) & 1);
      // page of this lane (paged form): lanes [0, pages_per_tile) each fetch one page
      int page = 0, row_off = 0;
      if (a.paged && lane < pa.pages_per_tile) {
        const int tok = j * BN + lane * pa.page_rows;
        int pg = tok / a.block_size;
        row_off = tok - pg * a.block_size;
        pg = min(pg, last_page);  // pages past the end of the sequence: refetch a valid one (masked later)
        page = max(0, min(bt_row[pg], a.num_blocks - 1));
      }
      for (int which = 0; which < 2 && ok; ++which) {
        uint64_t* full = which ? &v_full[stg] : &k_full[stg];
        uint64_t* empty = which ? &v_empty[stg] : &k_empty[stg];
        const CUtensorMap* tm = which ? &tmap_v : &tmap_k;
        uint8_t* dst = (which ? sV : sK) + stg * TILE_BYTES;
        if (!mbar_wait(empty, ph ^ 1, abort_flag, a.status, st_code)) {
          ok = false;
          break;
        }
        if (lane == 0) mbar_expect_tx(full, TILE_BYTES);
        __syncwarp();
        if (a.paged) {
          if (lane < pa.pages_per_tile) {
            for (int hf = 0; hf < 2; ++hf)
              tma_load_4d(dst + hf * HALF_BYTES + lane * pa.page_rows * 128, tm, full, hf * 64, hk, row_off, page);
          }
        } else if (lane == 0) {
          for (int hf = 0; hf < 2; ++hf)
            tma_load_3d(dst + hf * HALF_BYTES, tm, full, hf * 64, hk, s.k_begin + j * BN);
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer ==================================
    if (lane == 0) {
      const bool bf16 = pa.is_bf16 != 0;
      const uint32_t idesc_qk = umma_idesc_f16(bf16, false, false, BM, BN);  // A, B K-major
      const uint32_t idesc_pv = umma_idesc_f16(bf16, false, true, BM, HD);   // B (V) MN-major
      auto issue_qk = [&](int t, int stg) {
        const uint32_t qa = smem_u32(sQ + t * TILE_BYTES);
        const uint32_t ka = smem_u32(sK + stg * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          mma_f16_ss(tmem_base + t * 128, umma_desc_sw128(qa + off, 0, 1024), umma_desc_sw128(ka + off, 0, 1024),
                     idesc_qk, k != 0 ? 1u : 0u);
        }
      };
      auto issue_pv_half = [&](int t, int stg, int h, bool acc) {
        const uint32_t va = smem_u32(sV + stg * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // V: MN-major, 64-column blocks HALF_BYTES apart, 8-key groups 1024 B apart, 16 keys per step
          const uint64_t bdesc = umma_desc_sw128(va + (h * 4 + k) * 2048, HALF_BYTES, 1024);
          mma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + h * 64 + k * 8, bdesc, idesc_pv,
                     (acc || k != 0) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, a.status, st_code);
      ok = ok && mbar_wait(&k_full[0], 0, abort_flag, a.status, st_code);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < NT; ++t) {
          issue_qk(t, 0);
          tc_commit(&s_full[t]);
        }
        tc_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int stg = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!mbar_wait(&v_full[stg], ph, abort_flag, a.status, st_code)) break;
        for (int t = 0; t < NT; ++t) {
          for (int h = 0; h < 2 && ok; ++h) {
            if (!mbar_wait(&p_ready[t * 2 + h], (uint32_t)(j & 1), abort_flag, a.status, st_code)) {
              ok = false;
              break;
            }
            tc_fence_after();
            FG_TRACE(0 + t * 2 + h, j);
            issue_pv_half(t, stg, h, j > 0 || h > 0);
            tc_commit(&o_done[t * 2 + h]);
          }
          if (!ok) break;
          if (t == NT - 1) tc_commit(&v_empty[stg]);
          if (j + 1 < n_tiles) {
            const int nstg = (j + 1) & 1;
            if (t == 0 && !mbar_wait(&k_full[nstg], (uint32_t)(((j + 1) >> 1) & 1), abort_flag, a.status, st_code)) {
              ok = false;
              break;
            }
            tc_fence_after();
            issue_qk(t, nstg);
            tc_commit(&s_full[t]);
            if (t == NT - 1) tc_commit(&k_empty[nstg]);
          }
        }
      }
    }
  } else if (warp >= 4 && warp < 4 + 4 * NT) {
    // ================================ softmax / epilogue ===========================
    const int t = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;        // row inside the tile == TMEM lane
    const int qpos = m0 + r;                  // query position inside the sequence
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + t * 128;
    const uint32_t o_addr = tmem_base + lane_addr + 256 + t * 128;
    const bool bf16 = pa.is_bf16 != 0;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;

    const float scale = a.scale_log2;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!mbar_wait(&s_full[t], (uint32_t)(j & 1), abort_flag, a.status, st_code)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (quarter == 0) FG_TRACE(4 + t * 16, j);
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const uint32_t sh_addr = s_addr + h * 64;
        float sv[64];
        {
          uint32_t* u = reinterpret_cast<uint32_t*>(sv);
          tmem_ld32(sh_addr + 0, *reinterpret_cast<uint32_t(*)[32]>(u));
          tmem_ld32(sh_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(u + 32));
          tmem_ld_wait();
        }
        const int col0 = j * BN + h * 64;
        const bool need_mask = (col0 + 64 > s.k_len) || (a.causal && (col0 + 63 > m0 + shift));
        if (need_mask) {
          int lim = s.k_len - 1;                        // last visible column
          if (a.causal) lim = min(lim, qpos + shift);
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (col0 + i > lim) sv[i] = -INFINITY;
        }
        // four independent chains of three-input max
        float mx4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
        for (int i = 4; i < 64; i += 8) {
          mx4[0] = max3(mx4[0], sv[i], sv[i + 1]);
          mx4[1] = max3(mx4[1], sv[i + 2], sv[i + 3]);
          if (i + 4 < 64) {
            mx4[2] = max3(mx4[2], sv[i + 4], sv[i + 5]);
            mx4[3] = max3(mx4[3], sv[i + 6], sv[i + 7]);
          }
        }
        const float m_tile = fmaxf(max3(mx4[0], mx4[1], mx4[2]), mx4[3]) * scale;  // scale > 0
        // Raise the reference maximum only when it grows by more than the threshold:
        // probabilities then stay below 2^8 and the accumulator needs no rescale.
        const bool raise = m_tile > m_used + kRescaleThreshold || (m_used == -INFINITY && m_tile > -INFINITY);
        if ((j > 0 || h > 0) && __any_sync(0xffffffffu, raise)) {
          // every PV issued so far must have landed: the last one is the previous half
          const int ph = h ^ 1;
          const int pj = h ? j : j - 1;
          if (!mbar_wait(&o_done[t * 2 + ph], (uint32_t)(pj & 1), abort_flag, a.status, st_code)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const float f = raise ? ex2(m_used - m_tile) : 1.0f;  // m_used == -inf -> 0 (accumulator is 0 there)
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(o_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st32(o_addr + c * 32, o);
          }
          l_run *= f;
        }
        if (raise) m_used = m_tile;
        const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
        // probabilities of this half: 2 chunks of 32 -> 16 packed 32-bit columns each
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const bool poly = kPolyEvery > 0 && (i % (kPolyEvery > 0 ? kPolyEvery : 1)) == kPolyEvery - 1;
            const float x0 = fmaf(sv[c * 32 + 2 * i], scale, neg_m);
            const float x1 = fmaf(sv[c * 32 + 2 * i + 1], scale, neg_m);
            const float p0 = poly ? ex2_poly(x0) : ex2(x0);
            const float p1 = poly ? ex2_poly(x1) : ex2(x1);
            sum4[i & 3] += p0 + p1;
            pk[i] = bf16 ? pack_bf16(p0, p1) : pack_f16(p0, p1);
          }
          tmem_st16(sh_addr + c * 16, pk);
        }
        l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        tmem_st_wait();
        tc_fence_before();
        if (h == 0 && a.paged && t == 0 && j == n_tiles - 1 && j * BN + BN > s.k_len) {
          // Rows of the last V tile past the end of the sequence hold whatever the cache
          // page holds; zero them so 0 * garbage can never produce NaN.
          const int stg = j & 1;
          if (mbar_wait(&v_full[stg], (uint32_t)((j >> 1) & 1), abort_flag, a.status, st_code)) {
            const int first = s.k_len - j * BN;  // first invalid row of the tile
            uint8_t* vt = sV + stg * TILE_BYTES;
            for (int idx = r; idx < (BN - first) * 16; idx += 128) {
              const int row = first + idx / 16, ch = idx % 16;
              *reinterpret_cast<uint4*>(vt + (ch >> 3) * HALF_BYTES + row * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
          } else {
            ok = false;
          }
        }
        if (quarter == 0) FG_TRACE(5 + t * 16 + h, j);
        mbar_arrive(&p_ready[t * 2 + h]);
        if (!ok) break;
      }
    }

    if (ok && mbar_wait(&o_done[t * 2 + 1], (uint32_t)((n_tiles - 1) & 1), abort_flag, a.status, st_code)) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      const bool valid = qpos < s.q_len;
      char* orow = reinterpret_cast<char*>(a.out) +
                   ((int64_t)(s.q_begin + qpos) * a.o_rs + (int64_t)(h0 + t) * a.o_hs) * 2;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32(o_addr + c * 32, o);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float x0 = __uint_as_float(o[q4 * 8 + 2 * i]) * inv;
              const float x1 = __uint_as_float(o[q4 * 8 + 2 * i + 1]) * inv;
              wp[i] = bf16 ? pack_bf16(x0, x1) : pack_f16(x0, x1);
            }
            *reinterpret_cast<uint4*>(orow + c * 64 + q4 * 16) = w;
          }
        }
      }
      if (valid && a.lse)
        a.lse[(int64_t)(h0 + t) * a.total_q + s.q_begin + qpos] =
            l_run > 0.f ? m_used * 0.6931471805599453f + logf(l_run) : INFINITY;
    }
  }

  // ================================ teardown ======================================
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

static bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }

}  // namespace

bool attn_prefill_sm100_eligible(const fg_attn_params* p) {
  if (p->dtype != FG_BF16 && p->dtype != FG_F16) return false;
  if (p->head_dim != 128) return false;
  if (p->alibi_slopes != nullptr || p->softcap > 0.0 || !(p->softmax_scale > 0.0)) return false;
  if (p->max_seqlen_q < 64) return false;  // short query blocks: the general kernel wastes less
  const bool left = p->window_left >= 0 && p->window_left < p->max_seqlen_k;
  const bool right = !p->causal && p->window_right >= 0 && p->window_right < p->max_seqlen_k;
  if (left || right) return false;
  if (p->block_table != nullptr) {
    if (!is_pow2(p->block_size) || p->block_size < 8) return false;
    if (p->block_size > 128 && p->block_size % 128 != 0) return false;
  }
  if (p->batch > 65535 || p->num_heads > 65535) return false;
  return true;
}

int attn_prefill_sm100(const AttnArgs& a, int dtype, cudaStream_t st) {
  PrefillArgs pa;
  pa.a = a;
  pa.tiles = (a.group % 2 == 0) ? 2 : 1;
  pa.is_bf16 = dtype == FG_BF16;
  pa.page_rows = a.paged ? (a.block_size < 128 ? a.block_size : 128) : 128;
  pa.pages_per_tile = 128 / pa.page_rows;
  if (!pa.a.status) return fail(FG_ERR_CUDA, "flash_attn_varlen: device status word unavailable");

  CUtensorMap tq, tk, tv;
  {
    uint64_t dims[3] = {(uint64_t)HD, (uint64_t)a.H, (uint64_t)a.total_q};
    uint64_t strides[2] = {(uint64_t)a.q_hs * 2, (uint64_t)a.q_rs * 2};
    uint32_t box[3] = {64, 1, 128};
    int rc = encode_tmap_16bit(&tq, a.q, 3, dims, strides, box);
    if (rc != FG_OK) return rc;
  }
  if (a.paged) {
    uint64_t dims[4] = {(uint64_t)HD, (uint64_t)a.Hk, (uint64_t)a.block_size, (uint64_t)a.num_blocks};
    uint32_t box[4] = {64, 1, (uint32_t)pa.page_rows, 1};
    uint64_t ks[3] = {(uint64_t)a.k_hs * 2, (uint64_t)a.k_rs * 2, (uint64_t)a.k_bs * 2};
    uint64_t vs[3] = {(uint64_t)a.v_hs * 2, (uint64_t)a.v_rs * 2, (uint64_t)a.v_bs * 2};
    int rc = encode_tmap_16bit(&tk, a.k, 4, dims, ks, box);
    if (rc != FG_OK) return rc;
    rc = encode_tmap_16bit(&tv, a.v, 4, dims, vs, box);
    if (rc != FG_OK) return rc;
  } else {
    uint64_t dims[3] = {(uint64_t)HD, (uint64_t)a.Hk, (uint64_t)(a.total_k > 0 ? a.total_k : 1)};
    uint32_t box[3] = {64, 1, 128};
    uint64_t ks[2] = {(uint64_t)a.k_hs * 2, (uint64_t)a.k_rs * 2};
    uint64_t vs[2] = {(uint64_t)a.v_hs * 2, (uint64_t)a.v_rs * 2};
    int rc = encode_tmap_16bit(&tk, a.k, 3, dims, ks, box);
    if (rc != FG_OK) return rc;
    rc = encode_tmap_16bit(&tv, a.v, 3, dims, vs, box);
    if (rc != FG_OK) return rc;
  }
  static thread_local int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    FG_CUDA_OK(cudaFuncSetAttribute(attn_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_BYTES));
    attr_dev = dev;
  }
  dim3 grid((a.max_q + BM - 1) / BM, a.H / pa.tiles, a.batch);
  attn_prefill_tcgen05_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(tq, tk, tv, pa);
  FG_CHECK_LAUNCH("attn_prefill_tcgen05_kernel");
  return FG_OK;
}

}  // namespace fg
