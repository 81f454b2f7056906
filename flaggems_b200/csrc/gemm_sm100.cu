// Dense GEMM for the mm/addmm projections on sm_100a:
//   C[M,N] = alpha * A[M,K] @ B[K,N] (+ beta * bias), 16-bit inputs, fp32 accumulate.
//
// Persistent kernel, one CTA per SM, BK = 64, two tile shapes (template parameter MT):
//   MT = 1: 128x256 output tile, 4-stage ring of 48 KB stages, two 256-column fp32
//           accumulators in TMEM so that tile i+1's main loop overlaps the epilogue of tile i;
//   MT = 2: 256x256 output tile as two M128 MMAs per K step that share the B operand,
//           3-stage ring of 64 KB stages, the two accumulators fill TMEM (no overlap of the
//           epilogue).  A third less operand traffic from L2 per flop and a deeper ring in
//           clocks; taken for K-major A when the wave count does not eat the gain.
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of A and B into the
//               128-byte-swizzled shared-memory ring
//   warp 1      allocates TMEM and issues tcgen05.mma (M128 N256 K16) from one thread
//   warps 2-9   epilogue (two warps per TMEM lane quarter, 128 columns each): tcgen05.ld the
//               accumulator, alpha/beta/bias in fp32, round once, transpose 32 rows x 64 columns
//               through a per-warp shared-memory tile and store whole 128-byte row segments
// Both operands may be row- or column-major; the UMMA descriptors carry the
// majorness, the TMA boxes differ (one [64 x rows] box for a K-major operand, one
// [64 x 64] box per 64 rows for an MN-major operand).  M, N and K tails are handled
// by TMA zero fill on loads and predication on stores.
#include <cstdlib>

#include "common.cuh"
#include "sm100_common.cuh"

namespace fg {

int* device_status_ptr();

namespace {

constexpr int BM = 128, BN = 256, BK = 64;   // BM: rows of one MMA; a tile has MT * BM rows
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int MAX_STAGES = 4;
template <int MT>
struct Cfg {
  static constexpr int TILE_M = MT * BM;
  static constexpr int STAGES = MT == 1 ? 4 : 3;
  static constexpr int A_STAGE_BYTES = TILE_M * BK * 2;  // 16 / 32 KB
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
};
constexpr int EPI_STAGE_BYTES = 32 * 128;   // per epilogue warp: 32 rows x 64 output columns of 16 bits
constexpr int SMEM_BYTES = 4 * (BM * BK * 2 + B_STAGE_BYTES) + 1024 /*align*/ + 256 /*barriers*/ + 8 * EPI_STAGE_BYTES;  // ring 192 KB + 32 KB
constexpr int NUM_THREADS = 320;   // TMA warp, MMA warp, 8 epilogue warps
constexpr int TMEM_COLS = 512;

struct GemmArgs {
  void* c;
  const void* bias;
  int64_t M, N, K;
  int64_t c_s0;                // C row stride (unit column stride)
  int64_t bias_s0, bias_s1;
  float alpha, beta;
  int has_bias;
  int a_mn_major, b_mn_major;  // 0: K contiguous, 1: M / N contiguous
  int is_bf16;
  int group_m;
  int c_vec_ok;                // 16-byte stores legal for C
  int bias_vec;                // bias is one contiguous, 16-byte aligned row shared by all rows
  int64_t batch;               // independent problems sharing the shape (bmm); the tensor maps carry
  int64_t c_bs, bias_bs;       // the batch as their third dimension, C and bias by these strides
  int64_t full_units;          // work units [0, full_units) are whole tiles, the rest 128-row halves of the
  int64_t num_units;           // remaining tiles (MT = 2 only: balances the last, partly filled wave)
  int* status;
};

// Work unit -> (tile, first 128-row block of the tile, number of 128-row blocks).
template <int MT>
__device__ __forceinline__ void unit_decode(const GemmArgs& g, int64_t u, int64_t& tile, int& h0, int& nh) {
  if (MT == 1 || u < g.full_units) {
    tile = u;
    h0 = 0;
    nh = MT;
  } else {
    const int64_t r = u - g.full_units;
    tile = g.full_units + (r >> 1);
    h0 = (int)(r & 1);
    nh = 1;
  }
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int group_m,
                                            int64_t& tm, int64_t& tn) {
  // Grouped ordering: `group_m` row tiles share each sweep over the column tiles so
  // the A panels of a group and the B panels in flight stay L2 resident.
  const int64_t per_group = (int64_t)group_m * tiles_n;
  const int64_t g = tile / per_group;
  const int64_t first_m = g * group_m;
  const int64_t rows = (tiles_m - first_m) < group_m ? (tiles_m - first_m) : group_m;
  const int64_t r = tile - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

template <typename T, int MT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_a_half,
                    const __grid_constant__ CUtensorMap tmap_b, GemmArgs g) {
  using namespace sm100;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int STAGES = Cfg<MT>::STAGES, STAGE_BYTES = Cfg<MT>::STAGE_BYTES;
  constexpr int A_STAGE_BYTES = Cfg<MT>::A_STAGE_BYTES, TILE_M = Cfg<MT>::TILE_M;
  uint8_t* bars_base = smem + 4 * (BM * BK * 2 + B_STAGE_BYTES);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bars_base);
  uint64_t* empty_bar = full_bar + MAX_STAGES;
  uint64_t* acc_full = empty_bar + MAX_STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // a timed-out wait earlier on this device: drain the launch instead of repeating it
  // (one thread reads the word so that the whole CTA takes the same decision)
  __shared__ int s_drain;
  if (threadIdx.x == 0) s_drain = *reinterpret_cast<volatile int*>(g.status);
  __syncthreads();
  if (s_drain != 0) return;

  const int64_t tiles_m = (g.M + TILE_M - 1) / TILE_M;
  const int64_t tiles_n = (g.N + BN - 1) / BN;
  const int64_t tiles_per_batch = tiles_m * tiles_n;
  const int64_t num_units = g.num_units;
  const int num_kb = (int)((g.K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 256);   // every epilogue thread arrives
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    if (MT == 2) prefetch_tmap(&tmap_a_half);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        int64_t tile, tm, tn;
        int h0, nh;
        unit_decode<MT>(g, u, tile, h0, nh);
        const int bi = (int)(tile / tiles_per_batch);
        tile_coords(tile - bi * tiles_per_batch, tiles_m, tiles_n, g.group_m, tm, tn);
        const int m0 = (int)(tm * TILE_M) + h0 * BM, n0 = (int)(tn * BN);
        const bool whole = nh == MT;
        const uint32_t tx_bytes = (uint32_t)(whole ? STAGE_BYTES : BM * BK * 2 + B_STAGE_BYTES);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, g.status, kStatusGemmTimeout)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], tx_bytes);
          const int k0 = kb * BK;
          if (!g.a_mn_major) {
            tma_load_3d(sa, whole ? &tmap_a : &tmap_a_half, &full_bar[stage], k0, m0, bi);
          } else {
#pragma unroll
            for (int b = 0; b < TILE_M / 64; ++b)
              tma_load_3d(sa + b * (64 * BK * 2), &tmap_a, &full_bar[stage], m0 + 64 * b, k0, bi);
          }
          if (!g.b_mn_major) {
            tma_load_3d(sb, &tmap_b, &full_bar[stage], k0, n0, bi);
          } else {
#pragma unroll
            for (int b = 0; b < BN / 64; ++b)
              tma_load_3d(sb + b * (64 * BK * 2), &tmap_b, &full_bar[stage], n0 + 64 * b, k0, bi);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(g.is_bf16 != 0, g.a_mn_major != 0, g.b_mn_major != 0, BM, BN);
      // Per-operand descriptor geometry.
      const uint32_t a_lbo = g.a_mn_major ? 64 * BK * 2 : 0, b_lbo = g.b_mn_major ? 64 * BK * 2 : 0;
      const uint32_t a_kstep = g.a_mn_major ? 16 * 128 : 32;  // bytes per K=16 step
      const uint32_t b_kstep = g.b_mn_major ? 16 * 128 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int64_t local = 0;
      bool ok = true;
      for (int64_t u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++local) {
        const int nh = (MT == 1 || u < g.full_units) ? MT : 1;
        // MT = 1: two accumulators, used alternately.  MT = 2: both halves of TMEM hold this tile.
        const int buf = MT == 1 ? (int)(local & 1) : 0;
        const uint32_t acc_phase = MT == 1 ? (uint32_t)((local >> 1) & 1) : (uint32_t)(local & 1);
        if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag, g.status, kStatusGemmTimeout)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, g.status, kStatusGemmTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t bdesc = umma_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              if (mt >= nh) break;
              // rows mt*128.. of the A stage: 128 rows x 128 B further on (K-major A only for MT = 2)
              const uint64_t adesc = umma_desc_sw128(sa + mt * (BM * BK * 2) + k * a_kstep, a_lbo, 1024);
              mma_f16_ss(d_tmem + (uint32_t)(mt * BN), adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          tc_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const int chalf = (warp - 2) >> 2;     // two warps share a quarter: columns [0,128) and [128,256) of the tile
    int64_t local = 0;
    for (int64_t u = blockIdx.x; u < num_units; u += gridDim.x, ++local) {
      const int buf = MT == 1 ? (int)(local & 1) : 0;
      const uint32_t acc_phase = MT == 1 ? (uint32_t)((local >> 1) & 1) : (uint32_t)(local & 1);
      int64_t tile, tm, tn;
      int h0, nh;
      unit_decode<MT>(g, u, tile, h0, nh);
      const int64_t bi = tile / tiles_per_batch;
      tile_coords(tile - bi * tiles_per_batch, tiles_m, tiles_n, g.group_m, tm, tn);
      if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag, g.status, kStatusGemmTimeout)) break;
      tc_fence_after();
      const int64_t col0 = tn * BN;
      const T* bias = reinterpret_cast<const T*>(g.bias) + bi * g.bias_bs;
      // alpha * acc (+ beta * bias) of one 32-column chunk of this lane's row
      auto scale_chunk = [&](const uint32_t (&r)[32], int64_t row, int64_t col, float (&v)[32]) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (g.has_bias) {
          if (g.bias_vec && col + 32 <= g.N) {
            // the usual addmm bias, a row vector: four 16-byte loads (the same addresses in
            // every lane) instead of 32 strided scalar ones
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float bv[8];
              Vec16<T>::unpack(ldg16(bias + col + q * 8), bv);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[q * 8 + j] = fmaf(v[q * 8 + j], g.alpha, bv[j] * g.beta);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int64_t cj = col + j;
              const float bv = (cj < g.N && row < g.M) ? Cvt<T>::to_f32(bias[row * g.bias_s0 + cj * g.bias_s1]) : 0.f;
              v[j] = v[j] * g.alpha + bv * g.beta;
            }
          }
        }
      };
      // Whole 64-column groups inside N with 16-byte stores allowed go through a per-warp staging
      // tile in shared memory: a lane converts its own row (TMEM lane = row), the warp then writes
      // four rows x 128 contiguous bytes per store instruction instead of 32 rows x 16 bytes.
      const bool staged = g.c_vec_ok && col0 + BN <= g.N;
      uint8_t* stage = bars_base + 256 + (warp - 2) * EPI_STAGE_BYTES;
#pragma unroll 1
      for (int mt = 0; mt < nh; ++mt) {
        const int64_t row0 = tm * TILE_M + (h0 + mt) * BM + quarter * 32;
        const int64_t row = row0 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((buf + mt) * BN);
        T* cbase = reinterpret_cast<T*>(g.c) + bi * g.c_bs;
        if (staged) {
#pragma unroll 1
          for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); c += 2) {
            const int64_t col = col0 + c * 32;
#pragma unroll
            for (int hc = 0; hc < 2; ++hc) {
              uint32_t r[32];
              tmem_ld32(taddr + (c + hc) * 32, r);
              tmem_ld_wait();
              float v[32];
              scale_chunk(r, row, col + hc * 32, v);
              // 16-byte packet j of the row goes to slot j ^ (row & 7): conflict-free both ways
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack2<T>(v[q * 8 + 0], v[q * 8 + 1]);
                o.y = pack2<T>(v[q * 8 + 2], v[q * 8 + 3]);
                o.z = pack2<T>(v[q * 8 + 4], v[q * 8 + 5]);
                o.w = pack2<T>(v[q * 8 + 6], v[q * 8 + 7]);
                *reinterpret_cast<uint4*>(stage + lane * 128 + (((hc * 4 + q) ^ (lane & 7)) << 4)) = o;
              }
            }
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + (lane >> 3), j = lane & 7;
              const uint4 o = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((j ^ (rr & 7)) << 4));
              if (row0 + rr < g.M) *reinterpret_cast<uint4*>(cbase + (row0 + rr) * g.c_s0 + col + j * 8) = o;
            }
            __syncwarp();
          }
        } else {
          T* crow = cbase + row * g.c_s0;
#pragma unroll 1
          for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); ++c) {
            uint32_t r[32];
            tmem_ld32(taddr + c * 32, r);
            tmem_ld_wait();
            const int64_t col = col0 + c * 32;
            if (row < g.M && col < g.N) {
              float v[32];
              scale_chunk(r, row, col, v);
              if (g.c_vec_ok && col + 32 <= g.N) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 o;
                  o.x = pack2<T>(v[q * 8 + 0], v[q * 8 + 1]);
                  o.y = pack2<T>(v[q * 8 + 2], v[q * 8 + 3]);
                  o.z = pack2<T>(v[q * 8 + 4], v[q * 8 + 5]);
                  o.w = pack2<T>(v[q * 8 + 6], v[q * 8 + 7]);
                  *reinterpret_cast<uint4*>(crow + col + q * 8) = o;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col + j < g.N) crow[col + j] = Cvt<T>::from_f32(v[j]);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);
    }
  }

  // ------------------------------ teardown -------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // Give copies and MMAs still in flight a bounded time to land before the
      // accumulator columns are handed back.
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

// Cost of a 256x256 tile relative to two 128x256 tiles (tile-shape choice below).
constexpr double kBigTileCost = 0.85;
// Cost of a 128-row half of a 256x256 tile in tile times.
constexpr double kHalfTileCost = 0.56;
// 0: choose; 1 / 2: force the tile shape (set from the environment variable FLAGGEMS_B200_GEMM_MT,
// for measurements).
static const int g_force_mt = []() {
  const char* e = getenv("FLAGGEMS_B200_GEMM_MT");
  return e ? atoi(e) : 0;
}();

// FLAGGEMS_B200_GEMM_GROUP_MB: megabytes of A rows one group of row tiles may take (default 32; for
// measurements).
static const int g_group_mb = []() {
  const char* e = getenv("FLAGGEMS_B200_GEMM_GROUP_MB");
  const int v = e ? atoi(e) : 0;
  return v > 0 ? v : 32;
}();

// FLAGGEMS_B200_GEMM_SPLIT_TAIL=0 keeps the last wave of 256x256 tiles whole (for measurements).
static const bool g_split_tail = []() {
  const char* e = getenv("FLAGGEMS_B200_GEMM_SPLIT_TAIL");
  return !(e && atoi(e) == 0);
}();

static bool tcgen05_eligible(const fg_gemm_params* p) {
  if (p->dtype != FG_BF16 && p->dtype != FG_F16) return false;
  if (p->M < 1 || p->N < 1 || p->K < 1) return false;
  if (p->M > 2147483647LL || p->N > 2147483647LL || p->K > 2147483647LL) return false;
  // Tiny problems are launch-bound; the generic kernel handles them without a
  // tensor map.  (Also keeps odd test shapes off the TMA alignment rules.)
  if (p->M * p->N < 64 * 64 || p->K < 32) return false;
  auto operand_ok = [](const void* ptr, int64_t s0, int64_t s1, int64_t rows, int64_t cols) {
    // either unit stride along dim1 (row-major) or along dim0 (column-major); the
    // other stride a multiple of 8 elements (16 B); base 16-byte aligned
    if (!aligned16(ptr)) return false;
    if (s1 == 1 && (s0 % 8 == 0) && s0 >= cols) return true;
    if (s0 == 1 && (s1 % 8 == 0) && s1 >= rows) return true;
    return false;
  };
  if (!operand_ok(p->a, p->a_stride0, p->a_stride1, p->M, p->K)) return false;
  if (!operand_ok(p->b, p->b_stride0, p->b_stride1, p->K, p->N)) return false;
  if (p->c_stride1 != 1) return false;
  return true;
}

// Tile shape and work units of a launch: pure host arithmetic, also served by fg_gemm_tile_plan.
struct TilePlan {
  int mt;              // 1: 128x256 tiles, 2: 256x256 tiles
  int sms, grid, group_m;
  int64_t tiles_m, tiles_n, tiles;   // row tiles (of mt * 128 rows), column tiles, tiles over the batch
  int64_t full_units, num_units;     // units [0, full_units) are whole tiles, the rest 128-row halves
};

static TilePlan plan_tiles(const fg_gemm_params* p, int64_t batch, int sms, bool a_mn) {
  // Tile shape: 256x256 needs a third less operand traffic per flop but has half as many,
  // twice as long tiles; it is taken when its last, partly filled wave costs less than that
  // gains, for K-major A only.  Measured at M = 8192 (bf16, B200): 1461 against 1392 TFLOP/s
  // for N = 28672, K = 4096 with bias, 1504 against 1356 for N = 4096, K = 14336, a tie for
  // N = 6144 where the big tile's sixth wave is a fifth full.
  TilePlan t;
  t.sms = sms;
  const int64_t tn = (p->N + BN - 1) / BN;
  const int64_t tiles1 = ((p->M + BM - 1) / BM) * tn * batch;
  const int64_t tiles2 = ((p->M + 2 * BM - 1) / (2 * BM)) * tn * batch;
  const int64_t waves1 = (tiles1 + sms - 1) / sms;
  // A last wave of 256x256 tiles that fills at most half of the SMs is cut into 128-row halves,
  // one per CTA: it then takes about 0.56 of a tile time (one MMA per K step, B no longer shared).
  const int64_t rest2 = tiles2 % sms;
  const bool split_tail = g_split_tail && tiles2 > sms && rest2 > 0 && 2 * rest2 <= sms;
  const double waves2 = (double)(tiles2 / sms) + (rest2 == 0 ? 0.0 : split_tail ? kHalfTileCost : 1.0);
  t.mt = (!a_mn && p->M > BM && waves2 * 2.0 * kBigTileCost < (double)waves1) ? 2 : 1;
  if (g_force_mt == 1 || (g_force_mt == 2 && !a_mn)) t.mt = g_force_mt;
  const int tile_m = t.mt * BM;
  t.tiles_m = (p->M + tile_m - 1) / tile_m;
  t.tiles_n = tn;
  t.tiles = t.mt == 2 ? tiles2 : tiles1;
  t.grid = t.tiles < sms ? (int)t.tiles : sms;
  t.full_units = (t.mt == 2 && split_tail) ? t.tiles - rest2 : t.tiles;
  t.num_units = t.full_units + 2 * (t.tiles - t.full_units);
  // Row tiles per sweep over the column tiles: as many as keep the A panel of a group
  // (group_m x tile rows x K) around 32 MB, so that it stays L2-resident while B streams
  // through once per group instead of once per few row tiles.
  const int64_t panel = (int64_t)tile_m * p->K * 2;
  int64_t gm = ((int64_t)g_group_mb << 20) / (panel > 0 ? panel : 1);
  if (gm < 4) gm = 4;
  if (gm > 64) gm = 64;
  t.group_m = (int)gm;
  return t;
}

static bool a_is_mn_major(const fg_gemm_params* p) {
  // A: K-major if a_stride1 == 1 (row-major), else M-major.  Degenerate shapes with
  // both strides 1 are treated as row-major.
  return !(p->a_stride1 == 1 && p->a_stride0 % 8 == 0 && p->a_stride0 >= p->K);
}

template <typename T, int MT>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& ta_half, const CUtensorMap& tb, const GemmArgs& g,
                       int grid, cudaStream_t st) {
  static thread_local int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    FG_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<T, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_BYTES));
    attr_dev = dev;
  }
  gemm_tcgen05_kernel<T, MT><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, ta_half, tb, g);
  FG_CHECK_LAUNCH("gemm_tcgen05_kernel");
  return FG_OK;
}

int gemm_tcgen05(const fg_gemm_params* p, const GemmBatch& bt, cudaStream_t st) {
  using namespace fg;
  const bool a_mn = a_is_mn_major(p);
  // B [K,N]: K-major if b_stride0 == 1 (column-major storage), else N-major.
  const bool b_mn = !(p->b_stride0 == 1 && p->b_stride1 % 8 == 0 && p->b_stride1 >= p->K);

  const TilePlan plan = plan_tiles(p, bt.batch, sm_budget(), a_mn);
  const int sms = plan.sms, mt = plan.mt, tile_m = mt * BM;

  CUtensorMap ta, ta_half, tb;
  {
    // third dimension: the batch (extent 1 and a dummy stride for a plain GEMM)
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    dims[2] = (uint64_t)bt.batch;
    box[2] = 1;
    if (!a_mn) {
      dims[0] = (uint64_t)p->K; dims[1] = (uint64_t)p->M; strides[0] = (uint64_t)p->a_stride0 * 2;
      box[0] = 64; box[1] = (uint32_t)tile_m;
    } else {
      dims[0] = (uint64_t)p->M; dims[1] = (uint64_t)p->K; strides[0] = (uint64_t)p->a_stride1 * 2;
      box[0] = 64; box[1] = BK;
    }
    strides[1] = bt.batch > 1 ? (uint64_t)bt.a_bs * 2 : strides[0] * dims[1];
    int rc = encode_tmap_16bit(&ta, p->a, 3, dims, strides, box);
    if (rc != FG_OK) return rc;
    ta_half = ta;
    if (mt == 2) {  // the same matrix in boxes of 128 rows, for the halved tiles of the last wave
      box[1] = BM;
      rc = encode_tmap_16bit(&ta_half, p->a, 3, dims, strides, box);
      if (rc != FG_OK) return rc;
    }
    if (!b_mn) {
      dims[0] = (uint64_t)p->K; dims[1] = (uint64_t)p->N; strides[0] = (uint64_t)p->b_stride1 * 2;
      box[0] = 64; box[1] = BN;
    } else {
      dims[0] = (uint64_t)p->N; dims[1] = (uint64_t)p->K; strides[0] = (uint64_t)p->b_stride0 * 2;
      box[0] = 64; box[1] = BK;
    }
    strides[1] = bt.batch > 1 ? (uint64_t)bt.b_bs * 2 : strides[0] * dims[1];
    rc = encode_tmap_16bit(&tb, p->b, 3, dims, strides, box);
    if (rc != FG_OK) return rc;
  }
  GemmArgs g;
  g.c = p->c; g.bias = p->bias;
  g.M = p->M; g.N = p->N; g.K = p->K;
  g.c_s0 = p->c_stride0;
  g.bias_s0 = p->bias_stride0; g.bias_s1 = p->bias_stride1;
  g.alpha = (float)p->alpha; g.beta = (float)p->beta;
  g.has_bias = p->bias != nullptr;
  g.a_mn_major = a_mn; g.b_mn_major = b_mn;
  g.is_bf16 = p->dtype == FG_BF16;
  g.group_m = plan.group_m;
  g.c_vec_ok = aligned16(p->c) && (p->c_stride0 % 8 == 0) && (bt.batch == 1 || bt.c_bs % 8 == 0);
  g.bias_vec = p->bias != nullptr && p->bias_stride0 == 0 && p->bias_stride1 == 1 && aligned16(p->bias) &&
               (bt.batch == 1 || bt.bias_bs % 8 == 0);
  g.batch = bt.batch; g.c_bs = bt.c_bs; g.bias_bs = bt.bias_bs;
  g.status = device_status_ptr();
  if (!g.status) return fail(FG_ERR_CUDA, "gemm: device status word unavailable");

  const int grid = plan.grid;   // persistent: one CTA per SM it may use
  g.full_units = plan.full_units;
  g.num_units = plan.num_units;
  (void)sms;
  if (p->dtype == FG_BF16)
    return mt == 2 ? launch_gemm<__nv_bfloat16, 2>(ta, ta_half, tb, g, grid, st)
                   : launch_gemm<__nv_bfloat16, 1>(ta, ta_half, tb, g, grid, st);
  return mt == 2 ? launch_gemm<__half, 2>(ta, ta_half, tb, g, grid, st) : launch_gemm<__half, 1>(ta, ta_half, tb, g, grid, st);
}

bool gemm_tcgen05_eligible(const fg_gemm_params* p) { return tcgen05_eligible(p); }

int gemm_tile_plan(const fg_gemm_params* p, int64_t batch, int num_sms, fg_gemm_plan* out) {
  if (!p || !out) return fail(FG_ERR_INVALID, "gemm_tile_plan: null pointer");
  if (batch < 1 || num_sms < 1) return fail(FG_ERR_INVALID, "gemm_tile_plan: batch and num_sms must be positive");
  if (!tcgen05_eligible(p)) return fail(FG_ERR_UNSUPPORTED, "gemm_tile_plan: the generic kernel takes this problem");
  const TilePlan t = plan_tiles(p, batch, num_sms, a_is_mn_major(p));
  out->tile_m = t.mt * BM;
  out->tile_n = BN;
  out->grid = t.grid;
  out->group_m = t.group_m;
  out->tiles_m = t.tiles_m;
  out->tiles_n = t.tiles_n;
  out->full_units = t.full_units;
  out->num_units = t.num_units;
  return FG_OK;
}

}  // namespace fg
