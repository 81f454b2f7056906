// fp32 GEMM on the tcgen05 tensor cores without TF32: C[M,N] = alpha * A @ B (+ beta * bias) for
// fp32 A, B, bias and C, with an error at the level of fp32 arithmetic on CUDA cores.
//
// Each operand is first written as three bf16 pieces, x = hi + mid + lo exactly (8 + 8 + 8
// mantissa bits; values below about 2^-100, whose third piece is a bf16 denormal, lose less than
// 2^-133), by `split3_kernel`.  The product is then the sum of six piece products in
// ascending order of magnitude,
//     mid*mid, hi*lo, lo*hi      (2^-16 of the result)
//     hi*mid, mid*hi             (2^-8)
//     hi*hi
// (the three dropped products are below 2^-24 of a term).  Every piece product is exact in the
// tensor core's fp32 accumulator; what is not exact is the accumulation itself, which truncates:
// a single accumulator over K = 4096 shows a relative bias of 1e-5 on same-signed data.  The
// kernel therefore closes the accumulator every few K blocks (`hi_chunk` x 64 for the hi*hi
// products, `low_chunk` x 64 for the small ones) and the epilogue warps add the chunks in fp32
// registers with round-to-nearest.  Measured against fp64 at 4096^3 with hi*hi chunks of 256: mean
// relative error 2.4e-7 on normal data and 3.1e-7 on same-signed data, where an fp32 FMA loop
// gives 1.0e-6 and 6.7e-7 (chunks of 512: 4.7e-7 and 7.1e-7, at the same speed); 183 TFLOP/s of
// fp32 work against 40 for the CUDA-core kernel and 63 for cuBLAS without TF32.
//
// One 128 x 256 output tile per work unit, persistent CTAs, BK = 64, four 48 KB stages:
//   warp 0      TMA producer: walks the six piece pairs, K block by K block, with the piece
//               index as the third tensor-map coordinate
//   warp 1      allocates TMEM (two 256-column accumulators, used alternately chunk by chunk)
//               and issues tcgen05.mma from one thread; the first MMA of a chunk overwrites
//   warps 2-9   tcgen05.ld each finished chunk and add it to 128 running sums per thread
//               (TMEM lane = row), hand the accumulator back, and after a tile's last chunk
//               apply alpha/beta/bias and store the row segment
// Operands keep their row- or column-major order through the split (the UMMA descriptors carry
// the majorness, as in the 16-bit kernel).  A non-finite input would turn into NaN here where
// fp32 arithmetic gives an infinity (inf * 0-piece), so the split pass raises a device flag for
// any such element; the kernel returns at once when the flag is up and the CUDA-core kernel,
// launched behind it and gated on the same flag, computes the result instead.  No host
// synchronisation is involved.
#include <cstdlib>

#include "common.cuh"
#include "sm100_common.cuh"

namespace fg {

int* device_status_ptr();
int gemm_simt_gated(const fg_gemm_params* p, const int* only_if_nonzero, cudaStream_t st);

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int NUM_THREADS = 320;   // TMA warp, MMA warp, 8 epilogue warps
constexpr int TMEM_COLS = 512;
constexpr int kPairs = 6;
// piece (0 = hi, 1 = mid, 2 = lo) of A and of B for pair p, two bits per pair, ascending magnitude
constexpr uint32_t kPieceA = 1u | (0u << 2) | (2u << 4) | (0u << 6) | (1u << 8) | (0u << 10);
constexpr uint32_t kPieceB = 1u | (2u << 2) | (0u << 4) | (1u << 6) | (0u << 8) | (0u << 10);

struct SplitArgs {
  float* c;
  const float* bias;
  int64_t M, N, K;
  int64_t c_s0;
  int64_t bias_s0, bias_s1;
  float alpha, beta;
  int has_bias;
  int a_mn_major, b_mn_major;   // 0: K contiguous, 1: M / N contiguous
  int group_m;
  int kb_per_pair;              // K blocks of 64 per piece pair
  int low_chunk, hi_chunk;      // K blocks per accumulator chunk: the five small pairs / hi*hi
  int c_vec_ok;                 // 16-byte stores legal for C
  int64_t num_tiles;
  const int* nonfinite;         // raised by the split pass: leave the work to the CUDA-core kernel
  int* status;
};

// End of the accumulator chunk that starts at K block `kb` (blocks [0, low_kb) are the small
// pairs, [low_kb, total_kb) the hi*hi pair).
__device__ __forceinline__ int chunk_end(int kb, int low_kb, int total_kb, int low_chunk, int hi_chunk) {
  if (kb < low_kb) {
    const int e = kb + low_chunk;
    return e < low_kb ? e : low_kb;
  }
  const int e = kb + hi_chunk;
  return e < total_kb ? e : total_kb;
}

__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int group_m,
                                            int64_t& tm, int64_t& tn) {
  // `group_m` row tiles share each sweep over the column tiles (L2 reuse of the A panels)
  const int64_t per_group = (int64_t)group_m * tiles_n;
  const int64_t g = tile / per_group;
  const int64_t first_m = g * group_m;
  const int64_t rows = (tiles_m - first_m) < group_m ? (tiles_m - first_m) : group_m;
  const int64_t r = tile - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_f32_split_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                              SplitArgs g) {
  using namespace sm100;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bars_base = smem + STAGES * STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bars_base);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // A timed-out wait earlier on this device, or a non-finite input: nothing to do here.
  __shared__ int s_skip;
  if (threadIdx.x == 0)
    s_skip = *reinterpret_cast<volatile int*>(g.status) | *reinterpret_cast<const volatile int*>(g.nonfinite);
  __syncthreads();
  if (s_skip != 0) return;

  const int64_t tiles_m = (g.M + BM - 1) / BM;
  const int64_t tiles_n = (g.N + BN - 1) / BN;
  const int kbpp = g.kb_per_pair;
  const int low_kb = (kPairs - 1) * kbpp, total_kb = kPairs * kbpp;

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
      for (int64_t u = blockIdx.x; u < g.num_tiles && ok; u += gridDim.x) {
        int64_t tm, tn;
        tile_coords(u, tiles_m, tiles_n, g.group_m, tm, tn);
        const int m0 = (int)(tm * BM), n0 = (int)(tn * BN);
        for (int pair = 0; pair < kPairs && ok; ++pair) {
          const int pa = (int)((kPieceA >> (2 * pair)) & 3u), pb = (int)((kPieceB >> (2 * pair)) & 3u);
          for (int kk = 0; kk < kbpp; ++kk) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, g.status, kStatusGemmTimeout)) {
              ok = false;
              break;
            }
            uint8_t* sa = smem + stage * STAGE_BYTES;
            uint8_t* sb = sa + A_STAGE_BYTES;
            mbar_expect_tx(&full_bar[stage], (uint32_t)STAGE_BYTES);
            const int k0 = kk * BK;
            if (!g.a_mn_major) {
              tma_load_3d(sa, &tmap_a, &full_bar[stage], k0, m0, pa);
            } else {
#pragma unroll
              for (int b = 0; b < BM / 64; ++b)
                tma_load_3d(sa + b * (64 * BK * 2), &tmap_a, &full_bar[stage], m0 + 64 * b, k0, pa);
            }
            if (!g.b_mn_major) {
              tma_load_3d(sb, &tmap_b, &full_bar[stage], k0, n0, pb);
            } else {
#pragma unroll
              for (int b = 0; b < BN / 64; ++b)
                tma_load_3d(sb + b * (64 * BK * 2), &tmap_b, &full_bar[stage], n0 + 64 * b, k0, pb);
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(true, g.a_mn_major != 0, g.b_mn_major != 0, BM, BN);
      const uint32_t a_lbo = g.a_mn_major ? 64 * BK * 2 : 0, b_lbo = g.b_mn_major ? 64 * BK * 2 : 0;
      const uint32_t a_kstep = g.a_mn_major ? 16 * 128 : 32;  // bytes per K = 16 step
      const uint32_t b_kstep = g.b_mn_major ? 16 * 128 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int64_t chunks = 0;   // accumulator chunks this CTA has started
      bool ok = true;
      for (int64_t u = blockIdx.x; u < g.num_tiles && ok; u += gridDim.x) {
        int kb = 0;
        while (kb < total_kb && ok) {
          const int ke = chunk_end(kb, low_kb, total_kb, g.low_chunk, g.hi_chunk);
          const int buf = (int)(chunks & 1);
          const uint32_t acc_phase = (uint32_t)((chunks >> 1) & 1);
          if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, abort_flag, g.status, kStatusGemmTimeout)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
          for (int k2 = kb; k2 < ke; ++k2) {
            if (!mbar_wait(&full_bar[stage], phase, abort_flag, g.status, kStatusGemmTimeout)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
            const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t adesc = umma_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
              const uint64_t bdesc = umma_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
              mma_f16_ss(d_tmem, adesc, bdesc, idesc, (k2 != kb || k != 0) ? 1u : 0u);
            }
            tc_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (ok) tc_commit(&acc_full[buf]);
          ++chunks;
          kb = ke;
        }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const int chalf = (warp - 2) >> 2;     // two warps share a quarter: columns [0,128) and [128,256) of the tile
    int64_t chunks = 0;
    bool ok = true;
    for (int64_t u = blockIdx.x; u < g.num_tiles && ok; u += gridDim.x) {
      float sum[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) sum[j] = 0.f;
      int kb = 0;
      while (kb < total_kb) {
        const int ke = chunk_end(kb, low_kb, total_kb, g.low_chunk, g.hi_chunk);
        const int buf = (int)(chunks & 1);
        const uint32_t acc_phase = (uint32_t)((chunks >> 1) & 1);
        if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag, g.status, kStatusGemmTimeout)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + chalf * 128);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[c * 32 + j] += __uint_as_float(r[j]);   // fp32, round to nearest
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[buf]);
        ++chunks;
        kb = ke;
      }
      if (!ok) break;
      int64_t tm, tn;
      tile_coords(u, tiles_m, tiles_n, g.group_m, tm, tn);
      const int64_t row = tm * BM + quarter * 32 + lane;
      const int64_t col0 = tn * BN + chalf * 128;
      if (row < g.M) {
        float* crow = g.c + row * g.c_s0;
#pragma unroll
        for (int q = 0; q < 32; ++q) {
          const int64_t col = col0 + q * 4;
          if (col >= g.N) break;
          float v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[j] = sum[q * 4 + j];
            if (g.has_bias) {
              const float z = col + j < g.N ? g.bias[row * g.bias_s0 + (col + j) * g.bias_s1] : 0.f;
              v[j] = v[j] * g.alpha + z * g.beta;
            }
          }
          if (g.c_vec_ok && col + 4 <= g.N) {
            *reinterpret_cast<float4*>(crow + col) = make_float4(v[0], v[1], v[2], v[3]);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (col + j < g.N) crow[col + j] = v[j];
          }
        }
      }
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

// x [outer, inner] fp32 with `inner` contiguous and `ld_in` elements between rows -> three bf16
// planes [outer, ld_out] (`plane_stride` elements apart) with x = hi + mid + lo exactly; the pad
// columns [inner, ld_out) are written as zeros.  Eight elements per thread.
__global__ void __launch_bounds__(256) split3_kernel(const float* __restrict__ x, int64_t outer, int64_t inner,
                                                      int64_t ld_in, __nv_bfloat16* __restrict__ planes,
                                                      int64_t ld_out, int64_t plane_stride, int vec_ok,
                                                      int* nonfinite) {
  const int64_t groups = ld_out >> 3;
  const int64_t total = outer * groups;
  bool bad = false;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / groups, c0 = (idx - r * groups) << 3;
    const float* src = x + r * ld_in + c0;
    float v[8];
    if (vec_ok && c0 + 8 <= inner) {
      const uint4 u0 = ldg16_stream(src), u1 = ldg16_stream(src + 4);
      v[0] = __uint_as_float(u0.x); v[1] = __uint_as_float(u0.y); v[2] = __uint_as_float(u0.z); v[3] = __uint_as_float(u0.w);
      v[4] = __uint_as_float(u1.x); v[5] = __uint_as_float(u1.y); v[6] = __uint_as_float(u1.z); v[7] = __uint_as_float(u1.w);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = c0 + j < inner ? src[j] : 0.f;
    }
    float h[8], m[8], l[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float xv = v[j];
      bad |= !isfinite(xv);
      float fh = __bfloat162float(__float2bfloat16_rn(xv));
      // rounding up past the largest finite bf16: take the truncated piece instead
      if (isinf(fh)) fh = __uint_as_float(__float_as_uint(xv) & 0xffff0000u);
      const float r1 = xv - fh;                                   // exact
      const float fm = __bfloat162float(__float2bfloat16_rn(r1));
      const float r2 = r1 - fm;                                   // exact; fits 8 bits unless denormal as bf16
      h[j] = fh; m[j] = fm; l[j] = r2;
    }
    __nv_bfloat16* dst = planes + r * ld_out + c0;
    stg16(dst, Vec16<__nv_bfloat16>::pack(h));
    stg16(dst + plane_stride, Vec16<__nv_bfloat16>::pack(m));
    stg16(dst + 2 * plane_stride, Vec16<__nv_bfloat16>::pack(l));
  }
  if (bad) *nonfinite = 1;
}

// FLAGGEMS_B200_F32_CHUNK: K blocks of 64 per hi*hi accumulator chunk (default 4; for measurements).
const int g_hi_chunk = []() {
  const char* e = getenv("FLAGGEMS_B200_F32_CHUNK");
  const int v = e ? atoi(e) : 0;
  return v > 0 ? v : 4;
}();
constexpr int kLowChunk = 32;

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// How an operand [rows, cols] with element strides (s0, s1) is laid out for the split.
struct Operand {
  bool ok = false;
  bool dim0_contiguous = false;   // column-major storage
  int64_t outer = 0, inner = 0, ld_in = 0, ld_out = 0;
  int64_t plane_elems() const { return outer * ld_out; }
};
Operand describe(int64_t rows, int64_t cols, int64_t s0, int64_t s1) {
  Operand o;
  if (s1 == 1 && s0 >= cols) {
    o.ok = true; o.dim0_contiguous = false; o.outer = rows; o.inner = cols; o.ld_in = s0;
  } else if (s0 == 1 && s1 >= rows) {
    o.ok = true; o.dim0_contiguous = true; o.outer = cols; o.inner = rows; o.ld_in = s1;
  }
  o.ld_out = round_up(o.inner, 8);
  return o;
}

bool split_eligible(const fg_gemm_params* p, Operand& a, Operand& b) {
  if (p->dtype != FG_F32) return false;
  if (p->M < 128 || p->N < 128 || p->K < 128) return false;
  if (p->M > 2147483647LL - BM || p->N > 2147483647LL - BN || p->K > 2147483647LL / 8) return false;
  // below this the CUDA-core kernel is as fast (measured: a tie at 3e8, 1.4x at 1e9): the split
  // passes and the extra launches cost about 60 us
  if ((double)p->M * (double)p->N * (double)p->K < 536870912.0) return false;
  if (p->c_stride1 != 1) return false;
  if (p->M > 65535LL * 64) return false;   // the gated CUDA-core launch behind the kernel must fit its grid
  a = describe(p->M, p->K, p->a_stride0, p->a_stride1);
  b = describe(p->K, p->N, p->b_stride0, p->b_stride1);
  return a.ok && b.ok;
}

constexpr int64_t kFlagBytes = 256;

}  // namespace

int64_t gemm_f32_split_workspace_bytes(const fg_gemm_params* p) {
  Operand a, b;
  if (!p || !split_eligible(p, a, b)) return 0;
  return kFlagBytes + round_up(3 * a.plane_elems() * 2, 256) + round_up(3 * b.plane_elems() * 2, 256);
}

int gemm_f32_split(const fg_gemm_params* p, void* workspace, int64_t workspace_bytes, cudaStream_t st) {
  using namespace fg;
  Operand a, b;
  if (!split_eligible(p, a, b))
    return fail(FG_ERR_UNSUPPORTED, "gemm_f32_split: fg_gemm takes this problem (fg_gemm_f32_split_workspace_bytes is 0)");
  const int64_t need = gemm_f32_split_workspace_bytes(p);
  FG_REQUIRE(workspace != nullptr && workspace_bytes >= need, "gemm_f32_split: workspace of %lld bytes, %lld needed",
             (long long)workspace_bytes, (long long)need);
  FG_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "gemm_f32_split: workspace must be 256-byte aligned");
  int* status = device_status_ptr();
  if (!status) return fail(FG_ERR_CUDA, "gemm_f32_split: device status word unavailable");

  int* flag = reinterpret_cast<int*>(workspace);
  __nv_bfloat16* pa = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(workspace) + kFlagBytes);
  __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(pa) + round_up(3 * a.plane_elems() * 2, 256));
  FG_CUDA_OK(cudaMemsetAsync(flag, 0, sizeof(int), st));
  auto run_split = [&](const void* src, const Operand& o, __nv_bfloat16* dst) -> int {
    const int64_t total = o.outer * (o.ld_out >> 3);
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)num_sms() * 16;
    if (blocks > cap) blocks = cap;
    const int vec_ok = aligned16(src) && o.ld_in % 4 == 0;
    split3_kernel<<<(unsigned)blocks, 256, 0, st>>>(reinterpret_cast<const float*>(src), o.outer, o.inner, o.ld_in, dst,
                                                     o.ld_out, o.plane_elems(), vec_ok, flag);
    FG_CHECK_LAUNCH("split3_kernel");
    return FG_OK;
  };
  int rc = run_split(p->a, a, pa);
  if (rc != FG_OK) return rc;
  rc = run_split(p->b, b, pb);
  if (rc != FG_OK) return rc;

  // A [M, K]: K contiguous unless stored column-major.  B [K, N]: N contiguous unless stored column-major.
  const bool a_mn = a.dim0_contiguous, b_mn = !b.dim0_contiguous;
  CUtensorMap ta, tb;
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    dims[2] = 3;
    box[2] = 1;
    if (!a_mn) {
      dims[0] = (uint64_t)p->K; dims[1] = (uint64_t)p->M; box[0] = 64; box[1] = BM;
    } else {
      dims[0] = (uint64_t)p->M; dims[1] = (uint64_t)p->K; box[0] = 64; box[1] = BK;
    }
    strides[0] = (uint64_t)a.ld_out * 2;
    strides[1] = (uint64_t)a.plane_elems() * 2;
    rc = encode_tmap_16bit(&ta, pa, 3, dims, strides, box);
    if (rc != FG_OK) return rc;
    if (!b_mn) {
      dims[0] = (uint64_t)p->K; dims[1] = (uint64_t)p->N; box[0] = 64; box[1] = BN;
    } else {
      dims[0] = (uint64_t)p->N; dims[1] = (uint64_t)p->K; box[0] = 64; box[1] = BK;
    }
    strides[0] = (uint64_t)b.ld_out * 2;
    strides[1] = (uint64_t)b.plane_elems() * 2;
    rc = encode_tmap_16bit(&tb, pb, 3, dims, strides, box);
    if (rc != FG_OK) return rc;
  }
  SplitArgs g;
  g.c = reinterpret_cast<float*>(p->c);
  g.bias = reinterpret_cast<const float*>(p->bias);
  g.M = p->M; g.N = p->N; g.K = p->K;
  g.c_s0 = p->c_stride0;
  g.bias_s0 = p->bias_stride0; g.bias_s1 = p->bias_stride1;
  g.alpha = (float)p->alpha; g.beta = (float)p->beta;
  g.has_bias = p->bias != nullptr;
  g.a_mn_major = a_mn; g.b_mn_major = b_mn;
  g.kb_per_pair = (int)((p->K + BK - 1) / BK);
  g.low_chunk = kLowChunk;
  g.hi_chunk = g_hi_chunk;
  g.c_vec_ok = aligned16(p->c) && p->c_stride0 % 4 == 0;
  const int64_t tiles_m = (p->M + BM - 1) / BM, tiles_n = (p->N + BN - 1) / BN;
  g.num_tiles = tiles_m * tiles_n;
  // row tiles per sweep: keep a group's A panels (three pieces) around 32 MB
  const int64_t panel = (int64_t)BM * p->K * 2 * 3;
  int64_t gm = ((int64_t)32 << 20) / panel;
  if (gm < 4) gm = 4;
  if (gm > 64) gm = 64;
  g.group_m = (int)gm;
  g.nonfinite = flag;
  g.status = status;

  static thread_local int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    FG_CUDA_OK(cudaFuncSetAttribute(gemm_f32_split_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_BYTES));
    attr_dev = dev;
  }
  const int sms = sm_budget();
  const int grid = g.num_tiles < sms ? (int)g.num_tiles : sms;
  gemm_f32_split_tcgen05_kernel<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ta, tb, g);
  FG_CHECK_LAUNCH("gemm_f32_split_tcgen05_kernel");
  // non-finite inputs: the CUDA-core kernel computes the result instead (it returns at once otherwise)
  return gemm_simt_gated(p, flag, st);
}

}  // namespace fg
