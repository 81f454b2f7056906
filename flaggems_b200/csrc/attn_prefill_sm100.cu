// Prefill attention for head dim 128 on sm_100a tensor cores (tcgen05 + TMEM).
//
// One work item = 128 query positions of one sequence x TWO query heads of the same KV
// group (one when the group size is odd): the two 128-row Q tiles share every K/V
// tile, which halves the K/V traffic and lets the tensor pipe work on one tile while
// the softmax warps work on the other.
//
//   warps 0-7    softmax, one warpgroup per Q tile, one thread per row (TMEM lane = row), so a
//                row needs no exchange between threads.  The score tile is produced in steps
//                of 64 keys into the tile's one score buffer.  Per step: tcgen05.ld the 64
//                scores into registers and hand the buffer back at once (the next step's scores
//                are computed while this step's softmax runs), row max, scale, mask, exp2, pack
//                P to 16 bit and tcgen05.st it into one of the tile's two probability buffers.
//                The running max is only raised when it grows by more than 8 (log2 units),
//                so the O accumulator in TMEM is rescaled rarely; the same warps write the
//                normalised output
//   warp 8       TMA producer: Q tiles once, then K and V tiles (128 keys x 128) through
//                two 2-stage rings; paged caches are fetched page by page with one
//                4-D box per page and 64-column half, so a tile lands as a dense,
//                128-byte-swizzled K-major tile
//   warps 9,10   one score-issuing thread per Q tile: S = Q K^T of a step as 8 SS MMAs (M128 N64
//                K16), issued as soon as the softmax warps hold the previous step's scores in
//                registers and the PV MMAs that read the probability buffer this step will fill
//                (two steps back) have completed
//   warp 11      one PV-issuing thread for both tiles: O += P V of a step as 4 TS MMAs per tile
//                (M128 N128 K16, P read from TMEM as the A operand), tile 0 then tile 1, each as
//                soon as its probabilities are stored.  Three issuing threads instead of one per
//                tile: a thread that issues a step's 12 MMAs and 3-4 commits beside the softmax
//                warps of its scheduler needs about as long as a softmax step, and with the score
//                MMAs on threads of their own the tensor pipe's round trip is off the softmax
//                warps' path (+2 % on the whole kernel; 12 warps still leave 170 registers a thread,
//                a 13th would cap them at 128)
// TMEM columns: tile t has its score buffer at t*128 (64 columns), its probability buffers at
// t*128+64 and t*128+96 (32 packed columns each: keys [16k,16k+16) in columns 8k..8k+8) and its
// output at 256+t*128.
// Every wait in the kernel is an mbarrier wait with a time limit (no named barriers, no
// register reallocation): a wait that gives up sets the device status word and the CTA drains.
// The kernel is persistent: one CTA per SM keeps its shared memory, TMEM, tensor maps and barriers
// and draws work items from a ticket counter (query blocks of a sequence from the longest causal
// prefix to the shortest).  Nothing synchronises the CTA between items: the producer warp publishes
// the next item through a two-slot ring and loads ahead, the roles follow the barrier phases with
// running counters, and the first score step of an item is computed while the previous output
// tile is still being normalised and stored.
//
// Measured costs that shaped this layout (B200, SM clocks, microbenchmarks on an otherwise
// idle SM): an mbarrier arrive reaches a waiting thread after 110-150; the first result of
// an MMA group lands ~180 after issue; the tensor pipe takes 59 for an SS M128 K16 MMA with
// N <= 64, 64 with N = 128 (SS and TS alike), 128 with N = 256; one diverged thread needs
// 45-50 to issue an MMA and ~95 for a tcgen05.commit; ex2 runs at 4 lanes per clock and
// scheduler (8 per warp instruction), one warp alone sustains 12.5 per element of the
// fma/ex2/add/pack mix and two or more warps per scheduler 8.3-8.7, i.e. the special-function
// unit, not the tensor pipe, bounds a 128-wide head: 2048 clocks per 128 keys and two Q tiles
// against 2080 of MMA time.
//
// Covers: fp16/bf16, head dim 128, causal or full attention, paged (block size a
// power of two >= 8) or contiguous KV.  ALiBi, soft-cap, windows and other head dims
// take the general kernel.
#include <atomic>

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
#define FG_SITE(n) (st_code + 1000 * (n))
#else
#define FG_SITE(n) (st_code)
#define FG_TRACE(slot, idx) \
  do {                      \
  } while (0)
#endif

namespace fg {

// Ticket counters of the persistent prefill kernel (one per launch in flight, see the launcher).
// A launch takes the next counter of the ring and zeroes it on its stream ahead of the kernel, so
// launches on different streams do not share one -- as long as fewer than kTicketRing prefill
// launches are queued or running on a device at the same time, across all streams (a launch that
// is still in flight when the ring comes round to its counter would have it zeroed under it and
// repeat or skip query blocks).  A captured CUDA graph bakes its counter in: do not replay such a
// graph concurrently with more than kTicketRing - 1 other prefill launches either.
constexpr unsigned int kTicketRing = 1024;
__device__ unsigned int g_prefill_tickets[kTicketRing];

int* device_status_ptr();

namespace {

constexpr int BM = 128, BN = 128, HD = 128;   // BN: keys per K/V tile in shared memory
constexpr int STEP = 64;                      // keys per score step (one TMEM score buffer)
constexpr int HALF_BYTES = 128 * 64 * 2;   // one [128 x 64] 128B-swizzled sub-tile
constexpr int TILE_BYTES = 2 * HALF_BYTES; // 32 KB
constexpr int TMA_WARP = 8, MMA_WARP0 = 9;
constexpr int NUM_THREADS = 12 * 32;   // 8 softmax warps, TMA producer, two score-MMA issuers, one PV-MMA issuer
constexpr int SMEM_BYTES = 6 * TILE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct PrefillArgs {
  AttnArgs a;
  int tiles;            // query tiles per CTA (1 or 2)
  int page_rows;        // rows fetched per TMA box for K/V (min(block_size, 128)); 128 when contiguous
  int pages_per_tile;   // 128 / page_rows
  int is_bf16;
  int num_mb, num_hp;          // work items: (query block, head pair, sequence), query block fastest
  int64_t num_items;
  unsigned int* ticket;        // next work item of this launch (zeroed on the stream before the launch)
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  // volatile: the exponentials of a step stay in program order, back to back
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed pairs of fp32 (two lanes of one 64-bit register): (a0, a1) = (a0, a1) * sc + ng and
// (s0, s1) += (p0, p1) as single instructions.
__device__ __forceinline__ uint64_t pack2f(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void fma2(float& a0, float& a1, uint64_t sc, uint64_t ng) {
  asm("{\n .reg .b64 x, r;\n mov.b64 x, {%0, %1};\n fma.rn.f32x2 r, x, %2, %3;\n mov.b64 {%0, %1}, r;\n}\n"
      : "+f"(a0), "+f"(a1)
      : "l"(sc), "l"(ng));
}
__device__ __forceinline__ void add2(float& s0, float& s1, float p0, float p1) {
  asm("{\n .reg .b64 x, y, r;\n mov.b64 x, {%0, %1};\n mov.b64 y, {%2, %3};\n add.rn.f32x2 r, x, y;\n mov.b64 {%0, %1}, r;\n}\n"
      : "+f"(s0), "+f"(s1)
      : "f"(p0), "f"(p1));
}
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

template <bool kBf16>   // element type of Q/K/V/P/out: bf16 or fp16 (a compile-time choice keeps the
                        // per-pair conversions of the softmax loop free of selects)
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, PrefillArgs pa) {
  using namespace sm100;
  const AttnArgs& a = pa.a;
  const int NT = pa.tiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A wait that timed out anywhere on this device left the status word set: finish the
  // launch quickly instead of letting every remaining CTA run into the same timeout
  // (one thread reads it so that the whole CTA takes the same decision).
  __shared__ int s_drain;
  __shared__ int64_t s_items[2];   // ring of work items published by the producer warp
  if (threadIdx.x == 0) s_drain = *reinterpret_cast<volatile int*>(a.status);
  __syncthreads();
  if (s_drain != 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                       // [2 tiles][2 halves][128 x 64]
  uint8_t* sK = smem + 2 * TILE_BYTES;      // [2 stages]
  uint8_t* sV = smem + 4 * TILE_BYTES;      // [2 stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  uint64_t* q_full = bars;            // [1]  Q tiles of an item have landed
  uint64_t* q_empty = bars + 1;       // [1]  every QK of an item has been executed: Q may be overwritten
  uint64_t* k_full = bars + 2;        // [2]
  uint64_t* k_empty = bars + 4;       // [2]
  uint64_t* v_full = bars + 6;        // [2]
  uint64_t* v_empty = bars + 8;       // [2]
  uint64_t* s_full = bars + 10;       // [2 tiles] scores of a step have landed in the tile's score buffer
  uint64_t* s_free = bars + 12;       // [2 tiles] ... and have been read into registers: the next may overwrite them
  uint64_t* p_ready = bars + 14;      // [2 tiles][2 probability buffers]
  uint64_t* o_done = bars + 18;       // [2 tiles][2]: PV of even / odd steps (a softmax warp can be two
                                      // steps ahead of the tensor pipe, one parity bit per barrier is not enough)
  uint64_t* o_free = bars + 22;       // [2 tiles] the output tile of the previous item has been read out
  uint64_t* item_full = bars + 24;    // [2]
  uint64_t* item_empty = bars + 26;   // [2]
  constexpr int NUM_BARS = 28;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(q_empty, NT);           // one commit per issuing thread
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], NT);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);        // the one PV-issuing thread commits for both tiles
      mbar_init(&o_free[i], 4);       // one arrival per softmax warp of the tile
      mbar_init(&item_full[i], 1);
      mbar_init(&item_empty[i], 5 * NT + 1);   // per tile: the score-issuing thread and four softmax warps; the PV thread
    }
    for (int i = 0; i < 2; ++i) mbar_init(&s_full[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&s_free[i], 4);    // one arrival per softmax warp of the tile
    for (int i = 0; i < 4; ++i) mbar_init(&p_ready[i], 4);   // one arrival per softmax warp of the tile
    for (int i = 0; i < 4; ++i) mbar_init(&o_done[i], 1);
    mbar_fence_init();
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == MMA_WARP0) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int st_code = kStatusAttnTimeout;
  // Every wait of a warp is polled by lane 0 and its outcome broadcast, so that a wait
  // that gave up takes the whole warp the same way.
  auto wwait = [&](uint64_t* bar, uint32_t parity, int site) -> bool {
    int r = 1;
    if (lane == 0) r = mbar_wait(bar, parity, abort_flag, a.status, FG_SITE(site)) ? 1 : 0;
    return __shfl_sync(0xffffffffu, r, 0) != 0;
  };

  // ---- persistent roles.  The CTA keeps its shared memory, TMEM, tensor maps and barriers for
  // the whole launch; the barriers are initialised once and every role follows their phases with
  // running counters (work items, K/V tiles, score steps), so nothing synchronises the CTA between
  // items: the producer warp draws the next item from the launch's ticket counter while the current
  // one is still being computed, publishes it through a two-slot ring and loads its Q and first K/V
  // tiles as soon as the stages are free; the score-issuing threads compute its first score step
  // while the softmax warps still normalise and store the previous output.
  struct Item {
    int m0, h0, b, n_steps, n_tiles, shift;
    SeqInfo s;
  };
  auto decode = [&](int64_t item, Item& it) {
    const int m_block = pa.num_mb - 1 - (int)(item % pa.num_mb);   // heaviest query block of a sequence first
    it.h0 = (int)((item / pa.num_mb) % pa.num_hp) * NT;
    it.b = (int)(item / ((int64_t)pa.num_mb * pa.num_hp));
    it.s = seq_info(a, it.b);
    it.m0 = m_block * BM;
    it.shift = it.s.k_len - it.s.q_len;
    int vis = it.s.k_len;               // keys visible to at least one row of this block
    if (a.causal) vis = max(0, min(vis, it.m0 + BM + it.shift));
    it.n_steps = (vis + STEP - 1) / STEP;
    it.n_tiles = (it.n_steps + 1) / 2;  // K/V tiles of 128 keys
  };
  // Next published item of a consumer role (lane 0 of a warp, or a single thread): -1 when the
  // launch has no more work or a wait gave up.
  auto next_item = [&](uint32_t n) -> int64_t {
    if (!mbar_wait(&item_full[n & 1], (n >> 1) & 1, abort_flag, a.status, FG_SITE(20))) return -1;
    const int64_t item = s_items[n & 1];
    mbar_arrive(&item_empty[n & 1]);
    return item;
  };

  if (warp == TMA_WARP) {
    // ================================ TMA producer ================================
    uint32_t n_pub = 0, n_q = 0, kv = 0;   // items published, items with a Q load, K/V tiles loaded
    bool ok = true;
    while (ok) {
      // draw tickets until one names a query block inside its sequence
      Item it;
      int64_t item = 0;
      for (;;) {
        if (lane == 0) item = (int64_t)atomicAdd(pa.ticket, 1u);
        item = __shfl_sync(0xffffffffu, item, 0);
        if (item >= pa.num_items) {
          item = -1;
          break;
        }
        decode(item, it);
        if (it.m0 < it.s.q_len) break;
      }
      if (!wwait(&item_empty[n_pub & 1], ((n_pub >> 1) & 1) ^ 1, 21)) break;
      if (lane == 0) {
        s_items[n_pub & 1] = item;
        mbar_arrive(&item_full[n_pub & 1]);   // release: the slot is written before the arrival is seen
      }
      ++n_pub;
      if (item < 0) break;
      if (it.n_tiles == 0) continue;          // no visible key: the softmax warps write zeros
      const SeqInfo& s = it.s;
      const int hk = it.h0 / a.group;
      if (n_q > 0 && !wwait(q_empty, (n_q - 1) & 1, 22)) break;
      if (lane == 0) {
        mbar_expect_tx(q_full, NT * TILE_BYTES);
        for (int t = 0; t < NT; ++t)
          for (int hf = 0; hf < 2; ++hf)
            tma_load_4d(sQ + t * TILE_BYTES + hf * HALF_BYTES, &tmap_q, q_full, hf * 64, it.h0 + t,
                        a.batch_strided ? it.m0 : s.q_begin + it.m0, a.batch_strided ? it.b : 0);
      }
      ++n_q;
      const int32_t* bt_row = a.paged ? a.block_table + (int64_t)it.b * a.bt_stride : nullptr;
      const int last_page = a.paged ? max(0, (s.k_len - 1) / a.block_size) : 0;
      for (int j = 0; j < it.n_tiles && ok; ++j, ++kv) {
        const int stg = kv & 1;
        const uint32_t ph = (kv >> 1) & 1;
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
          if (!wwait(empty, ph ^ 1, 1 + which)) {
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
              tma_load_4d(dst + hf * HALF_BYTES, tm, full, hf * 64, hk,
                          a.batch_strided ? j * BN : s.k_begin + j * BN, a.batch_strided ? it.b : 0);
          }
        }
      }
    }
  } else if (warp == MMA_WARP0 + 2 || (warp >= MMA_WARP0 && warp < MMA_WARP0 + NT)) {
    // ================================ MMA issuers =================================
    // One thread per Q tile for the score MMAs and one thread for the PV MMAs of both tiles: a single
    // thread per tile needs 1800-2000 clocks per step for both kinds beside the softmax warps of its
    // scheduler (45-50 clocks per MMA and ~95 per commit when alone), as long as a softmax step.  The
    // threads order their work through the barriers only (scores: S read out and the PV two steps
    // back completed; PV: probabilities stored), never through issue order.
    // The descriptors are kept as 32-bit low words plus one constant high word so that an
    // MMA costs one add per operand.
    const bool pv_role = warp == MMA_WARP0 + 2;     // warps 9, 10: scores of tile 0, 1; warp 11: PV of both tiles
    const int t = pv_role ? 0 : warp - MMA_WARP0;
    if (lane == 0) {
      constexpr bool bf16 = kBf16;
      const uint32_t idesc_qk = umma_idesc_f16(bf16, false, false, BM, STEP);  // A, B K-major, N = 64
      const uint32_t idesc_pv = umma_idesc_f16(bf16, false, true, BM, HD);     // B (V) MN-major
      // K-major operands: 8-row groups 1024 B apart.  V is MN-major: 64-column blocks HALF_BYTES
      // apart (leading offset), 8-key groups 1024 B apart, 16 keys (2048 B) per MMA.
      const uint32_t desc_hi = (uint32_t)(umma_desc_sw128(0, 0, 1024) >> 32);
      const uint32_t q_lo = (uint32_t)umma_desc_sw128(smem_u32(sQ + t * TILE_BYTES), 0, 1024);
      const uint32_t k_lo0 = (uint32_t)umma_desc_sw128(smem_u32(sK), 0, 1024);
      const uint32_t v_lo0 = (uint32_t)umma_desc_sw128(smem_u32(sV), HALF_BYTES, 1024);
      const uint32_t s_tmem = tmem_base + t * 128;   // the score thread's tile
      uint32_t n_it = 0, n_q = 0, kv0 = 0, g0 = 0;   // items read, items computed, K/V tiles and score steps before this item
      bool ok = true;
      while (ok) {
        const int64_t item = next_item(n_it++);
        if (item < 0) break;
        Item it;
        decode(item, it);
        const int n_steps = it.n_steps;
        if (n_steps == 0) continue;
#ifdef FG_PREFILL_TRACE
        const bool trace_on = blockIdx.x == 0 && g0 == 0;   // the first item this CTA computes
#endif
        if (!pv_role) {
          // ---- scores of step i: keys [64 i, 64 i + 64) = rows (i & 1) * 64 .. of K tile i >> 1, into the
          // tile's one score buffer as soon as the softmax warps hold the previous step's in registers
          if (!mbar_wait(q_full, n_q & 1, abort_flag, a.status, FG_SITE(3))) break;
          for (int i = 0; i < n_steps && ok; ++i) {
            const uint32_t tile = kv0 + (uint32_t)(i >> 1), stg = tile & 1, g = g0 + (uint32_t)i;
            if (!(i & 1) && !mbar_wait(&k_full[stg], (tile >> 1) & 1, abort_flag, a.status, FG_SITE(8))) {
              ok = false;
              break;
            }
            // the scores of the previous step (of this item or the one before) must have been read out
            if (g > 0 && !mbar_wait(&s_free[t], (g - 1) & 1, abort_flag, a.status, FG_SITE(9))) {
              ok = false;
              break;
            }
            // The softmax warps will store P(i) over the buffer that the PV MMAs of step i - 2, issued by
            // another thread, read: those must have completed before the scores of step i exist.  (Steps 0
            // and 1 of an item follow the previous item's last PV, which the softmax warps wait for in
            // their epilogue before they take the next item's first scores.)
            if (i >= 2 && !mbar_wait(&o_done[t * 2 + (g & 1)], ((g - 2) >> 1) & 1, abort_flag, a.status, FG_SITE(18))) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t k_lo = k_lo0 + stg * (TILE_BYTES >> 4) + (i & 1) * (STEP * 128 >> 4);
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) {
              const uint32_t off = ((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4;
              mma_f16_ss_lohi(s_tmem, q_lo + off, k_lo + off, desc_hi, idesc_qk, k != 0 ? 1u : 0u);
            }
            tc_commit(&s_full[t]);
            FG_TRACE(48 + t, i);
            if ((i & 1) || i == n_steps - 1) tc_commit(&k_empty[stg]);   // last step on this K tile
            if (i == n_steps - 1) tc_commit(q_empty);                    // last use of this item's Q
          }
        } else {
          // ---- O += P V of step i of both tiles, tile 0 first, once the probabilities are stored
          for (int i = 0; i < n_steps && ok; ++i) {
            const uint32_t tile = kv0 + (uint32_t)(i >> 1), stg = tile & 1, g = g0 + (uint32_t)i;
            if (!(i & 1) && !mbar_wait(&v_full[stg], (tile >> 1) & 1, abort_flag, a.status, FG_SITE(5))) {
              ok = false;
              break;
            }
            const uint32_t v_lo = v_lo0 + stg * (TILE_BYTES >> 4) + (i & 1) * (4 * 2048 >> 4);
            for (int tt = 0; tt < NT && ok; ++tt) {
              if (!mbar_wait(&p_ready[tt * 2 + (g & 1)], (g >> 1) & 1, abort_flag, a.status, FG_SITE(6))) {
                ok = false;
                break;
              }
              // the first PV of an item overwrites the output tile: the previous one must have been read out
              if (i == 0 && n_q > 0 && !mbar_wait(&o_free[tt], (n_q - 1) & 1, abort_flag, a.status, FG_SITE(7))) {
                ok = false;
                break;
              }
              tc_fence_after();
              FG_TRACE(0 + tt, i);
              const uint32_t p_tmem = tmem_base + tt * 128 + STEP + (g & 1) * 32;
              const uint32_t o_tm = tmem_base + 256 + tt * 128;
#pragma unroll
              for (int k = 0; k < 4; ++k)
                mma_f16_ts_lohi(o_tm, p_tmem + k * 8, v_lo + k * (2048 >> 4), desc_hi, idesc_pv, (i > 0 || k > 0) ? 1u : 0u);
              tc_commit(&o_done[tt * 2 + (g & 1)]);
            }
            if (ok && ((i & 1) || i == n_steps - 1)) tc_commit(&v_empty[stg]);     // last step on this V tile
          }
        }
        ++n_q;
        kv0 += (uint32_t)it.n_tiles;
        g0 += (uint32_t)n_steps;
      }
    }
  } else if (warp < 4 * NT) {
    // ================================ softmax / epilogue ===========================
    const int t = warp >> 2;                  // Q tile
    const int quarter = warp & 3;             // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;        // row inside the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_addr + t * 128;         // my row of the score tile
    const uint32_t o_addr = tmem_base + lane_addr + 256 + t * 128;   // my row of the output tile
    constexpr bool bf16 = kBf16;
    const float scale = a.scale_log2;
    uint32_t n_it = 0, kv0 = 0, g0 = 0;       // items read, K/V tiles and score steps before this item
    bool ok = true;

    while (ok) {
      int64_t item = 0;
      if (lane == 0) item = next_item(n_it);
      ++n_it;
      item = __shfl_sync(0xffffffffu, item, 0);
      if (item < 0) break;
      Item it;
      decode(item, it);
      const SeqInfo& s = it.s;
      const int m0 = it.m0, shift = it.shift, n_steps = it.n_steps;
      const int qpos = m0 + r;                  // query position inside the sequence
      const bool valid = qpos < s.q_len;
      char* orow = reinterpret_cast<char*>(a.out) +
                   ((a.batch_strided ? (int64_t)it.b * a.o_batch + (int64_t)qpos * a.o_rs
                                     : (int64_t)(s.q_begin + qpos) * a.o_rs) +
                    (int64_t)(it.h0 + t) * a.o_hs) * 2;
      float* lse_ptr = a.lse ? a.lse + (int64_t)(it.h0 + t) * a.total_q + s.q_begin + qpos : nullptr;
#ifdef FG_PREFILL_TRACE
      const bool trace_on = blockIdx.x == 0 && g0 == 0 && lane == 0;
#endif
      if (n_steps == 0) {
        // no visible key for any row of the block: zeros, lse = +inf
        if (valid) {
#pragma unroll
          for (int c = 0; c < HD / 8; ++c) *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(0, 0, 0, 0);
          if (lse_ptr) *lse_ptr = INFINITY;
        }
        continue;
      }
      float m_used = -INFINITY, l_run = 0.f;

      for (int i = 0; i < n_steps; ++i) {
        const uint32_t g = g0 + (uint32_t)i;
        const int sb = (int)(g & 1);                       // probability buffer of this step
        const uint32_t p_addr = s_addr + STEP + sb * 32;

        if (quarter == 0) FG_TRACE(8 + t * 16, i);
        if (!wwait(&s_full[t], g & 1, 10)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (quarter == 0) FG_TRACE(4 + t * 16, i);
        float sv[64];
        tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        tmem_ld_wait();
        // the scores are in registers: the next step's may be computed into the same columns
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[t]);
        const int col0 = i * STEP;
        if ((col0 + STEP > s.k_len) || (a.causal && (col0 + STEP - 1 > m0 + shift))) {
          int lim = s.k_len - 1;                         // last visible column of this row
          if (a.causal) lim = min(lim, qpos + shift);
#pragma unroll
          for (int e = 0; e < 64; ++e)
            if (col0 + e > lim) sv[e] = -INFINITY;
        }
        float m4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
        for (int e = 4; e < 64; e += 8) {
          m4[0] = max3(m4[0], sv[e], sv[e + 1]);
          m4[1] = max3(m4[1], sv[e + 2], sv[e + 3]);
          if (e + 4 < 64) {
            m4[2] = max3(m4[2], sv[e + 4], sv[e + 5]);
            m4[3] = max3(m4[3], sv[e + 6], sv[e + 7]);
          }
        }
        const float m_tile = fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]) * scale;  // scale > 0; -inf stays -inf
        if (quarter == 0) FG_TRACE(6 + t * 16, i);
        // Raise the reference maximum only when it grows by more than the threshold:
        // probabilities then stay below 2^8 and the accumulator needs no rescale.
        const bool raise = m_tile > m_used + kRescaleThreshold || (m_used == -INFINITY && m_tile > -INFINITY);
        if (i > 0 && __any_sync(0xffffffffu, raise)) {
          // every PV issued so far (steps 0 .. i-1; the pipe completes them in order) must have
          // landed before O is touched
          if (!wwait(&o_done[t * 2 + ((g - 1) & 1)], ((g - 1) >> 1) & 1, 14)) {
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
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
            tmem_st32(o_addr + c * 32, o);
          }
          l_run *= f;
        }
        if (raise) m_used = m_tile;
        const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
        if (a.paged && i == n_steps - 1 && col0 + STEP > s.k_len) {
          // Rows of the last V tile past the end of the sequence hold whatever the cache
          // page holds; zero the ones this step multiplies so 0 * garbage can never produce
          // NaN.  Each Q tile does it for itself (same zeros twice): its PV is ordered after
          // its own softmax only.
          const int tl = i >> 1;
          const uint32_t tile = kv0 + (uint32_t)tl, stg = tile & 1;
          if (!wwait(&v_full[stg], (tile >> 1) & 1, 15)) {
            ok = false;
            break;
          }
          const int first = s.k_len - tl * BN;               // first invalid row of the tile
          const int end = (i & 1) * STEP + STEP;             // this step's rows end here
          uint8_t* vt = sV + stg * TILE_BYTES;
          for (int idx = r; idx < (end - first) * 16; idx += 128) {
            const int row = first + idx / 16, ch = idx % 16;
            *reinterpret_cast<uint4*>(vt + (ch >> 3) * HALF_BYTES + row * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
        }
        // ---- probabilities -> 32 packed 32-bit columns over the start of the score buffer
        // (the scores are all in registers, so P may overwrite them in TMEM)
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        // Three passes over the 64 scores in registers -- exponent arguments, exponentials, then sums and
        // packing -- with the exponentials kept in program order (volatile): 64 independent
        // special-function instructions back to back instead of short fma -> ex2 -> add chains.  The
        // arguments and the row sums use the packed fp32 pair instructions (fma/add .f32x2): 2.5
        // instead of 3.5 instructions per score (+3 % on the whole kernel, measured).
        {
          const uint64_t sc2 = pack2f(scale, scale), ng2 = pack2f(neg_m, neg_m);
#pragma unroll
          for (int e = 0; e < 64; e += 2) fma2(sv[e], sv[e + 1], sc2, ng2);
        }
        if (quarter == 0) FG_TRACE(10 + t * 16, i);
#pragma unroll
        for (int e = 0; e < 64; ++e) sv[e] = ex2(sv[e]);
        if (quarter == 0) FG_TRACE(11 + t * 16, i);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = sv[q * 32 + 2 * e], p1 = sv[q * 32 + 2 * e + 1];
            add2(sum4[(e & 1) * 2], sum4[(e & 1) * 2 + 1], p0, p1);
            pk[e] = bf16 ? pack_bf16(p0, p1) : pack_f16(p0, p1);
          }
          tmem_st16(p_addr + q * 16, pk);
        }
        l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        if (quarter == 0) FG_TRACE(12 + t * 16, i);
        tmem_st_wait();
        if (quarter == 0) FG_TRACE(13 + t * 16, i);
        tc_fence_before();
        __syncwarp();
        if (quarter == 0) FG_TRACE(56 + t, i);
        if (lane == 0) mbar_arrive(&p_ready[t * 2 + sb]);
      }
      if (!ok) break;

      // ---- epilogue: normalise my row of O and write it out
      const uint32_t g_last = g0 + (uint32_t)n_steps - 1;
      if (!wwait(&o_done[t * 2 + (g_last & 1)], (g_last >> 1) & 1, 16)) break;
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32(o_addr + c * 32, o);
        tmem_ld_wait();
        if (c == 3) {
          // my row of the output tile is in registers: once the four warps of the tile have said
          // so, the next item's first PV may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&o_free[t]);
        }
        if (valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float x0 = __uint_as_float(o[q4 * 8 + 2 * j]) * inv;
              const float x1 = __uint_as_float(o[q4 * 8 + 2 * j + 1]) * inv;
              wp[j] = bf16 ? pack_bf16(x0, x1) : pack_f16(x0, x1);
            }
            *reinterpret_cast<uint4*>(orow + c * 64 + q4 * 16) = w;
          }
        }
      }
      if (valid && lse_ptr) *lse_ptr = l_run > 0.f ? m_used * 0.6931471805599453f + logf(l_run) : INFINITY;
      kv0 += (uint32_t)it.n_tiles;
      g0 += (uint32_t)n_steps;
    }
  }

  // ================================ teardown ======================================
  // Every role has left its loop: all MMAs and copies it issued have been waited for by the
  // role that consumes them (the last output tile was read after its o_done barrier).
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP0) {
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
  // Q and the contiguous K/V are four-dimensional maps [D, heads, rows, batches]: the packed form is
  // one "batch" of total rows, the batch-strided form (dense batches whose batch and sequence
  // dimensions do not pack, e.g. a transposed (batch, heads, seq, dim) tensor) has max_seqlen rows
  // per batch member and the batch stride as the outermost stride.
  {
    const uint64_t rows = a.batch_strided ? (uint64_t)a.max_q : (uint64_t)a.total_q;
    uint64_t dims[4] = {(uint64_t)HD, (uint64_t)a.H, rows, a.batch_strided ? (uint64_t)a.batch : 1ull};
    uint64_t strides[3] = {(uint64_t)a.q_hs * 2, (uint64_t)a.q_rs * 2,
                           a.batch_strided ? (uint64_t)a.q_batch * 2 : (uint64_t)a.q_rs * 2 * (rows > 0 ? rows : 1)};
    uint32_t box[4] = {64, 1, 128, 1};
    int rc = encode_tmap_16bit(&tq, a.q, 4, dims, strides, box);
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
    const uint64_t rows = a.batch_strided ? (uint64_t)(a.max_k > 0 ? a.max_k : 1) : (uint64_t)(a.total_k > 0 ? a.total_k : 1);
    uint64_t dims[4] = {(uint64_t)HD, (uint64_t)a.Hk, rows, a.batch_strided ? (uint64_t)a.batch : 1ull};
    uint32_t box[4] = {64, 1, 128, 1};
    uint64_t ks[3] = {(uint64_t)a.k_hs * 2, (uint64_t)a.k_rs * 2,
                      a.batch_strided ? (uint64_t)a.k_batch * 2 : (uint64_t)a.k_rs * 2 * rows};
    uint64_t vs[3] = {(uint64_t)a.v_hs * 2, (uint64_t)a.v_rs * 2,
                      a.batch_strided ? (uint64_t)a.v_batch * 2 : (uint64_t)a.v_rs * 2 * rows};
    int rc = encode_tmap_16bit(&tk, a.k, 4, dims, ks, box);
    if (rc != FG_OK) return rc;
    rc = encode_tmap_16bit(&tv, a.v, 4, dims, vs, box);
    if (rc != FG_OK) return rc;
  }
  static thread_local int attr_dev = -1;
  static thread_local unsigned int* tickets = nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_dev != dev) {
    FG_CUDA_OK(cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_BYTES));
    FG_CUDA_OK(cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_BYTES));
    void* sym = nullptr;
    FG_CUDA_OK(cudaGetSymbolAddress(&sym, g_prefill_tickets));
    tickets = reinterpret_cast<unsigned int*>(sym);
    attr_dev = dev;
  }
  pa.num_mb = (int)((a.max_q + BM - 1) / BM);
  pa.num_hp = a.H / pa.tiles;
  pa.num_items = (int64_t)pa.num_mb * pa.num_hp * a.batch;
  if (pa.num_items <= 0) return FG_OK;
  if (pa.num_items >= 4000000000LL) return fail(FG_ERR_TOO_LARGE, "flash_attn_varlen: too many query blocks");
  // One ticket counter per launch, taken round-robin from a small ring so that launches in
  // flight on different streams do not share one; zeroed on the stream ahead of the kernel.
  static std::atomic<unsigned int> launch_seq{0};
  pa.ticket = tickets + (launch_seq.fetch_add(1, std::memory_order_relaxed) % kTicketRing);
  FG_CUDA_OK(cudaMemsetAsync(pa.ticket, 0, sizeof(unsigned int), st));
  const int64_t ctas = pa.num_items < num_sms() ? pa.num_items : num_sms();
  dim3 grid((unsigned)ctas);
  if (pa.is_bf16)
    attn_prefill_tcgen05_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(tq, tk, tv, pa);
  else
    attn_prefill_tcgen05_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, st>>>(tq, tk, tv, pa);
  FG_CHECK_LAUNCH("attn_prefill_tcgen05_kernel");
  return FG_OK;
}

}  // namespace fg
