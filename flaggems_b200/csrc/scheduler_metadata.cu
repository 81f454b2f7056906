// get_scheduler_metadata: split-KV scheduling data for FlashAttention-3 style decode.
//
// Replaces get_scheduler_metadata (src/flag_gems/ops/get_scheduler_metadata.py:567-894) for
// compute capability >= 9.0, the only branch a B200 reaches.  The result is an int32 vector
//   [0]                         work-queue semaphore, zeroed
//   [1 .. batch]                KV splits of each sequence (only for batches of at most 992)
// Two parts:
//   * fg_scheduler_plan: pure host arithmetic (mask normalisation, pack-GQA choice, static split
//     count from the wave-efficiency heuristic, the tile the block counts are taken in);
//   * scheduler_metadata_kernel: ONE launch of one CTA that counts query and key tiles per
//     sequence, sums them over the batch in shared memory and derives the per-sequence splits.
//     The reference runs two kernels with a device-to-host read of the sum between them; here
//     nothing leaves the device, so the call neither synchronises nor breaks a stream capture.
#include "common.cuh"

namespace fg {
namespace {

struct TileMN {
  int m, n;
};

int round_head_dim(int d, int last) {
  const int steps[5] = {64, 96, 128, 192, 256};
  for (int s : steps)
    if (d <= s) return s;
  return last;
}

// Tile of the 16-bit forward kernel the block counts refer to.
TileMN tile_mn(int d, int dv, bool causal, bool local, bool paged_non_tma, bool one_wg) {
  if (d <= 64) {
    if (dv == 512) return {64, 64};
    if (dv == 256) return {128, 112};
    return {192, (causal || local) ? 128 : 192};
  }
  if (d <= 96) return {192, (local || paged_non_tma) ? 128 : 144};
  if (d <= 128) return {one_wg ? 64 : 128, (causal || local || paged_non_tma) ? 128 : 176};
  if (d <= 192) return {128, (paged_non_tma || local) ? 96 : (dv <= 128 ? 128 : 112)};
  return {128, local ? 64 : 80};
}

bool one_mma_warpgroup(int headdim, int seqlen_q, bool pack_gqa, int hq, int hk) {
  return headdim == 128 && (int64_t)seqlen_q * (pack_gqa ? hq / hk : 1) <= 64;
}

int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// Fewest splits whose last wave is at least 85 % as full as the best one (doubles, like the
// Python floats of the reference).
int split_heuristic(int64_t total_mblocks, int num_sm, int n_blocks, int m_blocks, int64_t bytes_one_kv_head,
                    bool causal_or_local, int max_splits) {
  if ((double)total_mblocks >= 0.8 * num_sm) {
    const int64_t l2 = 50ll * 1024 * 1024;
    if (bytes_one_kv_head > l2 && m_blocks >= num_sm * 2 && !causal_or_local) {
      const int64_t s = (bytes_one_kv_head + l2 - 1) / l2;
      return (int)(s < max_splits ? s : max_splits);
    }
    return 1;
  }
  if (n_blocks <= 4) return 1;
  if (num_sm < max_splits) max_splits = num_sm;
  if (n_blocks < max_splits) max_splits = n_blocks;
  double eff[128];
  double best = 0.0;
  for (int s = 1; s <= max_splits; ++s) {
    const double waves = (double)(total_mblocks * s) / num_sm;
    eff[s - 1] = waves / ceil(waves);
    if (eff[s - 1] > best) best = eff[s - 1];
  }
  for (int s = 1; s <= max_splits; ++s)
    if (eff[s - 1] >= 0.85 * best) return s;
  return 1;
}

struct KernelArgs {
  const int32_t *seqused_k, *cu_seqlens_q, *cu_seqlens_k_new, *seqused_q, *leftpad_k;
  int32_t* metadata;
  int batch, max_seqlen_q, max_seqlen_k_new, q_per_kv, heads, block_m, block_n, num_sm, num_splits;
  int pad_blocks;  // tiles the reference's unmasked 128-wide sum adds for the lanes past the batch
  int dynamic;
};

__device__ __forceinline__ void seq_blocks(const KernelArgs& a, int b, int& m_blocks, int& n_blocks) {
  int q_len = a.seqused_q ? a.seqused_q[b] : a.cu_seqlens_q ? a.cu_seqlens_q[b + 1] - a.cu_seqlens_q[b] : a.max_seqlen_q;
  q_len *= a.q_per_kv;
  m_blocks = (q_len + a.block_m - 1) / a.block_m;
  int k_len = a.seqused_k[b];
  if (a.max_seqlen_k_new > 0)
    k_len += a.cu_seqlens_k_new ? a.cu_seqlens_k_new[b + 1] - a.cu_seqlens_k_new[b] : a.max_seqlen_k_new;
  if (a.leftpad_k) k_len -= a.leftpad_k[b];
  n_blocks = (k_len + a.block_n - 1) / a.block_n;
}

constexpr int kThreads = 1024;

__global__ void __launch_bounds__(kThreads) scheduler_metadata_kernel(const KernelArgs a) {
  __shared__ int warp_sums[kThreads / 32];
  __shared__ int s_per_sm;
  const int tid = threadIdx.x;
  if (tid == 0) a.metadata[0] = 0;
  if (!a.dynamic) return;
  int sum = 0;
  for (int b = tid; b < a.batch; b += kThreads) {
    int m, n;
    seq_blocks(a, b, m, n);
    sum += m * n;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((tid & 31) == 0) warp_sums[tid >> 5] = sum;
  __syncthreads();
  if (tid < 32) {
    int v = warp_sums[tid];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (tid == 0) {
      const int total = v + a.pad_blocks;
      // KV tiles one SM should get, with 10 % slack: fp32, one rounding per operation
      const float per_sm =
          ceilf(__fdiv_rn(__fmul_rn(__fmul_rn((float)total, 1.1f), (float)a.heads), (float)a.num_sm));
      const int p = (int)per_sm;
      s_per_sm = p > 1 ? p : 1;
    }
  }
  __syncthreads();
  const int per_sm = s_per_sm;
  for (int b = tid; b < a.batch; b += kThreads) {
    int m, n;
    seq_blocks(a, b, m, n);
    int s = (n + per_sm - 1) / per_sm;
    s = s < a.num_splits ? s : a.num_splits;
    a.metadata[1 + b] = s > 1 ? s : 1;
  }
}

int make_plan(const FgSchedulerParams* p, FgSchedulerPlan* out) {
  FG_REQUIRE(p && out, "scheduler_plan: null pointer");
  FG_REQUIRE(p->batch_size >= 0 && p->max_seqlen_q >= 0 && p->max_seqlen_k >= 0, "scheduler_plan: negative size");
  FG_REQUIRE(p->num_heads > 0 && p->num_heads_k > 0 && p->num_heads % p->num_heads_k == 0,
             "scheduler_plan: %d query heads are not a multiple of %d KV heads", p->num_heads, p->num_heads_k);
  FG_REQUIRE(p->headdim > 0 && p->headdim_v > 0, "scheduler_plan: head dims must be positive");
  FG_REQUIRE(p->elem_size == 2, "scheduler_plan: FlashAttention only supports fp16 and bf16 data type");
  FG_REQUIRE(p->page_size >= 0 && p->max_seqlen_k_new >= 0, "scheduler_plan: negative page size or appended length");
  if (p->arch < 90)
    return fail(FG_ERR_UNSUPPORTED, "scheduler_plan: compute capability %d is below 9.0 (library built for sm_100a)",
                p->arch);
  const int num_sm = p->num_sm - p->sm_margin;
  FG_REQUIRE(num_sm > 0, "scheduler_plan: %d SMs minus a margin of %d leaves none", p->num_sm, p->sm_margin);

  int wl = p->window_size_left >= 0 ? p->window_size_left : -1;
  int wr = p->window_size_right;
  if (wl >= p->max_seqlen_k - 1) wl = -1;
  if (wr >= p->max_seqlen_q - 1) wr = -1;
  const bool paged = p->page_size > 0;
  bool causal = p->is_causal != 0;
  if (p->max_seqlen_q == 1 && wl == -1 && wr == -1 && ((p->headdim <= 64 || p->headdim > 128) || !paged))
    causal = false;
  if (causal) wr = 0;
  causal = wl < 0 && wr == 0;
  const bool local = (wl >= 0 || wr >= 0) && !causal;
  const int d_r = round_head_dim(p->headdim, 256), dv_r = round_head_dim(p->headdim_v, 512);
  const int group = p->num_heads / p->num_heads_k;
  const int64_t q_packed = (int64_t)p->max_seqlen_q * group;

  // paged K/V through TMA needs whole pages per key tile and more than one query tile
  bool paged_tma = false;
  const bool leftpad = p->has_leftpad || p->leftpad_k;
  const bool varlen_q = p->varlen_q || p->cu_seqlens_q || p->seqused_q;
  if (paged && !leftpad && p->max_seqlen_k_new == 0) {
    const TileMN t = tile_mn(d_r, dv_r, causal, local, false, false);
    paged_tma = p->page_size % t.n == 0 && q_packed > t.m;
  }
  bool pack;
  if (p->pack_gqa >= 0) {
    pack = p->pack_gqa != 0;
  } else if ((paged && !paged_tma) || p->num_splits > 1) {
    pack = true;
  } else if (p->num_heads == p->num_heads_k) {
    pack = false;
  } else if (varlen_q) {
    pack = true;
  } else {
    const int bm = tile_mn(d_r, dv_r, causal, local, paged && !paged_tma, false).m;
    auto up = [bm](int64_t a) { return (a + bm - 1) / bm * bm; };
    pack = (double)p->max_seqlen_q / (double)up(p->max_seqlen_q) < 0.9 * ((double)q_packed / (double)up(q_packed));
  }
  const bool dynamic = p->batch_size <= 992;
  int splits = p->num_splits;
  if (splits <= 0) {
    // the static count treats paged K/V as the non-TMA form whatever was found above
    const TileMN t = tile_mn(d_r, dv_r, causal, local, paged,
                             one_mma_warpgroup(p->headdim, p->max_seqlen_q, pack, p->num_heads, p->num_heads_k));
    int64_t k_loaded = p->max_seqlen_k;
    if (local) {
      k_loaded = (int64_t)wl + wr + 1 + t.m;
      if (k_loaded > p->max_seqlen_k) k_loaded = p->max_seqlen_k;
      if (k_loaded < 0) k_loaded = 0;
    }
    const int n_blocks = ceil_div(k_loaded, t.n), m_blocks = ceil_div(q_packed, t.m);
    splits = split_heuristic((int64_t)(dynamic ? 1 : p->batch_size) * p->num_heads_k * m_blocks, num_sm, n_blocks,
                             m_blocks, (int64_t)p->max_seqlen_k * (p->headdim + p->headdim_v) * p->elem_size,
                             causal || local, 128);
  }
  if (splits > 256) splits = 256;
  if (splits > num_sm) splits = num_sm;
  if (splits > 1) pack = true;
  const TileMN t = tile_mn(d_r, dv_r, causal, local, paged && !paged_tma,
                           one_mma_warpgroup(p->headdim, p->max_seqlen_q, pack, p->num_heads, p->num_heads_k));
  out->num_splits = splits;
  out->pack_gqa = pack;
  out->block_m = t.m;
  out->block_n = t.n;
  out->use_dynamic_split = dynamic;
  out->is_causal = causal;
  out->is_local = local;
  out->q_per_kv = pack ? (p->num_heads + p->num_heads_k - 1) / p->num_heads_k : 1;
  out->heads = pack ? p->num_heads_k : p->num_heads;
  out->metadata_len = 1 + (dynamic ? p->batch_size : 0);
  return FG_OK;
}

}  // namespace
}  // namespace fg

extern "C" int fg_scheduler_plan(const FgSchedulerParams* p, FgSchedulerPlan* plan) { return fg::make_plan(p, plan); }

extern "C" int fg_get_scheduler_metadata(const FgSchedulerParams* p, int32_t* metadata, void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("get_scheduler_metadata");
  FgSchedulerPlan plan;
  const int rc = make_plan(p, &plan);
  if (rc != FG_OK) return rc;
  FG_REQUIRE(metadata, "get_scheduler_metadata: null output");
  FG_REQUIRE(p->batch_size == 0 || p->seqused_k, "get_scheduler_metadata: seqused_k is required");
  FG_REQUIRE(!(p->varlen_q && !p->cu_seqlens_q && !p->seqused_q),
             "get_scheduler_metadata: varlen_q set without cu_seqlens_q or seqused_q");
  FG_REQUIRE(!(p->has_leftpad && !p->leftpad_k), "get_scheduler_metadata: has_leftpad set without leftpad_k");
  KernelArgs a;
  a.seqused_k = p->seqused_k;
  a.cu_seqlens_q = p->seqused_q ? nullptr : p->cu_seqlens_q;
  a.cu_seqlens_k_new = p->cu_seqlens_k_new;
  a.seqused_q = p->seqused_q;
  a.leftpad_k = p->leftpad_k;
  a.metadata = metadata;
  a.batch = p->batch_size;
  a.max_seqlen_q = p->max_seqlen_q;
  a.max_seqlen_k_new = p->max_seqlen_k_new;
  a.q_per_kv = plan.q_per_kv;
  a.heads = plan.heads;
  a.block_m = plan.block_m;
  a.block_n = plan.block_n;
  a.num_sm = p->num_sm - p->sm_margin;
  a.num_splits = plan.num_splits;
  a.dynamic = plan.use_dynamic_split;
  // The reference sums its first pass over programs of 128 sequences without masking the lanes past
  // the batch: such a lane reads 0 keys and 0 query tokens from the length vectors, but when the query
  // length and the appended length are the two constants it still counts one sequence of max_seqlen_q
  // queries and max_seqlen_k_new keys.  Added here so that the result stays identical.
  a.pad_blocks = 0;
  if (p->max_seqlen_k_new > 0 && !p->cu_seqlens_k_new && !p->seqused_q && !p->cu_seqlens_q) {
    const int pad = (128 - p->batch_size % 128) % 128;
    a.pad_blocks = pad * ceil_div((int64_t)p->max_seqlen_q * plan.q_per_kv, plan.block_m) *
                   ceil_div(p->max_seqlen_k_new, plan.block_n);
  }
  scheduler_metadata_kernel<<<1, kThreads, 0, (cudaStream_t)stream>>>(a);
  FG_CHECK_LAUNCH("scheduler_metadata_kernel");
  return FG_OK;
}
