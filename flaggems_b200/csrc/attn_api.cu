// fg_flash_attn_varlen: argument validation, kernel-family selection and the
// workspace contract of the attention entry point.
#include <cmath>

#include "attn_common.cuh"

namespace fg {

int attn_generic(const AttnArgs& a, int dtype, cudaStream_t st);
int attn_decode(const AttnArgs& a, int dtype, int chunk_tokens, cudaStream_t st);
int attn_prefill_sm100(const AttnArgs& a, int dtype, cudaStream_t st);
bool attn_prefill_sm100_eligible(const fg_attn_params* p);
void decode_split_plan(int64_t batch, int64_t num_heads_k, int64_t max_seqlen_k, int forced_splits, int sms,
                       int* chunk_tokens, int* num_splits);
int* device_status_ptr();

enum { kPathGeneric = 0, kPathPrefillSm100 = 1, kPathDecode = 2 };

static bool has_window(const fg_attn_params* p) {
  // a window that already spans every key is no window (the reference clears it too)
  const bool left = p->window_left >= 0 && p->window_left < p->max_seqlen_k;
  const bool right = !p->causal && p->window_right >= 0 && p->window_right < p->max_seqlen_k;
  return left || right;
}

static int pick_path(const fg_attn_params* p) {
  const int64_t group = p->num_heads_k > 0 ? p->num_heads / p->num_heads_k : 0;
  if (p->max_seqlen_q == 1 && p->alibi_slopes == nullptr && !has_window(p) && group >= 1 && group <= 16 &&
      p->total_q == p->batch)
    return kPathDecode;
  if (attn_prefill_sm100_eligible(p)) return kPathPrefillSm100;
  return kPathGeneric;
}

}  // namespace fg

extern "C" int fg_flash_attn_path(const fg_attn_params* p) { return p ? fg::pick_path(p) : 0; }

extern "C" int64_t fg_flash_attn_workspace_bytes(int64_t batch, int64_t num_heads, int64_t head_dim,
                                                 int64_t max_seqlen_q, int64_t max_seqlen_k) {
  // Only single-query batches split.  Size for the shortest chunk the planner may
  // pick (256 tokens) so that any plan fits: splits * batch * H * (D + 1) floats.
  if (max_seqlen_q != 1 || batch <= 0) return 0;
  const int64_t splits = (max_seqlen_k + 255) / 256;
  if (splits <= 1) return 0;
  return splits * batch * num_heads * (head_dim + 1) * 4;
}

extern "C" int fg_flash_attn_varlen(const fg_attn_params* p, void* stream) {
  using namespace fg;
  FG_REQUIRE_HEALTHY("flash_attn_varlen");
  FG_REQUIRE(p != nullptr, "flash_attn_varlen: null params");
  FG_REQUIRE(p->dtype == FG_F16 || p->dtype == FG_BF16, "FlashAttention only support fp16 and bf16 data type");
  FG_REQUIRE(p->batch >= 0 && p->total_q >= 0, "flash_attn_varlen: negative size");
  FG_REQUIRE(p->num_heads > 0 && p->num_heads_k > 0, "flash_attn_varlen: head counts must be positive");
  FG_REQUIRE(p->num_heads % p->num_heads_k == 0,
             "Number of heads in key/value must divide number of heads in query");
  FG_REQUIRE(p->head_dim > 0 && p->head_dim <= 256, "FlashAttention forward only supports head dimension at most 256");
  FG_REQUIRE(p->head_dim % 8 == 0, "head_size must be a multiple of 8");
  if (p->batch == 0 || p->total_q == 0) return FG_OK;
  FG_REQUIRE(p->q && p->k && p->v && p->out, "flash_attn_varlen: null tensor");
  FG_REQUIRE(p->cu_seqlens_q != nullptr, "flash_attn_varlen: cu_seqlens_q is required");
  const bool paged = p->block_table != nullptr;
  if (paged) {
    FG_REQUIRE(p->seqused_k != nullptr, "seqused_k must be provided if block_table is provided");
    FG_REQUIRE(p->block_size > 0 && p->num_blocks > 0, "flash_attn_varlen: paged KV needs block_size and num_blocks");
  } else {
    FG_REQUIRE(p->cu_seqlens_k != nullptr, "cu_seqlens_k or seqused_k must be provided");
    FG_REQUIRE(p->total_k >= 0, "flash_attn_varlen: negative total_k");
  }
  auto al = [](const void* ptr) { return aligned16(ptr); };
  FG_REQUIRE(al(p->q) && al(p->k) && al(p->v) && al(p->out), "flash_attn_varlen: tensors must be 16-byte aligned");
  FG_REQUIRE(p->q_row_stride % 8 == 0 && p->q_head_stride % 8 == 0 && p->k_row_stride % 8 == 0 &&
                 p->k_head_stride % 8 == 0 && p->v_row_stride % 8 == 0 && p->v_head_stride % 8 == 0 &&
                 p->o_row_stride % 8 == 0 && p->o_head_stride % 8 == 0 &&
                 (!paged || (p->k_block_stride % 8 == 0 && p->v_block_stride % 8 == 0)),
             "flash_attn_varlen: strides must be multiples of 8 elements");
  FG_REQUIRE(p->max_seqlen_q >= 0 && p->max_seqlen_k >= 0, "flash_attn_varlen: negative max_seqlen");
  FG_REQUIRE(p->max_seqlen_q <= 2147483647LL / 64 && p->max_seqlen_k <= 2147483647LL / 64 &&
                 p->total_q <= 2147483647LL,
             "flash_attn_varlen: sequence too long");
  FG_REQUIRE(p->softcap >= 0.0, "flash_attn_varlen: softcap must be >= 0");

  AttnArgs a;
  a.q = p->q; a.k = p->k; a.v = p->v; a.out = p->out; a.lse = p->lse;
  a.cu_q = p->cu_seqlens_q; a.cu_k = p->cu_seqlens_k; a.seqused_k = p->seqused_k;
  a.block_table = p->block_table; a.alibi = p->alibi_slopes;
  a.q_rs = p->q_row_stride; a.q_hs = p->q_head_stride;
  a.k_rs = p->k_row_stride; a.k_hs = p->k_head_stride; a.k_bs = p->k_block_stride;
  a.v_rs = p->v_row_stride; a.v_hs = p->v_head_stride; a.v_bs = p->v_block_stride;
  a.o_rs = p->o_row_stride; a.o_hs = p->o_head_stride;
  a.bt_stride = p->block_table_stride; a.alibi_bs = p->alibi_batch_stride;
  a.total_q = p->total_q;
  a.total_k = p->total_k;
  a.q_batch = p->q_batch_stride; a.k_batch = p->k_batch_stride;
  a.v_batch = p->v_batch_stride; a.o_batch = p->o_batch_stride;
  a.batch_strided = (p->q_batch_stride | p->k_batch_stride | p->v_batch_stride | p->o_batch_stride) != 0;
  if (a.batch_strided) {
    FG_REQUIRE(p->q_batch_stride > 0 && p->k_batch_stride > 0 && p->v_batch_stride > 0 && p->o_batch_stride > 0,
               "flash_attn_varlen: give all four batch strides or none");
    FG_REQUIRE(p->q_batch_stride % 8 == 0 && p->k_batch_stride % 8 == 0 && p->v_batch_stride % 8 == 0 &&
                   p->o_batch_stride % 8 == 0,
               "flash_attn_varlen: batch strides must be multiples of 8 elements");
    if (paged || pick_path(p) != kPathPrefillSm100)
      return fail(FG_ERR_UNSUPPORTED,
                  "flash_attn_varlen: batch strides are taken by the tensor-core prefill kernel only (head dim 128, "
                  "contiguous K/V, no ALiBi / soft-cap / window, at least 64 query rows); pack the tensors instead");
  }
  a.batch = (int)p->batch; a.H = (int)p->num_heads; a.Hk = (int)p->num_heads_k;
  a.group = a.H / a.Hk; a.D = (int)p->head_dim;
  a.max_q = (int)p->max_seqlen_q; a.max_k = (int)p->max_seqlen_k;
  a.block_size = (int)p->block_size; a.num_blocks = (int)p->num_blocks;
  a.paged = paged;
  a.has_alibi = p->alibi_slopes != nullptr;
  // Single-token queries see every key: causal masking is a no-op there (the
  // reference drops it unless ALiBi needs the causal bias form).
  a.causal = p->causal != 0;
  if (p->max_seqlen_q == 1 && !a.has_alibi) a.causal = 0;
  int64_t wl = p->window_left, wr = p->window_right;
  if (a.causal) wr = 0;
  if (wl >= p->max_seqlen_k) wl = -1;
  if (wr >= p->max_seqlen_k) wr = -1;
  a.wl = (int)(wl < 0 ? -1 : wl);
  a.wr = (int)(wr < 0 ? -1 : wr);
  a.local = a.wl >= 0 || (!a.causal && a.wr >= 0);
  a.has_softcap = p->softcap > 0.0;
  const double LOG2E = 1.4426950408889634074;
  if (a.has_softcap) {
    a.scale = (float)p->softcap;
    a.softcap_pre = (float)(p->softmax_scale / p->softcap);
    a.scale_log2 = (float)(p->softcap * LOG2E);
  } else {
    a.scale = (float)p->softmax_scale;
    a.softcap_pre = 0.f;
    a.scale_log2 = (float)(p->softmax_scale * LOG2E);
  }
  a.num_splits = 1;
  a.ws_o = nullptr;
  a.ws_lse = nullptr;
  a.status = device_status_ptr();
  cudaStream_t st = (cudaStream_t)stream;

  const int path = pick_path(p);
  if (path == kPathDecode) {
    int chunk = 0, splits = 1;
    decode_split_plan(p->batch, p->num_heads_k, p->max_seqlen_k, p->num_splits, num_sms(), &chunk, &splits);
    if (splits > 1) {
      const int64_t need = (int64_t)splits * p->total_q * p->num_heads * (p->head_dim + 1) * 4;
      if (p->workspace == nullptr || p->workspace_bytes < need) {
        if (p->num_splits > 1)
          return fail(FG_ERR_INVALID, "flash_attn_varlen: %d splits need a workspace of %lld bytes", splits,
                      (long long)need);
        // No (or too small a) workspace: run unsplit.
        splits = 1;
        chunk = (int)((p->max_seqlen_k + 63) / 64 * 64);
        if (chunk < 64) chunk = 64;
      } else {
        a.ws_o = reinterpret_cast<float*>(p->workspace);
        a.ws_lse = a.ws_o + (int64_t)splits * p->total_q * p->num_heads * p->head_dim;
      }
    }
    a.num_splits = splits;
    return attn_decode(a, p->dtype, chunk, st);
  }
  if (path == kPathPrefillSm100) return attn_prefill_sm100(a, p->dtype, st);
  return attn_generic(a, p->dtype, st);
}
