// Shared definitions of the attention kernels: the flat argument block (the
// analogue of FlashFwdParams) and the score post-processing shared by all paths.
#pragma once
#include "common.cuh"

namespace fg {

struct AttnArgs {
  const void *q, *k, *v;
  void* out;
  float* lse;
  const int32_t *cu_q, *cu_k, *seqused_k, *block_table;
  const float* alibi;
  int64_t q_rs, q_hs, k_rs, k_hs, k_bs, v_rs, v_hs, v_bs, o_rs, o_hs;
  int64_t bt_stride, alibi_bs;
  int64_t total_q, total_k;
  // batch-strided dense form (tensor-core prefill kernel only): member b's rows start b * *_batch
  // elements into the tensor instead of at row cu_seqlens[b]
  int64_t q_batch, k_batch, v_batch, o_batch;
  int batch_strided;
  int batch, H, Hk, group, D;
  int max_q, max_k, block_size, num_blocks;
  int wl, wr;         // window, -1 = unbounded (wr == 0 when causal)
  int causal, local, has_alibi, has_softcap, paged;
  float scale;        // softmax scale applied to q.k (== softcap when capping)
  float scale_log2;   // scale * log2(e)
  float softcap_pre;  // scale / softcap : S = tanh(S * softcap_pre) before `scale`
  // split-KV (decode)
  int num_splits;
  float* ws_o;        // [splits, total_q, H, D] fp32 partial outputs
  float* ws_lse;      // [splits, H, total_q] fp32 partial log-sum-exp (base 2 domain)
  int* status;
};

// Sequence geometry of batch element b.
struct SeqInfo {
  int q_begin, q_len, k_begin, k_len;
};
__device__ __forceinline__ SeqInfo seq_info(const AttnArgs& a, int b) {
  SeqInfo s;
  s.q_begin = a.cu_q[b];
  s.q_len = a.cu_q[b + 1] - s.q_begin;
  if (a.paged) {
    s.k_begin = 0;
    s.k_len = a.seqused_k[b];
  } else {
    s.k_begin = a.cu_k[b];
    s.k_len = a.cu_k[b + 1] - s.k_begin;
    if (a.seqused_k) s.k_len = min(s.k_len, a.seqused_k[b]);
  }
  if (s.k_len < 0) s.k_len = 0;
  if (s.q_len < 0) s.q_len = 0;
  return s;
}

// Row address (in elements) of key/value token `tok` of the current sequence.
// Paged: page = block_table[b][tok / block_size] (clamped into the cache so a bad
// table entry cannot fault), row inside the page = tok % block_size.
__device__ __forceinline__ int64_t kv_row_offset(const AttnArgs& a, const int32_t* bt_row, int k_begin, int tok,
                                                 int64_t rs, int64_t bs) {
  if (a.paged) {
    const int pg = tok / a.block_size;
    int page = bt_row[pg];
    page = max(0, min(page, a.num_blocks - 1));
    return (int64_t)page * bs + (int64_t)(tok - pg * a.block_size) * rs;
  }
  return (int64_t)(k_begin + tok) * rs;
}

}  // namespace fg
