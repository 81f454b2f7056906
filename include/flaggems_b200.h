/*
 * flaggems_b200 -- C ABI of the B200 (sm_100a) LLM-inference operator path.
 *
 * Every entry point takes plain device pointers, sizes and strides (strides are
 * in ELEMENTS, never bytes), a dtype code and the CUDA stream to launch on
 * (a cudaStream_t passed as void*; NULL is the legacy default stream).  Nothing
 * here allocates device memory unless stated otherwise and nothing synchronises the
 * stream: the call returns once the kernels are enqueued.  The device that owns the
 * pointers must be the current CUDA device of the calling thread.
 *
 * Return value: 0 on success, a negative FG_ERR_* code on failure.  After a
 * failure fg_last_error() returns a thread-local, human readable message; the
 * Python host layer raises it as RuntimeError, which is how the reference's
 * C++ wrappers report errors (TORCH_CHECK -> c10::Error).
 *
 * Each declaration cites the reference (FlagGems v3.0) interface it replaces, by
 * path inside the FlagGems source tree.
 */
#ifndef FLAGGEMS_B200_H_
#define FLAGGEMS_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FG_API __attribute__((visibility("default")))

/* dtype codes for floating-point tensors */
enum { FG_F32 = 0, FG_F16 = 1, FG_BF16 = 2 };

/* error codes */
enum {
  FG_OK = 0,
  FG_ERR_INVALID = -1,     /* bad argument (shape, stride, dtype, null pointer)   */
  FG_ERR_UNSUPPORTED = -2, /* valid in the reference, not implemented here        */
  FG_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed                   */
  FG_ERR_TOO_LARGE = -4,   /* size exceeds a documented limit of the entry point  */
  FG_ERR_DEVICE = -5       /* the device status word is set (see fg_device_status): nothing was launched */
};

/* ABI version of this header; bumped on any signature change. */
FG_API int fg_abi_version(void);
/* Message of the last failing call made by this thread ("" if none). */
FG_API const char* fg_last_error(void);
/* Number of kernels this library has launched since load (all threads). Used by
 * the benchmark to report how many of its own kernels ran in a timed region. */
FG_API int64_t fg_launch_count(void);
/* Persistent kernels (the tcgen05 GEMM) launch one CTA per SM and assume they get them
 * all.  When communication kernels run beside them (NCCL all-gather on another stream)
 * give the persistent kernels a smaller budget so that their CTAs are co-resident:
 * fg_set_num_sms(n) limits them to n SMs for the whole process (0 = all SMs).
 * No counterpart in the reference (it has no persistent kernels). */
FG_API int fg_set_num_sms(int sms);
FG_API int fg_get_num_sms(void);
/* Device status word of the current device: 0 when healthy, otherwise the code a
 * kernel stored when one of its bounded waits (mbarrier / TMEM hand-off) ran out of
 * time and it returned early (101 = GEMM, 102 = attention, 103 = the test hook below).
 * The kernel stores the code in device memory, where every later kernel with bounded waits
 * reads it and returns at once, and in a word of pinned host memory that each launching
 * entry point checks first, without synchronising: while the word is set every such entry
 * point returns FG_ERR_DEVICE and launches nothing, so a caller cannot consume output
 * buffers that a drained kernel left unwritten without being told.  (The first call that
 * needs the word on a device page-locks and maps that host word: make one call before
 * any stream capture.)  The reference has no such state: its kernels have no bounded waits.
 * fg_device_status synchronises with the device (a 4-byte read-back) and returns the code;
 * reset != 0 clears both words.  fg_device_status_nosync reads the host word only. */
FG_API int fg_device_status(int reset);
FG_API int fg_device_status_nosync(void);
/* Test hooks (no counterpart in the reference).  fg_debug_set_status stores `code` in both
 * status words of the current device as a kernel that gave up would (host word only when
 * there is no device).  fg_debug_wait_timeout enqueues one single-thread kernel that waits,
 * with the library's bounded wait and a limit of `limit_ns` (at most 100 ms), on an
 * mbarrier that nothing arrives at -- no copy or MMA is in flight -- and stores in
 * *outcome_dev (device int) 1 if the wait returned true, 2 if it gave up. */
FG_API int fg_debug_set_status(int code);
FG_API int fg_debug_wait_timeout(int64_t limit_ns, int* outcome_dev, void* stream);

/* Strided device-to-device copy of `rows` rows of `width_bytes` on `stream`
 * (cudaMemcpy2DAsync: DMA engines, no SM).  Source and destination may belong to different
 * GPUs when the destination is mapped into this process (peer access or symmetric memory).
 * The multi-GPU layer uses it to push a rank's column shard [M, N/G] into columns
 * [g N/G, (g+1) N/G) of every peer's row-major [M, N] result.  No counterpart in the
 * reference (it has no distributed code). */
FG_API int fg_copy_2d(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes,
                      int64_t width_bytes, int64_t rows, void* stream);

/* ------------------------------------------------------------------------
 * fused_add_rms_norm: residual += x ; x = rmsnorm(residual) * weight, in place.
 * Replaces flag_gems::fused_add_rms_norm (lib/fused_add_rms_norm.cpp:14-72) and
 * the Python op src/flag_gems/fused/fused_add_rms_norm.py:57-82.
 * x, residual: [M, N] with unit column stride and the given row strides.
 * The sum is kept in fp32; the variance uses the unrounded sum, residual
 * receives the sum rounded to `dtype`.
 * ---------------------------------------------------------------------- */
FG_API int fg_fused_add_rms_norm(void* x, void* residual, const void* weight,
                                 int64_t M, int64_t N, int64_t x_row_stride,
                                 int64_t r_row_stride, double eps, int dtype, void* stream);

/* rms_norm without residual: out = x * rsqrt(mean(x^2) + eps) * weight.
 * Replaces flag_gems::rms_norm (lib/rms_norm.cpp:15-72; Python
 * src/flag_gems/ops/rms_norm.py:221). out may alias x. */
FG_API int fg_rms_norm(const void* x, const void* weight, void* out, int64_t M, int64_t N,
                       int64_t x_row_stride, int64_t o_row_stride, double eps, int dtype,
                       void* stream);

/* ------------------------------------------------------------------------
 * silu_and_mul: out = silu(fp32(a)) * b, elementwise with broadcasting.
 * Replaces silu_and_mul / silu_and_mul_out
 * (src/flag_gems/fused/silu_and_mul.py:12-17,47-53).
 * All three tensors are described over the same `ndim` (<= 6) broadcast shape
 * `sizes`; a broadcast dimension has stride 0.  a, b and out share `dtype`.
 * ---------------------------------------------------------------------- */
FG_API int fg_silu_and_mul(const void* a, const void* b, void* out, int ndim,
                           const int64_t* sizes, const int64_t* a_strides,
                           const int64_t* b_strides, const int64_t* o_strides, int dtype,
                           void* stream);

/* ------------------------------------------------------------------------
 * gelu_and_mul: out = gelu(fp32(a)) * b with the exact (erf) form or, when
 * `approximate_tanh` is non-zero, the tanh form.  Replaces the forward of gelu_and_mul
 * (src/flag_gems/fused/gelu_and_mul.py:15-21,52-64,95-105); shapes and strides as for
 * fg_silu_and_mul.
 * ---------------------------------------------------------------------- */
FG_API int fg_gelu_and_mul(const void* a, const void* b, void* out, int ndim,
                           const int64_t* sizes, const int64_t* a_strides,
                           const int64_t* b_strides, const int64_t* o_strides, int approximate_tanh,
                           int dtype, void* stream);

/* ------------------------------------------------------------------------
 * reshape_and_cache: the same scatter into the vLLM v0 cache layout,
 *   key_cache   [num_blocks, num_heads, head_size / x, block_size, x]
 *   value_cache [num_blocks, num_heads, head_size, block_size]        (both contiguous).
 * Replaces reshape_and_cache (src/flag_gems/fused/reshape_and_cache.py:14-106).
 * key / value are [num_tokens, num_heads, head_size] with dense heads and the given
 * token strides (elements); slots < 0 or beyond the cache are skipped; bit-exact copy.
 * ---------------------------------------------------------------------- */
FG_API int fg_reshape_and_cache(const void* key, const void* value, void* key_cache, void* value_cache,
                                const int64_t* slot_mapping, int64_t num_tokens, int64_t num_heads,
                                int64_t head_size, int64_t block_size, int64_t num_blocks, int64_t x,
                                int64_t key_stride, int64_t value_stride, int elem_size, void* stream);

/* ------------------------------------------------------------------------
 * rotary_embedding: rotate q [T, Hq, D] and k [T, Hk, D] by cos/sin rows.
 * Replaces flag_gems::rotary_embedding / rotary_embedding_inplace
 * (lib/rotary_embedding.cpp:96-280) and apply_rotary_pos_emb
 * (src/flag_gems/fused/rotary_embedding.py:181-312).
 * q_out/k_out equal q/k for the in-place form.  cos, sin: [max_pos, D/2] with
 * unit column stride.  positions: int64 (pos_is_i64=1) or int32 token positions,
 * or NULL, in which case position = token % seq_len.  interleaved=0 is the
 * NeoX (half-split) layout, 1 the GPT-J (pairwise) layout.
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* q;
  const void* k;
  void* q_out;
  void* k_out;
  const void* cos;
  const void* sin;
  const void* positions;
  int64_t num_tokens, q_heads, k_heads, head_dim;
  int64_t q_stride_t, q_stride_h, q_stride_d;
  int64_t k_stride_t, k_stride_h, k_stride_d;
  int64_t qo_stride_t, qo_stride_h, qo_stride_d;
  int64_t ko_stride_t, ko_stride_h, ko_stride_d;
  int64_t pos_stride, cos_stride, sin_stride;
  int64_t seq_len;       /* used only when positions == NULL */
  int64_t max_positions; /* rows of cos/sin; positions are clamped into [0, max_positions) */
  int32_t pos_is_i64;
  int32_t interleaved;
  int32_t dtype;     /* dtype of q, k and the outputs */
  int32_t cos_dtype; /* dtype of cos and sin */
} fg_rope_params;
FG_API int fg_rotary_embedding(const fg_rope_params* p, void* stream);

/* ------------------------------------------------------------------------
 * reshape_and_cache_flash: scatter new K/V tokens into a paged cache.
 * Replaces flag_gems::reshape_and_cache_flash
 * (lib/reshape_and_cache_flash.cpp:11-67; Python
 * src/flag_gems/fused/reshape_and_cache_flash.py:61-112).
 * key/value: [T, H, D] (unit stride over D, head stride D, token stride given).
 * caches: [num_blocks, block_size, H, D] with the given block / page-row / head
 * strides.  slot_mapping: int64 [T]; a negative slot skips the token, and so does
 * a slot at or beyond num_blocks*block_size (the reference would write out of
 * bounds there).  A pure byte copy: `elem_size` is 1, 2 or 4 bytes.  Bit-exact.
 * ---------------------------------------------------------------------- */
FG_API int fg_reshape_and_cache_flash(const void* key, const void* value, void* key_cache,
                                      void* value_cache, const int64_t* slot_mapping,
                                      int64_t num_tokens, int64_t num_heads,
                                      int64_t head_size, int64_t block_size,
                                      int64_t num_blocks, int64_t key_stride,
                                      int64_t value_stride,
                                      int64_t cache_block_stride, int64_t cache_row_stride,
                                      int64_t cache_head_stride, int elem_size, void* stream);

/* ------------------------------------------------------------------------
 * gemm: C = alpha * A @ B (+ beta * bias), fp32 accumulation.
 * Replaces flag_gems::mm_tensor / mm_out_tensor (lib/mm.cpp:239-332), addmm /
 * addmm_out (lib/addmm.cpp:11-123) and the Python ops src/flag_gems/ops/mm.py:200-237,
 * src/flag_gems/ops/addmm.py:83-181.
 * A [M,K], B [K,N], C [M,N], bias broadcast to [M,N]; every tensor is given by
 * its two element strides so row-major, column-major and stride-0 (bias) forms
 * are all accepted.  bias == NULL means plain mm (alpha, beta ignored).
 * The epilogue is evaluated in fp32 and rounded once to the dtype of C.
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* a;
  const void* b;
  const void* bias;
  void* c;
  int64_t M, N, K;
  int64_t a_stride0, a_stride1;
  int64_t b_stride0, b_stride1;
  int64_t bias_stride0, bias_stride1;
  int64_t c_stride0, c_stride1;
  double alpha, beta;
  int32_t dtype; /* dtype of A, B, bias and C */
  int32_t reserved;
} fg_gemm_params;
FG_API int fg_gemm(const fg_gemm_params* p, void* stream);

/* `batch` independent problems of the shape in `p` (bmm): problem i reads a + i * a_batch_stride,
 * b + i * b_batch_stride, bias + i * bias_batch_stride and writes c + i * c_batch_stride (elements).
 * Replaces bmm (src/flag_gems/ops/bmm.py:23-136).  One launch of the tensor-core kernel when the
 * shape qualifies and the batch strides are multiples of 8 elements. */
FG_API int fg_gemm_batched(const fg_gemm_params* p, int64_t batch, int64_t a_batch_stride,
                           int64_t b_batch_stride, int64_t c_batch_stride, int64_t bias_batch_stride,
                           void* stream);
/* fp32 problems on the tensor cores, never TF32 (the reference multiplies fp32 with
 * allow_tf32=False, src/flag_gems/ops/mm.py:100-107, src/flag_gems/ops/addmm.py:60-66): each operand is
 * written into `workspace` as three bf16 pieces that add up to it exactly, six piece products are
 * accumulated by tcgen05.mma in short K chunks, and the chunks are added in fp32 with round to
 * nearest.  Error against fp64 is at or below that of an fp32 FMA loop.  If an input holds an
 * infinity or a NaN the CUDA-core kernel computes the result instead (decided on the device, no
 * host synchronisation), so special values propagate as in fp32 arithmetic.
 * fg_gemm_f32_split_workspace_bytes: bytes of scratch the call needs, or 0 when the problem does
 * not qualify (dtype other than fp32, a dimension below 128, M*N*K below 2^29, an operand without
 * a unit stride, c_stride1 != 1) and fg_gemm should be called.  Pure host logic.
 * fg_gemm_f32_split: `workspace` is device memory, 256-byte aligned, of at least that many bytes,
 * owned by the call until the work queued on `stream` has run.  FG_ERR_UNSUPPORTED when the
 * problem does not qualify. */
FG_API int64_t fg_gemm_f32_split_workspace_bytes(const fg_gemm_params* p);
FG_API int fg_gemm_f32_split(const fg_gemm_params* p, void* workspace, int64_t workspace_bytes, void* stream);
/* 1 if fg_gemm would take the tcgen05/TMA path for these arguments, 0 if the
 * generic path.  Pure host logic (no CUDA call). */
FG_API int fg_gemm_uses_tcgen05(const fg_gemm_params* p);

/* How the tcgen05 kernel would cut the problem up on `num_sms` SMs (pure host logic, no CUDA
 * call; FG_ERR_UNSUPPORTED when the generic kernel takes the problem).  The output is
 * tiles_m x tiles_n tiles of tile_m x tile_n per batch member; the persistent grid walks
 * num_units work units round-robin: units [0, full_units) are whole tiles (unit = tile index,
 * batch-major, then grouped: group_m row tiles share a sweep over the column tiles), each later
 * pair of units is the upper and lower 128-row half of one of the remaining tiles. */
typedef struct {
  int32_t tile_m, tile_n, grid, group_m;
  int64_t tiles_m, tiles_n, full_units, num_units;
} fg_gemm_plan;
FG_API int fg_gemm_tile_plan(const fg_gemm_params* p, int64_t batch, int num_sms, fg_gemm_plan* plan);

/* ------------------------------------------------------------------------
 * flash_attn_varlen: FlashAttention-2 style forward over variable-length
 * sequences with a paged or contiguous KV store.
 * Replaces flag_gems::flash_attn_varlen_func (lib/flash_attn_varlen_func.cpp:14-578)
 * and mha_varlan_fwd (src/flag_gems/ops/flash_api.py:230-569); the fields follow
 * FlashFwdParams (include/flag_gems/operators.h:126-194).
 *
 * q, out: [total_q, Hq, D].  Paged form (block_table != NULL): k, v are
 * [num_blocks, block_size, Hk, D] and k_len[b] = seqused_k[b].  Contiguous form
 * (block_table == NULL): k, v are [total_k, Hk, D] and sequence b owns rows
 * cu_seqlens_k[b] .. cu_seqlens_k[b+1]; seqused_k, when given, shortens it.
 * The causal mask is aligned to the bottom-right corner: key j is visible to
 * query i iff j <= i + k_len - q_len.  Rows with no visible key produce 0 and
 * an LSE of +inf.  lse (optional) is fp32 [Hq, total_q].
 *
 * workspace: device scratch for split-KV decode, at least
 * fg_flash_attn_workspace_bytes(...) bytes, or NULL to forbid splitting.
 * The tensor-core prefill kernel draws its work items from one of 1024 per-device ticket counters,
 * taken round-robin per launch: keep fewer than 1024 prefill launches in flight per device.
 * ---------------------------------------------------------------------- */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse; /* may be NULL */
  const int32_t* cu_seqlens_q;  /* [batch+1] */
  const int32_t* cu_seqlens_k;  /* [batch+1] or NULL */
  const int32_t* seqused_k;     /* [batch] or NULL */
  const int32_t* block_table;   /* [batch, max_blocks_per_seq] or NULL */
  const float* alibi_slopes;    /* [Hq] or [batch, Hq] or NULL */
  void* workspace;
  int64_t workspace_bytes;
  int64_t q_row_stride, q_head_stride;
  int64_t k_row_stride, k_head_stride, k_block_stride;
  int64_t v_row_stride, v_head_stride, v_block_stride;
  int64_t o_row_stride, o_head_stride;
  int64_t block_table_stride;
  int64_t alibi_batch_stride;
  int64_t total_q, batch, num_heads, num_heads_k, head_dim;
  int64_t max_seqlen_q, max_seqlen_k;
  int64_t block_size, num_blocks;
  int64_t window_left, window_right; /* -1 = unbounded */
  int64_t total_k;                   /* rows of k/v in the contiguous form (0 when paged) */
  /* Batch-strided dense form, all four zero (the packed form) or all four set: batch member b's rows
   * start b * *_batch_stride elements into q / k / v / out instead of at row cu_seqlens[b], and row i
   * of the member is i * *_row_stride further on; cu_seqlens_q / cu_seqlens_k still give the lengths
   * (and the lse columns).  For dense batches whose batch and sequence dimensions do not pack into
   * one row dimension, such as the (batch, seq, heads, dim) view of a (batch, heads, seq, dim) tensor
   * that scaled_dot_product_attention passes to aten::_flash_attention_forward (the reference kernel
   * takes batch strides there, src/flag_gems/ops/flash_api.py:572-916).  Contiguous K/V only, and
   * only where the tensor-core prefill kernel applies (fg_flash_attn_path == 1), else
   * FG_ERR_UNSUPPORTED. */
  int64_t q_batch_stride, k_batch_stride, v_batch_stride, o_batch_stride;
  double softmax_scale;
  double softcap; /* 0 = off */
  int32_t causal;
  int32_t dtype; /* FG_F16 or FG_BF16 */
  int32_t num_splits; /* 0 = choose, 1 = never split, >1 = force */
  int32_t reserved;
} fg_attn_params;
FG_API int fg_flash_attn_varlen(const fg_attn_params* p, void* stream);
FG_API int64_t fg_flash_attn_workspace_bytes(int64_t batch, int64_t num_heads,
                                             int64_t head_dim, int64_t max_seqlen_q,
                                             int64_t max_seqlen_k);
/* Which kernel family fg_flash_attn_varlen would pick: 0 generic (mma.sync),
 * 1 tcgen05 prefill, 2 split-KV decode.  Pure host logic. */
FG_API int fg_flash_attn_path(const fg_attn_params* p);

/* ------------------------------------------------------------------------
 * flash_attn_decode_static: single-token (decode) attention that allocates nothing.
 * No counterpart in the reference.
 *
 * Same arguments and result as fg_flash_attn_varlen for a decode batch (one query
 * token per sequence, no ALiBi, no window, at most 16 query heads per KV head), but the
 * scratch for the split-KV partial results is a fixed array inside the library image
 * (fg_flash_attn_decode_static_capacity() bytes, 64 MiB, resident on every GPU that
 * loads the library) instead of `workspace`, which is ignored.  It exists for callers
 * that cannot allocate device memory at call time: runtimes that gave all free memory
 * to their KV-cache pool at start-up, hosts that bind this ABI without an allocator of
 * their own, and decode loops that must not hit the device-wide synchronisation of
 * cudaMalloc/cudaFree.  The call itself performs no cudaMalloc, cudaFree or other
 * allocating library call.
 *
 * Limits and rules:
 *  - a batch whose chunk plan needs more than the capacity is rejected with
 *    FG_ERR_TOO_LARGE (need = chunks * batch * num_heads * (head_dim + 1) * 4 bytes, with
 *    chunks = ceil(max_seqlen_k / chunk) and chunk between 256 and 1024 tokens);
 *  - the first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and keeps it; make that call before
 *    any stream capture;
 *  - the array is part of the library's device code image, which CUDA loads onto a device at the
 *    first call into the library there (lazy module loading), not at dlopen: a runtime that hands
 *    all free device memory to its own pool must make one call into this library on every
 *    device (any fg_* entry that launches a kernel or resolves a symbol, e.g.
 *    fg_device_status(0)) BEFORE it does so, or that first call can fail for lack of the 64 MiB;
 *  - all calls on a device share the one array, which keeps whatever the last call
 *    left in it.  Nothing in it has to start at zero (every slot that is read was
 *    written by the same call), but two calls that may run at the same time on one GPU
 *    (different streams) would overwrite each other's partial results: serialise them.
 * ---------------------------------------------------------------------- */
FG_API int fg_flash_attn_decode_static(const fg_attn_params* p, void* stream);
FG_API int64_t fg_flash_attn_decode_static_capacity(void);

/* ------------------------------------------------------------------------
 * get_scheduler_metadata: split-KV scheduling vector of a FlashAttention-3 style
 * decode.  Replaces get_scheduler_metadata
 * (src/flag_gems/ops/get_scheduler_metadata.py:567-894; bound by vLLM as
 * _vllm_fa3_C.get_scheduler_metadata, src/flag_gems/patches/patch_vllm_all.py:279-368)
 * for compute capability >= 9.0; older parts return FG_ERR_UNSUPPORTED.
 *
 * fg_scheduler_plan is host arithmetic only (no CUDA call): the normalised mask kind,
 * the pack-GQA choice, the static split count and the tile (block_m x block_n) the
 * per-sequence block counts are taken in.  metadata_len = 1 + batch_size for batches
 * of at most 992 sequences, else 1.
 * fg_get_scheduler_metadata enqueues ONE kernel on `stream` that writes
 *   metadata[0] = 0 (work-queue semaphore), metadata[1 + b] = KV splits of sequence b
 * into `metadata` (device, metadata_len int32).  No host synchronisation (the reference
 * reads the block total back between its two kernels).  Integer result, identical to
 * the reference's.
 *   page_size 0 = no page table; pack_gqa -1 = decide by heuristic; num_splits <= 0 =
 *   decide by heuristic; arch = 10 * major + minor; num_sm = SMs of the device.
 *   cu_seqlens_k is accepted for signature parity and not read (nor does the reference).
 * ---------------------------------------------------------------------- */
typedef struct {
  int32_t batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k, headdim, headdim_v;
  int32_t elem_size;        /* bytes per q/k/v element: 2 */
  int32_t page_size, max_seqlen_k_new, is_causal, window_size_left, window_size_right;
  int32_t has_softcap, num_splits, pack_gqa, sm_margin, arch, num_sm;
  int32_t varlen_q, has_leftpad; /* for fg_scheduler_plan without device pointers */
  const int32_t* seqused_k;        /* [batch] device, required by fg_get_scheduler_metadata */
  const int32_t* cu_seqlens_q;     /* [batch + 1] or NULL */
  const int32_t* cu_seqlens_k;     /* unused */
  const int32_t* cu_seqlens_k_new; /* [batch + 1] or NULL */
  const int32_t* seqused_q;        /* [batch] or NULL */
  const int32_t* leftpad_k;        /* [batch] or NULL */
} FgSchedulerParams;

typedef struct {
  int32_t num_splits, pack_gqa, block_m, block_n, use_dynamic_split, is_causal, is_local;
  int32_t q_per_kv, heads, metadata_len;
} FgSchedulerPlan;

FG_API int fg_scheduler_plan(const FgSchedulerParams* p, FgSchedulerPlan* plan);
FG_API int fg_get_scheduler_metadata(const FgSchedulerParams* p, int32_t* metadata, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLAGGEMS_B200_H_ */
