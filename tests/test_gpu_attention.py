"""GPU parity: flash_attn_varlen_func (paged prefill, paged decode, contiguous varlen)
against the CPU oracle evaluated in fp32.

The parameter grids follow FlagGems' tests/test_attention_ops.py:886-1085 (sequence
mixes, head ratios, head sizes 128/192/256, ALiBi, soft-cap, fp16/bf16) with the
reference's tolerance atol=2e-2, rtol=1e-2; further cases cover the contiguous form,
sliding windows, empty rows, split-KV decode and the benchmark configurations."""
import ctypes

import pytest
import torch

from flaggems_b200 import _lib, workloads
from oracle import reference_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
ATOL, RTOL = 2e-2, 1e-2


def _oracle(q, kc, vc, qlens, klens, bt, scale, **kw):
    return O.paged_attention(q.cpu(), kc.cpu(), vc.cpu(), qlens, klens, bt.cpu(), scale,
                             compute_dtype=torch.float32, **kw)


def _make(seq_lens, num_heads, head_size, block_size, num_blocks, dtype, seed=1234567890):
    torch.manual_seed(seed)
    qlens = [x[0] for x in seq_lens]
    klens = [x[1] for x in seq_lens]
    hq, hk = num_heads
    q = torch.randn(sum(qlens), hq, head_size, dtype=dtype, device=DEV)
    kc = torch.randn(num_blocks, block_size, hk, head_size, dtype=dtype, device=DEV)
    vc = torch.randn_like(kc)
    cu = torch.tensor([0] + qlens, dtype=torch.int32).cumsum(0, dtype=torch.int32).to(DEV)
    used = torch.tensor(klens, dtype=torch.int32, device=DEV)
    maxb = (max(klens) + block_size - 1) // block_size
    bt = torch.randint(0, num_blocks, (len(seq_lens), maxb), dtype=torch.int32, device=DEV)
    return q, kc, vc, cu, used, bt, qlens, klens


@pytest.mark.parametrize("seq_lens", [[(1, 1328), (5, 18), (129, 463)]])
@pytest.mark.parametrize("num_heads", [(4, 4), (8, 2), (16, 2)])
@pytest.mark.parametrize("head_size", [128, 192, 256])
@pytest.mark.parametrize("block_size", [32])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("alibi", [False, True])
@pytest.mark.parametrize("soft_cap", [None, 10.0, 50.0])
@pytest.mark.parametrize("num_blocks", [2048])
def test_flash_attn_varlen_func(fg, seq_lens, num_heads, head_size, block_size, dtype, alibi, soft_cap, num_blocks):
    if alibi and soft_cap is not None:
        pytest.skip("combination excluded by the reference test (numerical stability)")
    q, kc, vc, cu, used, bt, qlens, klens = _make(seq_lens, num_heads, head_size, block_size, num_blocks, dtype)
    scale = head_size ** -0.5
    slopes = bias = None
    if alibi:
        slopes = torch.ones(len(seq_lens), num_heads[0], dtype=torch.float32, device=DEV) * 0.3
        bias = O.alibi_bias(slopes.cpu(), max(qlens), max(klens), causal=True)
    out = fg.flash_attn_varlen_func(
        q=q, k=kc, v=vc, cu_seqlens_q=cu, seqused_k=used, max_seqlen_q=max(qlens), max_seqlen_k=max(klens),
        softmax_scale=scale, causal=True, window_size=(-1, -1), block_table=bt,
        softcap=soft_cap if soft_cap is not None else 0, alibi_slopes=slopes, fa_version=2)
    ref = _oracle(q, kc, vc, qlens, klens, bt, scale, attn_bias=bias, soft_cap=soft_cap)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("seq_lens", [[(1, 1328), (1, 18), (1, 463)]])
@pytest.mark.parametrize("num_heads", [(8, 2), (32, 8), (4, 4)])
@pytest.mark.parametrize("head_size", [128, 64, 256])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("soft_cap", [None, 10.0])
def test_flash_attn_varlen_func_decode(fg, seq_lens, num_heads, head_size, dtype, soft_cap):
    q, kc, vc, cu, used, bt, qlens, klens = _make(seq_lens, num_heads, head_size, 32, 2048, dtype)
    scale = head_size ** -0.5
    out, lse = fg.flash_attn_varlen_func(
        q=q, k=kc, v=vc, cu_seqlens_q=cu, seqused_k=used, max_seqlen_q=1, max_seqlen_k=max(klens),
        softmax_scale=scale, causal=True, window_size=(-1, -1), block_table=bt,
        softcap=soft_cap if soft_cap is not None else 0, fa_version=2, return_softmax_lse=True)
    ref = _oracle(q, kc, vc, qlens, klens, bt, scale, soft_cap=soft_cap)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    assert lse.shape == (num_heads[0], len(seq_lens)) and torch.isfinite(lse).all()


def _params_for(q, kc, vc, cu, used, bt, max_q, max_k):
    p = _lib.AttnParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), q.data_ptr()
    p.cu_seqlens_q, p.seqused_k, p.block_table = cu.data_ptr(), used.data_ptr(), bt.data_ptr()
    p.total_q, p.batch, p.num_heads, p.head_dim = q.shape[0], cu.numel() - 1, q.shape[1], q.shape[2]
    p.num_heads_k = kc.shape[2]
    p.max_seqlen_q, p.max_seqlen_k = max_q, max_k
    p.block_size, p.num_blocks = kc.shape[1], kc.shape[0]
    p.window_left = p.window_right = -1
    p.softmax_scale = float(q.shape[2]) ** -0.5
    p.causal, p.dtype = 1, _lib.dtype_code(q.dtype)
    return p


def test_decode_takes_the_split_kv_path_and_lse_is_right(fg):
    seq_lens = [(1, 5000), (1, 64), (1, 1), (1, 777)]
    q, kc, vc, cu, used, bt, qlens, klens = _make(seq_lens, (32, 8), 128, 16, 4096, torch.bfloat16)
    assert _lib.load().fg_flash_attn_path(ctypes.byref(_params_for(q, kc, vc, cu, used, bt, 1, 5000))) == 2
    scale = 128 ** -0.5
    out, lse = fg.flash_attn_varlen_func(q, kc, vc, 1, cu, 5000, seqused_k=used, softmax_scale=scale, causal=True,
                                         block_table=bt, return_softmax_lse=True)
    ref = _oracle(q, kc, vc, qlens, klens, bt, scale)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    # lse[h, t] = logsumexp_j(scale * q.k)
    for i, (kl, row) in enumerate(zip(klens, bt.cpu())):
        nb = (kl + 15) // 16
        k = kc[row[:nb].long().to(DEV)].reshape(-1, 8, 128)[:kl].float().repeat_interleave(4, dim=1)
        s = torch.einsum("hd,khd->hk", q[i].float(), k) * scale
        torch.testing.assert_close(lse[:, i].cpu(), torch.logsumexp(s, dim=-1).cpu(), atol=2e-3, rtol=2e-3)


def test_contiguous_varlen_windows_and_empty_rows(fg):
    b = workloads.prefill_batch(seed=7, num_seqs=5, min_len=1, max_len=300, q_heads=8, kv_heads=2, head_dim=128,
                                block_size=16, dtype=torch.float16, device=DEV)
    ref = _oracle(b.q, b.key_cache, b.value_cache, b.query_lens, b.kv_lens, b.block_table, b.scale)
    paged = fg.flash_attn_varlen_func(b.q, b.key_cache, b.value_cache, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                      seqused_k=b.seqused_k, causal=True, block_table=b.block_table)
    contig = fg.flash_attn_varlen_func(b.q, b.k, b.v, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                       cu_seqlens_k=b.cu_seqlens_k, causal=True)
    torch.testing.assert_close(paged.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    torch.testing.assert_close(contig.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    # sliding window (left) with causal
    win = fg.flash_attn_varlen_func(b.q, b.key_cache, b.value_cache, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                    seqused_k=b.seqused_k, causal=True, window_size=(37, 0), block_table=b.block_table)
    refw = _oracle(b.q, b.key_cache, b.value_cache, b.query_lens, b.kv_lens, b.block_table, b.scale,
                   sliding_window=37 + 1)
    # oracle's sliding_window counts the diagonal: window_left = sliding_window - 1
    torch.testing.assert_close(win.cpu().float(), refw.float(), atol=ATOL, rtol=RTOL)
    # non-causal
    nc = fg.flash_attn_varlen_func(b.q, b.key_cache, b.value_cache, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                   seqused_k=b.seqused_k, causal=False, block_table=b.block_table)
    refn = _oracle(b.q, b.key_cache, b.value_cache, b.query_lens, b.kv_lens, b.block_table, b.scale, causal=False)
    torch.testing.assert_close(nc.cpu().float(), refn.float(), atol=ATOL, rtol=RTOL)
    # q longer than k: the first q_len - k_len rows see no key -> zeros, lse = +inf
    seq_lens = [(70, 20), (3, 3)]
    q, kc, vc, cu, used, bt, qlens, klens = _make(seq_lens, (4, 2), 64, 16, 64, torch.bfloat16)
    out, lse = fg.flash_attn_varlen_func(q, kc, vc, 70, cu, 20, seqused_k=used, causal=True, block_table=bt,
                                         return_softmax_lse=True)
    ref = _oracle(q, kc, vc, qlens, klens, bt, 64 ** -0.5)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    assert not out[:50].any() and torch.isinf(lse[:, :50]).all() and torch.isfinite(lse[:, 50:]).all()


def test_golden_paged_attention_and_custom_op(fg, golden_dir):
    for c in torch.load(golden_dir / "golden_paged_attn.pt", weights_only=False):
        q, kc, vc = c["q"].to(DEV), c["key_cache"].to(DEV), c["value_cache"].to(DEV)
        cu = torch.tensor([0] + c["query_lens"], dtype=torch.int32).cumsum(0, dtype=torch.int32).to(DEV)
        used = torch.tensor(c["kv_lens"], dtype=torch.int32, device=DEV)
        slopes = None if c["alibi_slopes"] is None else c["alibi_slopes"].to(DEV)
        out, lse = torch.ops.flag_gems.flash_attn_varlen_func(
            q, kc, vc, max(c["query_lens"]), cu, max(c["kv_lens"]), None, used, None, 0.0, c["scale"], True, None,
            c["soft_cap"] or 0.0, slopes, False, False, c["block_tables"].to(DEV), False, None)
        torch.testing.assert_close(out.cpu().float(), c["out"].float(), atol=ATOL, rtol=RTOL, msg=c["name"])


def test_argument_errors(fg):
    q, kc, vc, cu, used, bt, qlens, klens = _make([(4, 40)], (4, 2), 64, 16, 16, torch.bfloat16)
    with pytest.raises(AssertionError, match="cu_seqlens_k or seqused_k"):
        fg.flash_attn_varlen_func(q, kc, vc, 4, cu, 40, block_table=bt)
    with pytest.raises(RuntimeError, match="Only FA2"):
        fg.flash_attn_varlen_func(q, kc, vc, 4, cu, 40, seqused_k=used, block_table=bt, fa_version=3)
    with pytest.raises(RuntimeError, match="num_splits"):
        fg.flash_attn_varlen_func(q, kc, vc, 4, cu, 40, seqused_k=used, block_table=bt, num_splits=2)
    with pytest.raises(AssertionError):
        fg.flash_attn_varlen_func(q.float(), kc.float(), vc.float(), 4, cu, 40, seqused_k=used, block_table=bt)
    # max_seqlen given as tensors is accepted (one host sync, as in the reference)
    out = fg.flash_attn_varlen_func(q, kc, vc, torch.tensor(4), cu, torch.tensor(40), seqused_k=used, causal=True,
                                    block_table=bt)
    ref = _oracle(q, kc, vc, qlens, klens, bt, 64 ** -0.5)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)


def test_prefill_config3_reduced_and_out_argument(fg):
    # config-3 structure (16 seqs, 32/8 heads, d 128, bf16) at lengths the CPU oracle handles
    b = workloads.prefill_batch(seed=11, num_seqs=16, min_len=16, max_len=400, device=DEV)
    ref = _oracle(b.q, b.key_cache, b.value_cache, b.query_lens, b.kv_lens, b.block_table, b.scale)
    out = torch.empty_like(b.q)
    ret = fg.flash_attn_varlen_func(b.q, b.key_cache, b.value_cache, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                    seqused_k=b.seqused_k, causal=True, block_table=b.block_table, out=out)
    assert ret is out
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    contig = fg.flash_attn_varlen_func(b.q, b.k, b.v, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                       cu_seqlens_k=b.cu_seqlens_k, causal=True)
    torch.testing.assert_close(contig.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)


def test_prefill_config3_full_size_properties(fg):
    # Full config 3 (lengths up to 4096): oracle on the two shortest sequences, plus
    # size-independent properties: paged == contiguous, and softmax rows are convex
    # combinations (|out| <= max |v| per head-dim column).
    b = workloads.prefill_batch(seed=0, device=DEV)
    paged = fg.flash_attn_varlen_func(b.q, b.key_cache, b.value_cache, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                      seqused_k=b.seqused_k, causal=True, block_table=b.block_table)
    contig = fg.flash_attn_varlen_func(b.q, b.k, b.v, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                       cu_seqlens_k=b.cu_seqlens_k, causal=True)
    torch.testing.assert_close(paged.float(), contig.float(), atol=ATOL, rtol=RTOL)
    assert torch.isfinite(paged).all()
    assert paged.float().abs().max() <= b.v.float().abs().max() + 1e-2
    cu = b.cu_seqlens_q.cpu().tolist()
    order = sorted(range(len(b.query_lens)), key=lambda i: b.query_lens[i])[:2]
    for i in order:
        sl = slice(cu[i], cu[i + 1])
        ref = O.varlen_attention(b.q[sl].cpu(), b.k[sl].cpu(), b.v[sl].cpu(),
                                 torch.tensor([0, cu[i + 1] - cu[i]]), torch.tensor([0, cu[i + 1] - cu[i]]), b.scale,
                                 compute_dtype=torch.float32)
        torch.testing.assert_close(paged[sl].cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    # the first token of every sequence attends only to itself: out == v (per KV group)
    first = b.cu_seqlens_q[:-1].long()
    torch.testing.assert_close(paged[first].float(), b.v[first].repeat_interleave(4, dim=1).float(), atol=1e-2, rtol=1e-2)


def test_prefill_full_size_is_deterministic(fg):
    # The kernel has no atomics and a fixed reduction order: repeated launches on the same
    # inputs must agree bit for bit.  A difference means a missed wait between the tensor
    # pipe and the softmax warps (one was caught this way: 32-row blocks read before the last
    # PV had landed).
    b = workloads.prefill_batch(seed=0, device=DEV)

    def paged():
        return fg.flash_attn_varlen_func(b.q, b.key_cache, b.value_cache, b.max_seqlen_q, b.cu_seqlens_q,
                                         b.max_seqlen_k, seqused_k=b.seqused_k, causal=True, block_table=b.block_table)

    def contig():
        return fg.flash_attn_varlen_func(b.q, b.k, b.v, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                         cu_seqlens_k=b.cu_seqlens_k, causal=True)

    for f in (paged, contig):
        ref = f().clone()
        for _ in range(10):
            assert torch.equal(f(), ref)
    assert torch.equal(paged(), contig())


def test_decode_config4_reduced_with_cache_write(fg):
    # config-4 structure: write the new token with reshape_and_cache_flash, then decode
    b = workloads.decode_batch(seed=5, batch=24, min_ctx=30, max_ctx=2100, device=DEV)
    fg.reshape_and_cache_flash(b.new_key, b.new_value, b.key_cache, b.value_cache, b.slot_mapping, "auto", None, None)
    kc_ref, vc_ref = b.key_cache.cpu().clone(), b.value_cache.cpu().clone()
    out = fg.flash_attn_varlen_func(b.q, b.key_cache, b.value_cache, 1, b.cu_seqlens_q, b.max_seqlen_k,
                                    seqused_k=b.seqused_k, causal=True, block_table=b.block_table)
    ref = O.paged_attention(b.q.cpu(), kc_ref, vc_ref, b.query_lens, b.kv_lens, b.block_table.cpu(), b.scale,
                            compute_dtype=torch.float32)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    # the last key of each context is the token just written
    last = b.slot_mapping
    assert torch.equal(b.key_cache.view(-1, 8, 128)[last], b.new_key)


@pytest.mark.parametrize("block_size", [8, 16, 64, 128, 256])
@pytest.mark.parametrize("num_heads", [(8, 2), (4, 4), (6, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [True, False])
def test_prefill_tcgen05_path(fg, block_size, num_heads, dtype, causal):
    # q_len == k_len, q_len < k_len (chunked prefill) and q_len > k_len (rows without keys),
    # lengths straddling the 128-row tiles
    seq_lens = [(300, 300), (128, 129), (65, 700), (200, 90), (257, 1024)]
    num_blocks = max(64, 4096 // block_size)
    q, kc, vc, cu, used, bt, qlens, klens = _make(seq_lens, num_heads, 128, block_size, num_blocks, dtype, seed=3)
    assert _lib.load().fg_flash_attn_path(ctypes.byref(_params_for(q, kc, vc, cu, used, bt, 300, 1024))) == 1
    # poison the cache rows past each sequence end in its last page: they must not leak
    out, lse = fg.flash_attn_varlen_func(q, kc, vc, max(qlens), cu, max(klens), seqused_k=used, causal=causal,
                                         block_table=bt, return_softmax_lse=True)
    ref = _oracle(q, kc, vc, qlens, klens, bt, 128 ** -0.5, causal=causal)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    assert torch.isfinite(out).all()


def test_prefill_tcgen05_ignores_garbage_past_sequence_end(fg):
    # a cache whose unused slots hold NaN / Inf (torch.empty caches do): results unchanged
    b = workloads.prefill_batch(seed=21, num_seqs=3, min_len=130, max_len=500, q_heads=8, kv_heads=2, device=DEV)
    clean = fg.flash_attn_varlen_func(b.q, b.key_cache, b.value_cache, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                      seqused_k=b.seqused_k, causal=True, block_table=b.block_table)
    kc, vc = b.key_cache.clone(), b.value_cache.clone()
    for i, n in enumerate(b.kv_lens):
        if n % 16:
            page = int(b.block_table[i, (n - 1) // 16])
            kc[page, n % 16:] = float("nan")
            vc[page, n % 16:] = float("inf")
    dirty = fg.flash_attn_varlen_func(b.q, kc, vc, b.max_seqlen_q, b.cu_seqlens_q, b.max_seqlen_k,
                                      seqused_k=b.seqused_k, causal=True, block_table=b.block_table)
    assert torch.equal(clean, dirty)


@pytest.mark.parametrize("block_size", [8, 16, 24, 48, 64, 128, 256])
@pytest.mark.parametrize("head_size", [64, 96, 128, 192])
def test_decode_block_sizes_and_head_dims(fg, block_size, head_size):
    # power-of-two pages take the TMA-fed kernel, the others the cp.async kernel; head dims
    # that are not multiples of 64 rely on TMA zero fill of the last 64-column box
    seq_lens = [(1, 700), (1, 64), (1, 3), (1, 1025)]
    q, kc, vc, cu, used, bt, qlens, klens = _make(seq_lens, (8, 2), head_size, block_size, 300, torch.bfloat16, seed=5)
    out = fg.flash_attn_varlen_func(q, kc, vc, 1, cu, 1025, seqused_k=used, causal=True, block_table=bt)
    ref = _oracle(q, kc, vc, qlens, klens, bt, head_size ** -0.5)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)


def test_decode_contiguous_kv_and_garbage_tail(fg):
    # packed K/V with cu_seqlens_k (no page table), one query token per sequence
    torch.manual_seed(9)
    klens = [300, 17, 1000]
    cu_k = torch.tensor([0] + klens, dtype=torch.int32).cumsum(0, dtype=torch.int32).to(DEV)
    cu_q = torch.arange(4, dtype=torch.int32, device=DEV)
    q = torch.randn(3, 8, 128, dtype=torch.float16, device=DEV)
    k = torch.randn(sum(klens), 2, 128, dtype=torch.float16, device=DEV)
    v = torch.randn_like(k)
    out = fg.flash_attn_varlen_func(q, k, v, 1, cu_q, 1000, cu_seqlens_k=cu_k, causal=True)
    ref = O.varlen_attention(q.cpu(), k.cpu(), v.cpu(), cu_q.cpu(), cu_k.cpu(), 128 ** -0.5, causal=False,
                             compute_dtype=torch.float32)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)
    # paged: NaN/Inf in the unused tail of the last page must not leak
    b = workloads.decode_batch(seed=6, batch=6, min_ctx=20, max_ctx=900, device=DEV)
    clean = fg.flash_attn_varlen_func(b.q, b.key_cache, b.value_cache, 1, b.cu_seqlens_q, b.max_seqlen_k,
                                      seqused_k=b.seqused_k, causal=True, block_table=b.block_table)
    kc, vc = b.key_cache.clone(), b.value_cache.clone()
    for i, n in enumerate(b.kv_lens):
        if n % 16:
            page = int(b.block_table[i, (n - 1) // 16])
            kc[page, n % 16:] = float("nan")
            vc[page, n % 16:] = float("inf")
    dirty = fg.flash_attn_varlen_func(b.q, kc, vc, 1, b.cu_seqlens_q, b.max_seqlen_k, seqused_k=b.seqused_k,
                                      causal=True, block_table=b.block_table)
    assert torch.equal(clean, dirty)


# ---- aten::_flash_attention_forward (dense batches), reached from F.scaled_dot_product_attention
def _sdpa_oracle(q, k, v, scale, causal):
    """fp32 CPU math on (batch, heads, seq, dim) tensors; bottom-right aligned causal mask,
    KV heads repeated for GQA (the reference's oracle: tests/test_attention_ops.py:200-229)."""
    q, k, v = q.cpu().float(), k.cpu().float(), v.cpu().float()
    g = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
    s = torch.einsum("bhqd,bhkd->bhqk", q, k) * scale
    if causal:
        sq, sk = q.shape[2], k.shape[2]
        mask = torch.ones(sq, sk, dtype=torch.bool).triu(diagonal=sk - sq + 1)
        s = s.masked_fill(mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)   # rows without a visible key
    return torch.einsum("bhqk,bhkd->bhqd", p, v), torch.logsumexp(s, dim=-1)


@pytest.mark.parametrize("shape", [(1, 1, 128, 2048), (4, 8, 1024, 128), (4, 8, 17, 1030), (2, 8, 1024, 1024)])
@pytest.mark.parametrize("head_size", [64, 128, 192, 256])
@pytest.mark.parametrize("is_causal", [False, True])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_flash_attention_forward_dense(fg, shape, head_size, is_causal, dtype):
    # shapes of tests/test_attention_ops.py:473-797 (square, non-square, q shorter and longer than k)
    batch, heads, sq, sk = shape
    torch.manual_seed(0)
    q = torch.randn(batch, heads, sq, head_size, dtype=dtype, device=DEV)
    k = torch.randn(batch, heads, sk, head_size, dtype=dtype, device=DEV)
    v = torch.randn(batch, heads, sk, head_size, dtype=dtype, device=DEV)
    scale = head_size ** -0.5
    ref, ref_lse = _sdpa_oracle(q, k, v, scale, is_causal)
    # the ATen entry takes (batch, seq, heads, dim): transposed views, as SDPA passes them
    out, lse, seed, offset, dbg = fg.flash_attention_forward(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), None, None, sq, sk, 0.0, is_causal, False, scale=scale)
    assert out.shape == (batch, sq, heads, head_size) and lse.shape == (batch, heads, sq)
    torch.testing.assert_close(out.transpose(1, 2).cpu().float(), ref, atol=ATOL, rtol=RTOL)
    finite = torch.isfinite(ref_lse)
    torch.testing.assert_close(lse.cpu()[finite], ref_lse[finite], atol=2e-2, rtol=1e-2)


def test_sdpa_through_use_gems_and_gqa(fg):
    # F.scaled_dot_product_attention -> aten::_flash_attention_forward -> this library
    torch.manual_seed(1)
    q = torch.randn(2, 8, 512, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.randn(2, 8, 512, 128, dtype=torch.bfloat16, device=DEV)
    v = torch.randn(2, 8, 512, 128, dtype=torch.bfloat16, device=DEV)
    ref, _ = _sdpa_oracle(q, k, v, 128 ** -0.5, True)
    before = _lib.launch_count()
    with fg.use_gems():
        from torch.nn.attention import SDPBackend, sdpa_kernel
        with sdpa_kernel(backends=[SDPBackend.FLASH_ATTENTION]):
            out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    assert _lib.launch_count() > before, "SDPA did not reach this library's kernels"
    torch.testing.assert_close(out.cpu().float(), ref, atol=ATOL, rtol=RTOL)
    # grouped-query form through the operator itself (packed layout, no copy)
    qg = torch.randn(2, 256, 8, 128, dtype=torch.float16, device=DEV)
    kg = torch.randn(2, 300, 2, 128, dtype=torch.float16, device=DEV)
    vg = torch.randn(2, 300, 2, 128, dtype=torch.float16, device=DEV)
    o, lse, *_ = fg.flash_attention_forward(qg, kg, vg, None, None, 256, 300, 0.0, True, False)
    refg, _ = _sdpa_oracle(qg.transpose(1, 2), kg.transpose(1, 2), vg.transpose(1, 2), 128 ** -0.5, True)
    torch.testing.assert_close(o.transpose(1, 2).cpu().float(), refg, atol=ATOL, rtol=RTOL)
    with pytest.raises(NotImplementedError):
        fg.flash_attention_forward(qg, kg, vg, None, None, 256, 300, 0.1, True, False)


@pytest.mark.parametrize("B,H,Hk,Sq,Sk", [(3, 8, 2, 300, 300), (2, 4, 4, 129, 1000), (2, 16, 8, 1024, 1024)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_flash_attention_forward_batch_strided_views_need_no_copy(fg, B, H, Hk, Sq, Sk, dtype):
    """(batch, seq, heads, dim) views of (batch, heads, seq, dim) tensors do not pack into one row
    dimension; the tensor-core kernel takes their batch strides: one launch, no copy kernel, and the
    same bits as the packed layout gives."""
    torch.manual_seed(5)
    q = torch.randn(B, H, Sq, 128, dtype=dtype, device=DEV)
    k = torch.randn(B, Hk, Sk, 128, dtype=dtype, device=DEV)
    v = torch.randn(B, Hk, Sk, 128, dtype=dtype, device=DEV)
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    assert qt.stride(0) != Sq * qt.stride(1)
    before = _lib.launch_count()
    out, lse, *_ = fg.flash_attention_forward(qt, kt, vt, None, None, Sq, Sk, 0.0, True, False)
    assert _lib.launch_count() - before == 1
    out_p, lse_p, *_ = fg.flash_attention_forward(qt.contiguous(), kt.contiguous(), vt.contiguous(), None, None, Sq, Sk,
                                                  0.0, True, False)
    assert torch.equal(out, out_p) and torch.equal(lse, lse_p)
    ref, _ = _sdpa_oracle(q, k.repeat_interleave(H // Hk, dim=1), v.repeat_interleave(H // Hk, dim=1), 128 ** -0.5, True)
    torch.testing.assert_close(out.transpose(1, 2).cpu().float(), ref, atol=ATOL, rtol=RTOL)


def test_batch_strides_are_rejected_where_no_kernel_takes_them(fg):
    import ctypes as C
    lib = _lib.load()
    p = _lib.AttnParams()
    x = torch.zeros(16, dtype=torch.bfloat16, device=DEV)
    cu = torch.zeros(3, dtype=torch.int32, device=DEV)
    p.q = p.k = p.v = p.out = x.data_ptr()
    p.cu_seqlens_q = p.cu_seqlens_k = cu.data_ptr()
    p.total_q, p.total_k, p.batch, p.num_heads, p.num_heads_k, p.head_dim = 256, 256, 2, 4, 4, 64   # head dim 64
    p.max_seqlen_q = p.max_seqlen_k = 128
    for f in ("q_row_stride", "k_row_stride", "v_row_stride", "o_row_stride"):
        setattr(p, f, 64)
    for f in ("q_head_stride", "k_head_stride", "v_head_stride", "o_head_stride"):
        setattr(p, f, 128 * 64)
    p.q_batch_stride = p.k_batch_stride = p.v_batch_stride = p.o_batch_stride = 4 * 128 * 64
    p.window_left = p.window_right = -1
    p.softmax_scale, p.dtype = 0.125, _lib.dtype_code(torch.bfloat16)
    assert lib.fg_flash_attn_varlen(C.byref(p), None) == -2          # FG_ERR_UNSUPPORTED, nothing launched
    p.head_dim = 128
    p.k_batch_stride = 0
    assert lib.fg_flash_attn_varlen(C.byref(p), None) == -1          # all four or none


# ---------------------------------------------------------------------------------------
# get_scheduler_metadata: integer work, bit-exact against the fixture recorded from the
# reference function itself, against the oracle on fresh random inputs, and for the
# reference test's own grid (tests/test_attention_ops.py:1618-1695).
# ---------------------------------------------------------------------------------------

def _sched_to(kw, device):
    return {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in kw.items()}


@pytest.mark.gpu
def test_scheduler_metadata_golden(fg, golden_dir):
    props = torch.cuda.get_device_properties(0)
    cases = torch.load(golden_dir / "golden_scheduler_metadata.pt", weights_only=False)
    if props.multi_processor_count != cases[0]["sm_count"]:
        pytest.skip(f"fixture recorded for {cases[0]['sm_count']} SMs, this GPU has {props.multi_processor_count}")
    for i, c in enumerate(cases):
        got = fg.get_scheduler_metadata(**_sched_to(c["kwargs"], DEV))
        assert got.dtype == torch.int32 and got.is_cuda
        assert torch.equal(got.cpu(), c["metadata"]), (i, {k: v for k, v in c["kwargs"].items()
                                                          if not torch.is_tensor(v)})


@pytest.mark.gpu
@pytest.mark.parametrize("batch_size", [1, 8, 256, 512])
@pytest.mark.parametrize("max_seqlen_k", [512, 2048])
@pytest.mark.parametrize("headdim", [64, 128])
@pytest.mark.parametrize("num_splits_static", [0, 4])
def test_scheduler_metadata_reference_grid(fg, batch_size, max_seqlen_k, headdim, num_splits_static):
    g = torch.Generator().manual_seed(42 + batch_size + max_seqlen_k)
    seqused_k = torch.randint(1, max_seqlen_k, (batch_size,), dtype=torch.int32, generator=g)
    kw = dict(batch_size=batch_size, max_seqlen_q=1, max_seqlen_k=max_seqlen_k, num_heads=32, num_heads_k=8,
              headdim=headdim, headdim_v=headdim, cu_seqlens_q=None, cu_seqlens_k_new=None, seqused_q=None,
              leftpad_k=None, page_size=None, max_seqlen_k_new=0, is_causal=False, window_size_left=-1,
              window_size_right=-1, has_softcap=False, num_splits=num_splits_static, pack_gqa=True, sm_margin=0)
    with fg.use_gems():
        got = fg.get_scheduler_metadata(qkv_dtype=torch.float16, seqused_k=seqused_k.to(DEV), cu_seqlens_k=None, **kw)
    want = O.get_scheduler_metadata(seqused_k=seqused_k, sm_count=torch.cuda.get_device_properties(0).multi_processor_count,
                                    **kw)
    assert torch.equal(got.cpu(), want)


@pytest.mark.gpu
def test_scheduler_metadata_random_and_edges(fg):
    import random

    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rng = random.Random(11)
    g = torch.Generator().manual_seed(11)
    ri = lambda lo, hi, n: torch.randint(lo, hi, (n,), dtype=torch.int32, generator=g)
    for _ in range(150):
        b = rng.choice([0, 1, 2, 5, 127, 128, 129, 992, 993, 1024, 1025, 5000])
        hk = rng.choice([1, 2, 8])
        hq = hk * rng.choice([1, 4, 7, 16])
        d = rng.choice([64, 96, 128, 192, 256])
        sq, sk = rng.choice([1, 1, 3, 64, 500]), rng.choice([16, 512, 8192, 70000, 300000])
        kw = dict(batch_size=b, max_seqlen_q=sq, max_seqlen_k=sk, num_heads=hq, num_heads_k=hk, headdim=d,
                  headdim_v=rng.choice([d, 128, 512]), seqused_k=ri(1, sk + 1, b), cu_seqlens_q=None,
                  cu_seqlens_k_new=None, seqused_q=None, leftpad_k=None, page_size=rng.choice([None, 16, 128]),
                  max_seqlen_k_new=rng.choice([0, 0, 4, 300]), is_causal=rng.random() < 0.5,
                  window_size_left=rng.choice([-1, -1, 100]), window_size_right=rng.choice([-1, 0, 50]),
                  has_softcap=rng.random() < 0.2, num_splits=rng.choice([0, 0, 1, 3, 300]),
                  pack_gqa=rng.choice([None, True, False]), sm_margin=rng.choice([0, 16]))
        r = rng.random()
        if r < 0.25:
            ql = ri(1, sq + 1, b)
            kw["cu_seqlens_q"] = torch.cat([torch.zeros(1, dtype=torch.int32), ql.cumsum(0).to(torch.int32)])
        elif r < 0.5:
            kw["seqused_q"] = ri(1, sq + 1, b)
        if rng.random() < 0.3:
            kw["leftpad_k"] = torch.minimum(ri(0, 40, b), kw["seqused_k"] - 1)
        if kw["max_seqlen_k_new"] and rng.random() < 0.5:
            kn = ri(1, kw["max_seqlen_k_new"] + 1, b)
            kw["cu_seqlens_k_new"] = torch.cat([torch.zeros(1, dtype=torch.int32), kn.cumsum(0).to(torch.int32)])
        want = O.get_scheduler_metadata(sm_count=sms, **kw)
        got = fg.get_scheduler_metadata(qkv_dtype=torch.bfloat16, cu_seqlens_k=None, **_sched_to(kw, DEV))
        assert torch.equal(got.cpu(), want), {k: v for k, v in kw.items() if not torch.is_tensor(v)}
    # int64 length vectors are converted; too short a vector is refused
    sk = torch.tensor([700, 9000, 33], dtype=torch.int64, device=DEV)
    a = fg.get_scheduler_metadata(3, 1, 9000, 32, 8, 128, 128, torch.bfloat16, sk, page_size=16)
    assert torch.equal(a.cpu(), O.get_scheduler_metadata(3, 1, 9000, 32, 8, 128, 128, sk.cpu(), page_size=16, sm_count=sms))
    with pytest.raises(RuntimeError, match="entries"):
        fg.get_scheduler_metadata(4, 1, 9000, 32, 8, 128, 128, torch.bfloat16, sk)
