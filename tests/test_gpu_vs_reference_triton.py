"""Parity against the reference itself on the same GPU: the unmodified FlagGems package
(installed under ``baseline/_ref``) runs its Triton kernels on the same seeded inputs and
the results are compared operator by operator -- with the reference's own tolerances, and
with atol = rtol = 1e-2 (bf16, fp32 accumulation) on top; bit-exact for the cache scatter.

Small cases first, then the benchmark configurations at full size built by
``flaggems_b200.workloads`` with the benchmark's own seeds: the T=4096 elementwise block,
all 16 prefill sequences (128..4096 tokens), the batch-256 decode (contexts up to 8192)
after the cache write, and every row of the four M=8192 projections.  The observed
maximum absolute / relative errors are written to the file named by the environment variable
``FLAGGEMS_B200_PARITY_REPORT`` when it is set.

Skipped when the reference install is absent or does not import (it needs a GPU and Triton).
"""
import json
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from baseline import triton_reference as tref  # noqa: E402
from flaggems_b200 import workloads  # noqa: E402
from flaggems_b200.testing import assert_close  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-2  # atol = rtol for bf16 results
_observed = {}


@pytest.fixture(scope="module")
def ref():
    try:
        return tref.load()
    except tref.ReferenceUnavailable as e:
        pytest.skip(str(e))


@pytest.fixture(scope="module", autouse=True)
def _write_observed():
    yield
    report = os.environ.get("FLAGGEMS_B200_PARITY_REPORT")
    if _observed and report:
        Path(report).parent.mkdir(parents=True, exist_ok=True)
        Path(report).write_text(json.dumps(_observed, indent=1))


def check(name, got, want, atol=TOL, rtol=TOL):
    """Record max abs / max rel error of `got` against the reference's result and assert
    |got - want| <= atol + rtol |want| everywhere."""
    g, w = got.float(), want.float()
    assert g.shape == w.shape, (name, g.shape, w.shape)
    err = (g - w).abs()
    bound = atol + rtol * w.abs()
    big = w.abs() > 0.05
    rel = (err[big] / w.abs()[big]).max().item() if big.any() else 0.0
    bad = int((err > bound).sum().item())
    _observed[name] = {"max_abs": err.max().item(), "max_rel_where_ref_above_0.05": rel,
                       "violations_of_1e-2": bad, "elements": g.numel(),
                       "identical_fraction": float((g == w).float().mean().item())}
    assert torch.isfinite(g).all(), name
    assert bad == 0, f"{name}: {bad} of {g.numel()} elements beyond atol={atol}, rtol={rtol}; max abs {err.max().item()}"


# ------------------------------------------------------------------------------- small cases
def test_fused_add_rms_norm_vs_triton(fg, ref):
    x, r, w, eps = workloads.norm_inputs(seed=1, T=512, device=DEV)
    x2, r2 = x.clone(), r.clone()
    tref.call(ref.fused_add_rms_norm, x2, r2, [4096], w, eps)
    fg.fused_add_rms_norm(x, r, [4096], w, eps)
    assert_close(x, x2, torch.bfloat16)
    assert_close(r, r2, torch.bfloat16)


def test_rotary_embedding_vs_triton(fg, ref):
    q, k, cos, sin, pos = workloads.rope_inputs(seed=2, T=512, device=DEV)
    for interleaved in (False, True):
        rq, rk = tref.call(ref.apply_rotary_pos_emb, q, k, cos, sin, pos, interleaved, False)
        oq, ok = fg.apply_rotary_pos_emb(q, k, cos, sin, pos, interleaved, False)
        assert_close(oq, rq, torch.bfloat16)
        assert_close(ok, rk, torch.bfloat16)


def test_silu_and_mul_vs_triton(fg, ref):
    x = workloads.silu_inputs(seed=3, T=256, device=DEV)
    d = x.shape[1] // 2
    assert_close(fg.silu_and_mul(x[:, :d], x[:, d:]), tref.call(ref.silu_and_mul, x[:, :d], x[:, d:]),
                 torch.bfloat16)


def test_reshape_and_cache_flash_vs_triton(fg, ref):
    b = workloads.decode_batch(seed=4, batch=64, min_ctx=16, max_ctx=400, device=DEV)
    kc, vc = b.key_cache.clone(), b.value_cache.clone()
    tref.call(ref.reshape_and_cache_flash, b.new_key, b.new_value, kc, vc, b.slot_mapping, "auto", None, None)
    fg.reshape_and_cache_flash(b.new_key, b.new_value, b.key_cache, b.value_cache, b.slot_mapping, "auto", None, None)
    assert torch.equal(kc, b.key_cache) and torch.equal(vc, b.value_cache)


def test_mm_addmm_vs_triton(fg, ref):
    torch.manual_seed(5)
    a = torch.randn(512, 1024, dtype=torch.bfloat16, device=DEV)
    b = torch.randn(1024, 768, dtype=torch.bfloat16, device=DEV) / 32
    bias = torch.randn(768, dtype=torch.bfloat16, device=DEV) * 0.02
    assert_close(fg.mm(a, b), tref.call(ref.mm, a, b), torch.bfloat16, reduce_dim=1024)
    assert_close(fg.addmm(bias, a, b, alpha=0.5, beta=2.0), tref.call(ref.addmm, bias, a, b, alpha=0.5, beta=2.0),
                 torch.bfloat16, reduce_dim=1024)


def test_flash_attn_varlen_prefill_and_decode_vs_triton(fg, ref):
    p = workloads.prefill_batch(seed=6, num_seqs=4, min_len=60, max_len=500, device=DEV)
    kw = dict(max_seqlen_q=p.max_seqlen_q, cu_seqlens_q=p.cu_seqlens_q, max_seqlen_k=p.max_seqlen_k,
              seqused_k=p.seqused_k, causal=True, block_table=p.block_table, softmax_scale=p.scale)
    torch.testing.assert_close(fg.flash_attn_varlen_func(p.q, p.key_cache, p.value_cache, **kw).float(),
                               tref.call(ref.flash_attn_varlen_func, p.q, p.key_cache, p.value_cache, **kw).float(),
                               atol=2e-2, rtol=1e-2)
    d = workloads.decode_batch(seed=7, batch=16, min_ctx=30, max_ctx=1500, device=DEV)
    kw = dict(max_seqlen_q=1, cu_seqlens_q=d.cu_seqlens_q, max_seqlen_k=d.max_seqlen_k, seqused_k=d.seqused_k,
              causal=True, block_table=d.block_table, softmax_scale=d.scale)
    torch.testing.assert_close(fg.flash_attn_varlen_func(d.q, d.key_cache, d.value_cache, **kw).float(),
                               tref.call(ref.flash_attn_varlen_func, d.q, d.key_cache, d.value_cache, **kw).float(),
                               atol=2e-2, rtol=1e-2)


def test_get_scheduler_metadata_vs_triton(fg, ref):
    g = torch.Generator().manual_seed(42)
    for b, sk, d, ns, page, knew in [(1, 512, 64, 0, None, 0), (8, 2048, 128, 0, None, 0), (256, 2048, 128, 4, None, 0),
                                     (512, 512, 64, 0, None, 0), (256, 8192, 128, 0, 16, 0), (64, 32768, 128, 0, 16, 0),
                                     (993, 8192, 128, 0, 16, 0), (5, 6000, 64, 0, None, 5), (130, 6000, 128, 0, 16, 0)]:
        seqused_k = torch.randint(1, sk, (b,), dtype=torch.int32, generator=g).to(DEV)
        kw = dict(batch_size=b, max_seqlen_q=1, max_seqlen_k=sk, num_heads=32, num_heads_k=8, headdim=d, headdim_v=d,
                  qkv_dtype=torch.float16, seqused_k=seqused_k, cu_seqlens_q=None, cu_seqlens_k=None,
                  cu_seqlens_k_new=None, seqused_q=None, leftpad_k=None, page_size=page, max_seqlen_k_new=knew,
                  is_causal=False, window_size_left=-1, window_size_right=-1, has_softcap=False, num_splits=ns,
                  pack_gqa=None if page else True, sm_margin=0)
        try:
            want = tref.call(ref.get_scheduler_metadata, **kw)
        except Exception as e:  # the reference's kernels against this image's Triton
            pytest.skip(f"reference get_scheduler_metadata does not run here: {type(e).__name__}: {e}")
        got = fg.get_scheduler_metadata(**kw)
        assert torch.equal(got, want.to(torch.int32)), (b, sk, d, ns, page, knew)


@pytest.mark.parametrize("num_heads", [(4, 4), (8, 2), (16, 2)])
@pytest.mark.parametrize("head_size", [128, 192, 256])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("alibi,soft_cap", [(False, None), (True, None), (False, 10.0), (False, 50.0)])
def test_reference_attention_grid_vs_triton(fg, ref, num_heads, head_size, dtype, alibi, soft_cap):
    """The reference's own varlen grid (tests/test_attention_ops.py:886-995: mixed query lengths,
    GQA, head dims 128-256, ALiBi, soft-cap; paged cache with random block tables), this time
    against its Triton kernel instead of the oracle: the kernels behind ALiBi, soft-cap and the
    other head dims (mma.sync path) are compared with the reference's on the same GPU."""
    torch.manual_seed(1234567890)
    seq_lens = [(1, 1328), (5, 18), (129, 463)]
    qlens, klens = [x[0] for x in seq_lens], [x[1] for x in seq_lens]
    hq, hk = num_heads
    block_size, num_blocks = 32, 2048
    q = torch.randn(sum(qlens), hq, head_size, dtype=dtype, device=DEV)
    kc = torch.randn(num_blocks, block_size, hk, head_size, dtype=dtype, device=DEV)
    vc = torch.randn_like(kc)
    cu = torch.tensor([0] + qlens, dtype=torch.int32).cumsum(0, dtype=torch.int32).to(DEV)
    used = torch.tensor(klens, dtype=torch.int32, device=DEV)
    bt = torch.randint(0, num_blocks, (len(seq_lens), (max(klens) + block_size - 1) // block_size), dtype=torch.int32,
                       device=DEV)
    slopes = torch.ones(len(seq_lens), hq, dtype=torch.float32, device=DEV) * 0.3 if alibi else None
    kw = dict(q=q, k=kc, v=vc, cu_seqlens_q=cu, seqused_k=used, max_seqlen_q=max(qlens), max_seqlen_k=max(klens),
              softmax_scale=head_size ** -0.5, causal=True, window_size=(-1, -1), block_table=bt,
              softcap=soft_cap if soft_cap is not None else 0, alibi_slopes=slopes, fa_version=2)
    want = tref.call(ref.flash_attn_varlen_func, **kw)
    got = fg.flash_attn_varlen_func(**kw)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=1e-2)


# ------------------------------------------- the reference's own test grids of the other operators
@pytest.mark.parametrize("shape", [(1, 2), (4096, 256), (200, 40999)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.bfloat16])
def test_reference_norm_shapes_vs_triton(fg, ref, shape, dtype):
    """Shapes of tests/test_norm_ops.py:597-632 (the last one takes the two-pass kernel for long rows)."""
    torch.manual_seed(0)
    x = torch.randn(shape, dtype=dtype, device=DEV)
    r = torch.randn(shape, dtype=dtype, device=DEV)
    w = torch.randn(shape[1:], dtype=dtype, device=DEV)
    x2, r2 = x.clone(), r.clone()
    tref.call(ref.fused_add_rms_norm, x2, r2, list(shape[1:]), w, 1e-5)
    fg.fused_add_rms_norm(x, r, list(shape[1:]), w, 1e-5)
    assert_close(x, x2, dtype)
    assert_close(r, r2, dtype)


@pytest.mark.parametrize("q_heads,k_heads", [(8, 1), (6, 2)])
@pytest.mark.parametrize("head_dim", [64, 96, 128, 256])
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("has_pos_id", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_reference_rope_grid_vs_triton(fg, ref, q_heads, k_heads, head_dim, interleaved, has_pos_id, dtype):
    """Grid of tests/test_special_ops.py:164-219: 4-D inputs, with position ids or positions = index in the sequence."""
    torch.manual_seed(0)
    batch, seq, max_seq = 4, 97, 512
    q = torch.randn((batch, seq, q_heads, head_dim), dtype=dtype, device=DEV)
    k = torch.randn((batch, seq, k_heads, head_dim), dtype=dtype, device=DEV)
    pos = torch.randint(0, max_seq, (batch, seq), device=DEV) if has_pos_id else None
    cos, sin = workloads.rope_tables(max_seq, head_dim, dtype, DEV)
    want_q, want_k = tref.call(ref.apply_rotary_pos_emb, q, k, cos, sin, pos, interleaved, False)
    got_q, got_k = fg.apply_rotary_pos_emb(q, k, cos, sin, pos, interleaved, False)
    assert_close(got_q, want_q, dtype)
    assert_close(got_k, want_k, dtype)


@pytest.mark.parametrize("M,N,K,dtype", [(1, 1, 32, torch.bfloat16), (15, 160, 1024, torch.bfloat16),
                                         (495, 5333, 71, torch.bfloat16), (495, 5333, 71, torch.float32)])
@pytest.mark.parametrize("scalar", [-0.999])   # (every shape and dtype costs an autotuning run of the reference: kept small)
def test_reference_blas_grid_vs_triton(fg, ref, M, N, K, dtype, scalar):
    """Shapes and scalars of tests/test_blas_ops.py:24-92 (tiny, skinny and odd shapes; fp32 without TF32)."""
    torch.manual_seed(0)
    a = torch.randn((M, K), dtype=dtype, device=DEV)
    b = torch.randn((K, N), dtype=dtype, device=DEV)
    bias = torch.randn((N,), dtype=dtype, device=DEV)
    assert_close(fg.mm(a, b), tref.call(ref.mm, a, b), dtype, reduce_dim=K)
    assert_close(fg.addmm(bias, a, b, alpha=scalar, beta=scalar),
                 tref.call(ref.addmm, bias, a, b, alpha=scalar, beta=scalar), dtype, reduce_dim=K)


def test_fp32_mm_on_tensor_cores_is_as_accurate_as_the_reference(fg, ref):
    """A large fp32 product: the reference multiplies with `allow_tf32=False` (ops/mm.py:100-107); here it
    runs on the tensor cores from three bf16 pieces per operand.  Both against fp64: the error of
    this library's result must not exceed the reference's."""
    torch.manual_seed(0)
    M = N = K = 2048
    a = torch.randn((M, K), dtype=torch.float32, device=DEV)
    b = torch.randn((K, N), dtype=torch.float32, device=DEV)
    exact = a.double() @ b.double()
    got, want = fg.mm(a, b), tref.call(ref.mm, a, b)
    assert_close(got, want, torch.float32, reduce_dim=K)
    err = lambda x: float((x.double() - exact).abs().mean() / exact.abs().mean())
    assert err(got) <= err(want) * 1.1 + 1e-8, (err(got), err(want))


@pytest.mark.parametrize("head_size", [64, 80, 120, 256])
@pytest.mark.parametrize("block_size", [8, 16, 32])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_reference_cache_write_grid_vs_triton(fg, ref, head_size, block_size, dtype):
    """Grid of tests/test_attention_ops.py:1389-1470: 42 tokens into random distinct slots, bit for bit."""
    import random

    random.seed(2025)
    torch.manual_seed(2025)
    num_tokens, num_heads, num_blocks = 42, 8, 1024
    slots = torch.tensor(random.sample(range(num_blocks * block_size), num_tokens), dtype=torch.long, device=DEV)
    key = torch.randn((num_tokens, num_heads, head_size), dtype=dtype, device=DEV)
    value = torch.randn_like(key)
    kc = torch.randn((num_blocks, block_size, num_heads, head_size), dtype=dtype, device=DEV)
    vc = torch.randn_like(kc)
    kc2, vc2 = kc.clone(), vc.clone()
    tref.call(ref.reshape_and_cache_flash, key, value, kc2, vc2, slots, "auto", None, None)
    fg.reshape_and_cache_flash(key, value, kc, vc, slots, "auto", None, None)
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)


# ------------------------------------------------------------- benchmark configurations, full size
def test_config2_elementwise_block_full_size_vs_triton(fg, ref):
    """T=4096, hidden 4096: fused_add_rms_norm; rope on q [4096,32,128] / k [4096,8,128];
    silu_and_mul on the halves of [4096, 22016] (the benchmark's seeds 1, 2, 3)."""
    x, r, w, eps = workloads.norm_inputs(seed=1, device=DEV)
    x2, r2 = x.clone(), r.clone()
    tref.call(ref.fused_add_rms_norm, x2, r2, [4096], w, eps)
    fg.fused_add_rms_norm(x, r, [4096], w, eps)
    check("config2/fused_add_rms_norm/out", x, x2)
    check("config2/fused_add_rms_norm/residual", r, r2)
    assert_close(x, x2, torch.bfloat16)
    q, k, cos, sin, pos = workloads.rope_inputs(seed=2, device=DEV)
    rq, rk = tref.call(ref.apply_rotary_pos_emb, q, k, cos, sin, pos, False, False)
    oq, ok = fg.apply_rotary_pos_emb(q, k, cos, sin, pos, False, False)
    check("config2/rotary_embedding/q", oq, rq)
    check("config2/rotary_embedding/k", ok, rk)
    q2, k2 = q.clone(), k.clone()
    fg.apply_rotary_pos_emb(q2, k2, cos, sin, pos, False, True)      # the in-place form the benchmark times
    assert torch.equal(q2, oq) and torch.equal(k2, ok)
    act = workloads.silu_inputs(seed=3, device=DEV)
    d = act.shape[1] // 2
    want = tref.call(ref.silu_and_mul, act[:, :d], act[:, d:])
    got = torch.empty_like(want)
    fg.silu_and_mul_out(act[:, :d], act[:, d:], got)
    check("config2/silu_and_mul", got, want)


def test_config3_prefill_all_sequences_vs_triton(fg, ref):
    """All 16 sequences (128..4096 tokens) of the benchmark's prefill batch, paged form."""
    p = workloads.prefill_batch(seed=4, device=DEV)
    kw = dict(max_seqlen_q=p.max_seqlen_q, cu_seqlens_q=p.cu_seqlens_q, max_seqlen_k=p.max_seqlen_k,
              seqused_k=p.seqused_k, causal=True, block_table=p.block_table, softmax_scale=p.scale)
    want = tref.call(ref.flash_attn_varlen_func, p.q, p.key_cache, p.value_cache, **kw)
    got = fg.flash_attn_varlen_func(p.q, p.key_cache, p.value_cache, **kw)
    check("config3/prefill_paged", got, want)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=1e-2)
    # the contiguous form of the same batch (which the reference does not take) must agree with the paged one
    got_c = fg.flash_attn_varlen_func(p.q, p.k, p.v, p.max_seqlen_q, p.cu_seqlens_q, p.max_seqlen_k,
                                      cu_seqlens_k=p.cu_seqlens_k, causal=True, softmax_scale=p.scale)
    check("config3/prefill_contiguous", got_c, want)


def test_config4_cache_write_then_decode_batch256_vs_triton(fg, ref):
    """Batch 256, contexts 512..8192, block 16: the cache write (bit-exact) followed by the
    decode of one query token per sequence over the written cache."""
    d = workloads.decode_batch(seed=5, device=DEV)
    # the reference writes first, into the same caches; the token rows it wrote are kept for the bit comparison
    slots = d.slot_mapping
    hk, hd = d.key_cache.shape[2], d.key_cache.shape[3]
    before_k = d.key_cache.view(-1, hk, hd)[slots].clone()
    before_v = d.value_cache.view(-1, hk, hd)[slots].clone()
    tref.call(ref.reshape_and_cache_flash, d.new_key, d.new_value, d.key_cache, d.value_cache, slots, "auto", None, None)
    ref_k = d.key_cache.view(-1, hk, hd)[slots].clone()
    ref_v = d.value_cache.view(-1, hk, hd)[slots].clone()
    d.key_cache.view(-1, hk, hd)[slots] = before_k       # undo, then write with this library
    d.value_cache.view(-1, hk, hd)[slots] = before_v
    fg.reshape_and_cache_flash(d.new_key, d.new_value, d.key_cache, d.value_cache, slots, "auto", None, None)
    assert torch.equal(d.key_cache.view(-1, hk, hd)[slots], ref_k)
    assert torch.equal(d.value_cache.view(-1, hk, hd)[slots], ref_v)
    assert torch.equal(ref_k, d.new_key) and torch.equal(ref_v, d.new_value)
    kw = dict(max_seqlen_q=1, cu_seqlens_q=d.cu_seqlens_q, max_seqlen_k=d.max_seqlen_k, seqused_k=d.seqused_k,
              causal=True, block_table=d.block_table, softmax_scale=d.scale)
    want = tref.call(ref.flash_attn_varlen_func, d.q, d.key_cache, d.value_cache, **kw)
    got = fg.flash_attn_varlen_func(d.q, d.key_cache, d.value_cache, **kw)
    check("config4/decode_batch256", got, want)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("name", list(workloads.GEMM_SHAPES))
def test_config5_projection_every_row_vs_triton(fg, ref, name):
    """M=8192 at the four projection shapes: mm and addmm (bias [N], alpha = beta = 1), all rows."""
    K, N = workloads.GEMM_SHAPES[name]
    a, b, bias = workloads.gemm_inputs(name, seed=10 + list(workloads.GEMM_SHAPES).index(name), device=DEV)
    want = tref.call(ref.mm, a, b)
    got = fg.mm(a, b)
    check(f"config5/mm[{name}]", got, want)
    assert_close(got, want, torch.bfloat16, reduce_dim=K)
    del want, got
    want = tref.call(ref.addmm, bias, a, b)
    with fg.use_gems():
        got = torch.addmm(bias, a, b)         # through the ATen override
    check(f"config5/addmm[{name}]", got, want)
    assert_close(got, want, torch.bfloat16, reduce_dim=K)
