"""Parity against the reference itself on the same GPU: the unmodified FlagGems package
(installed under ``baseline/_ref``) runs its Triton kernels on the same seeded inputs and
the results are compared operator by operator with the reference's own tolerances
(bit-exact for the cache scatter).  Skipped when the reference install is absent or does
not import (it needs a GPU and Triton)."""
import sys
from pathlib import Path

import pytest
import torch

from flaggems_b200 import workloads
from flaggems_b200.testing import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"
REF_DIR = Path(__file__).resolve().parent.parent / "baseline" / "_ref"


@pytest.fixture(scope="module")
def ref():
    if not (REF_DIR / "flag_gems").exists():
        pytest.skip("reference install baseline/_ref is not present")
    sys.path.insert(0, str(REF_DIR))
    try:
        import flag_gems  # the reference, unmodified
    except Exception as e:  # no GPU, Triton mismatch, ...
        pytest.skip(f"reference does not import here: {type(e).__name__}: {e}")
    finally:
        sys.path.remove(str(REF_DIR))
    return flag_gems


def test_fused_add_rms_norm_vs_triton(fg, ref):
    x, r, w, eps = workloads.norm_inputs(seed=1, T=512, device=DEV)
    x2, r2 = x.clone(), r.clone()
    ref.fused_add_rms_norm(x2, r2, [4096], w, eps)
    fg.fused_add_rms_norm(x, r, [4096], w, eps)
    assert_close(x, x2, torch.bfloat16)
    assert_close(r, r2, torch.bfloat16)


def test_rotary_embedding_vs_triton(fg, ref):
    q, k, cos, sin, pos = workloads.rope_inputs(seed=2, T=512, device=DEV)
    for interleaved in (False, True):
        rq, rk = ref.apply_rotary_pos_emb(q, k, cos, sin, pos, interleaved, False)
        oq, ok = fg.apply_rotary_pos_emb(q, k, cos, sin, pos, interleaved, False)
        assert_close(oq, rq, torch.bfloat16)
        assert_close(ok, rk, torch.bfloat16)


def test_silu_and_mul_vs_triton(fg, ref):
    x = workloads.silu_inputs(seed=3, T=256, device=DEV)
    d = x.shape[1] // 2
    assert_close(fg.silu_and_mul(x[:, :d], x[:, d:]), ref.silu_and_mul(x[:, :d], x[:, d:]), torch.bfloat16)


def test_reshape_and_cache_flash_vs_triton(fg, ref):
    b = workloads.decode_batch(seed=4, batch=64, min_ctx=16, max_ctx=400, device=DEV)
    kc, vc = b.key_cache.clone(), b.value_cache.clone()
    ref.reshape_and_cache_flash(b.new_key, b.new_value, kc, vc, b.slot_mapping, "auto", None, None)
    fg.reshape_and_cache_flash(b.new_key, b.new_value, b.key_cache, b.value_cache, b.slot_mapping, "auto", None, None)
    assert torch.equal(kc, b.key_cache) and torch.equal(vc, b.value_cache)


def test_mm_addmm_vs_triton(fg, ref):
    torch.manual_seed(5)
    a = torch.randn(512, 1024, dtype=torch.bfloat16, device=DEV)
    b = torch.randn(1024, 768, dtype=torch.bfloat16, device=DEV) / 32
    bias = torch.randn(768, dtype=torch.bfloat16, device=DEV) * 0.02
    assert_close(fg.mm(a, b), ref.mm(a, b), torch.bfloat16, reduce_dim=1024)
    assert_close(fg.addmm(bias, a, b, alpha=0.5, beta=2.0), ref.addmm(bias, a, b, alpha=0.5, beta=2.0),
                 torch.bfloat16, reduce_dim=1024)


def test_flash_attn_varlen_prefill_and_decode_vs_triton(fg, ref):
    p = workloads.prefill_batch(seed=6, num_seqs=4, min_len=60, max_len=500, device=DEV)
    kw = dict(max_seqlen_q=p.max_seqlen_q, cu_seqlens_q=p.cu_seqlens_q, max_seqlen_k=p.max_seqlen_k,
              seqused_k=p.seqused_k, causal=True, block_table=p.block_table, softmax_scale=p.scale)
    torch.testing.assert_close(fg.flash_attn_varlen_func(p.q, p.key_cache, p.value_cache, **kw).float(),
                               ref.flash_attn_varlen_func(p.q, p.key_cache, p.value_cache, **kw).float(),
                               atol=2e-2, rtol=1e-2)
    d = workloads.decode_batch(seed=7, batch=16, min_ctx=30, max_ctx=1500, device=DEV)
    kw = dict(max_seqlen_q=1, cu_seqlens_q=d.cu_seqlens_q, max_seqlen_k=d.max_seqlen_k, seqused_k=d.seqused_k,
              causal=True, block_table=d.block_table, softmax_scale=d.scale)
    torch.testing.assert_close(fg.flash_attn_varlen_func(d.q, d.key_cache, d.value_cache, **kw).float(),
                               ref.flash_attn_varlen_func(d.q, d.key_cache, d.value_cache, **kw).float(),
                               atol=2e-2, rtol=1e-2)


@pytest.mark.gpu
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
            want = ref.get_scheduler_metadata(**kw)
        except Exception as e:  # the reference's kernels against this image's Triton
            pytest.skip(f"reference get_scheduler_metadata does not run here: {type(e).__name__}: {e}")
        got = fg.get_scheduler_metadata(**kw)
        assert torch.equal(got, want.to(torch.int32)), (b, sk, d, ns, page, knew)
