"""GPU parity: fused_add_rms_norm, rms_norm, rotary embedding, silu_and_mul and the
paged-cache scatter against the CPU oracle, through the Python host layer and the C ABI.

Shapes follow FlagGems' own tests (tests/test_norm_ops.py:597-632,
tests/test_special_ops.py:164-219, tests/test_binary_pointwise_ops.py:1377-1403,
tests/test_attention_ops.py:1389-1470) plus the benchmark configuration sizes.
Tolerances are the reference's: rtol = dtype resolution, atol = 1e-4 (x reduce_dim);
the cache scatter is bit-exact."""
import random

import pytest
import torch

from flaggems_b200 import workloads
from flaggems_b200.testing import assert_close
from oracle import reference_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
FLOAT_DTYPES = [torch.float16, torch.float32, torch.bfloat16]


# ------------------------------------------------------------------ fused_add_rms_norm
@pytest.mark.parametrize("shape", [(1, 2), (4096, 256), (200, 40999), (33, 4096), (5, 8192), (3, 16384), (2, 24)])
@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
def test_fused_add_rms_norm(fg, shape, dtype):
    torch.manual_seed(0)
    x = torch.randn(shape, dtype=dtype, device=DEV)
    r = torch.randn(shape, dtype=dtype, device=DEV)
    w = torch.randn(shape[1], dtype=dtype, device=DEV)
    ref_out, ref_res = O.fused_add_rms_norm(x.cpu(), r.cpu(), w.cpu(), 1e-5)
    out, res = fg.fused_add_rms_norm(x, r, [shape[1]], weight=w, eps=1e-5)
    assert out.data_ptr() == x.data_ptr() and res.data_ptr() == r.data_ptr()  # in place
    assert_close(out.cpu(), ref_out, dtype)
    assert_close(res.cpu(), ref_res, dtype)


def test_fused_add_rms_norm_config2_and_strided(fg):
    x, r, w, eps = workloads.norm_inputs(seed=1, device=DEV)
    ref_out, ref_res = O.fused_add_rms_norm(x.cpu(), r.cpu(), w.cpu(), eps, upcast=torch.float32)
    fg.fused_add_rms_norm(x, r, [4096], w, eps)
    assert_close(x.cpu(), ref_out, torch.bfloat16)
    assert_close(r.cpu(), ref_res, torch.bfloat16)
    # row-strided views (a slice of a wider buffer) are updated in place
    big = torch.randn(64, 1024, dtype=torch.bfloat16, device=DEV)
    bigr = torch.randn(64, 768, dtype=torch.bfloat16, device=DEV)
    xs, rs = big[:, 256:768], bigr[:, :512]
    w2 = torch.randn(512, dtype=torch.bfloat16, device=DEV)
    keep = big.clone()
    ref_out, ref_res = O.fused_add_rms_norm(xs.cpu(), rs.cpu(), w2.cpu(), 1e-6)
    fg.fused_add_rms_norm(xs, rs, [512], w2, 1e-6)
    assert_close(xs.cpu(), ref_out, torch.bfloat16)
    assert_close(rs.cpu(), ref_res, torch.bfloat16)
    assert torch.equal(big[:, :256], keep[:, :256]) and torch.equal(big[:, 768:], keep[:, 768:])


def test_fused_add_rms_norm_golden_and_custom_op(fg, golden_dir):
    for c in torch.load(golden_dir / "golden_fused_add_rms_norm.pt", weights_only=False):
        x, r, w = c["x"].to(DEV), c["residual"].to(DEV), c["weight"].to(DEV)
        torch.ops.flag_gems.fused_add_rms_norm(x, r, w, c["eps"])
        assert_close(x.cpu(), c["out"], x.dtype)
        assert_close(r.cpu(), c["new_residual"], x.dtype)


@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
def test_rms_norm(fg, dtype):
    torch.manual_seed(0)
    x = torch.randn(37, 2048, dtype=dtype, device=DEV)
    w = torch.randn(2048, dtype=dtype, device=DEV)
    out = fg.rms_norm(x, [2048], w, 1e-5)
    assert_close(out.cpu(), O.rms_norm(x.cpu(), w.cpu(), 1e-5), dtype)
    m = fg.GemsRMSNorm(2048, eps=1e-5, device=DEV, dtype=dtype)
    with torch.no_grad():
        m.weight.copy_(w)
        assert_close(m(x).cpu(), O.rms_norm(x.cpu(), w.cpu(), 1e-5), dtype)


# ------------------------------------------------------------------ rotary embedding
@pytest.mark.parametrize("batch_size", [4])
@pytest.mark.parametrize("max_seq_len", [512])
@pytest.mark.parametrize("q_heads,k_heads", [(8, 1), (6, 2), (1, 1), (8, 8)])
@pytest.mark.parametrize("head_dim", [64, 96, 128, 256])
@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
@pytest.mark.parametrize("rotary_interleaved", [True, False])
@pytest.mark.parametrize("has_pos_id", [True, False])
def test_apply_rotary_pos_emb(fg, batch_size, max_seq_len, q_heads, k_heads, head_dim, dtype, rotary_interleaved,
                              has_pos_id):
    torch.manual_seed(0)
    seq_len = torch.randint(1, max_seq_len, (1,)).item()
    q = torch.randn((batch_size, seq_len, q_heads, head_dim), dtype=dtype, device=DEV)
    k = torch.randn((batch_size, seq_len, k_heads, head_dim), dtype=dtype, device=DEV)
    pos = torch.randint(0, max_seq_len, (batch_size, seq_len), device=DEV)
    cos, sin = O.rope_cos_sin(max_seq_len, head_dim, dtype)
    ref_q, ref_k = O.apply_rotary_pos_emb(q.cpu(), k.cpu(), cos, sin, pos.cpu() if has_pos_id else None,
                                          rotary_interleaved, upcast=torch.float64)
    cos, sin = cos.to(DEV), sin.to(DEV)
    q_e, k_e = fg.apply_rotary_pos_emb(q, k, cos, sin, pos if has_pos_id else None, rotary_interleaved)
    assert_close(q_e.cpu(), ref_q, dtype)
    assert_close(k_e.cpu(), ref_k, dtype)
    # in place: same numbers, same storage
    q2, k2 = q.clone(), k.clone()
    qi, ki = fg.apply_rotary_pos_emb(q2, k2, cos, sin, pos if has_pos_id else None, rotary_interleaved, inplace=True)
    assert qi.data_ptr() == q2.data_ptr() and torch.equal(qi, q_e) and torch.equal(ki, k_e)


def test_rope_config2_partial_rotary_and_int32_positions(fg):
    q, k, cos, sin, pos = workloads.rope_inputs(seed=2, device=DEV)
    ref_q, ref_k = O.apply_rotary_pos_emb(q.cpu(), k.cpu(), cos.cpu(), sin.cpu(), pos.cpu())
    qe, ke = fg.apply_rotary_pos_emb(q, k, cos, sin, pos)
    assert_close(qe.cpu(), ref_q, torch.bfloat16)
    assert_close(ke.cpu(), ref_k, torch.bfloat16)
    qe32, _ = fg.apply_rotary_pos_emb(q, k, cos, sin, pos.to(torch.int32))
    assert torch.equal(qe32, qe)
    # vLLM calling form: rotate only the first rotary_dim of each head, in place, on a
    # strided view, with an fp32 cos/sin cache
    T, rd = 50, 64
    qq = torch.randn(T, 4, 128, dtype=torch.float16, device=DEV)
    kk = torch.randn(T, 2, 128, dtype=torch.float16, device=DEV)
    c32, s32 = O.rope_cos_sin(128, rd, torch.float32)
    p = torch.randint(0, 128, (T,), device=DEV)
    ref_q, ref_k = O.apply_rotary_pos_emb(qq[..., :rd].cpu(), kk[..., :rd].cpu(), c32, s32, p.cpu())
    keep = qq.clone()
    torch.ops.flag_gems.rotary_embedding_inplace(qq[..., :rd], kk[..., :rd], c32.to(DEV), s32.to(DEV), p, False)
    assert_close(qq[..., :rd].cpu(), ref_q, torch.float16)
    assert_close(kk[..., :rd].cpu(), ref_k, torch.float16)
    assert torch.equal(qq[..., rd:], keep[..., rd:])


def test_rope_golden(fg, golden_dir):
    for c in torch.load(golden_dir / "golden_rope.pt", weights_only=False):
        dev = lambda t: None if t is None else t.to(DEV)
        qe, ke = fg.apply_rotary_pos_emb(dev(c["q"]), dev(c["k"]), dev(c["cos"]), dev(c["sin"]),
                                         dev(c["position_ids"]), c["interleaved"])
        assert_close(qe.cpu(), c["q_out"], c["q"].dtype)
        assert_close(ke.cpu(), c["k_out"], c["q"].dtype)


# ------------------------------------------------------------------ silu_and_mul
POINTWISE_SHAPES = [(), (1,), (1024, 1024), (20, 320, 15), (16, 128, 64, 60), (16, 7, 57, 32, 29), (3, 11008)]


@pytest.mark.parametrize("shape", POINTWISE_SHAPES)
@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
def test_silu_and_mul(fg, shape, dtype):
    torch.manual_seed(0)
    a = torch.randn(shape, dtype=dtype, device=DEV)
    b = torch.randn(shape, dtype=dtype, device=DEV)
    out = fg.silu_and_mul(a, b)
    assert out.dtype == dtype and out.shape == a.shape
    assert_close(out.cpu(), O.silu_and_mul(a.cpu(), b.cpu()), dtype)


@pytest.mark.parametrize("shape", POINTWISE_SHAPES)
@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_gelu_and_mul(fg, shape, dtype, approximate):
    # forward of tests/test_binary_pointwise_ops.py:962-978
    torch.manual_seed(0)
    a = torch.randn(shape, dtype=dtype, device=DEV)
    b = torch.randn(shape, dtype=dtype, device=DEV)
    out = fg.gelu_and_mul(a, b, approximate)
    assert out.dtype == dtype and out.shape == a.shape
    assert_close(out.cpu(), O.gelu_and_mul(a.cpu(), b.cpu(), approximate), dtype)


def test_gelu_and_mul_halves_and_errors(fg):
    x = workloads.silu_inputs(seed=3, T=512, device=DEV)
    d = x.shape[1] // 2
    for approximate in ("none", "tanh"):
        assert_close(fg.gelu_and_mul(x[:, :d], x[:, d:], approximate).cpu(),
                     O.gelu_and_mul(x[:, :d].cpu(), x[:, d:].cpu(), approximate), torch.bfloat16)
    with pytest.raises(ValueError):
        fg.gelu_and_mul(x[:, :d], x[:, d:], "fast")
    with pytest.raises(RuntimeError, match="backward"):
        fg.gelu_and_mul(x[:, :d].clone().requires_grad_(), x[:, d:])


def test_silu_and_mul_halves_broadcast_and_out(fg):
    x = workloads.silu_inputs(seed=3, T=512, device=DEV)
    d = x.shape[-1] // 2
    ref = O.silu_and_mul(x[:, :d].cpu(), x[:, d:].cpu())
    assert_close(fg.silu_and_mul(x[:, :d], x[:, d:]).cpu(), ref, torch.bfloat16)
    out = torch.empty(512, d, dtype=torch.bfloat16, device=DEV)
    assert fg.silu_and_mul_out(x[:, :d], x[:, d:], out) is out
    assert_close(out.cpu(), ref, torch.bfloat16)
    assert_close(fg.GemsSiluAndMul()(x[:, :d], x[:, d:]).cpu(), ref, torch.bfloat16)
    # broadcasting and extreme inputs
    a = torch.randn(4, 1, 33, dtype=torch.float32, device=DEV) * 30
    b = torch.randn(5, 33, dtype=torch.float32, device=DEV)
    assert_close(fg.silu_and_mul(a, b).cpu(), O.silu_and_mul(a.cpu(), b.cpu()), torch.float32)
    # odd strides: transposed operand takes the strided kernel
    at = torch.randn(40, 24, dtype=torch.float16, device=DEV).t()
    bt = torch.randn(24, 40, dtype=torch.float16, device=DEV)
    assert_close(fg.silu_and_mul(at, bt).cpu(), O.silu_and_mul(at.cpu(), bt.cpu()), torch.float16)
    with pytest.raises(RuntimeError):
        fg.silu_and_mul_out(a, b, torch.empty(3, 3, device=DEV))
    e = fg.silu_and_mul(torch.empty(0, 8, device=DEV), torch.empty(0, 8, device=DEV))
    assert e.shape == (0, 8)


# ------------------------------------------------------------------ reshape_and_cache_flash
@pytest.mark.parametrize("head_size", [64, 80, 120, 256])
@pytest.mark.parametrize("block_size", [8, 16, 32])
@pytest.mark.parametrize("num_blocks", [128, 1000])
@pytest.mark.parametrize("dtype", [torch.half, torch.bfloat16, torch.float])
def test_reshape_and_cache_flash(fg, head_size, block_size, num_blocks, dtype):
    random.seed(2025)
    torch.manual_seed(2025)
    num_tokens, num_heads = 42, 8
    slots = torch.tensor(random.sample(range(num_blocks * block_size), num_tokens), dtype=torch.long, device=DEV)
    qkv = torch.randn(num_tokens, 3, num_heads, head_size, dtype=dtype, device=DEV)
    _, key, value = qkv.unbind(dim=1)  # strided views of a fused qkv, as vLLM passes them
    kv = torch.randn(2, num_blocks, block_size, num_heads, head_size, dtype=dtype, device=DEV)
    key_cache, value_cache = kv.unbind(0)
    ref_k, ref_v = key_cache.cpu().clone(), value_cache.cpu().clone()
    O.reshape_and_cache_flash(key.cpu(), value.cpu(), ref_k, ref_v, slots.cpu())
    assert fg.reshape_and_cache_flash(key, value, key_cache, value_cache, slots, "auto", None, None) is None
    assert torch.equal(key_cache.cpu(), ref_k) and torch.equal(value_cache.cpu(), ref_v)  # bit-exact


@pytest.mark.parametrize("head_size", [64, 80, 120, 256])
@pytest.mark.parametrize("block_size", [8, 16, 32])
@pytest.mark.parametrize("num_blocks", [128, 1000])
@pytest.mark.parametrize("dtype", [torch.half, torch.bfloat16, torch.float])
def test_reshape_and_cache_v0_layout(fg, head_size, block_size, num_blocks, dtype):
    # tests/test_attention_ops.py:1254-1324: K cache [blocks, heads, D/x, block, x], V cache [blocks, heads, D, block]
    random.seed(2025)
    torch.manual_seed(2025)
    num_tokens, num_heads = 42, 8
    x = 16 // torch.tensor([], dtype=dtype).element_size()
    slots = random.sample(range(num_blocks * block_size), num_tokens)
    slots[5] = -1  # a padded token
    slots = torch.tensor(slots, dtype=torch.long, device=DEV)
    qkv = torch.randn(num_tokens, 3, num_heads, head_size, dtype=dtype, device=DEV)
    _, key, value = qkv.unbind(dim=1)
    key_cache = torch.randn(num_blocks, num_heads, head_size // x, block_size, x, dtype=dtype, device=DEV)
    value_cache = torch.randn(num_blocks, num_heads, head_size, block_size, dtype=dtype, device=DEV)
    ref_k, ref_v = key_cache.cpu().clone(), value_cache.cpu().clone()
    O.reshape_and_cache(key.cpu(), value.cpu(), ref_k, ref_v, slots.cpu())
    assert fg.reshape_and_cache(key, value, key_cache, value_cache, slots, "auto", None, None) is None
    assert torch.equal(key_cache.cpu(), ref_k) and torch.equal(value_cache.cpu(), ref_v)  # bit-exact


def test_reshape_and_cache_flash_edges(fg, golden_dir):
    c = torch.load(golden_dir / "golden_reshape_and_cache_flash.pt", weights_only=False)
    kc, vc = c["key_cache"].to(DEV), c["value_cache"].to(DEV)
    torch.ops.flag_gems.reshape_and_cache_flash(c["key"].to(DEV), c["value"].to(DEV), kc, vc,
                                                c["slot_mapping"].to(DEV), "auto")
    assert torch.equal(kc.cpu(), c["key_cache_out"]) and torch.equal(vc.cpu(), c["value_cache_out"])
    # padding slots (-1) and slots beyond the cache are skipped; zero tokens is a no-op
    slots = c["slot_mapping"].clone()
    slots[::2] = -1
    slots[1] = 10 ** 9
    kc2, vc2 = c["key_cache"].to(DEV), c["value_cache"].to(DEV)
    fg.reshape_and_cache_flash(c["key"].to(DEV), c["value"].to(DEV), kc2, vc2, slots.to(DEV), "auto", None, None)
    rk, rv = c["key_cache"].clone(), c["value_cache"].clone()
    s2 = slots.clone()
    s2[1] = -1
    O.reshape_and_cache_flash(c["key"], c["value"], rk, rv, s2)
    assert torch.equal(kc2.cpu(), rk) and torch.equal(vc2.cpu(), rv)
    fg.reshape_and_cache_flash(c["key"][:0].to(DEV), c["value"][:0].to(DEV), kc2, vc2,
                               slots[:0].to(DEV), "auto", None, None)
    assert torch.equal(kc2.cpu(), rk)


def test_reshape_and_cache_flash_full_size_round_trip(fg):
    # Config-3 sized scatter (~34k tokens, 8 heads x 128): every token written through a
    # random permutation of slots must read back bit-exactly, untouched slots stay zero.
    torch.manual_seed(5)
    T, H, D, BS = 33800, 8, 128, 16
    NB = (T + BS - 1) // BS + 7
    key = torch.randn(T, H, D, dtype=torch.bfloat16, device=DEV)
    value = torch.randn(T, H, D, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(NB, BS, H, D, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(NB * BS, device=DEV)[:T]
    fg.reshape_and_cache_flash(key, value, kc, vc, slots, "auto", None, None)
    assert torch.equal(kc.view(-1, H, D)[slots], key) and torch.equal(vc.view(-1, H, D)[slots], value)
    untouched = torch.ones(NB * BS, dtype=torch.bool, device=DEV)
    untouched[slots] = False
    assert not kc.view(-1, H, D)[untouched].any() and not vc.view(-1, H, D)[untouched].any()
