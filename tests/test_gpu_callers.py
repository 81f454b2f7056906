"""The callers of the operator path on the GPU: the module wrappers (``GemsRope``,
``gems_rope_forward``) and the functions vLLM's classes are patched with
(``custom_gems_rope_forward_cuda``, ``custom_gems_flash_attention_impl_forward``,
``custom_gems_write_to_paged_cache``, ``custom_silu_and_mul``, ``custom_gems_silu_and_mul``,
``custom_gems_rms_forward_cuda``), called with minimal stand-ins for ``self`` / ``layer`` /
``attn_metadata`` and checked against the CPU oracle -- and against vLLM's own
``RotaryEmbedding.forward_native`` / ``vllm_flash_attn`` when those can be used on the box.

Mirrors the reference's ``modules_tests/test_gems_rotary_embedding.py:20-86``,
``modules_tests/test_gems_attn.py:49-166`` and the patch bodies
``src/flag_gems/patches/patch_vllm_all.py:9-92,142-247``.
"""
from types import SimpleNamespace

import pytest
import torch

from flaggems_b200 import patches, workloads
from flaggems_b200.testing import assert_close
from oracle import reference_oracle as O  # checker only

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _vllm_rotary(head_size, rotary_dim, max_pos, base, is_neox_style, dtype):
    """vLLM's RotaryEmbedding when this vLLM can build one outside an engine, else None."""
    try:
        from vllm.config import VllmConfig, set_current_vllm_config
        from vllm.model_executor.layers.rotary_embedding import RotaryEmbedding

        with set_current_vllm_config(VllmConfig()):
            return RotaryEmbedding(head_size, rotary_dim, max_pos, base, is_neox_style, dtype)
    except Exception:  # noqa: BLE001
        return None


# ------------------------------------------------------------------------------------ GemsRope
@pytest.mark.parametrize("q_heads, k_heads", [(8, 1), (8, 8)])
@pytest.mark.parametrize("head_dim", [64, 128, 256])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rotary_interleaved", [True, False])
def test_gems_rope_module(fg, q_heads, k_heads, head_dim, dtype, rotary_interleaved):
    torch.manual_seed(42)
    batch, max_seq_len, base = 8, 2048, 10000
    seq_len = int(torch.randint(1, max_seq_len // 2, (1,)).item())
    query = torch.randn((batch, seq_len, q_heads, head_dim), dtype=dtype, device=DEV)
    key = torch.randn((batch, seq_len, k_heads, head_dim), dtype=dtype, device=DEV)
    position_ids = torch.randint(0, max_seq_len, (batch, seq_len), device=DEV)
    rope = fg.GemsRope(rotary_dim=head_dim, max_position_embeddings=max_seq_len, base=base,
                       rotary_interleaved=rotary_interleaved, dtype=dtype, device=DEV)
    assert rope.cos_cached.shape == (max_seq_len, head_dim // 2) and rope.cos_cached.dtype == dtype
    oc, os_ = O.rope_cos_sin(max_seq_len, head_dim, dtype, base)
    torch.testing.assert_close(rope.cos_cached.cpu().float(), oc.float(), atol=2e-3 if dtype == torch.float32 else 1e-2,
                               rtol=0)
    q_out, k_out = rope(query, key, position_ids=position_ids, inplace=False)
    assert q_out.data_ptr() != query.data_ptr() and q_out.shape == query.shape
    want_q, want_k = O.apply_rotary_pos_emb(query.cpu(), key.cpu(), rope.cos_cached.cpu(), rope.sin_cached.cpu(),
                                            position_ids.cpu(), rotary_interleaved)
    assert_close(q_out.cpu(), want_q, dtype)
    assert_close(k_out.cpu(), want_k, dtype)
    # in-place form: same numbers, written into the inputs
    q2, k2 = query.clone(), key.clone()
    rq, rk = rope(q2, k2, position_ids=position_ids, inplace=True)
    assert rq.data_ptr() == q2.data_ptr() and rk.data_ptr() == k2.data_ptr()
    assert torch.equal(q2, q_out) and torch.equal(k2, k_out)
    # vLLM's module on the same inputs (reference test: modules_tests/test_gems_rotary_embedding.py:49-83)
    vr = _vllm_rotary(head_dim, head_dim, max_seq_len, base, not rotary_interleaved, dtype)
    if vr is not None:
        vcos, vsin = vr.cos_sin_cache.to(DEV).chunk(2, dim=-1)
        assert_close(rope.cos_cached, vcos, dtype)
        assert_close(rope.sin_cached, vsin, dtype)
        vq, vk = vr.forward_native(position_ids, query.clone().view(batch, seq_len, -1),
                                   key.clone().view(batch, seq_len, -1))
        if dtype == torch.float32:   # the reference compares with vLLM in fp32 only: vLLM's native form rounds
            assert_close(q_out, vq.view_as(q_out), dtype)          # every intermediate to the tensor dtype
            assert_close(k_out, vk.view_as(k_out), dtype)
        else:
            torch.testing.assert_close(q_out.float(), vq.view_as(q_out).float(), atol=3e-2, rtol=2e-2)
            torch.testing.assert_close(k_out.float(), vk.view_as(k_out).float(), atol=3e-2, rtol=2e-2)


def test_gems_rope_forward_partial_rotary_dim_on_strided_slices(fg):
    """The vLLM calling form: the rotary slice of each head of a fused qkv buffer, in place."""
    torch.manual_seed(7)
    T, hq, hk, hd, rot = 96, 8, 2, 128, 64
    qkv = torch.randn((T, (hq + 2 * hk) * hd), dtype=torch.bfloat16, device=DEV)
    q = qkv[:, : hq * hd].view(T, hq, hd)
    k = qkv[:, hq * hd: (hq + hk) * hd].view(T, hk, hd)
    before = qkv.clone()
    cos, sin = (t.to(DEV) for t in O.rope_cos_sin(512, rot, torch.bfloat16))
    pos = torch.randint(0, 512, (T,), device=DEV)
    want_q, want_k = O.apply_rotary_pos_emb(q[..., :rot].cpu(), k[..., :rot].cpu(), cos.cpu(), sin.cpu(), pos.cpu())
    rq, rk = fg.gems_rope_forward(q[..., :rot], k[..., :rot], cos, sin, position_ids=pos, rotary_interleaved=False,
                                  inplace=True)
    assert_close(q[..., :rot].cpu(), want_q, torch.bfloat16)
    assert_close(k[..., :rot].cpu(), want_k, torch.bfloat16)
    # the pass-through tail of every head and the value part of the buffer are untouched
    assert torch.equal(q[..., rot:], before[:, : hq * hd].view(T, hq, hd)[..., rot:])
    assert torch.equal(k[..., rot:], before[:, hq * hd: (hq + hk) * hd].view(T, hk, hd)[..., rot:])
    assert torch.equal(qkv[:, (hq + hk) * hd:], before[:, (hq + hk) * hd:])
    # out of place on the same kind of views
    qkv2 = before.clone()
    q2 = qkv2[:, : hq * hd].view(T, hq, hd)
    k2 = qkv2[:, hq * hd: (hq + hk) * hd].view(T, hk, hd)
    oq, ok = fg.gems_rope_forward(q2[..., :rot], k2[..., :rot], cos, sin, position_ids=pos, inplace=False)
    assert torch.equal(qkv2, before)
    assert torch.equal(oq, q[..., :rot]) and torch.equal(ok, k[..., :rot])


# -------------------------------------------------------------- RotaryEmbedding.forward_cuda patch
@pytest.mark.parametrize("is_neox_style", [True, False])
@pytest.mark.parametrize("rotary_dim, head_size", [(128, 128), (64, 128), (32, 64)])
@pytest.mark.parametrize("use_offsets", [False, True])
def test_custom_gems_rope_forward_cuda(fg, is_neox_style, rotary_dim, head_size, use_offsets):
    torch.manual_seed(11)
    max_pos, T, hq, hk, dtype = 1024, 77, 8, 2, torch.bfloat16
    cos, sin = O.rope_cos_sin(max_pos, rotary_dim, dtype)
    self = SimpleNamespace(cos_sin_cache=torch.cat((cos, sin), dim=-1), head_size=head_size, rotary_dim=rotary_dim,
                           is_neox_style=is_neox_style)      # cache on the CPU: the patch moves it
    positions = torch.randint(0, max_pos // 2, (T,), device=DEV)
    offsets = torch.randint(0, max_pos // 2, (T,), device=DEV) if use_offsets else None
    query = torch.randn((T, hq * head_size), dtype=dtype, device=DEV)
    key = torch.randn((T, hk * head_size), dtype=dtype, device=DEV)
    q0, k0 = query.clone(), key.clone()
    out_q, out_k = patches.custom_gems_rope_forward_cuda(self, positions, query, key, offsets)
    assert out_q.shape == q0.shape and out_k.shape == k0.shape
    assert self.cos_sin_cache.device.type == "cuda"
    pos = positions + offsets if use_offsets else positions
    q3, k3 = q0.view(T, hq, head_size).cpu(), k0.view(T, hk, head_size).cpu()
    want_q, want_k = O.apply_rotary_pos_emb(q3[..., :rotary_dim], k3[..., :rotary_dim], cos, sin, pos.cpu(),
                                            not is_neox_style)
    got_q, got_k = out_q.view(T, hq, head_size).cpu(), out_k.view(T, hk, head_size).cpu()
    assert_close(got_q[..., :rotary_dim], want_q, dtype)
    assert_close(got_k[..., :rotary_dim], want_k, dtype)
    assert torch.equal(got_q[..., rotary_dim:], q3[..., rotary_dim:])
    assert torch.equal(got_k[..., rotary_dim:], k3[..., rotary_dim:])
    vr = _vllm_rotary(head_size, rotary_dim, max_pos, 10000, is_neox_style, dtype)
    if vr is not None and not use_offsets:
        vr.cos_sin_cache = vr.cos_sin_cache.to(DEV)
        vq, vk = vr.forward_native(positions, q0.clone(), k0.clone())
        # vLLM's native form rounds every intermediate to bf16: a bf16-sized tolerance
        torch.testing.assert_close(out_q.float(), vq.float(), atol=3e-2, rtol=2e-2)
        torch.testing.assert_close(out_k.float(), vk.float(), atol=3e-2, rtol=2e-2)


# -------------------------------------------------------------- FlashAttentionImpl.forward patch
def _attention_case(dtype, hq, hk, hd, block_size, seq_lens, seed=0, pad_tokens=3):
    """A mixed prefill + decode batch as vLLM v1 hands it to FlashAttentionImpl.forward: new
    tokens of every sequence packed in `query/key/value` (plus padding rows beyond
    num_actual_tokens), contexts already in the cache, the new tokens' slots in slot_mapping."""
    g = torch.Generator().manual_seed(seed)
    q_lens = [q for q, _ in seq_lens]
    kv_lens = [k for _, k in seq_lens]
    n = sum(q_lens)
    blocks = [(k + block_size - 1) // block_size for k in kv_lens]
    num_blocks = sum(blocks) + 5
    perm = torch.randperm(num_blocks, generator=g)
    bt = torch.zeros((len(seq_lens), max(blocks)), dtype=torch.int32)
    o = 0
    for i, nb in enumerate(blocks):
        bt[i, :nb] = perm[o:o + nb].to(torch.int32)
        o += nb
    kv_cache = torch.randn((2, num_blocks, block_size, hk, hd), generator=g, dtype=torch.float32).to(dtype)
    query = torch.randn((n + pad_tokens, hq, hd), generator=g, dtype=torch.float32).to(dtype)
    key = torch.randn((n + pad_tokens, hk, hd), generator=g, dtype=torch.float32).to(dtype)
    value = torch.randn((n + pad_tokens, hk, hd), generator=g, dtype=torch.float32).to(dtype)
    slots = []
    for i, (ql, kl) in enumerate(seq_lens):     # the new tokens are the last ql positions of each context
        for t in range(kl - ql, kl):
            slots.append(int(bt[i, t // block_size]) * block_size + t % block_size)
    slot_mapping = torch.tensor(slots + [-1] * pad_tokens, dtype=torch.int64)
    qsl = torch.zeros(len(seq_lens) + 1, dtype=torch.int32)
    qsl[1:] = torch.tensor(q_lens, dtype=torch.int32).cumsum(0)
    md = SimpleNamespace(num_actual_tokens=n, slot_mapping=slot_mapping, query_start_loc=qsl,
                         seq_lens=torch.tensor(kv_lens, dtype=torch.int32), max_query_len=max(q_lens),
                         max_seq_len=max(kv_lens), block_table=bt, use_cascade=False)
    return kv_cache, query, key, value, md, q_lens, kv_lens


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hq, hk, hd", [(8, 2, 128), (4, 4, 64), (16, 2, 256)])
def test_custom_gems_flash_attention_impl_forward(fg, dtype, hq, hk, hd):
    seq_lens = [(1, 1328), (5, 18), (129, 463), (1, 77), (200, 200)]
    kv_cache, query, key, value, md, q_lens, kv_lens = _attention_case(dtype, hq, hk, hd, 16, seq_lens, seed=hd)
    # oracle first, on CPU copies: scatter the new tokens, then attention over the cache
    kc, vc = kv_cache[0].clone(), kv_cache[1].clone()
    O.reshape_and_cache_flash(key, value, kc, vc, md.slot_mapping)
    n = md.num_actual_tokens
    scale = hd ** -0.5
    want = O.paged_attention(query[:n], kc, vc, q_lens, kv_lens, md.block_table, scale, compute_dtype=torch.float32)
    # the patched method on device tensors
    to = lambda t: t.to(DEV)
    md_dev = SimpleNamespace(**{k: (to(v) if torch.is_tensor(v) else v) for k, v in vars(md).items()})
    self = SimpleNamespace(kv_cache_dtype="auto", scale=scale, alibi_slopes=None, sliding_window=(-1, -1),
                           logits_soft_cap=0.0, use_irope=False)
    layer = SimpleNamespace(_k_scale=None, _v_scale=None)
    kv_dev = to(kv_cache)
    output = torch.full((query.shape[0], hq, hd), 7.0, dtype=dtype, device=DEV)
    ret = patches.custom_gems_flash_attention_impl_forward(self, layer, to(query), to(key), to(value), kv_dev, md_dev,
                                                           output=output)
    assert ret is output
    assert torch.equal(kv_dev[0].cpu(), kc) and torch.equal(kv_dev[1].cpu(), vc)       # cache write: bit-exact
    torch.testing.assert_close(output[:n].cpu().float(), want.float(), atol=2e-2, rtol=1e-2)
    assert (output[n:] == 7.0).all()                                                  # padding rows are not written
    # profiling run (no metadata) returns the output untouched
    assert patches.custom_gems_flash_attention_impl_forward(self, layer, to(query), to(key), to(value), kv_dev, None,
                                                            output=output) is output
    # vLLM's FlashAttention-2 on the same cache, when it runs on this GPU
    try:
        import vllm.vllm_flash_attn.flash_attn_interface as vfa

        vout = vfa.flash_attn_varlen_func(
            q=to(query)[:n], k=kv_dev[0], v=kv_dev[1], max_seqlen_q=md.max_query_len, cu_seqlens_q=md_dev.query_start_loc,
            max_seqlen_k=md.max_seq_len, seqused_k=md_dev.seq_lens, softmax_scale=scale, causal=True,
            window_size=[-1, -1], block_table=md_dev.block_table, fa_version=2)
    except Exception:  # noqa: BLE001  (no FA2 build for this GPU, other signature, ...)
        vout = None
    if vout is not None:
        torch.testing.assert_close(output[:n].float(), vout.float(), atol=2e-2, rtol=1e-2)


def test_custom_gems_flash_attention_impl_forward_rejects_what_the_reference_rejects(fg):
    kv_cache, query, key, value, md, _, _ = _attention_case(torch.bfloat16, 8, 2, 128, 16, [(4, 40)])
    self = SimpleNamespace(kv_cache_dtype="auto", scale=0.1, alibi_slopes=None, sliding_window=(-1, -1),
                           logits_soft_cap=0.0, use_irope=False)
    layer = SimpleNamespace()
    with pytest.raises(AssertionError, match="Output tensor must be provided"):
        patches.custom_gems_flash_attention_impl_forward(self, layer, query, key, value, kv_cache, md)
    with pytest.raises(NotImplementedError, match="output quantization"):
        patches.custom_gems_flash_attention_impl_forward(self, layer, query, key, value, kv_cache, md,
                                                         output=query, output_scale=torch.ones(1))
    md.use_cascade = True
    to = lambda t: t.to(DEV)
    md_dev = SimpleNamespace(**{k: (to(v) if torch.is_tensor(v) else v) for k, v in vars(md).items()})
    with pytest.raises(NotImplementedError, match="Cascade"):
        patches.custom_gems_flash_attention_impl_forward(self, layer, to(query), to(key), to(value), to(kv_cache),
                                                         md_dev, output=torch.empty_like(to(query)))


# -------------------------------------------------------------- PagedAttention.write_to_paged_cache patch
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_custom_gems_write_to_paged_cache(fg, dtype):
    torch.manual_seed(2025)
    T, H, D, bs, nb = 42, 8, 128, 16, 64
    x = 16 // torch.tensor([], dtype=dtype).element_size()
    key = torch.randn((T, H, D), dtype=dtype)
    value = torch.randn((T, H, D), dtype=dtype)
    key_cache = torch.randn((nb, H, D // x, bs, x), dtype=dtype)
    value_cache = torch.randn((nb, H, D, bs), dtype=dtype)
    slot_mapping = torch.randperm(nb * bs)[:T].to(torch.int64).view(T, 1)       # vLLM passes it unflattened
    slot_mapping[5] = -1
    want_k, want_v = key_cache.clone(), value_cache.clone()
    O.reshape_and_cache(key, value, want_k, want_v, slot_mapping.flatten())
    kc, vc = key_cache.to(DEV), value_cache.to(DEV)
    patches.custom_gems_write_to_paged_cache(key.to(DEV), value.to(DEV), kc, vc, slot_mapping.to(DEV), "auto",
                                             None, None)
    assert torch.equal(kc.cpu(), want_k) and torch.equal(vc.cpu(), want_v)


# -------------------------------------------------------------- SiluAndMul / _C.silu_and_mul / RMSNorm patches
def test_custom_silu_and_mul_patches(fg):
    x = workloads.silu_inputs(seed=9, T=33, width=2 * 1408, device=DEV)
    d = x.shape[-1] // 2
    want = O.silu_and_mul(x[:, :d].cpu(), x[:, d:].cpu())
    out = torch.empty((33, d), dtype=x.dtype, device=DEV)
    assert patches.custom_silu_and_mul(out, x) is None          # torch.ops._C.silu_and_mul(out, input)
    assert_close(out.cpu(), want, x.dtype)
    got = patches.custom_gems_silu_and_mul(SimpleNamespace(), x)   # SiluAndMul.forward_cuda(self, x)
    assert torch.equal(got, out)
    x3 = x.view(3, 11, 2 * d)                                     # leading batch dims
    assert torch.equal(patches.custom_gems_silu_and_mul(SimpleNamespace(), x3), out.view(3, 11, d))


def test_custom_gems_rms_forward_cuda_patch(fg):
    x, r, w, eps = workloads.norm_inputs(seed=10, T=37, hidden=2048, device=DEV)
    self = SimpleNamespace(weight=w, variance_epsilon=eps)
    want_o, want_r = O.fused_add_rms_norm(x.cpu(), r.cpu(), w.cpu(), eps)
    want_plain = O.rms_norm(x.cpu(), w.cpu(), eps)
    plain = patches.custom_gems_rms_forward_cuda(self, x)          # RMSNorm.forward_cuda(self, x)
    assert_close(plain.cpu(), want_plain, x.dtype)
    o, res = patches.custom_gems_rms_forward_cuda(self, x, r)      # ... (self, x, residual): in place on both
    assert o.data_ptr() == x.data_ptr() and res.data_ptr() == r.data_ptr()
    assert_close(x.cpu(), want_o, x.dtype)
    assert_close(r.cpu(), want_r, x.dtype)
