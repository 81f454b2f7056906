"""Pin the CPU oracle against fixtures produced by the reference's own test oracles
(``tests/golden/make_golden.py`` ran them from the FlagGems checkout)."""
import torch

from oracle import reference_oracle as O


def _load(golden_dir, name):
    return torch.load(golden_dir / name, weights_only=False)


def test_paged_attention_matches_reference_oracle(golden_dir):
    for c in _load(golden_dir, "golden_paged_attn.pt"):
        bias = None
        if c["alibi_slopes"] is not None:
            bias = O.alibi_bias(c["alibi_slopes"], max(c["query_lens"]), max(c["kv_lens"]), causal=True)
        out = O.paged_attention(c["q"], c["key_cache"], c["value_cache"], c["query_lens"], c["kv_lens"],
                                c["block_tables"], c["scale"], attn_bias=bias, soft_cap=c["soft_cap"])
        # same formula, same dtype flow as ref_paged_attn -> identical results
        torch.testing.assert_close(out, c["out"], atol=0, rtol=0, msg=c["name"])
        # and the fp32 evaluation of the formula stays within the reference's own
        # tolerance (tests/test_attention_ops.py:990-992) of the input-dtype evaluation
        out32 = O.paged_attention(c["q"], c["key_cache"], c["value_cache"], c["query_lens"], c["kv_lens"],
                                  c["block_tables"], c["scale"], attn_bias=bias, soft_cap=c["soft_cap"],
                                  compute_dtype=torch.float32)
        torch.testing.assert_close(out32.float(), c["out"].float(), atol=2e-2, rtol=1e-2, msg=c["name"])


def test_sdpa_matches_reference_oracle(golden_dir):
    c = _load(golden_dir, "golden_sdpa.pt")
    out = O.sdpa_causal(c["q"], c["k"], c["v"], c["scale"])
    torch.testing.assert_close(out, c["out"], atol=2e-6, rtol=1e-5)


def test_sdpa_config1_matches_torch_sdpa():
    # Config 1 at full size; F.scaled_dot_product_attention is what the reference's
    # torch_sdpa calls (tests/test_attention_ops.py:200-229).
    from flaggems_b200 import workloads

    q, k, v, scale = workloads.sdpa_inputs(seed=0)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, scale=scale, is_causal=True)
    torch.testing.assert_close(O.sdpa_causal(q, k, v, scale), ref, atol=5e-6, rtol=1e-5)


def test_varlen_contiguous_equals_paged_form():
    from flaggems_b200 import workloads

    b = workloads.prefill_batch(seed=3, num_seqs=3, min_len=5, max_len=50, q_heads=4, kv_heads=2,
                                head_dim=32, block_size=8, dtype=torch.float32, device="cpu")
    a = O.paged_attention(b.q, b.key_cache, b.value_cache, b.query_lens, b.kv_lens, b.block_table, b.scale)
    c = O.varlen_attention(b.q, b.k, b.v, b.cu_seqlens_q, b.cu_seqlens_k, b.scale)
    torch.testing.assert_close(a, c, atol=1e-6, rtol=1e-6)


def test_rope_matches_reference_oracle(golden_dir):
    for c in _load(golden_dir, "golden_rope.pt"):
        cos, sin = O.rope_cos_sin(c["max_seq"], c["q"].shape[-1], c["q"].dtype)
        torch.testing.assert_close(cos, c["cos"], atol=0, rtol=0)
        torch.testing.assert_close(sin, c["sin"], atol=0, rtol=0)
        qe, ke = O.apply_rotary_pos_emb(c["q"], c["k"], c["cos"], c["sin"], c["position_ids"], c["interleaved"])
        torch.testing.assert_close(qe, c["q_out"], atol=0, rtol=0)
        torch.testing.assert_close(ke, c["k_out"], atol=0, rtol=0)


def test_fused_add_rms_norm_matches_reference_oracle(golden_dir):
    for c in _load(golden_dir, "golden_fused_add_rms_norm.pt"):
        out, res = O.fused_add_rms_norm(c["x"], c["residual"], c["weight"], c["eps"])
        torch.testing.assert_close(out, c["out"], atol=0, rtol=0)
        torch.testing.assert_close(res, c["new_residual"], atol=0, rtol=0)


def test_reshape_and_cache_flash_matches_reference_oracle(golden_dir):
    c = _load(golden_dir, "golden_reshape_and_cache_flash.pt")
    kc, vc = c["key_cache"].clone(), c["value_cache"].clone()
    O.reshape_and_cache_flash(c["key"], c["value"], kc, vc, c["slot_mapping"])
    assert torch.equal(kc, c["key_cache_out"]) and torch.equal(vc, c["value_cache_out"])
    # negative slots are padding: nothing is written
    kc2, vc2 = c["key_cache"].clone(), c["value_cache"].clone()
    O.reshape_and_cache_flash(c["key"], c["value"], kc2, vc2, torch.full_like(c["slot_mapping"], -1))
    assert torch.equal(kc2, c["key_cache"]) and torch.equal(vc2, c["value_cache"])


def test_pointwise_and_blas_match_reference_oracle(golden_dir):
    c = _load(golden_dir, "golden_pointwise_blas.pt")
    torch.testing.assert_close(O.silu_and_mul(c["x"], c["y"]), c["silu_and_mul"], atol=0, rtol=0)
    torch.testing.assert_close(O.mm(c["a"], c["b"]), c["mm"], atol=0, rtol=0)
    torch.testing.assert_close(O.addmm(c["bias"], c["a"], c["b"], c["alpha"], c["beta"]), c["addmm"], atol=0, rtol=0)


def _scheduler_kwargs(case):
    kw = dict(case["kwargs"])
    kw.pop("qkv_dtype")
    kw.pop("cu_seqlens_k")  # accepted and never read by the reference
    return kw


def test_scheduler_metadata_matches_reference_run(golden_dir):
    """The fixture holds the reference function's own results (its Triton kernels run under
    the interpreter, device queries answered as a B200)."""
    cases = _load(golden_dir, "golden_scheduler_metadata.pt")
    assert len(cases) >= 150
    for i, c in enumerate(cases):
        got = O.get_scheduler_metadata(sm_count=c["sm_count"], **_scheduler_kwargs(c))
        assert got.dtype == torch.int32 and torch.equal(got, c["metadata"]), i


def test_cache_oracles_replay_what_the_reference_tests_accepted(golden_dir):
    """``golden_cache_tests.pt``: inputs drawn by the reference's own ``test_reshape_and_cache`` and
    ``test_reshape_and_cache_flash`` and the caches those tests accepted (the tests ran from the
    reference checkout with the oracle standing in for the operator)."""
    cases = _load(golden_dir, "golden_cache_tests.pt")
    assert {c["layout"] for c in cases} == {"v0", "flash"} and len(cases) >= 7
    for c in cases:
        kc, vc = c["key_cache"].clone(), c["value_cache"].clone()
        fn = O.reshape_and_cache if c["layout"] == "v0" else O.reshape_and_cache_flash
        fn(c["key"], c["value"], kc, vc, c["slot_mapping"])
        assert torch.equal(kc, c["key_cache_out"]) and torch.equal(vc, c["value_cache_out"])
        assert not torch.equal(kc, c["key_cache"])
