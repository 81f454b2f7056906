"""Host-side logic that needs no GPU: registration filter, the enable()/use_gems() API
surface, custom-op schemas, kernel-path selection, shard helpers and the no-fallback rule."""
import ctypes
import logging

import pytest
import torch

import flaggems_b200 as fg
from flaggems_b200 import _lib, custom_ops, dist as fdist
from flaggems_b200.register import Register


class _FakeLib:
    def __init__(self):
        self.calls = []

    def impl(self, key, fn, dispatch_key):
        self.calls.append((key, fn.__name__, dispatch_key))


def test_register_filters_unused_and_native_keys():
    cfg = (("mm", fg.mm), ("mm.out", fg.mm_out), ("addmm", fg.addmm), ("addmm.out", fg.addmm_out))
    lib = _FakeLib()
    r = Register(cfg, user_unused_ops_list=["mm"], cpp_patched_ops_list=["addmm.out"], lib=lib)
    assert r.get_all_ops() == ["mm.out", "addmm"]
    assert lib.calls == [("mm.out", "mm_out", "CUDA"), ("addmm", "addmm", "CUDA")]
    assert r.get_unused_ops() == ["mm"] and r.get_vendor_name() == "nvidia" and r.get_current_device() == "cuda"


def test_enable_and_use_gems_surface(tmp_path):
    assert fg.device == "cuda" and fg.vendor_name == "nvidia" and fg.__version__.startswith("3.0")
    lib = _FakeLib()
    log = tmp_path / "oplist.log"
    fg.enable(lib=lib, unused=["addmm_out"], record=True, once=True, path=str(log))
    assert fg.all_ops() == ["addmm", "mm", "mm.out", "bmm", "_flash_attention_forward"]
    logging.getLogger("flag_gems.ops").debug("GEMS TEST RECORD")
    fg.logging_utils.teardown_flaggems_logging()
    assert "GEMS TEST RECORD" in log.read_text()
    # the scoped form registers on a private Library and destroys it on exit; CPU
    # tensors are untouched by CUDA-key overrides
    with fg.use_gems():
        assert set(fg.all_ops()) == {"mm", "mm.out", "addmm", "addmm.out", "bmm", "_flash_attention_forward"}
        a = torch.randn(3, 4)
        torch.testing.assert_close(torch.mm(a, a.t()), a @ a.t())
    for name in ("flash_attn_varlen_func", "reshape_and_cache_flash", "fused_add_rms_norm", "apply_rotary_pos_emb",
                 "silu_and_mul", "silu_and_mul_out", "mm", "mm_out", "addmm", "addmm_out", "flash_attention_forward", "GemsRMSNorm", "GemsRope",
                 "GemsSiluAndMul", "apply_gems_patches_to_vllm", "gems_rms_forward", "gems_rope_forward"):
        assert callable(getattr(fg, name)), name
    assert callable(fg.ops.flash_attn_varlen_func) and callable(fg.testing.assert_close)


def test_custom_op_schemas_match_the_reference_strings():
    for name in ("fused_add_rms_norm", "rotary_embedding_inplace", "rotary_embedding", "reshape_and_cache_flash",
                 "flash_attn_varlen_func", "mm", "addmm", "rms_norm"):
        op = getattr(torch.ops.flag_gems, name)
        schema = str(op.default._schema)
        assert schema.startswith(f"flag_gems::{name}(")
    s = str(torch.ops.flag_gems.flash_attn_varlen_func.default._schema)
    assert "SymInt max_seqlen_q, Tensor cu_seqlens_q, SymInt max_seqlen_k" in s and "SymInt fa_version=2" in s
    s = str(torch.ops.flag_gems.reshape_and_cache_flash.default._schema)
    assert "Tensor(a!) key_cache, Tensor(b!) value_cache" in s and "str kv_cache_dtype" in s
    far = torch.ops.flag_gems.fused_add_rms_norm.default._schema
    assert [a.name for a in far.arguments] == ["input", "residual", "weight", "epsilon"]
    assert [bool(a.alias_info and a.alias_info.is_write) for a in far.arguments] == [True, True, False, False]
    assert len(far.returns) == 0
    assert set(custom_ops.SCHEMAS) == set(custom_ops._IMPLS)


def test_no_cpu_fallback():
    x = torch.randn(4, 8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fg.fused_add_rms_norm(x, x.clone(), [8], torch.ones(8))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fg.silu_and_mul(x, x)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fg.mm(x, x.t())
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fg.reshape_and_cache_flash(torch.zeros(1, 1, 8), torch.zeros(1, 1, 8), torch.zeros(1, 4, 1, 8),
                                   torch.zeros(1, 4, 1, 8), torch.zeros(1, dtype=torch.long), "auto", None, None)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("FLAGGEMS_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_LIB", None)
    with pytest.raises(RuntimeError, match="missing"):
        _lib.load()


def _gemm_params(M, N, K, dtype=_lib.FG_BF16, a_strides=None, b_strides=None, base=0x7f0000000000):
    p = _lib.GemmParams()
    p.a, p.b, p.c = base, base + (1 << 30), base + (2 << 30)
    p.M, p.N, p.K = M, N, K
    p.a_stride0, p.a_stride1 = a_strides or (K, 1)
    p.b_stride0, p.b_stride1 = b_strides or (N, 1)
    p.c_stride0, p.c_stride1 = N, 1
    p.dtype = dtype
    return p


def test_gemm_path_selection_is_pure_host_logic():
    uses = lambda p: _lib.load().fg_gemm_uses_tcgen05(ctypes.byref(p))
    assert uses(_gemm_params(8192, 6144, 4096)) == 1
    assert uses(_gemm_params(8192, 6144, 4096, b_strides=(1, 4096))) == 1       # column-major B
    assert uses(_gemm_params(8192, 6144, 4096, a_strides=(1, 8192))) == 1       # column-major A
    assert uses(_gemm_params(8192, 6144, 4096, dtype=_lib.FG_F32)) == 0         # fp32: CUDA-core path
    assert uses(_gemm_params(495, 5333, 71)) == 0                               # rows not 16-byte multiples
    assert uses(_gemm_params(1, 1, 32)) == 0
    assert uses(_gemm_params(8192, 6144, 4096, base=0x7f0000000002)) == 0       # misaligned base


def test_f32_split_workspace_is_pure_host_logic():
    """fg_gemm_f32_split_workspace_bytes: 0 when fg_gemm should take the problem, else a 256-byte
    flag block plus three bf16 pieces per operand with the leading dimension rounded up to 8."""
    need = lambda p: _lib.load().fg_gemm_f32_split_workspace_bytes(ctypes.byref(p))
    up = lambda v, m: (v + m - 1) // m * m
    f32 = _lib.FG_F32
    assert need(_gemm_params(4096, 4096, 4096, dtype=f32)) == 256 + 2 * 3 * 4096 * 4096 * 2
    # odd sizes: A [1000, 1300] row-major -> 1000 rows of 1304; B [1300, 1111] row-major -> 1300 rows of 1112
    assert need(_gemm_params(1000, 1111, 1300, dtype=f32)) == 256 + up(3 * 1000 * 1304 * 2, 256) + up(3 * 1300 * 1112 * 2, 256)
    # column-major A [1000, 1300] (stride0 == 1): 1300 rows of 1000
    assert need(_gemm_params(1000, 1111, 1300, dtype=f32, a_strides=(1, 1000))) == \
        256 + up(3 * 1300 * 1000 * 2, 256) + up(3 * 1300 * 1112 * 2, 256)
    assert need(_gemm_params(4096, 4096, 4096)) == 0                              # bf16: fg_gemm's tensor-core kernel
    assert need(_gemm_params(512, 1024, 512, dtype=f32)) == 0                     # M*N*K below 2^29
    assert need(_gemm_params(512, 1024, 1024, dtype=f32)) > 0
    assert need(_gemm_params(4096, 4096, 127, dtype=f32)) == 0                    # a dimension below 128
    assert need(_gemm_params(4096, 4096, 4096, dtype=f32, a_strides=(8192, 2))) == 0   # no unit stride
    p = _gemm_params(4096, 4096, 4096, dtype=f32)
    p.c_stride0, p.c_stride1 = 1, 4096
    assert need(p) == 0                                                           # column-major output
    assert _lib.load().fg_gemm_f32_split(ctypes.byref(p), None, 0, None) == -2    # FG_ERR_UNSUPPORTED, nothing launched


def test_three_bf16_pieces_carry_an_fp32_value_exactly():
    """The arithmetic of the fp32 tensor-core GEMM's split pass (csrc/gemm_f32_split_sm100.cu, split3_kernel),
    restated with numpy: hi = bf16(x) rounded to nearest even (truncated when rounding would overflow to
    infinity), mid = bf16(x - hi), lo = x - hi - mid.  The three pieces must add up to x exactly and be bf16
    values (the third one outside the denormal range), and the three piece products the kernel drops must stay below 2^-22 of |a b|."""
    import numpy as np

    def bf16_rn(x):                                   # float32 -> nearest-even bfloat16, kept as float32
        u = x.astype(np.float32).view(np.uint32).astype(np.uint64)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
        return r.view(np.float32)

    def split3(x):
        with np.errstate(over="ignore", invalid="ignore"):
            hi = bf16_rn(x)
            trunc = (x.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
            hi = np.where(np.isinf(hi), trunc, hi)
            r1 = x - hi
            mid = bf16_rn(r1)
            lo = r1 - mid
        return hi, mid, lo

    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32),
        (rng.standard_normal(50000) * 1e30).astype(np.float32),
        (rng.standard_normal(50000) * 1e-30).astype(np.float32),
        np.array([3.4e38, -3.4e38, 3.3895314e38, 1.0, -1.0, 0.0, 1.0 + 2.0 ** -23, 255.99998, 2.0 ** -100], np.float32),
        rng.integers(0x00800000, 0x7F7FFFFF, 200000, dtype=np.uint32).view(np.float32),     # every exponent and mantissa
    ])
    hi, mid, lo = split3(x)
    for piece in (hi, mid, lo):
        assert np.all(np.isfinite(piece))
    assert np.array_equal(hi.astype(np.float64) + mid.astype(np.float64) + lo.astype(np.float64), x.astype(np.float64))
    is_bf16 = lambda v: (v.view(np.uint32) & 0xFFFF) == 0
    assert np.all(is_bf16(hi)) and np.all(is_bf16(mid))
    # the third piece is a bfloat16 value too unless it falls into the denormal range (|x| below 2^-100 or so);
    # there the kernel's final rounding of it costs less than the denormal spacing 2^-133
    big = np.abs(x) >= 2.0 ** -100
    assert np.all(is_bf16(lo[big]))
    assert np.max(np.abs(bf16_rn(lo).astype(np.float64) - lo.astype(np.float64))) <= 2.0 ** -134
    # the kernel multiplies hi*hi, hi*mid, mid*hi, hi*lo, lo*hi, mid*mid; what it leaves out:
    a, b = x[:200000].astype(np.float64), x[200000 - 1::-1][:200000].astype(np.float64)
    ah, am, al = (v[:200000].astype(np.float64) for v in (hi, mid, lo))
    bh, bm, bl = (v[200000 - 1::-1][:200000].astype(np.float64) for v in (hi, mid, lo))
    kept = ah * bh + ah * bm + am * bh + ah * bl + al * bh + am * bm
    assert np.max(np.abs(a * b - kept) / np.abs(a * b)) < 2.0 ** -22


def test_attention_path_selection():
    def params(max_q, batch, total_q, hq=32, hk=8, d=128, alibi=False, wl=-1):
        p = _lib.AttnParams()
        p.max_seqlen_q, p.max_seqlen_k, p.batch, p.total_q = max_q, 4096, batch, total_q
        p.num_heads, p.num_heads_k, p.head_dim = hq, hk, d
        p.window_left, p.window_right = wl, -1
        p.alibi_slopes = 0x1000 if alibi else None
        p.causal, p.dtype = 1, _lib.FG_BF16
        return p
    path = lambda p: _lib.load().fg_flash_attn_path(ctypes.byref(p))
    assert path(params(1, 256, 256)) == 2            # single-token decode -> split-KV kernel
    assert path(params(1, 256, 256, alibi=True)) == 0
    assert path(params(1, 256, 256, wl=128)) == 0
    assert path(params(1, 256, 256, hq=64, hk=2)) == 0   # 32 query heads per KV head exceed one MMA tile
    assert path(params(4096, 16, 30000)) in (0, 1)
    ws = _lib.load().fg_flash_attn_workspace_bytes
    assert ws(256, 32, 128, 1, 8192) == 32 * 256 * 32 * 129 * 4
    assert ws(256, 32, 128, 1, 200) == 0 and ws(16, 32, 128, 4096, 4096) == 0


def test_shard_helpers():
    assert [fdist.shard_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    qs, ks = fdist.kv_head_shard(32, 8, 3, 4)
    assert (qs.start, qs.stop, ks.start, ks.stop) == (24, 32, 6, 8)
    with pytest.raises(ValueError):
        fdist.kv_head_shard(32, 8, 0, 3)
    w = torch.arange(24.0).reshape(2, 12).repeat(1, 4)  # [2, 48]
    parts = [fdist.column_shard(w, torch.arange(48.0), r, 2) for r in range(2)]
    assert torch.equal(torch.cat([p[0] for p in parts], dim=1), w)
    assert torch.equal(torch.cat([p[1] for p in parts]), torch.arange(48.0))
    with pytest.raises(ValueError):
        fdist.column_shard(torch.zeros(2, 20), None, 0, 2)
    assert fdist.all_gather_columns(w, 1) is w


def test_workload_generators_are_seeded_and_consistent():
    from flaggems_b200 import workloads

    a = workloads.prefill_batch(seed=9, num_seqs=4, min_len=3, max_len=60, q_heads=4, kv_heads=2, head_dim=16,
                                block_size=8, dtype=torch.float32, device="cpu")
    b = workloads.prefill_batch(seed=9, num_seqs=4, min_len=3, max_len=60, q_heads=4, kv_heads=2, head_dim=16,
                                block_size=8, dtype=torch.float32, device="cpu")
    assert a.query_lens == b.query_lens and torch.equal(a.q, b.q) and torch.equal(a.block_table, b.block_table)
    # the paged cache holds exactly the packed K/V rows
    cu = a.cu_seqlens_q.tolist()
    for i, n in enumerate(a.kv_lens):
        pages = a.block_table[i, : (n + 7) // 8].long()
        rows = a.key_cache[pages].reshape(-1, 2, 16)[:n]
        assert torch.equal(rows, a.k[cu[i]:cu[i + 1]])
    d = workloads.decode_batch(seed=9, batch=5, min_ctx=9, max_ctx=70, q_heads=4, kv_heads=2, head_dim=16,
                               block_size=8, dtype=torch.float32, device="cpu")
    for i, n in enumerate(d.kv_lens):
        assert d.slot_mapping[i] == d.block_table[i, (n - 1) // 8] * 8 + (n - 1) % 8
    assert len(set(d.block_table[d.block_table > 0].tolist())) == int((d.block_table > 0).sum())  # disjoint pages
    assert workloads.prefill_flops([4], q_heads=1, head_dim=1) == 4 * 10


def test_scheduler_plan_matches_the_oracle_plan():
    """fg_scheduler_plan is host arithmetic: it runs without a GPU and must agree with the
    restated reference heuristics on every field."""
    import random

    from oracle import reference_oracle as O

    rng = random.Random(5)
    for _ in range(3000):
        hk = rng.choice([1, 2, 4, 8, 16])
        hq = hk * rng.choice([1, 2, 4, 7, 8, 16])
        d = rng.choice([32, 64, 72, 96, 128, 160, 192, 256])
        dv = rng.choice([d, d, 64, 128, 256, 512])
        args = (rng.choice([1, 2, 17, 128, 300, 992, 993, 100000]), rng.choice([1, 1, 2, 7, 64, 128, 500, 40000]),
                rng.choice([16, 100, 512, 3000, 8192, 70000, 5000000]), hq, hk, d, dv)
        kw = dict(page_size=rng.choice([None, None, 16, 64, 128, 256]), max_seqlen_k_new=rng.choice([0, 0, 3, 200]),
                  is_causal=rng.random() < 0.5, window_size_left=rng.choice([-1, -1, 0, 100, 5000]),
                  window_size_right=rng.choice([-1, -1, 0, 50]), has_softcap=rng.random() < 0.2,
                  num_splits=rng.choice([0, 0, 0, 1, 2, 4, 300]), pack_gqa=rng.choice([None, None, True, False]),
                  varlen_q=rng.random() < 0.3, has_leftpad=rng.random() < 0.2)
        margin = rng.choice([0, 0, 8, 100])
        a = fg.scheduler_plan(*args, sm_margin=margin, **kw)
        b = O.scheduler_plan(*args, num_sm=148 - margin, **kw)
        got = (a["num_splits"], bool(a["pack_gqa"]), a["block_m"], a["block_n"], bool(a["use_dynamic_split"]),
               bool(a["is_causal"]), bool(a["is_local"]), a["q_per_kv"], a["heads"])
        want = (b["num_splits"], b["pack_gqa"], b["block_m"], b["block_n"], b["dynamic"], b["causal"], b["local"],
                b["q_per_kv"], b["heads"])
        assert got == want, (args, margin, kw)
        assert a["metadata_len"] == 1 + (args[0] if args[0] <= 992 else 0)
    # argument errors of the reference (ops/get_scheduler_metadata.py:596-603) and the sm_100a-only rule
    with pytest.raises(AssertionError, match="fp16 and bf16"):
        fg.scheduler_plan(4, 1, 512, 8, 8, 128, 128, torch.float32)
    with pytest.raises(AssertionError, match="must divide"):
        fg.scheduler_plan(4, 1, 512, 9, 4, 128, 128)
    with pytest.raises(RuntimeError, match="below 9.0"):
        fg.scheduler_plan(4, 1, 512, 8, 8, 128, 128, arch=80)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fg.get_scheduler_metadata(2, 1, 512, 8, 8, 128, 128, torch.bfloat16, torch.tensor([5, 9], dtype=torch.int32))


def test_gemm_tile_plan_covers_every_output_block_once():
    """fg_gemm_tile_plan is the host half of the tensor-core GEMM launch: tile shape, persistent
    grid and work units (whole tiles, then 128-row halves of the tiles of a last wave that fills at
    most half of the SMs).  Walking the units the way the kernel does must touch every 128-row
    block of every column tile of every batch member exactly once."""
    lib = _lib.load()

    def plan(M, N, K, batch=1, sms=148, **kw):
        out = _lib.GemmPlan()
        p = _gemm_params(M, N, K, **kw)
        rc = lib.fg_gemm_tile_plan(ctypes.byref(p), batch, sms, ctypes.byref(out))
        return rc, out

    def walk(pl, M, batch):
        seen = {}
        tiles_per_batch = pl.tiles_m * pl.tiles_n
        halves = pl.tile_m // 128
        for cta in range(pl.grid):
            for u in range(cta, pl.num_units, pl.grid):
                if halves == 1 or u < pl.full_units:
                    tile, h0, nh = u, 0, halves
                else:
                    r = u - pl.full_units
                    tile, h0, nh = pl.full_units + r // 2, r % 2, 1
                bi, t = divmod(tile, tiles_per_batch)
                per_group = pl.group_m * pl.tiles_n          # grouped order of the kernel's tile_coords
                g = t // per_group
                first_m = g * pl.group_m
                rows = min(pl.tiles_m - first_m, pl.group_m)
                r = t - g * per_group
                tm, tn = first_m + r % rows, r // rows
                for h in range(h0, h0 + nh):
                    key = (bi, tm * halves + h, tn)
                    seen[key] = seen.get(key, 0) + 1
        blocks_m = pl.tiles_m * halves
        assert len(seen) == batch * blocks_m * pl.tiles_n and set(seen.values()) == {1}
        assert blocks_m * 128 >= M

    cases = [(8192, 28672, 4096, 1), (8192, 6144, 4096, 1), (8192, 4096, 14336, 1), (8192, 4096, 4096, 1),
             (2100, 4608, 512, 1), (2048, 28672, 256, 1), (129, 264, 72, 1), (300, 16, 4096, 1), (1024, 1024, 1024, 32),
             (1000, 520, 264, 7), (4096, 4096, 4096, 1), (8192, 4096, 512, 1)]
    for M, N, K, batch in cases:
        for sms in (148, 132, 20):
            rc, pl = plan(M, N, K, batch, sms)
            assert rc == 0, (M, N, K, batch, sms)
            assert pl.tile_n == 256 and pl.tile_m in (128, 256) and 1 <= pl.grid <= sms
            assert pl.tiles_m == -(-M // pl.tile_m) and pl.tiles_n == -(-N // 256)
            assert pl.full_units <= pl.num_units and (pl.num_units - pl.full_units) % 2 == 0
            # halves only for 256-row tiles, at most one per CTA, after whole waves
            if pl.num_units > pl.full_units:
                assert pl.tile_m == 256 and pl.full_units % pl.grid == 0 and pl.num_units - pl.full_units <= pl.grid
            walk(pl, M, batch)
    # the benchmark projections take the big tile; the last wave of o / down (68 tiles) is halved
    rc, pl = plan(8192, 4096, 4096)
    assert (pl.tile_m, pl.full_units, pl.num_units) == (256, 444, 444 + 136)
    # column-major A keeps the 128-row tile; the generic kernel's problems have no plan
    rc, pl = plan(8192, 6144, 4096, a_strides=(1, 8192))
    assert rc == 0 and pl.tile_m == 128
    assert plan(495, 5333, 71)[0] == -2 and plan(8192, 6144, 4096, 0)[0] == -1
