"""Generate the golden fixtures in this folder from the reference checkout.

Run it on a machine that has the FlagGems tree:

    python tests/golden/make_golden.py --ref /path/to/FlagGems      (or FLAGGEMS_REF=/path/to/FlagGems)

FlagGems' test modules import ``flag_gems`` at the top, which needs a GPU, so they
cannot be imported on a CPU-only machine.  Their *oracle functions* are plain torch,
though: this script cuts those function definitions out of the reference's test files
with ``ast`` (no source is copied into this repository), executes them on seeded
inputs on the CPU, and stores inputs and outputs in ``golden_*.pt``.  The committed
fixtures pin ``oracle/reference_oracle.py`` (see ``tests/test_oracle_golden.py``) and
serve as fixed parity cases for the GPU tests.
"""
from __future__ import annotations

import argparse
import os
import ast
import random
import types
from pathlib import Path
from typing import List, Optional, Tuple  # noqa: F401  (names used by the extracted code)

import torch

HERE = Path(__file__).resolve().parent


def extract(path: Path, names, namespace):
    """exec the (possibly nested) function definitions called ``names`` from ``path``."""
    tree = ast.parse(path.read_text())
    found = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in names and node.name not in found:
            node.decorator_list = []
            found[node.name] = node
    missing = set(names) - set(found)
    if missing:
        raise SystemExit(f"{path}: oracle functions not found: {sorted(missing)}")
    mod = ast.Module(body=[found[n] for n in names], type_ignores=[])
    ast.fix_missing_locations(mod)
    exec(compile(mod, str(path), "exec"), namespace)
    return [namespace[n] for n in names]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("FLAGGEMS_REF"), required="FLAGGEMS_REF" not in os.environ,
                    help="root of the FlagGems checkout the oracle functions are cut out of")
    args = ap.parse_args()
    ref = Path(args.ref)
    stub = types.SimpleNamespace(vendor_name="nvidia", device="cpu")
    ns = {"torch": torch, "List": List, "Optional": Optional, "Tuple": Tuple, "flag_gems": stub,
          "TO_CPU": True}
    ref_paged_attn, attn_bias_from_alibi_slopes, torch_sdpa = extract(
        ref / "tests/test_attention_ops.py",
        ["ref_paged_attn", "attn_bias_from_alibi_slopes", "torch_sdpa"], ns)
    get_rope_cos_sin, _, _, torch_apply_rotary_pos_emb = extract(
        ref / "tests/test_special_ops.py",
        ["get_rope_cos_sin", "rotate_half", "rotate_interleave", "torch_apply_rotary_pos_emb"], ns)
    (_torch_fused_add_rms_norm,) = extract(ref / "tests/test_norm_ops.py", ["_torch_fused_add_rms_norm"], ns)

    # ------------------------------------------------------------ attention (paged)
    cases = []
    specs = [
        ("prefill_bf16", [(1, 200), (5, 18), (70, 131)], (4, 2), 64, 16, torch.bfloat16, False, None),
        ("prefill_fp16_softcap", [(1, 200), (5, 18), (70, 131)], (4, 2), 64, 16, torch.float16, False, 10.0),
        ("prefill_fp16_alibi", [(3, 90), (33, 33)], (4, 4), 64, 16, torch.float16, True, None),
        ("decode_bf16", [(1, 130), (1, 18), (1, 77)], (8, 2), 128, 16, torch.bfloat16, False, None),
        ("prefill_bf16_d128", [(40, 40), (17, 96)], (8, 2), 128, 32, torch.bfloat16, False, None),
    ]
    for name, seq_lens, heads, d, bs, dtype, alibi, cap in specs:
        torch.manual_seed(1234567890)
        qlens = [x[0] for x in seq_lens]
        klens = [x[1] for x in seq_lens]
        hq, hk = heads
        num_blocks = 12
        q = torch.randn(sum(qlens), hq, d, dtype=dtype)
        kc = torch.randn(num_blocks, bs, hk, d, dtype=dtype)
        vc = torch.randn_like(kc)
        maxb = (max(klens) + bs - 1) // bs
        bt = torch.randint(0, num_blocks, (len(seq_lens), maxb), dtype=torch.int32)
        scale = d ** -0.5
        slopes = bias = None
        if alibi:
            slopes = torch.ones(len(seq_lens), hq, dtype=torch.float32) * 0.3
            bias = attn_bias_from_alibi_slopes(slopes, max(qlens), max(klens), causal=True)
        out = ref_paged_attn(query=q, key_cache=kc, value_cache=vc, query_lens=qlens, kv_lens=klens,
                             block_tables=bt, scale=scale, attn_bias=bias, sliding_window=None, soft_cap=cap)
        cases.append(dict(name=name, q=q, key_cache=kc, value_cache=vc, query_lens=qlens, kv_lens=klens,
                          block_tables=bt, scale=scale, alibi_slopes=slopes, soft_cap=cap, out=out))
    torch.save(cases, HERE / "golden_paged_attn.pt")

    # ------------------------------------------------------------ dense SDPA (config-1 form, reduced)
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 2, 96, 64) for _ in range(3))
    out = torch_sdpa(q, k, v, 0.125, True)
    torch.save(dict(q=q, k=k, v=v, scale=0.125, out=out), HERE / "golden_sdpa.pt")

    # ------------------------------------------------------------ rope
    cases = []
    for dtype in (torch.bfloat16, torch.float32):
        for interleaved in (False, True):
            for use_pos in (False, True):
                torch.manual_seed(7)
                b, s, hq, hk, d, max_seq = 2, 8, 4, 2, 32, 16
                q = torch.randn(b, s, hq, d, dtype=dtype)
                k = torch.randn(b, s, hk, d, dtype=dtype)
                pos = torch.randint(0, max_seq, (b, s)) if use_pos else None
                cos, sin = get_rope_cos_sin(max_seq, d, dtype, device="cpu")
                qe, ke = torch_apply_rotary_pos_emb(q, k, cos, sin, pos, interleaved)
                cases.append(dict(q=q, k=k, cos=cos, sin=sin, position_ids=pos, interleaved=interleaved,
                                  max_seq=max_seq, q_out=qe, k_out=ke))
    torch.save(cases, HERE / "golden_rope.pt")

    # ------------------------------------------------------------ fused_add_rms_norm
    cases = []
    for dtype, shape in ((torch.bfloat16, (7, 256)), (torch.float16, (3, 520)), (torch.float32, (5, 77))):
        torch.manual_seed(11)
        x = torch.randn(shape, dtype=dtype)
        r = torch.randn(shape, dtype=dtype)
        w = torch.randn(shape[1], dtype=dtype)
        out, new_res = _torch_fused_add_rms_norm(x.double(), r.double(), weight=w.double(), eps=1e-5)
        cases.append(dict(x=x, residual=r, weight=w, eps=1e-5, out=out, new_residual=new_res))
    torch.save(cases, HERE / "golden_fused_add_rms_norm.pt")

    # ------------------------------------------------------------ reshape_and_cache_flash
    # the reference oracle is the in-test loop tests/test_attention_ops.py:1459-1467
    random.seed(2025)
    torch.manual_seed(2025)
    T, H, D, BS, NB = 10, 2, 24, 8, 6
    key = torch.randn(T, H, D, dtype=torch.float16)
    value = torch.randn(T, H, D, dtype=torch.float16)
    kc = torch.randn(NB, BS, H, D, dtype=torch.float16)
    vc = torch.randn(NB, BS, H, D, dtype=torch.float16)
    slot_mapping = torch.tensor(random.sample(range(NB * BS), T), dtype=torch.long)
    kc_out, vc_out = kc.clone(), vc.clone()
    blk = torch.div(slot_mapping, BS, rounding_mode="floor").tolist()
    off = (slot_mapping % BS).tolist()
    for i in range(T):
        kc_out[blk[i], off[i], :, :] = key[i]
        vc_out[blk[i], off[i], :, :] = value[i]
    torch.save(dict(key=key, value=value, key_cache=kc, value_cache=vc, slot_mapping=slot_mapping,
                    key_cache_out=kc_out, value_cache_out=vc_out), HERE / "golden_reshape_and_cache_flash.pt")

    # ------------------------------------------------------------ silu_and_mul / mm / addmm
    # oracles are one-line torch expressions: tests/test_binary_pointwise_ops.py:1386,
    # tests/test_blas_ops.py:38-44,129-132 (inputs upcast to float64)
    torch.manual_seed(3)
    x = torch.randn(5, 48, dtype=torch.bfloat16)
    y = torch.randn(5, 48, dtype=torch.bfloat16)
    silu = torch.mul(torch.nn.functional.silu(x.double()), y.double())
    a = torch.randn(15, 160, dtype=torch.float16)
    b = torch.randn(33, 160, dtype=torch.float16).t()
    bias = torch.randn(33, dtype=torch.float16)
    mm = torch.mm(a.double(), b.double())
    addmm = torch.addmm(bias.double(), a.double(), b.double(), alpha=-0.999, beta=-0.999)
    torch.save(dict(x=x, y=y, silu_and_mul=silu, a=a, b=b, bias=bias, alpha=-0.999, beta=-0.999, mm=mm,
                    addmm=addmm), HERE / "golden_pointwise_blas.pt")
    for f in sorted(HERE.glob("golden_*.pt")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
