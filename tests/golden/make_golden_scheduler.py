"""Generate ``golden_scheduler_metadata.pt`` by running the reference's own
``get_scheduler_metadata`` on the CPU.

    python tests/golden/make_golden_scheduler.py --ref /path/to/FlagGems   (or FLAGGEMS_REF=...)

The reference function launches two small Triton kernels and asks the device for its
compute capability and SM count.  Here the kernels run under Triton's interpreter
(``TRITON_INTERPRET=1``, CPU tensors) and the two device queries are answered with the
values of a B200: capability (10, 0) and 148 SMs.  The module is loaded from the
reference checkout by path; nothing of it is copied.  Every case stores the keyword
arguments and the int32 result.
"""
from __future__ import annotations

import argparse
import importlib.util
import itertools
import os
import types
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent
SM_COUNT = 148


def load_reference(ref: Path):
    torch.cuda.get_device_capability = lambda device=None: (10, 0)
    torch.cuda.get_device_properties = lambda device=None: types.SimpleNamespace(multi_processor_count=SM_COUNT)
    spec = importlib.util.spec_from_file_location("reference_scheduler_metadata",
                                                  ref / "src/flag_gems/ops/get_scheduler_metadata.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cases():
    g = torch.Generator().manual_seed(42)
    rnd = lambda lo, hi, n: torch.randint(lo, hi, (n,), dtype=torch.int32, generator=g)
    base = dict(max_seqlen_q=1, num_heads=32, num_heads_k=8, qkv_dtype=torch.float16, cu_seqlens_q=None,
                cu_seqlens_k=None, cu_seqlens_k_new=None, seqused_q=None, leftpad_k=None, page_size=None,
                max_seqlen_k_new=0, is_causal=False, window_size_left=-1, window_size_right=-1, has_softcap=False,
                num_splits=0, pack_gqa=True, sm_margin=0)
    # the grid of the reference's own test (tests/test_attention_ops.py:1618-1695)
    for b, sk, d, ns in itertools.product([1, 8, 256, 512], [512, 2048], [64, 128], [0, 4]):
        yield dict(base, batch_size=b, max_seqlen_k=sk, headdim=d, headdim_v=d, num_splits=ns, seqused_k=rnd(1, sk, b))
    # the shapes of its benchmark (benchmark/test_attention_perf.py:417-423): pack_gqa left to the heuristic
    for b, sq, sk, hq, hk, d, dv in [(8, 8, 1024, 16, 4, 128, 128), (32, 32, 512, 8, 8, 64, 64),
                                    (256, 256, 2048, 32, 32, 128, 128), (512, 512, 4096, 32, 8, 128, 128),
                                    (1024, 1024, 8192, 64, 16, 128, 128)]:
        yield dict(base, batch_size=b, max_seqlen_q=sq, max_seqlen_k=sk, num_heads=hq, num_heads_k=hk, headdim=d,
                   headdim_v=dv, pack_gqa=None, seqused_k=rnd(1, sk + 1, b))
    # paged decode of the benchmark configuration and its neighbours
    for b, sk, page, causal in itertools.product([3, 64, 256, 992, 993], [8192, 32768], [None, 16, 128], [False, True]):
        yield dict(base, batch_size=b, max_seqlen_k=sk, headdim=128, headdim_v=128, page_size=page, is_causal=causal,
                   pack_gqa=None, seqused_k=rnd(sk // 16, sk + 1, b))
    # head dims across the tile table, margins, windows, soft-cap, MHA
    for d, dv in [(32, 32), (64, 256), (64, 512), (80, 80), (96, 96), (128, 128), (160, 160), (192, 128), (192, 192),
                  (256, 256)]:
        for extra in [dict(), dict(window_size_left=255, window_size_right=0), dict(is_causal=True, page_size=64),
                      dict(sm_margin=20, has_softcap=True)]:
            yield dict(base, batch_size=5, max_seqlen_k=16384, headdim=d, headdim_v=dv, pack_gqa=None,
                       seqused_k=rnd(1, 16385, 5), **extra)
    for hq, hk in [(8, 8), (32, 32), (64, 8), (28, 4)]:
        yield dict(base, batch_size=7, max_seqlen_k=20000, num_heads=hq, num_heads_k=hk, headdim=128, headdim_v=128,
                   pack_gqa=None, seqused_k=rnd(1, 20001, 7))
        yield dict(base, batch_size=7, max_seqlen_q=40, max_seqlen_k=20000, num_heads=hq, num_heads_k=hk, headdim=128,
                   headdim_v=128, pack_gqa=False, is_causal=True, seqused_k=rnd(1, 20001, 7))
    # ragged queries, explicit query lengths, left padding, appended keys
    for b in (4, 130):
        ql = rnd(1, 300, b)
        cu = torch.cat([torch.zeros(1, dtype=torch.int32), ql.cumsum(0).to(torch.int32)])
        yield dict(base, batch_size=b, max_seqlen_q=int(ql.max()), max_seqlen_k=6000, headdim=128, headdim_v=128,
                   pack_gqa=None, is_causal=True, cu_seqlens_q=cu, seqused_k=rnd(300, 6001, b))
        yield dict(base, batch_size=b, max_seqlen_q=300, max_seqlen_k=6000, headdim=128, headdim_v=128,
                   pack_gqa=None, is_causal=True, seqused_q=ql, page_size=16, seqused_k=rnd(300, 6001, b))
        yield dict(base, batch_size=b, max_seqlen_k=6000, headdim=128, headdim_v=128, page_size=16,
                   leftpad_k=rnd(0, 100, b), seqused_k=rnd(300, 6001, b))
        yield dict(base, batch_size=b, max_seqlen_k=6000, headdim=64, headdim_v=64, max_seqlen_k_new=5,
                   seqused_k=rnd(300, 6001, b))
        kn = rnd(1, 9, b)
        yield dict(base, batch_size=b, max_seqlen_k=6000, headdim=128, headdim_v=128, max_seqlen_k_new=8,
                   cu_seqlens_k_new=torch.cat([torch.zeros(1, dtype=torch.int32), kn.cumsum(0).to(torch.int32)]),
                   seqused_k=rnd(300, 6001, b))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("FLAGGEMS_REF"), required="FLAGGEMS_REF" not in os.environ)
    ref = load_reference(Path(ap.parse_args().ref))
    out = []
    for kw in cases():
        res = ref.get_scheduler_metadata(**kw)
        out.append(dict(kwargs=kw, sm_count=SM_COUNT, metadata=res.to(torch.int32).clone()))
    torch.save(out, HERE / "golden_scheduler_metadata.pt")
    print(len(out), "cases", (HERE / "golden_scheduler_metadata.pt").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
