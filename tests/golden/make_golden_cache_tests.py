"""Pin the two KV-cache oracles by running the reference's own test functions against them.

    python tests/golden/make_golden_cache_tests.py --ref /path/to/FlagGems   (or FLAGGEMS_REF=...)

``test_reshape_and_cache`` and ``test_reshape_and_cache_flash`` of the reference
(tests/test_attention_ops.py:1254-1330, :1390-1472) build their inputs, call
``flag_gems.reshape_and_cache[_flash]`` and compare the caches with an in-test loop.  Here the
two test functions (and the helpers they use) are cut out of the reference checkout with ``ast``
-- nothing is copied -- and executed on the CPU with ``flag_gems`` replaced by a stub whose two
operators are the functions of ``oracle/reference_oracle.py``.  A test that returns without an
assertion error means the reference's own check accepts the oracle; the inputs the test drew and the
caches it accepted are then stored in ``golden_cache_tests.pt`` for replay without the checkout.
"""
from __future__ import annotations

import argparse
import os
import random
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE))

from make_golden import extract  # noqa: E402
from oracle import reference_oracle as O  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("FLAGGEMS_REF"), required="FLAGGEMS_REF" not in os.environ)
    ref = Path(ap.parse_args().ref)
    record = []

    def capture(layout, fn):
        def op(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale, v_scale):
            before = (key_cache.clone(), value_cache.clone())
            fn(key, value, key_cache, value_cache, slot_mapping)
            record.append(dict(layout=layout, key=key.clone(), value=value.clone(), slot_mapping=slot_mapping.clone(),
                               key_cache=before[0], value_cache=before[1], key_cache_out=key_cache.clone(),
                               value_cache_out=value_cache.clone()))
        return op

    stub = types.SimpleNamespace(device="cpu", vendor_name="nvidia",
                                 reshape_and_cache=capture("v0", O.reshape_and_cache),
                                 reshape_and_cache_flash=capture("flash", O.reshape_and_cache_flash))
    ns = {"torch": torch, "random": random, "np": np, "flag_gems": stub, "device": "cpu"}
    extract(ref / "tests/accuracy_utils.py", ["init_seed"], ns)
    _, _, test_v0, test_flash = extract(
        ref / "tests/test_attention_ops.py",
        ["create_kv_caches_with_random", "create_kv_caches_with_random_flash", "test_reshape_and_cache",
         "test_reshape_and_cache_flash"], ns)
    # the reference's head sizes, block sizes and dtypes with few tokens, heads and blocks (its own
    # sizes would make a 100 MB fixture)
    for head_size, block_size, dtype in [(64, 8, torch.half), (80, 16, torch.bfloat16), (120, 8, torch.float),
                                         (256, 8, torch.half)]:
        test_v0(20, 2, head_size, block_size, 4, dtype, "auto", 2025)
    for head_size, block_size, dtype in [(64, 8, torch.half), (120, 16, torch.bfloat16), (256, 8, torch.float)]:
        test_flash(20, 2, head_size, block_size, 4, dtype, "auto", 2025)
    torch.save(record, HERE / "golden_cache_tests.pt")
    print(len(record), "cases accepted by the reference's tests;", (HERE / "golden_cache_tests.pt").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
