"""The C-ABI library loads on a machine without a GPU and exports every symbol that
``include/flaggems_b200.h`` declares (no compute call is made here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "flaggems_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"FG_API\s+[\w\s\*]+?\b(fg_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("fg_fused_add_rms_norm", "fg_silu_and_mul", "fg_rotary_embedding", "fg_reshape_and_cache_flash",
                 "fg_gemm", "fg_flash_attn_varlen", "fg_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from flaggems_b200 import _lib

    path = _lib.library_path()
    assert path.exists(), f"{path} missing: run python -m flaggems_b200.build"
    lib = ctypes.CDLL(str(path))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_bindings_cover_the_header():
    from flaggems_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()
    lib = _lib.load()
    assert lib.fg_abi_version() == _lib.ABI_VERSION
    assert lib.fg_last_error() == b""
    assert lib.fg_launch_count() == 0 or lib.fg_launch_count() > 0


def test_struct_sizes_match_the_header():
    # sizeof of each parameter block, computed from the header's field list
    from flaggems_b200 import _lib

    assert ctypes.sizeof(_lib.RopeParams) == 7 * 8 + 21 * 8 + 4 * 4
    assert ctypes.sizeof(_lib.GemmParams) == 4 * 8 + 11 * 8 + 2 * 8 + 2 * 4
    assert ctypes.sizeof(_lib.AttnParams) == 11 * 8 + 29 * 8 + 2 * 8 + 4 * 4


def test_argument_errors_are_reported_without_a_gpu():
    from flaggems_b200 import _lib

    lib = _lib.load()
    # invalid arguments are rejected on the host, before any CUDA call
    rc = lib.fg_silu_and_mul(None, None, None, 9, None, None, None, None, 0, None)
    assert rc == -1
    assert b"ndim" in lib.fg_last_error()
    with pytest.raises(RuntimeError, match="ndim"):
        _lib.check(rc)
    p = _lib.GemmParams()
    p.M, p.N, p.K = 4, 4, -1
    assert lib.fg_gemm(ctypes.byref(p), None) == -1
