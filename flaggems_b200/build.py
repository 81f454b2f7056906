"""Build recipe of the C-ABI library (``libflaggems_b200.so``).

The kernels are compiled with ``nvcc`` for sm_100a only and linked into one shared
object that sits inside the package (``flaggems_b200/lib``), so that it travels with
a copy of the source tree.  No torch headers are involved: the library's interface is
the plain C header ``include/flaggems_b200.h``.

Run ``python -m flaggems_b200.build`` (add ``--force`` to rebuild everything).
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libflaggems_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build flaggems_b200")
    return exe


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list((PKG_DIR.parent / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: Path, force: bool, hdr_mtime: float) -> tuple[Path, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_mtime):
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link ``libflaggems_b200.so``; returns its path."""
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    hdr_mtime = _newest_header_mtime()
    srcs = _sources()
    logs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(lambda s: _compile(s, force, hdr_mtime), srcs))
    objs = [o for o, _ in results]
    logs = [log for _, log in results if log]
    newest_obj = max(o.stat().st_mtime for o in objs)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest_obj:
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking libflaggems_b200.so failed:\n{r.stdout}\n{r.stderr}")
    if logs:
        (OBJ_DIR / "ptxas.log").write_text("\n".join(logs))
        if verbose:
            print("\n".join(logs))
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
