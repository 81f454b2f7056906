"""Loading and calling the unmodified reference (FlagGems, its Triton kernels) from
``baseline/_ref`` on a GPU box.  Used by the parity tests that compare this library with the
reference on the same GPU and by ``bench.py``'s Triton-path timings; nothing in the product
package imports it.

The reference's launcher keeps compiled kernels in a cache of its own and re-launches them
with the argument list of Triton 3.3-3.5 (``src/flag_gems/utils/libentry.py:883-903``); with
Triton 3.6 every call of an operator after its first fails with "function takes exactly N
arguments".  The first call of a kernel in a process goes through Triton's own launch path and
works, so ``forget()`` empties those caches (run-time state of the imported package; the
installed files are untouched) and every call takes the path that works.  Autotuning results
live elsewhere and are kept.
"""
from __future__ import annotations

import gc
import importlib
import sys
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"

_ref = None
_lib_entries = None


class ReferenceUnavailable(RuntimeError):
    pass


def load():
    """Import the reference package (once); raises ReferenceUnavailable with the reason."""
    global _ref
    if _ref is not None:
        return _ref
    if not (REF_DIR / "flag_gems").is_dir():
        raise ReferenceUnavailable("reference install baseline/_ref is not present")
    sys.path.insert(0, str(REF_DIR))
    try:
        import flag_gems
    except Exception as e:  # noqa: BLE001  (no GPU, Triton mismatch, ...)
        raise ReferenceUnavailable(f"reference does not import: {type(e).__name__}: {e}") from e
    finally:
        sys.path.remove(str(REF_DIR))
    _ref = flag_gems
    return _ref


def module_attr(module: str, name: str):
    """An attribute of a reference module fetched by module path (the packages re-export
    functions under the names of their modules, which hides the modules)."""
    load()
    return getattr(importlib.import_module(module), name)


def forget(rescan: bool = True):
    """Empty the reference launcher's per-device kernel caches (see the module docstring).
    The launcher objects are found by a scan of the garbage collector's object list; new ones
    appear when a reference module is first imported or generates a kernel, so a caller that
    has already run every operator once may pass ``rescan=False`` to reuse the last list."""
    global _lib_entries
    load()
    if rescan or _lib_entries is None:
        cls = importlib.import_module("flag_gems.utils.libentry").LibEntry
        _lib_entries = [o for o in gc.get_objects() if isinstance(o, cls)]
    for entry in _lib_entries:
        for dev_cache in entry.kernel_cache:
            dev_cache.clear()


def call(fn, *args, **kwargs):
    """``fn(*args, **kwargs)`` on a reference operator with the launcher caches emptied first."""
    forget()
    return fn(*args, **kwargs)
