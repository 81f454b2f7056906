"""flaggems_b200 -- the LLM-inference operator path of FlagGems rebuilt for NVIDIA B200.

The public surface follows ``flag_gems`` (``src/flag_gems/__init__.py``) for this path:
``enable()`` / ``use_gems()`` install ATen overrides for ``mm``, ``mm.out``, ``addmm``
and ``addmm.out`` on dispatch key CUDA; the fused operators, ``flash_attn_varlen_func``,
the ``torch.ops.flag_gems.*`` custom ops, the module wrappers and the vLLM patch
functions keep their reference names and signatures, so ``import flaggems_b200 as
flag_gems`` is a drop-in for code that uses only these operators.

Every operator is a hand-written sm_100a CUDA kernel reached through the C ABI of
``libflaggems_b200.so`` (``include/flaggems_b200.h``).  There is no Triton, no
autotuner, no multi-backend dispatch and no CPU fallback: a call on a CPU tensor, or
without the built library, raises.
"""
from __future__ import annotations

import logging

import torch

from . import testing  # noqa: F401
from . import _lib, config, custom_ops, dist, fused, modules, ops, patches  # noqa: F401
from .config import aten_patch_list
from .fused import *  # noqa: F401,F403
from .logging_utils import setup_flaggems_logging, teardown_flaggems_logging
from .modules import *  # noqa: F401,F403
from .ops import *  # noqa: F401,F403
from .patches import *  # noqa: F401,F403
from .register import Register

__version__ = "3.0+b200"
device = "cuda"
vendor_name = "nvidia"

registrar = Register
current_work_registrar = None
_aten_lib = None

custom_ops.register_custom_ops()


def _default_lib():
    global _aten_lib
    if _aten_lib is None:
        _aten_lib = torch.library.Library("aten", "IMPL")
    return _aten_lib


def _config():
    # (ATen key, implementation): the hot-path subset of the reference's table
    # (src/flag_gems/__init__.py:55-56, 213-214).
    return (
        ("addmm", ops.addmm),
        ("addmm.out", ops.addmm_out),
        ("mm", ops.mm),
        ("mm.out", ops.mm_out),
        ("bmm", ops.bmm),
        ("_flash_attention_forward", ops.flash_attention_forward),
    )


def enable(lib=None, unused=None, registrar=registrar, record=False, once=False, path=None):
    """Register the ATen overrides of this package on dispatch key CUDA.

    ``unused`` lists implementation function names to leave alone (e.g. ``["mm"]``);
    ``record/once/path`` control the operator-call log."""
    global current_work_registrar
    current_work_registrar = registrar(
        _config(),
        user_unused_ops_list=list(set(unused or [])),
        cpp_patched_ops_list=list(set(aten_patch_list)),
        lib=lib if lib is not None else _default_lib(),
    )
    setup_flaggems_logging(path=path, record=record, once=once)


class use_gems:
    """Scoped ``enable()``: the overrides live for the duration of the ``with`` block."""

    def __init__(self, unused=None, record=False, once=False, path=None):
        self.lib = torch.library.Library("aten", "IMPL")
        self.unused = [] if unused is None else unused
        self.registrar = Register
        self.record = record
        self.once = once
        self.path = path

    def __enter__(self):
        enable(lib=self.lib, unused=self.unused, registrar=self.registrar, record=self.record,
               once=self.once, path=self.path)

    def __exit__(self, exc_type, exc_val, exc_tb):
        global current_work_registrar
        self.lib._destroy()
        del self.lib
        current_work_registrar = None
        if self.record:
            teardown_flaggems_logging()


def all_ops():
    return current_work_registrar.get_all_ops()


__all__ = ["enable", "use_gems", "all_ops"] + fused.__all__ + ops.__all__ + modules.__all__ + patches.__all__
