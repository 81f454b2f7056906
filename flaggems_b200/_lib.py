"""ctypes binding of the C-ABI library ``libflaggems_b200.so``.

The structures mirror ``include/flaggems_b200.h`` field for field.  There is no other
route to the kernels: if the shared object is missing, loading raises and every
operator of the package fails loudly (there is no CPU or eager fallback).
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import torch

FG_F32, FG_F16, FG_BF16 = 0, 1, 2
ABI_VERSION = 2

_DTYPE_CODE = {torch.float32: FG_F32, torch.float16: FG_F16, torch.bfloat16: FG_BF16}

_LIB = None
_LIB_LOCK = threading.Lock()


def library_path() -> Path:
    env = os.environ.get("FLAGGEMS_B200_LIB")
    if env:
        return Path(env)
    return Path(__file__).resolve().parent / "lib" / "libflaggems_b200.so"


class RopeParams(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in ("q", "k", "q_out", "k_out", "cos", "sin", "positions")]
        + [(n, C.c_int64) for n in (
            "num_tokens", "q_heads", "k_heads", "head_dim",
            "q_stride_t", "q_stride_h", "q_stride_d",
            "k_stride_t", "k_stride_h", "k_stride_d",
            "qo_stride_t", "qo_stride_h", "qo_stride_d",
            "ko_stride_t", "ko_stride_h", "ko_stride_d",
            "pos_stride", "cos_stride", "sin_stride", "seq_len", "max_positions")]
        + [(n, C.c_int32) for n in ("pos_is_i64", "interleaved", "dtype", "cos_dtype")]
    )


class GemmParams(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in ("a", "b", "bias", "c")]
        + [(n, C.c_int64) for n in (
            "M", "N", "K", "a_stride0", "a_stride1", "b_stride0", "b_stride1",
            "bias_stride0", "bias_stride1", "c_stride0", "c_stride1")]
        + [("alpha", C.c_double), ("beta", C.c_double), ("dtype", C.c_int32), ("reserved", C.c_int32)]
    )


class AttnParams(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in (
            "q", "k", "v", "out", "lse", "cu_seqlens_q", "cu_seqlens_k", "seqused_k",
            "block_table", "alibi_slopes", "workspace")]
        + [(n, C.c_int64) for n in (
            "workspace_bytes",
            "q_row_stride", "q_head_stride",
            "k_row_stride", "k_head_stride", "k_block_stride",
            "v_row_stride", "v_head_stride", "v_block_stride",
            "o_row_stride", "o_head_stride",
            "block_table_stride", "alibi_batch_stride",
            "total_q", "batch", "num_heads", "num_heads_k", "head_dim",
            "max_seqlen_q", "max_seqlen_k", "block_size", "num_blocks",
            "window_left", "window_right", "total_k",
            "q_batch_stride", "k_batch_stride", "v_batch_stride", "o_batch_stride")]
        + [("softmax_scale", C.c_double), ("softcap", C.c_double)]
        + [(n, C.c_int32) for n in ("causal", "dtype", "num_splits", "reserved")]
    )


class GemmPlan(C.Structure):
    _fields_ = ([(n, C.c_int32) for n in ("tile_m", "tile_n", "grid", "group_m")]
                + [(n, C.c_int64) for n in ("tiles_m", "tiles_n", "full_units", "num_units")])


class SchedulerParams(C.Structure):
    _fields_ = (
        [(n, C.c_int32) for n in (
            "batch_size", "max_seqlen_q", "max_seqlen_k", "num_heads", "num_heads_k", "headdim", "headdim_v",
            "elem_size", "page_size", "max_seqlen_k_new", "is_causal", "window_size_left", "window_size_right",
            "has_softcap", "num_splits", "pack_gqa", "sm_margin", "arch", "num_sm", "varlen_q", "has_leftpad")]
        + [(n, C.c_void_p) for n in (
            "seqused_k", "cu_seqlens_q", "cu_seqlens_k", "cu_seqlens_k_new", "seqused_q", "leftpad_k")]
    )


class SchedulerPlan(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "num_splits", "pack_gqa", "block_m", "block_n", "use_dynamic_split", "is_causal", "is_local",
        "q_per_kv", "heads", "metadata_len")]


_I64 = C.c_int64
_P = C.c_void_p
_PI64 = C.POINTER(C.c_int64)

# name -> (restype, argtypes); the CPU-side symbol test walks this table too.
SIGNATURES = {
    "fg_abi_version": (C.c_int, []),
    "fg_last_error": (C.c_char_p, []),
    "fg_launch_count": (C.c_int64, []),
    "fg_device_status": (C.c_int, [C.c_int]),
    "fg_device_status_nosync": (C.c_int, []),
    "fg_debug_set_status": (C.c_int, [C.c_int]),
    "fg_debug_wait_timeout": (C.c_int, [C.c_int64, C.c_void_p, C.c_void_p]),
    "fg_copy_2d": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "fg_set_num_sms": (C.c_int, [C.c_int]),
    "fg_get_num_sms": (C.c_int, []),
    "fg_fused_add_rms_norm": (C.c_int, [_P, _P, _P, _I64, _I64, _I64, _I64, C.c_double, C.c_int, _P]),
    "fg_rms_norm": (C.c_int, [_P, _P, _P, _I64, _I64, _I64, _I64, C.c_double, C.c_int, _P]),
    "fg_silu_and_mul": (C.c_int, [_P, _P, _P, C.c_int, _PI64, _PI64, _PI64, _PI64, C.c_int, _P]),
    "fg_gelu_and_mul": (C.c_int, [_P, _P, _P, C.c_int, _PI64, _PI64, _PI64, _PI64, C.c_int, C.c_int, _P]),
    "fg_rotary_embedding": (C.c_int, [C.POINTER(RopeParams), _P]),
    "fg_reshape_and_cache_flash": (C.c_int, [_P, _P, _P, _P, _P] + [_I64] * 10 + [C.c_int, _P]),
    "fg_reshape_and_cache": (C.c_int, [_P, _P, _P, _P, _P] + [_I64] * 8 + [C.c_int, _P]),
    "fg_gemm": (C.c_int, [C.POINTER(GemmParams), _P]),
    "fg_gemm_batched": (C.c_int, [C.POINTER(GemmParams)] + [_I64] * 5 + [_P]),
    "fg_gemm_uses_tcgen05": (C.c_int, [C.POINTER(GemmParams)]),
    "fg_gemm_f32_split_workspace_bytes": (_I64, [C.POINTER(GemmParams)]),
    "fg_gemm_f32_split": (C.c_int, [C.POINTER(GemmParams), _P, _I64, _P]),
    "fg_gemm_tile_plan": (C.c_int, [C.POINTER(GemmParams), _I64, C.c_int, C.POINTER(GemmPlan)]),
    "fg_flash_attn_varlen": (C.c_int, [C.POINTER(AttnParams), _P]),
    "fg_flash_attn_workspace_bytes": (C.c_int64, [_I64] * 5),
    "fg_flash_attn_path": (C.c_int, [C.POINTER(AttnParams)]),
    "fg_flash_attn_decode_static": (C.c_int, [C.POINTER(AttnParams), _P]),
    "fg_flash_attn_decode_static_capacity": (C.c_int64, []),
    "fg_scheduler_plan": (C.c_int, [C.POINTER(SchedulerParams), C.POINTER(SchedulerPlan)]),
    "fg_get_scheduler_metadata": (C.c_int, [C.POINTER(SchedulerParams), _P, _P]),
}


def load():
    """Load (once) and return the ctypes handle of the C-ABI library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LIB_LOCK:
        if _LIB is not None:
            return _LIB
        path = library_path()
        if not path.exists():
            raise RuntimeError(
                f"flaggems_b200: the CUDA library {path} is missing. Build it with "
                "`python -m flaggems_b200.build`; there is no fallback path."
            )
        lib = C.CDLL(str(path))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        if lib.fg_abi_version() != ABI_VERSION:
            raise RuntimeError(
                f"flaggems_b200: ABI mismatch (library {lib.fg_abi_version()}, bindings {ABI_VERSION}); rebuild"
            )
        _LIB = lib
        return lib


def check(rc: int) -> None:
    """Turn a negative return code into the RuntimeError the reference would raise."""
    if rc < 0:
        msg = load().fg_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"flaggems_b200: {msg} (code {rc})")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise RuntimeError(f"flaggems_b200: unsupported dtype {dtype}") from None


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "flaggems_b200 operators run on CUDA tensors only; there is no CPU fallback "
                f"(got a tensor on {t.device})"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"flaggems_b200: tensors on different devices ({dev} and {t.device})")
    return dev


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def set_num_sms(sms: int) -> None:
    """Limit the persistent kernels to ``sms`` SMs (0 = all); see ``fg_set_num_sms``."""
    check(load().fg_set_num_sms(int(sms)))


def launch_count() -> int:
    return int(load().fg_launch_count())


def device_status(reset: bool = False) -> int:
    """Status word of the current device (0 = healthy); synchronises with the device."""
    rc = load().fg_device_status(1 if reset else 0)
    check(rc)
    return rc


def device_status_nosync() -> int:
    """The host-visible copy of the status word (no synchronisation).  Every launching entry
    point of the library checks it itself and fails with FG_ERR_DEVICE while it is set, which
    the wrappers of this package raise as RuntimeError."""
    return int(load().fg_device_status_nosync())
