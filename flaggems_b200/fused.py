"""Fused memory-bound operators of the inference path.

Same names, argument meaning and error behaviour as ``flag_gems.fused``
(``src/flag_gems/fused/__init__.py``); each function validates on the host, then
enqueues one sm_100a kernel through the C ABI on the tensor's device and current
stream.
"""
from __future__ import annotations

import ctypes as C
import logging
import math
from typing import Optional

import torch

from . import _lib

logger = logging.getLogger("flag_gems." + __name__.split(".")[-1])

__all__ = [
    "fused_add_rms_norm",
    "apply_rotary_pos_emb",
    "silu_and_mul",
    "silu_and_mul_out", "gelu_and_mul",
    "reshape_and_cache_flash",
    "reshape_and_cache",
]


# ---------------------------------------------------------------------------
# fused_add_rms_norm  (src/flag_gems/fused/fused_add_rms_norm.py:57-82)
# ---------------------------------------------------------------------------
def _rows_view(t: torch.Tensor, n: int):
    """``(rows, row_stride)`` when ``t`` is a stack of rows of ``n`` unit-stride elements
    under one uniform row stride (torch's own view rules decide), else None."""
    if n == 0 or t.numel() == 0:
        return 0, n
    try:
        t2 = t.view(-1, n)
    except RuntimeError:
        return None
    if n > 1 and t2.stride(1) != 1:
        return None
    return t2.shape[0], (t2.stride(0) if t2.shape[0] > 1 else n)


def fused_add_rms_norm(x, residual, normalized_shape, weight, eps=1e-5):
    """In place: ``residual += x`` then ``x = rmsnorm(residual) * weight``.

    Returns ``(x, residual)``.  The reference makes non-contiguous inputs contiguous
    first, which silently drops the in-place update for them
    (fused_add_rms_norm.py:74-76); here row-strided views are updated in place and
    anything that cannot be described as rows raises.
    """
    logger.debug(
        "GEMS FUSED_ADD_RMS_NORM FORWARD, [input shape]: %s, [residual shape]: %s, [weight shape]: %s",
        x.size(), residual.size(), weight.size(),
    )
    dev = _lib.require_cuda(x, residual, weight)
    if x.shape != residual.shape:
        raise RuntimeError("fused_add_rms_norm: input and residual must have the same shape")
    if x.dtype != residual.dtype or x.dtype != weight.dtype:
        raise RuntimeError("fused_add_rms_norm: input, residual and weight must share a dtype")
    N = math.prod(normalized_shape)
    if tuple(x.shape[x.ndim - len(normalized_shape):]) != tuple(normalized_shape):
        raise RuntimeError("fused_add_rms_norm: normalized_shape does not match the trailing dims of input")
    if weight.numel() != N:
        raise RuntimeError("fused_add_rms_norm: weight must have prod(normalized_shape) elements")
    weight = weight.contiguous()
    xv, rv = _rows_view(x, N), _rows_view(residual, N)
    if xv is None or rv is None:
        raise RuntimeError("fused_add_rms_norm: input and residual must be row-strided views (unit inner stride)")
    M = x.numel() // N if N else 0
    with torch.cuda.device(dev):
        _lib.check(_lib.load().fg_fused_add_rms_norm(
            x.data_ptr(), residual.data_ptr(), weight.data_ptr(), M, N, xv[1], rv[1], float(eps),
            _lib.dtype_code(x.dtype), _lib.stream_ptr(dev)))
    return x, residual


# ---------------------------------------------------------------------------
# apply_rotary_pos_emb  (src/flag_gems/fused/rotary_embedding.py:181-312)
# ---------------------------------------------------------------------------
def apply_rotary_pos_emb(
    q, k, cos, sin,
    position_ids: Optional[torch.Tensor] = None,
    rotary_interleaved: bool = False,
    inplace: bool = False,
):
    """Apply rotary position embedding to q ``(*, q_heads, head_dim)`` and k
    ``(*, k_heads, head_dim)``; cos/sin are ``(max_seq_len, head_dim // 2)``.

    Returns ``(q_embed, k_embed)`` shaped like the inputs (the inputs themselves when
    ``inplace``)."""
    logger.debug("GEMS ROTARY_POS_EMBEDDING")
    dev = _lib.require_cuda(q, k, cos, sin, position_ids)
    assert k.shape[-1] == q.shape[-1], (
        f"q and k must have the same last dimension, got {q.shape} and {k.shape}")
    assert cos.shape[-1] == sin.shape[-1], (
        f"cos and sin must have the same last dimension, got {cos.shape} and {sin.shape}")
    assert cos.shape[-1] * 2 == q.shape[-1], (
        f"cos/sin dim must be half of q/k dim, got {cos.shape} and {q.shape}")
    assert cos.stride(-1) == 1, "cos must be contiguous at the last dimension"
    assert sin.stride(-1) == 1, "sin must be contiguous at the last dimension"
    q_shape, k_shape = q.shape, k.shape
    assert q.shape[:-2] == k.shape[:-2], (
        f"q and k must have the same length, got {q.shape[:-2]} and {k.shape[:-2]}")
    if position_ids is None:
        assert len(q.shape) == 4, (
            f"q must have 4 dimensions if position_ids is not provided, got {q.shape}")
        seq_len = q.shape[-3]
    else:
        assert position_ids.shape == q.shape[:-2], (
            f"position_ids must have the same length as q, got {position_ids.shape} and {q.shape[:-2]}")
        position_ids = position_ids.reshape(-1)
        if position_ids.dtype not in (torch.int64, torch.int32):
            raise RuntimeError("position_ids must be int32 or int64")
        seq_len = 0
    if q.dtype != k.dtype:
        raise RuntimeError("apply_rotary_pos_emb: q and k must share a dtype")
    if cos.dtype != sin.dtype:
        raise RuntimeError("apply_rotary_pos_emb: cos and sin must share a dtype")
    if cos.dim() != 2 or sin.dim() != 2:
        cos = cos.reshape(-1, cos.shape[-1])
        sin = sin.reshape(-1, sin.shape[-1])

    q3 = q.view(-1, q.shape[-2], q.shape[-1])
    k3 = k.view(-1, k.shape[-2], k.shape[-1])
    n_tokens, q_heads, head_dim = q3.shape
    if inplace:
        qo, ko = q3, k3
    else:
        qo = torch.empty_like(q3)
        ko = torch.empty_like(k3)

    p = _lib.RopeParams()
    p.q, p.k, p.q_out, p.k_out = q3.data_ptr(), k3.data_ptr(), qo.data_ptr(), ko.data_ptr()
    p.cos, p.sin = cos.data_ptr(), sin.data_ptr()
    p.positions = None if position_ids is None else position_ids.data_ptr()
    p.num_tokens, p.q_heads, p.k_heads, p.head_dim = n_tokens, q_heads, k3.shape[1], head_dim
    p.q_stride_t, p.q_stride_h, p.q_stride_d = q3.stride()
    p.k_stride_t, p.k_stride_h, p.k_stride_d = k3.stride()
    p.qo_stride_t, p.qo_stride_h, p.qo_stride_d = qo.stride()
    p.ko_stride_t, p.ko_stride_h, p.ko_stride_d = ko.stride()
    p.pos_stride = 0 if position_ids is None else position_ids.stride(0)
    p.cos_stride, p.sin_stride = cos.stride(0), sin.stride(0)
    p.seq_len = seq_len
    p.max_positions = cos.shape[0]
    p.pos_is_i64 = 1 if (position_ids is not None and position_ids.dtype == torch.int64) else 0
    p.interleaved = 1 if rotary_interleaved else 0
    p.dtype = _lib.dtype_code(q.dtype)
    p.cos_dtype = _lib.dtype_code(cos.dtype)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().fg_rotary_embedding(C.byref(p), _lib.stream_ptr(dev)))
    return qo.view(q_shape), ko.view(k_shape)


# ---------------------------------------------------------------------------
# silu_and_mul  (src/flag_gems/fused/silu_and_mul.py:12-53)
# ---------------------------------------------------------------------------
def _silu_and_mul_launch(A, B, out, gelu=None):
    """``gelu``: None for silu, else the ``approximate`` string of gelu_and_mul."""
    dev = _lib.require_cuda(A, B, out)
    shape = out.shape
    if len(shape) > 6:
        raise RuntimeError("silu_and_mul: more than 6 dimensions are not supported")
    Ae, Be = A.expand(shape), B.expand(shape)
    nd = len(shape)
    arr = C.c_int64 * max(nd, 1)
    with torch.cuda.device(dev):
        if gelu is None:
            _lib.check(_lib.load().fg_silu_and_mul(
                Ae.data_ptr(), Be.data_ptr(), out.data_ptr(), nd,
                arr(*shape), arr(*Ae.stride()), arr(*Be.stride()), arr(*out.stride()),
                _lib.dtype_code(out.dtype), _lib.stream_ptr(dev)))
        else:
            _lib.check(_lib.load().fg_gelu_and_mul(
                Ae.data_ptr(), Be.data_ptr(), out.data_ptr(), nd,
                arr(*shape), arr(*Ae.stride()), arr(*Be.stride()), arr(*out.stride()),
                1 if gelu == "tanh" else 0, _lib.dtype_code(out.dtype), _lib.stream_ptr(dev)))
    return out


def _promote(A, B):
    dt = torch.result_type(A, B)
    if dt not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError(f"silu_and_mul: unsupported dtype {dt}")
    if A.dtype != dt:
        A = A.to(dt)
    if B.dtype != dt:
        B = B.to(dt)
    return A, B, dt


def silu_and_mul(A, B):
    """``silu(A) * B`` with broadcasting; the result has the promoted dtype of A and B."""
    logger.debug("GEMS SILU AND MUL FORWARD")
    _lib.require_cuda(A, B)
    A, B, dt = _promote(A, B)
    shape = torch.broadcast_shapes(A.shape, B.shape)
    out = torch.empty(shape, dtype=dt, device=A.device)
    return _silu_and_mul_launch(A, B, out)


def gelu_and_mul(x, y, approximate="none"):
    """``gelu(x, approximate) * y`` with broadcasting (forward of
    ``src/flag_gems/fused/gelu_and_mul.py:95-139``; the reference's autograd backward is
    not part of the inference path: tensors that require grad are refused)."""
    logger.debug("GEMS GELU AND MUL FORWARD")
    if approximate not in ("none", "tanh"):
        raise ValueError(f"Invalid approximate value: {approximate}")
    _lib.require_cuda(x, y)
    if torch.is_grad_enabled() and (x.requires_grad or y.requires_grad):
        raise RuntimeError("gelu_and_mul: backward is not implemented (inference path); call under torch.no_grad()")
    x, y, dt = _promote(x, y)
    shape = torch.broadcast_shapes(x.shape, y.shape)
    out = torch.empty(shape, dtype=dt, device=x.device)
    return _silu_and_mul_launch(x, y, out, gelu=approximate)


def silu_and_mul_out(A, B, out):
    """``out = silu(A) * B``; ``out`` must have the broadcast shape and no internal overlap."""
    logger.debug("GEMS SILU AND MUL OUT")
    _lib.require_cuda(A, B, out)
    A, B, dt = _promote(A, B)
    shape = torch.broadcast_shapes(A.shape, B.shape)
    if tuple(out.shape) != tuple(shape):
        raise RuntimeError(f"silu_and_mul_out: out has shape {tuple(out.shape)}, expected {tuple(shape)}")
    if out.dtype != dt:
        raise RuntimeError(f"silu_and_mul_out: out has dtype {out.dtype}, expected {dt}")
    if any(s == 0 and n > 1 for s, n in zip(out.stride(), out.shape)):
        raise RuntimeError("silu_and_mul_out: out must not have internal overlap")
    return _silu_and_mul_launch(A, B, out)


# ---------------------------------------------------------------------------
# reshape_and_cache_flash  (src/flag_gems/fused/reshape_and_cache_flash.py:61-112)
# ---------------------------------------------------------------------------
def reshape_and_cache_flash(
    key,           # [num_tokens, num_heads, head_size]
    value,         # [num_tokens, num_heads, head_size]
    key_cache,     # [num_blocks, block_size, num_heads, head_size]
    value_cache,   # [num_blocks, block_size, num_heads, head_size]
    slot_mapping,  # [num_tokens]
    kv_cache_dtype,
    k_scale,
    v_scale,
):
    """Scatter new K/V tokens into the paged cache: ``cache[slot // bs, slot % bs] = key[tok]``.

    ``kv_cache_dtype``, ``k_scale`` and ``v_scale`` are accepted and ignored, as in the
    reference (no fp8 cache).  Negative slots are skipped.  Returns None."""
    logger.debug("GEMS RESHAPE_AND_CACHE_FLASH")
    dev = _lib.require_cuda(key, value, key_cache, value_cache, slot_mapping)
    num_tokens = slot_mapping.size(0)
    num_heads, head_size = key.size(1), key.size(2)
    block_size = key_cache.size(1)
    if key.dtype != key_cache.dtype or value.dtype != value_cache.dtype or key.dtype != value.dtype:
        raise RuntimeError("reshape_and_cache_flash: key/value and the caches must share a dtype")
    assert key_cache.stride(0) == value_cache.stride(0)
    if key_cache.stride() != value_cache.stride():
        raise RuntimeError("reshape_and_cache_flash: key_cache and value_cache must have equal strides")
    if key_cache.stride(3) != 1 or key.stride(2) != 1 or value.stride(2) != 1:
        raise RuntimeError("reshape_and_cache_flash: head_size must be the unit-stride dimension")
    if (num_heads > 1 and (key.stride(1) != head_size or value.stride(1) != head_size)):
        raise RuntimeError("reshape_and_cache_flash: key/value heads must be densely packed per token")
    if slot_mapping.dtype != torch.int64:
        slot_mapping = slot_mapping.to(torch.int64)
    slot_mapping = slot_mapping.contiguous()
    with torch.cuda.device(dev):
        _lib.check(_lib.load().fg_reshape_and_cache_flash(
            key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
            slot_mapping.data_ptr(), num_tokens, num_heads, head_size, block_size, key_cache.size(0),
            key.stride(0), value.stride(0), key_cache.stride(0), key_cache.stride(1), key_cache.stride(2),
            key.element_size(), _lib.stream_ptr(dev)))
    return None


def reshape_and_cache(
    key,           # [num_tokens, num_heads, head_size]
    value,         # [num_tokens, num_heads, head_size]
    key_cache,     # [num_blocks, num_heads, head_size/x, block_size, x]
    value_cache,   # [num_blocks, num_heads, head_size, block_size]
    slot_mapping,  # [num_tokens]
    kv_cache_dtype,
    k_scale,
    v_scale,
):
    """Scatter new K/V tokens into the vLLM v0 cache layout
    (``src/flag_gems/fused/reshape_and_cache.py:70-106``).  ``kv_cache_dtype``, ``k_scale``
    and ``v_scale`` are accepted and ignored, as in the reference.  Returns None."""
    logger.debug("GEMS RESHAPE_AND_CACHE")
    dev = _lib.require_cuda(key, value, key_cache, value_cache, slot_mapping)
    num_tokens = slot_mapping.size(0)
    num_heads, head_size = key.size(1), key.size(2)
    block_size, x = key_cache.size(3), key_cache.size(4)
    if key.dtype != key_cache.dtype or value.dtype != value_cache.dtype or key.dtype != value.dtype:
        raise RuntimeError("reshape_and_cache: key/value and the caches must share a dtype")
    if not key_cache.is_contiguous() or not value_cache.is_contiguous():
        raise RuntimeError("reshape_and_cache: the caches must be contiguous")
    if key_cache.size(1) != num_heads or key_cache.size(2) * x != head_size or \
            tuple(value_cache.shape[1:]) != (num_heads, head_size, block_size):
        raise RuntimeError("reshape_and_cache: cache shapes do not match key/value")
    if key.stride(2) != 1 or value.stride(2) != 1 or \
            (num_heads > 1 and (key.stride(1) != head_size or value.stride(1) != head_size)):
        raise RuntimeError("reshape_and_cache: key/value heads must be densely packed per token")
    if slot_mapping.dtype != torch.int64:
        slot_mapping = slot_mapping.to(torch.int64)
    slot_mapping = slot_mapping.contiguous()
    with torch.cuda.device(dev):
        _lib.check(_lib.load().fg_reshape_and_cache(
            key.data_ptr(), value.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
            slot_mapping.data_ptr(), num_tokens, num_heads, head_size, block_size, key_cache.size(0), x,
            key.stride(0), value.stride(0), key.element_size(), _lib.stream_ptr(dev)))
    return None
