"""Tensor-core operators of the inference path: the mm/addmm projections,
``flash_attn_varlen_func`` and plain ``rms_norm``.

Same names, argument meaning and error behaviour as ``flag_gems.ops``
(``src/flag_gems/ops/mm.py``, ``addmm.py``, ``attention.py``, ``flash_api.py``,
``rms_norm.py``).  Host code validates and allocates outputs with torch; all
arithmetic runs in the sm_100a kernels behind the C ABI.
"""
from __future__ import annotations

import ctypes as C
import logging
import math
import os

import torch

from . import _lib

logger = logging.getLogger("flag_gems." + __name__.split(".")[-1])

__all__ = ["mm", "mm_out", "addmm", "addmm_out", "bmm", "flash_attn_varlen_func", "flash_attention_forward", "rms_norm",
           "get_scheduler_metadata", "scheduler_plan", "get_higher_dtype"]

_ordered_datatypes = [torch.float16, torch.bfloat16, torch.float32]


def get_higher_dtype(a, b):
    """Output dtype rule of the reference mm (src/flag_gems/ops/mm.py:140-151)."""
    if a is b:
        return a
    assert a in _ordered_datatypes
    assert b in _ordered_datatypes
    for d in _ordered_datatypes:
        if a is d:
            return b
        if b is d:
            return a


def broadcastable_to(s1, s2) -> bool:
    r1, r2 = len(s1), len(s2)
    if r1 == 0:
        return True
    if r2 == 0:
        return False
    if r1 > r2:
        return False
    for i in range(1, r1 + 1):
        if s1[-i] != 1 and s1[-i] != s2[-i]:
            return False
    return True


# FLAGGEMS_B200_F32_SPLIT=0 keeps fp32 matrix products on the CUDA-core kernel (for measurements).
_F32_SPLIT = os.environ.get("FLAGGEMS_B200_F32_SPLIT", "1") != "0"


def _tma_ready(x):
    """A 16-bit matrix in a form the tensor-core kernel can fetch with TMA: 16-byte aligned base
    and a leading dimension that is a multiple of 8 elements.  A matrix that is not (odd sizes
    such as K = 1023, or a view that starts mid-row) is copied once into a buffer with the leading
    dimension rounded up, keeping its row- or column-major order; the padding is never read (the
    tensor map carries the true extents).  Small operands go to the CUDA-core kernel as they are."""
    if x.dtype not in (torch.float16, torch.bfloat16) or x.dim() != 2:
        return x
    rows, cols = x.shape
    if rows * cols < 64 * 64:
        return x
    col_major = x.stride(0) == 1 and x.stride(1) != 1
    lead = x.stride(1) if col_major else x.stride(0)
    unit = x.stride(0) if col_major else x.stride(1)
    if x.data_ptr() % 16 == 0 and lead % 8 == 0 and lead >= (rows if col_major else cols) and unit == 1:
        return x
    if col_major:
        buf = torch.empty((cols, (rows + 7) // 8 * 8), dtype=x.dtype, device=x.device)
        out = buf[:, :rows].t()
    else:
        buf = torch.empty((rows, (cols + 7) // 8 * 8), dtype=x.dtype, device=x.device)
        out = buf[:, :cols]
    out.copy_(x)
    return out


def _gemm(a, b, c, bias=None, alpha=1.0, beta=1.0):
    dev = _lib.require_cuda(a, b, c, bias)
    if a.shape[0] * b.shape[1] >= 128 * 128 and a.shape[1] >= 32:
        a, b = _tma_ready(a), _tma_ready(b)
    p = _lib.GemmParams()
    p.a, p.b, p.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    p.bias = None if bias is None else bias.data_ptr()
    p.M, p.K = a.shape
    p.N = b.shape[1]
    p.a_stride0, p.a_stride1 = a.stride()
    p.b_stride0, p.b_stride1 = b.stride()
    p.c_stride0, p.c_stride1 = c.stride()
    if bias is not None:
        p.bias_stride0, p.bias_stride1 = bias.stride()
    p.alpha, p.beta = float(alpha), float(beta)
    p.dtype = _lib.dtype_code(c.dtype)
    lib = _lib.load()
    with torch.cuda.device(dev):
        # Large fp32 problems run on the tensor cores from three bf16 pieces per operand (fp32-level
        # error, never TF32); the pieces live in a scratch buffer for the duration of the call.
        need = lib.fg_gemm_f32_split_workspace_bytes(C.byref(p)) if c.dtype == torch.float32 and _F32_SPLIT else 0
        scratch = None
        if need > 0:
            try:
                scratch = torch.empty(need, dtype=torch.uint8, device=c.device)
            except torch.cuda.OutOfMemoryError:
                scratch = None      # no room for the pieces (1.5 x the operands): the CUDA-core kernel needs none
        if scratch is not None:
            _lib.check(lib.fg_gemm_f32_split(C.byref(p), scratch.data_ptr(), need, _lib.stream_ptr(dev)))
            # (freed on return: the caching allocator hands the block out again only to work queued
            # behind this call on the same stream)
        else:
            _lib.check(lib.fg_gemm(C.byref(p), _lib.stream_ptr(dev)))
    return c


def _prep_mm(a, b):
    _lib.require_cuda(a, b)
    if a.dim() != 2 or b.dim() != 2:
        raise RuntimeError("mm: both arguments must be 2-D")
    assert a.shape[1] == b.shape[0], "incompatible dimensions"
    # same normalisation as the reference: only a tensor strided in BOTH dims is copied
    if a.stride(0) > 1 and a.stride(1) > 1:
        a = a.contiguous()
    if b.stride(0) > 1 and b.stride(1) > 1:
        b = b.contiguous()
    c_dtype = get_higher_dtype(a.dtype, b.dtype)
    if a.dtype != c_dtype:
        a = a.to(c_dtype)
    if b.dtype != c_dtype:
        b = b.to(c_dtype)
    return a, b, c_dtype


def mm(a, b):
    """``a @ b`` with fp32 accumulation (aten::mm override)."""
    a, b, c_dtype = _prep_mm(a, b)
    M, K = a.shape
    N = b.shape[1]
    logger.debug("GEMS MM, [shape info]: [-, %s, %s, %s](batch, M, N, K), [A column-major]: %s, "
                 "[B column-major]: %s", M, N, K, a.stride(0) == 1, b.stride(0) == 1)
    c = torch.empty((M, N), device=a.device, dtype=c_dtype)
    return _gemm(a, b, c)


def mm_out(a, b, *, out):
    """``out = a @ b`` (aten::mm.out override)."""
    a, b, c_dtype = _prep_mm(a, b)
    M, K = a.shape
    N = b.shape[1]
    if tuple(out.shape) != (M, N):
        raise RuntimeError(f"mm_out: out has shape {tuple(out.shape)}, expected {(M, N)}")
    if out.dtype != c_dtype:
        raise RuntimeError(f"mm_out: out has dtype {out.dtype}, expected {c_dtype}")
    logger.debug("GEMS MM_OUT, [shape info]: [-, %s, %s, %s](batch, M, N, K)", M, N, K)
    return _gemm(a, b, out)


def bmm(A, B):
    """``torch.bmm(A, B)`` with fp32 accumulation (aten::bmm override; ``src/flag_gems/ops/bmm.py:122-136``).
    The batch is the third dimension of the GEMM kernel's tensor maps: one launch for all
    problems.  Only the inner two dimensions are normalised (a matrix strided in both
    dimensions is copied, as in ``mm``); the batch stride is passed as it is."""
    logger.debug("GEMS BMM")
    dev = _lib.require_cuda(A, B)
    if A.dim() != 3 or B.dim() != 3:
        raise RuntimeError("bmm: both arguments must be 3-D")
    batch, M, K = A.shape
    assert B.shape[0] == batch and B.shape[1] == K, "incompatible dimensions"
    N = B.shape[2]
    c_dtype = get_higher_dtype(A.dtype, B.dtype)
    A = A.to(c_dtype) if A.dtype != c_dtype else A
    B = B.to(c_dtype) if B.dtype != c_dtype else B
    if (A.stride(1) > 1 and A.stride(2) > 1) or (batch > 1 and A.stride(0) == 0):
        A = A.contiguous()
    if (B.stride(1) > 1 and B.stride(2) > 1) or (batch > 1 and B.stride(0) == 0):
        B = B.contiguous()
    out = torch.empty((batch, M, N), dtype=c_dtype, device=A.device)
    if batch == 0 or M == 0 or N == 0:
        return out
    p = _lib.GemmParams()
    p.a, p.b, p.c = A.data_ptr(), B.data_ptr(), out.data_ptr()
    p.bias = None
    p.M, p.K, p.N = M, K, N
    p.a_stride0, p.a_stride1 = A.stride(1), A.stride(2)
    p.b_stride0, p.b_stride1 = B.stride(1), B.stride(2)
    p.c_stride0, p.c_stride1 = out.stride(1), out.stride(2)
    p.alpha, p.beta = 1.0, 0.0
    p.dtype = _lib.dtype_code(c_dtype)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().fg_gemm_batched(C.byref(p), batch, A.stride(0), B.stride(0), out.stride(0), 0,
                                               _lib.stream_ptr(dev)))
    return out


def _prep_addmm(bias, mat1, mat2):
    _lib.require_cuda(bias, mat1, mat2)
    assert mat1.shape[1] == mat2.shape[0], "Incompatible dimensions"
    assert broadcastable_to(bias.shape, (mat1.shape[0], mat2.shape[1])), "Incompatible input shape"
    if mat1.dtype != mat2.dtype or bias.dtype != mat1.dtype:
        raise RuntimeError("addmm: bias, mat1 and mat2 must share a dtype")
    mat1 = mat1.contiguous()
    if mat2.stride(0) > 1 and mat2.stride(1) > 1:
        mat2 = mat2.contiguous()
    return mat1, mat2


def addmm(bias, mat1, mat2, *, beta=1, alpha=1):
    """``beta * bias + alpha * (mat1 @ mat2)``, epilogue in fp32 (aten::addmm override)."""
    mat1, mat2 = _prep_addmm(bias, mat1, mat2)
    M, K = mat1.shape
    N = mat2.shape[1]
    logger.debug("GEMS ADDMM, [shape info]: [-, %s, %s, %s](batch, M, N, K), [A column-major]: %s, "
                 "[B column-major]: %s, [bias column-major]: %s", M, N, K, mat1.stride(0) == 1,
                 mat2.stride(0) == 1, bias.dim() > 0 and bias.stride(0) == 1)
    out = torch.empty((M, N), device=mat1.device, dtype=mat1.dtype)
    return _gemm(mat1, mat2, out, bias.broadcast_to(out.shape), alpha, beta)


def addmm_out(bias, mat1, mat2, *, beta=1, alpha=1, out=None):
    """``out = beta * bias + alpha * (mat1 @ mat2)`` (aten::addmm.out override)."""
    mat1, mat2 = _prep_addmm(bias, mat1, mat2)
    M, K = mat1.shape
    N = mat2.shape[1]
    if out is None:
        out = torch.empty((M, N), device=mat1.device, dtype=mat1.dtype)
    else:
        assert out.shape == (M, N), "Incompatible output shape"
        if out.dtype != mat1.dtype:
            raise RuntimeError("addmm_out: out must have the dtype of mat1")
    logger.debug("GEMS ADDMM_OUT, [shape info]: [-, %s, %s, %s](batch, M, N, K)", M, N, K)
    return _gemm(mat1, mat2, out, bias.broadcast_to(out.shape), alpha, beta)


# ---------------------------------------------------------------------------
# rms_norm (src/flag_gems/ops/rms_norm.py:221; inference forward only)
# ---------------------------------------------------------------------------
def rms_norm(x, normalized_shape, weight, eps=1e-5):
    """``x * rsqrt(mean(x^2) + eps) * weight`` over the trailing ``normalized_shape``."""
    logger.debug("GEMS RMS_NORM FORWARD")
    dev = _lib.require_cuda(x, weight)
    N = math.prod(normalized_shape)
    if tuple(x.shape[x.ndim - len(normalized_shape):]) != tuple(normalized_shape):
        raise RuntimeError("rms_norm: normalized_shape does not match the trailing dims of input")
    if weight.numel() != N or weight.dtype != x.dtype:
        raise RuntimeError("rms_norm: weight must match normalized_shape and the input dtype")
    xc = x.contiguous()
    out = torch.empty_like(xc)
    M = xc.numel() // N if N else 0
    with torch.cuda.device(dev):
        _lib.check(_lib.load().fg_rms_norm(
            xc.data_ptr(), weight.contiguous().data_ptr(), out.data_ptr(), M, N, N, N, float(eps),
            _lib.dtype_code(x.dtype), _lib.stream_ptr(dev)))
    return out


# ---------------------------------------------------------------------------
# flash_attn_varlen_func (src/flag_gems/ops/attention.py:1118-1287,
#                         src/flag_gems/ops/flash_api.py:230-569)
# ---------------------------------------------------------------------------
def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


_workspaces: dict = {}


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Per-(device, stream) scratch for split-KV decode; grows monotonically so that
    steady-state decode steps allocate nothing."""
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def flash_attn_varlen_func(
    q,
    k,
    v,
    max_seqlen_q,
    cu_seqlens_q,
    max_seqlen_k,
    cu_seqlens_k=None,  # only used for non-paged prefill
    seqused_k=None,
    q_v=None,
    dropout_p=0.0,
    softmax_scale=None,
    causal=False,
    window_size=None,
    softcap=0.0,  # 0.0 means deactivated
    alibi_slopes=None,
    deterministic=False,
    return_attn_probs=False,
    block_table=None,
    return_softmax_lse=False,
    out=None,
    # Dummy FA3 arguments
    scheduler_metadata=None,
    q_descale=None,
    k_descale=None,
    v_descale=None,
    num_splits: int = 0,
    fa_version: int = 2,
):
    """FlashAttention-2 forward over variable-length sequences (vLLM-compatible signature).

    q: ``(total_q, nheads, headdim)``.  Paged form (``block_table`` given): k, v are
    ``(num_blocks, block_size, nheads_k, headdim)`` and ``seqused_k`` holds the key
    lengths.  Contiguous form: k, v are ``(total_k, nheads_k, headdim)`` indexed by
    ``cu_seqlens_k`` (the reference accepts the paged form only, flash_api.py:272).
    The causal mask is aligned to the bottom-right corner; rows that see no key
    produce zeros.  Returns ``out`` or ``(out, softmax_lse)`` with lse ``(nheads, total_q)``.
    """
    logger.debug("GEMS FLASH_ATTN_VARLEN_FUNC")
    assert cu_seqlens_k is not None or seqused_k is not None, "cu_seqlens_k or seqused_k must be provided"
    assert cu_seqlens_k is None or seqused_k is None, (
        "cu_seqlens_k and seqused_k cannot be provided at the same time")
    assert block_table is None or seqused_k is not None, "seqused_k must be provided if block_table is provided"
    if block_table is None and cu_seqlens_k is None:
        raise RuntimeError("flash_attn_varlen_func: the contiguous KV form needs cu_seqlens_k")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if window_size is None:
        real_window_size = (-1, -1)
    else:
        assert len(window_size) == 2
        real_window_size = (int(window_size[0]), int(window_size[1]))
    if fa_version != 2:
        raise RuntimeError("Only FA2 is implemented.")
    if num_splits > 0:
        raise RuntimeError("num_splits > 0 is not implemented in GEMS.")
    if dropout_p != 0.0:
        raise RuntimeError("flash_attn_varlen_func: dropout is not supported on the inference path")
    if q_v is not None:
        raise RuntimeError("flash_attn_varlen_func: q_v is not supported")
    if return_attn_probs:
        raise RuntimeError("flash_attn_varlen_func: return_attn_probs needs dropout, which is not supported")
    dev = _lib.require_cuda(q, k, v, cu_seqlens_q, cu_seqlens_k, seqused_k, block_table, alibi_slopes, out)
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    max_seqlen_q = max_seqlen_q.item() if hasattr(max_seqlen_q, "item") else max_seqlen_q
    max_seqlen_k = max_seqlen_k.item() if hasattr(max_seqlen_k, "item") else max_seqlen_k

    assert q.dtype in (torch.float16, torch.bfloat16), "FlashAttention only support fp16 and bf16 data type"
    assert q.dtype == k.dtype
    assert q.dtype == v.dtype
    assert cu_seqlens_q.dtype == torch.int32
    assert cu_seqlens_q.is_contiguous()
    total_q, num_heads, head_size = q.size()
    batch_size = cu_seqlens_q.numel() - 1
    paged = block_table is not None
    if paged:
        assert k.dim() == 4 and k.size() == v.size()
        num_blocks, block_size, num_heads_k = k.size(0), k.size(1), k.size(2)
        assert k.shape == (num_blocks, block_size, num_heads_k, head_size)
        assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
        assert block_table.size(0) == batch_size
    else:
        assert k.dim() == 3 and k.size() == v.size()
        num_blocks, block_size, num_heads_k = 0, 0, k.size(1)
        assert k.shape[2] == head_size
        assert cu_seqlens_k.dtype == torch.int32 and cu_seqlens_k.is_contiguous()
        assert cu_seqlens_k.size() == (batch_size + 1,)
    assert k.stride() == v.stride()
    if seqused_k is not None:
        assert seqused_k.dtype == torch.int32
        assert seqused_k.is_contiguous()
        assert seqused_k.size() == (batch_size,)
    assert head_size <= 256, "FlashAttention forward only supports head dimension at most 256"
    assert head_size % 8 == 0, "head_size must be a multiple of 8, this is ensured by padding!"
    assert num_heads % num_heads_k == 0, "Number of heads in key/value must divide number of heads in query"
    if out is not None:
        assert out.stride(-1) == 1
        assert out.dtype == q.dtype
        assert out.size() == (total_q, num_heads, head_size)
    else:
        out = torch.empty_like(q)
    if alibi_slopes is not None:
        assert alibi_slopes.dtype == torch.float32
        assert alibi_slopes.stride(-1) == 1
        assert alibi_slopes.shape == (num_heads,) or alibi_slopes.shape == (batch_size, num_heads)
    lse = torch.empty((num_heads, total_q), dtype=torch.float32, device=q.device)

    p = _lib.AttnParams()
    p.q, p.k, p.v, p.out, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.cu_seqlens_q = cu_seqlens_q.data_ptr()
    p.cu_seqlens_k = _lib.ptr(cu_seqlens_k)
    p.seqused_k = _lib.ptr(seqused_k)
    p.block_table = _lib.ptr(block_table)
    p.alibi_slopes = _lib.ptr(alibi_slopes)
    p.q_row_stride, p.q_head_stride = q.stride(0), q.stride(1)
    p.o_row_stride, p.o_head_stride = out.stride(0), out.stride(1)
    if paged:
        p.k_block_stride, p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1), k.stride(2)
        p.v_block_stride, p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1), v.stride(2)
        p.block_table_stride = block_table.stride(0)
    else:
        p.k_row_stride, p.k_head_stride = k.stride(0), k.stride(1)
        p.v_row_stride, p.v_head_stride = v.stride(0), v.stride(1)
        p.total_k = k.size(0)
    p.alibi_batch_stride = alibi_slopes.stride(0) if (alibi_slopes is not None and alibi_slopes.dim() == 2) else 0
    p.total_q, p.batch, p.num_heads, p.num_heads_k, p.head_dim = total_q, batch_size, num_heads, num_heads_k, head_size
    p.max_seqlen_q, p.max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    p.block_size, p.num_blocks = block_size, num_blocks
    p.window_left, p.window_right = real_window_size
    p.softmax_scale, p.softcap = float(softmax_scale), float(softcap)
    p.causal = 1 if causal else 0
    p.dtype = _lib.dtype_code(q.dtype)
    p.num_splits = 0
    lib = _lib.load()
    with torch.cuda.device(dev):
        nbytes = lib.fg_flash_attn_workspace_bytes(batch_size, num_heads, head_size, int(max_seqlen_q),
                                                   int(max_seqlen_k))
        if nbytes > 0:
            ws = _workspace(dev, nbytes)
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(lib.fg_flash_attn_varlen(C.byref(p), _lib.stream_ptr(dev)))
    return (out, lse) if return_softmax_lse else out


def _dense_batch_strided(query, key, value, out, cu_q, cu_k, softmax_scale, causal, wl, wr, softcap, alibi_slopes):
    """Dense attention on (batch, seq, heads, dim) tensors with arbitrary batch strides through the
    batch-stride fields of the C ABI.  Returns the lse ``(heads, batch * seq_q)`` or None when the
    tensor-core prefill kernel, the only one that takes batch strides, does not apply."""
    if alibi_slopes is not None or softcap or any(x.stride(-1) != 1 for x in (query, key, value)):
        return None
    if query.dtype not in (torch.float16, torch.bfloat16) or key.dtype != query.dtype or value.dtype != query.dtype:
        return None
    if key.stride() != value.stride():
        return None
    B, Sq, H, D = query.shape
    Sk, Hk = key.shape[1], key.shape[2]
    dev = _lib.require_cuda(query, key, value, out)
    lse = torch.empty((H, B * Sq), dtype=torch.float32, device=query.device)
    p = _lib.AttnParams()
    p.q, p.k, p.v, p.out, p.lse = query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.cu_seqlens_q, p.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
    p.q_batch_stride, p.q_row_stride, p.q_head_stride = query.stride(0), query.stride(1), query.stride(2)
    p.k_batch_stride, p.k_row_stride, p.k_head_stride = key.stride(0), key.stride(1), key.stride(2)
    p.v_batch_stride, p.v_row_stride, p.v_head_stride = value.stride(0), value.stride(1), value.stride(2)
    p.o_batch_stride, p.o_row_stride, p.o_head_stride = Sq * H * D, H * D, D
    p.total_q, p.total_k, p.batch = B * Sq, B * Sk, B
    p.num_heads, p.num_heads_k, p.head_dim = H, Hk, D
    p.max_seqlen_q, p.max_seqlen_k = Sq, Sk
    p.window_left, p.window_right = wl, wr
    p.softmax_scale, p.softcap = float(softmax_scale), 0.0
    p.causal, p.dtype = int(causal), _lib.dtype_code(query.dtype)
    strides = (p.q_batch_stride, p.q_row_stride, p.q_head_stride, p.k_batch_stride, p.k_row_stride, p.k_head_stride,
               p.v_batch_stride, p.v_row_stride, p.v_head_stride)
    if any(st % 8 or st <= 0 for st in strides) or any(x.data_ptr() % 16 for x in (query, key, value)):
        return None
    lib = _lib.load()
    if H % Hk or lib.fg_flash_attn_path(C.byref(p)) != 1:
        return None
    with torch.cuda.device(dev):
        _lib.check(lib.fg_flash_attn_varlen(C.byref(p), _lib.stream_ptr(dev)))
    return lse


_cu_cache: dict = {}


def _dense_cu_seqlens(batch: int, seqlen: int, device) -> torch.Tensor:
    """``[0, S, 2S, ...]`` int32 on the device, cached per (batch, seqlen, device)."""
    key = (batch, seqlen, device)
    cu = _cu_cache.get(key)
    if cu is None:
        if len(_cu_cache) > 64:
            _cu_cache.clear()
        cu = torch.arange(0, (batch + 1) * seqlen, seqlen, dtype=torch.int32, device=device)
        _cu_cache[key] = cu
    return cu


def flash_attention_forward(
    query,
    key,
    value,
    cumulative_sequence_length_q,
    cumulative_sequence_length_k,
    max_q,
    max_k,
    dropout_p,
    is_causal,
    return_debug_mask,
    *,
    scale=None,
    softcap=0.0,
    window_size_left=None,
    window_size_right=None,
    seqused_k=None,
    alibi_slopes=None,
    disable_splitkv=False,
):
    """``aten::_flash_attention_forward`` for dense batches, the override FlagGems installs
    with ``enable()`` and ``F.scaled_dot_product_attention`` reaches on CUDA
    (``src/flag_gems/ops/attention.py:1028-1110``, ``ops/flash_api.py:572-916``).

    ``query`` is ``(batch, seqlen_q, heads, head_dim)``, ``key``/``value``
    ``(batch, seqlen_k, kv_heads, head_dim)``; returns
    ``(out, logsumexp (batch, heads, seqlen_q) fp32, rng_state, unused, debug_mask)``.
    A dense batch is the packed form with equally long sequences, so the call goes to the
    same kernels as ``flash_attn_varlen_func`` (tcgen05 prefill for head dim 128, split-KV
    decode for single-token queries, the general kernel otherwise).  Like the reference the
    varlen form of this ATen entry is not supported; unlike it, dropout is not either (this is
    the inference path).  Tensors whose batch and sequence dimensions do not pack (the
    transposed views SDPA passes) go to the tensor-core prefill kernel with their batch
    strides, as the reference kernel takes them; where that kernel does not apply they are
    made contiguous first.
    """
    assert cumulative_sequence_length_q is None and cumulative_sequence_length_k is None, \
        "varlen is not supported yet."
    assert query.dim() == 4 and key.dim() == 4 and value.dim() == 4, "expected (batch, seqlen, heads, head_dim)"
    hq, hk, hv = query.shape[-1], key.shape[-1], value.shape[-1]
    assert hq == hk and hk == hv
    assert hk in {16, 32, 64, 96, 128, 192, 256}
    if dropout_p and dropout_p > 0.0:
        raise NotImplementedError("flash_attention_forward: dropout is not part of the inference path")
    B, Sq, H, D = query.shape
    Sk = key.shape[1]
    softmax_scale = scale or 1.0 / (D ** 0.5)

    def packable(x):
        # (batch, seq) -> one token dimension needs stride(0) == seq * stride(1) and unit inner stride
        return x.stride(-1) == 1 and x.stride(0) == x.shape[1] * x.stride(1)

    def packed(x):
        if packable(x):
            return x.as_strided((x.shape[0] * x.shape[1], x.shape[2], x.shape[3]), (x.stride(1), x.stride(2), 1),
                                x.storage_offset())
        return x.contiguous().view(x.shape[0] * x.shape[1], x.shape[2], x.shape[3])

    wl = -1 if window_size_left is None else int(window_size_left)
    wr = -1 if window_size_right is None else int(window_size_right)
    out = torch.empty((B * Sq, H, D), dtype=query.dtype, device=query.device)
    cu_q, cu_k = _dense_cu_seqlens(B, Sq, query.device), _dense_cu_seqlens(B, Sk, query.device)
    if not (packable(query) and packable(key) and packable(value)):
        # Tensors whose batch and sequence dimensions do not pack (the transposed views of
        # (batch, heads, seq, dim) that scaled_dot_product_attention passes): the tensor-core prefill
        # kernel takes a batch stride, so no copy is needed where it applies.
        got = _dense_batch_strided(query, key, value, out, cu_q, cu_k, softmax_scale, bool(is_causal), wl, wr,
                                   softcap, alibi_slopes)
        if got is not None:
            lse = got.view(H, B, Sq).permute(1, 0, 2).contiguous()
            rng_state = torch.zeros(2, dtype=torch.int64, device=query.device)
            unused = torch.empty(0, dtype=torch.int64, device=query.device)
            debug_mask = torch.empty(0, dtype=query.dtype, device=query.device)
            return out.view(B, Sq, H, D), lse, rng_state, unused, debug_mask
    q, k, v = packed(query), packed(key), packed(value)
    res, lse = flash_attn_varlen_func(
        q, k, v, Sq, cu_q, Sk, cu_seqlens_k=cu_k,
        softmax_scale=softmax_scale, causal=bool(is_causal), window_size=(wl, wr), softcap=softcap,
        alibi_slopes=alibi_slopes, return_softmax_lse=True, out=out)
    lse = lse.view(H, B, Sq).permute(1, 0, 2).contiguous()
    rng_state = torch.zeros(2, dtype=torch.int64, device=query.device)
    unused = torch.empty(0, dtype=torch.int64, device=query.device)
    debug_mask = torch.empty(0, dtype=query.dtype, device=query.device)
    return res.view(B, Sq, H, D), lse, rng_state, unused, debug_mask


def _scheduler_params(batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k, headdim, headdim_v, qkv_dtype,
                      page_size, max_seqlen_k_new, is_causal, window_size_left, window_size_right, has_softcap,
                      num_splits, pack_gqa, sm_margin, arch, num_sm, varlen_q=False, has_leftpad=False):
    if qkv_dtype not in (torch.half, torch.bfloat16):
        raise AssertionError("FlashAttention only supports fp16 and bf16 data type")
    if num_heads % num_heads_k != 0:
        raise AssertionError("Number of heads in key/value must divide number of heads in query")
    p = _lib.SchedulerParams()
    p.batch_size, p.max_seqlen_q, p.max_seqlen_k = batch_size, max_seqlen_q, max_seqlen_k
    p.num_heads, p.num_heads_k, p.headdim, p.headdim_v = num_heads, num_heads_k, headdim, headdim_v
    p.elem_size = qkv_dtype.itemsize
    p.page_size = 0 if page_size is None else int(page_size)
    p.max_seqlen_k_new, p.is_causal = max_seqlen_k_new, int(bool(is_causal))
    p.window_size_left, p.window_size_right = window_size_left, window_size_right
    p.has_softcap, p.num_splits = int(bool(has_softcap)), num_splits
    p.pack_gqa = -1 if pack_gqa is None else int(bool(pack_gqa))
    p.sm_margin, p.arch, p.num_sm = sm_margin, arch, num_sm
    p.varlen_q, p.has_leftpad = int(varlen_q), int(has_leftpad)
    return p


def scheduler_plan(batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k, headdim, headdim_v,
                   qkv_dtype=torch.bfloat16, *, page_size=None, max_seqlen_k_new=0, is_causal=False,
                   window_size_left=-1, window_size_right=-1, has_softcap=False, num_splits=0, pack_gqa=None,
                   sm_margin=0, varlen_q=False, has_leftpad=False, arch=100, num_sm=148) -> dict:
    """The host half of ``get_scheduler_metadata`` (no device work): static split count,
    pack-GQA choice and the tile the block counts refer to, as a dict."""
    p = _scheduler_params(batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k, headdim, headdim_v,
                          qkv_dtype, page_size, max_seqlen_k_new, is_causal, window_size_left, window_size_right,
                          has_softcap, num_splits, pack_gqa, sm_margin, arch, num_sm, varlen_q, has_leftpad)
    plan = _lib.SchedulerPlan()
    _lib.check(_lib.load().fg_scheduler_plan(C.byref(p), C.byref(plan)))
    return {name: getattr(plan, name) for name, _ in plan._fields_}


def get_scheduler_metadata(
    batch_size: int,
    max_seqlen_q: int,
    max_seqlen_k: int,
    num_heads: int,
    num_heads_k: int,
    headdim: int,
    headdim_v: int,
    qkv_dtype: torch.dtype,
    seqused_k: torch.Tensor,
    cu_seqlens_q=None,
    cu_seqlens_k=None,
    cu_seqlens_k_new=None,
    seqused_q=None,
    leftpad_k=None,
    page_size=None,
    max_seqlen_k_new: int = 0,
    is_causal: bool = False,
    window_size_left: int = -1,
    window_size_right: int = -1,
    has_softcap: bool = False,
    num_splits: int = 0,
    pack_gqa=None,
    sm_margin: int = 0,
) -> torch.Tensor:
    """Split-KV scheduling vector ``[semaphore, splits per sequence]`` (int32) of a
    FlashAttention-3 style decode; signature and result of
    ``src/flag_gems/ops/get_scheduler_metadata.py:567-894``.  One kernel launch and no
    device-to-host read (the reference reads the block total back between two kernels)."""
    logger.debug("GEMS GET_SCHEDULER_METADATA")
    dev = _lib.require_cuda(seqused_k, cu_seqlens_q, cu_seqlens_k_new, seqused_q, leftpad_k)
    cap = torch.cuda.get_device_capability(dev)
    p = _scheduler_params(batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k, headdim, headdim_v,
                          qkv_dtype, page_size, max_seqlen_k_new, is_causal, window_size_left, window_size_right,
                          has_softcap, num_splits, pack_gqa, sm_margin, cap[0] * 10 + cap[1],
                          torch.cuda.get_device_properties(dev).multi_processor_count)
    keep = []

    def ptr(t, n, name):
        if t is None:
            return None
        if t.numel() < n:
            raise RuntimeError(f"get_scheduler_metadata: {name} has {t.numel()} entries, {n} needed")
        if t.dtype != torch.int32 or not t.is_contiguous():
            t = t.to(torch.int32).contiguous()
        keep.append(t)
        return t.data_ptr()

    p.seqused_k = ptr(seqused_k, batch_size, "seqused_k")
    p.cu_seqlens_q = ptr(cu_seqlens_q, batch_size + 1, "cu_seqlens_q")
    p.cu_seqlens_k_new = ptr(cu_seqlens_k_new, batch_size + 1, "cu_seqlens_k_new")
    p.seqused_q = ptr(seqused_q, batch_size, "seqused_q")
    p.leftpad_k = ptr(leftpad_k, batch_size, "leftpad_k")
    out = torch.empty(1 + (batch_size if batch_size <= 992 else 0), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().fg_get_scheduler_metadata(C.byref(p), out.data_ptr(), _lib.stream_ptr(dev)))
    return out
