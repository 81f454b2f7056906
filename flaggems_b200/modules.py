"""Module-level entry points (mirror of ``src/flag_gems/modules``): the functions vLLM's
layers are patched with, and drop-in ``nn.Module`` wrappers around them."""
from __future__ import annotations

import logging
import numbers
from typing import List, Optional, Tuple, Union

import torch
import torch.nn as nn
from torch import Size
from torch.nn import init
from torch.nn.parameter import Parameter

from . import fused, ops
from .config import use_c_extension

logger = logging.getLogger("flag_gems.modules")

__all__ = [
    "gems_rms_forward",
    "GemsRMSNorm",
    "gems_rope_forward",
    "GemsRope",
    "gems_silu_and_mul",
    "GemsSiluAndMul",
]


def gems_rms_forward(
    x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float
) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    """RMSNorm with optional fused residual add (modules/normalization.py:33-53)."""
    if residual is not None:
        if use_c_extension:
            logger.debug("GEMS CUSTOM FUSED_ADD_RMS_NORM(C EXTENSION)")
            torch.ops.flag_gems.fused_add_rms_norm(x, residual, weight, eps)
            return x, residual
        logger.debug("GEMS CUSTOM FUSED_ADD_RMS_NORM")
        return fused.fused_add_rms_norm(x, residual, list(weight.size()), weight, eps)
    if use_c_extension:
        logger.debug("GEMS CUSTOM RMS_NORM(C EXTENSION)")
        return torch.ops.flag_gems.rms_norm(x, weight, eps)
    logger.debug("GEMS CUSTOM RMS_NORM")
    return ops.rms_norm(x, list(weight.size()), weight, eps)


class GemsRMSNorm(nn.Module):
    """RMSNorm compatible with ``torch.nn.RMSNorm`` and vLLM's ``RMSNorm``; ``forward(x,
    residual)`` performs the fused in-place residual add (modules/normalization.py:56-121)."""

    __constants__ = ["normalized_shape", "eps", "elementwise_affine"]
    normalized_shape: Union[int, List[int], Size]
    eps: Optional[float]
    elementwise_affine: bool

    def __init__(self, normalized_shape, eps: float = 1e-6, elementwise_affine: bool = True,
                 device=None, dtype=None) -> None:
        super().__init__()
        if isinstance(normalized_shape, numbers.Integral):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if self.elementwise_affine:
            self.weight = Parameter(torch.empty(self.normalized_shape, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.elementwise_affine:
            init.ones_(self.weight)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        return gems_rms_forward(x, residual, self.weight, self.eps)

    def extra_repr(self) -> str:
        return "{normalized_shape}, eps={eps}, elementwise_affine={elementwise_affine}".format(**self.__dict__)


def gems_rope_forward(
    query: torch.Tensor,
    key: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    position_ids: Optional[torch.Tensor] = None,
    rotary_interleaved: bool = False,
    inplace: bool = False,
):
    """Rotary embedding entry point (modules/rotary_embedding.py:36-61)."""
    if use_c_extension:
        logger.debug("GEMS CUSTOM ROPE FORWARD(C EXTENSION)")
        if inplace:
            torch.ops.flag_gems.rotary_embedding_inplace(query, key, cos, sin, position_ids, rotary_interleaved)
            return query, key
        return torch.ops.flag_gems.rotary_embedding(query, key, cos, sin, position_ids, rotary_interleaved)
    logger.debug("GEMS CUSTOM ROPE FORWARD")
    return fused.apply_rotary_pos_emb(query, key, cos, sin, position_ids, rotary_interleaved, inplace)


class GemsRope(nn.Module):
    """Vanilla RoPE with a precomputed ``[max_position_embeddings, rotary_dim // 2]`` cos/sin
    cache in ``dtype`` (modules/rotary_embedding.py:64-155)."""

    def __init__(self, rotary_dim, max_position_embeddings, base, rotary_interleaved, dtype, device):
        super().__init__()
        self.rotary_dim = rotary_dim
        self.max_position_embeddings = max_position_embeddings
        self.base = base
        self.rotary_interleaved = rotary_interleaved
        self.dtype = dtype
        self.device = device
        self._set_cos_sin_cache()

    def _compute_inv_freq(self) -> torch.Tensor:
        return 1.0 / (
            self.base ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32, device=self.device)
                          / self.rotary_dim))

    def _set_cos_sin_cache(self):
        inv_freq = self._compute_inv_freq()
        t = torch.arange(self.max_position_embeddings, device=self.device, dtype=torch.float32)
        freqs = torch.outer(t, inv_freq)
        self.register_buffer("cos_cached", freqs.cos().to(self.dtype), persistent=False)
        self.register_buffer("sin_cached", freqs.sin().to(self.dtype), persistent=False)

    def forward(self, query, key, position_ids: Optional[torch.Tensor] = None, inplace: bool = False):
        if not hasattr(self, "cos_cached") or not hasattr(self, "sin_cached"):
            self._set_cos_sin_cache()
        return gems_rope_forward(query, key, self.cos_cached, self.sin_cached, position_ids,
                                 self.rotary_interleaved, inplace)


def gems_silu_and_mul(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """``silu(x) * y`` (modules/activation.py:18-24)."""
    logger.debug("GEMS CUSTOM SILU_AND_MUL FORWARD")
    return fused.silu_and_mul(x, y)


class GemsSiluAndMul(nn.Module):
    """Fused ``torch.mul(torch.nn.functional.silu(x), y)`` (modules/activation.py:27-37)."""

    def forward(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        return gems_silu_and_mul(x, y)
