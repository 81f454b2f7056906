"""``torch.ops.flag_gems.*`` custom operators.

The schema strings are the ones the reference's C++ extension defines
(``src/flag_gems/csrc/cstub.cpp:26-89``), so code written against
``torch.ops.flag_gems.fused_add_rms_norm`` etc. (the vLLM integration, the module
layer) keeps working.  The CUDA implementations forward to the Python host wrappers,
which call the C ABI.
"""
from __future__ import annotations

import torch

from . import fused, ops

SCHEMAS = {
    "rms_norm": "rms_norm(Tensor input, Tensor weight, float epsilon) -> Tensor",
    "fused_add_rms_norm":
        "fused_add_rms_norm(Tensor! input, Tensor! residual, Tensor weight, float epsilon) -> ()",
    "rotary_embedding_inplace":
        "rotary_embedding_inplace(Tensor! q, Tensor! k, Tensor cos, Tensor sin, Tensor? position_ids=None, "
        "bool rotary_interleaved=False) -> ()",
    "rotary_embedding":
        "rotary_embedding(Tensor q, Tensor k, Tensor cos, Tensor sin, Tensor? position_ids=None, "
        "bool rotary_interleaved=False) -> (Tensor, Tensor)",
    "reshape_and_cache_flash":
        "reshape_and_cache_flash(Tensor key, Tensor value, Tensor(a!) key_cache, Tensor(b!) value_cache, "
        "Tensor slot_mapping, str kv_cache_dtype, Tensor? k_scale=None, Tensor? v_scale=None) -> ()",
    "flash_attn_varlen_func":
        "flash_attn_varlen_func(Tensor q, Tensor k, Tensor v, SymInt max_seqlen_q, Tensor cu_seqlens_q, "
        "SymInt max_seqlen_k, Tensor? cu_seqlens_k=None, Tensor? seqused_k=None, Tensor? q_v=None, "
        "float dropout_p=0.0, float? softmax_scale=None, bool causal=False, SymInt[]? window_size=None, "
        "float softcap=0.0, Tensor? alibi_slopes=None, bool deterministic=False, bool return_attn_probs=False, "
        "Tensor? block_table=None, bool return_softmax_lse=False, Tensor? out=None, "
        "Tensor? scheduler_metadata=None, Tensor? q_descale=None, Tensor? k_descale=None, "
        "Tensor? v_descale=None, SymInt fa_version=2) -> (Tensor, Tensor)",
    "mm": "mm(Tensor self, Tensor mat2) -> Tensor",
    "addmm": "addmm(Tensor self, Tensor mat1, Tensor mat2, *, Scalar beta=1, Scalar alpha=1) -> Tensor",
}


def _rms_norm(input, weight, epsilon):
    return ops.rms_norm(input, list(weight.size()), weight, epsilon)


def _fused_add_rms_norm(input, residual, weight, epsilon):
    fused.fused_add_rms_norm(input, residual, list(weight.size()), weight, epsilon)


def _rotary_embedding_inplace(q, k, cos, sin, position_ids=None, rotary_interleaved=False):
    fused.apply_rotary_pos_emb(q, k, cos, sin, position_ids, rotary_interleaved, inplace=True)


def _rotary_embedding(q, k, cos, sin, position_ids=None, rotary_interleaved=False):
    return fused.apply_rotary_pos_emb(q, k, cos, sin, position_ids, rotary_interleaved, inplace=False)


def _reshape_and_cache_flash(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype,
                             k_scale=None, v_scale=None):
    fused.reshape_and_cache_flash(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype,
                                  k_scale, v_scale)


def _flash_attn_varlen_func(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k=None,
                            seqused_k=None, q_v=None, dropout_p=0.0, softmax_scale=None, causal=False,
                            window_size=None, softcap=0.0, alibi_slopes=None, deterministic=False,
                            return_attn_probs=False, block_table=None, return_softmax_lse=False, out=None,
                            scheduler_metadata=None, q_descale=None, k_descale=None, v_descale=None,
                            fa_version=2):
    return ops.flash_attn_varlen_func(
        q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k, seqused_k, q_v, dropout_p,
        softmax_scale, causal, window_size, softcap, alibi_slopes, deterministic, return_attn_probs,
        block_table, True, out, scheduler_metadata, q_descale, k_descale, v_descale, 0, fa_version)


_IMPLS = {
    "rms_norm": _rms_norm,
    "fused_add_rms_norm": _fused_add_rms_norm,
    "rotary_embedding_inplace": _rotary_embedding_inplace,
    "rotary_embedding": _rotary_embedding,
    "reshape_and_cache_flash": _reshape_and_cache_flash,
    "flash_attn_varlen_func": _flash_attn_varlen_func,
    "mm": ops.mm,
    "addmm": ops.addmm,
}

_def_lib = None
_impl_lib = None


def register_custom_ops() -> None:
    """Define the ``flag_gems`` operator namespace once per process."""
    global _def_lib, _impl_lib
    if _def_lib is not None:
        return
    _def_lib = torch.library.Library("flag_gems", "DEF")
    _impl_lib = torch.library.Library("flag_gems", "IMPL")
    for name, schema in SCHEMAS.items():
        _def_lib.define(schema)
        _impl_lib.impl(name, _IMPLS[name], "CUDA")
