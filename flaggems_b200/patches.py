"""vLLM integration (mirror of ``src/flag_gems/patches/patch_vllm_all.py`` for the
inference path): the replacement methods keep the reference's signatures; the MLA /
MoE / top-k patches of the reference are outside this path.

``apply_gems_patches_to_vllm`` looks the vLLM classes up defensively because their
module paths move between vLLM releases; a class that cannot be found is skipped and
reported instead of aborting the whole patch.
"""
from __future__ import annotations

import importlib
from typing import Optional, Tuple

import torch

from . import fused, ops

__all__ = [
    "apply_gems_patches_to_vllm",
    "patch_module_method",
    "patch_vllm_lib",
    "custom_gems_rms_forward_cuda",
    "custom_gems_rope_forward_cuda",
    "custom_gems_silu_and_mul",
    "custom_gems_write_to_paged_cache",
    "custom_gems_flash_attention_impl_forward",
    "custom_silu_and_mul",
    "custom_get_scheduler_metadata",
]

_libs: dict = {}


def patch_module_method(cls, method_name: str, new_method, verbose=True):
    old_method = getattr(cls, method_name, None)
    setattr(cls, method_name, new_method)
    if verbose:
        print(f"Patched {cls.__name__}.{method_name} with FLAGGEMS {new_method.__name__}")
    return old_method


def patch_vllm_lib(lib_name, fn_name, fn, key, verbose=True):
    if lib_name not in ("_C", "_moe_C", "_vllm_fa3_C"):
        raise ValueError(f"Library {lib_name} is not recognized.")
    lib = _libs.get(lib_name)
    if lib is None:
        lib = _libs[lib_name] = torch.library.Library(lib_name, "IMPL")
    lib.impl(fn_name, fn, key)
    if verbose:
        print(f"Patched torch.ops.{lib_name}.{fn_name} with FLAGGEMS {fn.__name__}")


def custom_gems_rms_forward_cuda(self, x, residual=None):
    from .modules import gems_rms_forward

    return gems_rms_forward(x, residual, self.weight, self.variance_epsilon)


def custom_gems_rope_forward_cuda(
    self,
    positions: torch.Tensor,
    query: torch.Tensor,
    key: torch.Tensor,
    offsets: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    from .modules import gems_rope_forward

    self.cos_sin_cache = self.cos_sin_cache.to(positions.device)
    if offsets is not None:
        positions = positions + offsets
    positions = positions.flatten()
    num_tokens = positions.shape[0]
    query_shape, key_shape = query.shape, key.shape
    query = query.view(num_tokens, -1, self.head_size)
    key = key.view(num_tokens, -1, self.head_size)
    query_rot = query[..., : self.rotary_dim]
    key_rot = key[..., : self.rotary_dim]
    cos, sin = self.cos_sin_cache.chunk(2, dim=-1)
    # in place on the rotary slice: the pass-through tail of each head is untouched,
    # so no concatenation is needed afterwards
    gems_rope_forward(query_rot, key_rot, cos, sin, position_ids=positions,
                      rotary_interleaved=not self.is_neox_style, inplace=True)
    return query.reshape(query_shape), key.reshape(key_shape)


def custom_gems_silu_and_mul(self, x: torch.Tensor) -> torch.Tensor:
    from .modules import gems_silu_and_mul

    d = x.shape[-1] // 2
    return gems_silu_and_mul(x[..., :d], x[..., d:])


def custom_gems_write_to_paged_cache(key, value, key_cache, value_cache, slot_mapping, kv_cache_dtype, k_scale,
                                     v_scale):
    """``PagedAttention.write_to_paged_cache`` (vLLM v0 cache layout), patch_vllm_all.py:71-92."""
    fused.reshape_and_cache(key, value, key_cache, value_cache, slot_mapping.flatten(), kv_cache_dtype, k_scale,
                            v_scale)


def custom_get_scheduler_metadata(batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k, headdim, headdim_v,
                                  qkv_dtype, seqused_k, cu_seqlens_q=None, cu_seqlens_k=None, cu_seqlens_k_new=None,
                                  seqused_q=None, leftpad_k=None, page_size=None, max_seqlen_k_new=0, is_causal=False,
                                  window_size_left=-1, window_size_right=-1, has_softcap=False, num_splits=0,
                                  pack_gqa=None, sm_margin=0):
    """Replacement of ``torch.ops._vllm_fa3_C.get_scheduler_metadata`` (patch_vllm_all.py:279-328)."""
    return ops.get_scheduler_metadata(
        batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k, headdim, headdim_v, qkv_dtype, seqused_k,
        cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k, cu_seqlens_k_new=cu_seqlens_k_new, seqused_q=seqused_q,
        leftpad_k=leftpad_k, page_size=page_size, max_seqlen_k_new=max_seqlen_k_new, is_causal=is_causal,
        window_size_left=window_size_left, window_size_right=window_size_right, has_softcap=has_softcap,
        num_splits=num_splits, pack_gqa=pack_gqa, sm_margin=sm_margin)


def custom_silu_and_mul(out: torch.Tensor, input: torch.Tensor):
    """Replacement of ``torch.ops._C.silu_and_mul(out, input)``."""
    d = input.size(-1) // 2
    x, y = input.split(d, dim=-1)
    fused.silu_and_mul_out(x, y, out)


def custom_gems_flash_attention_impl_forward(
    self,
    layer: torch.nn.Module,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    kv_cache: torch.Tensor,
    attn_metadata,
    output: Optional[torch.Tensor] = None,
    output_scale: Optional[torch.Tensor] = None,
    output_block_scale: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``FlashAttentionImpl.forward``: write the new K/V tokens into the paged cache, then
    run varlen attention over the cache (patch_vllm_all.py:142-241)."""
    assert output is not None, "Output tensor must be provided."
    if output_scale is not None or output_block_scale is not None:
        raise NotImplementedError("fused output quantization is not yet supported for FlashAttentionImpl")
    if attn_metadata is None:  # profiling run
        return output
    num_actual_tokens = attn_metadata.num_actual_tokens
    key_cache, value_cache = kv_cache.unbind(0)
    fused.reshape_and_cache_flash(key, value, key_cache, value_cache, attn_metadata.slot_mapping,
                                  self.kv_cache_dtype, getattr(layer, "_k_scale", None),
                                  getattr(layer, "_v_scale", None))
    if self.kv_cache_dtype.startswith("fp8"):
        raise NotImplementedError("FP8 quantization is not yet supported for FlashAttentionImpl")
    local_md = getattr(attn_metadata, "local_attn_metadata", None)
    use_local_attn = getattr(self, "use_irope", False) and local_md is not None
    if getattr(attn_metadata, "use_cascade", False) and not use_local_attn:
        raise NotImplementedError("Cascade attention is not implemented in flag_gems.")
    if use_local_attn:
        cu_seqlens_q = local_md.local_query_start_loc
        seqused_k = local_md.local_seqused_k
        max_seqlen_q = local_md.local_max_query_len
        max_seqlen_k = local_md.local_max_seq_len
        block_table = local_md.local_block_table
    else:
        cu_seqlens_q = attn_metadata.query_start_loc
        seqused_k = attn_metadata.seq_lens
        max_seqlen_q = attn_metadata.max_query_len
        max_seqlen_k = attn_metadata.max_seq_len
        block_table = attn_metadata.block_table
    ops.flash_attn_varlen_func(
        q=query[:num_actual_tokens],
        k=key_cache,
        v=value_cache,
        out=output[:num_actual_tokens],
        cu_seqlens_q=cu_seqlens_q,
        max_seqlen_q=max_seqlen_q,
        seqused_k=seqused_k,
        max_seqlen_k=max_seqlen_k,
        softmax_scale=self.scale,
        causal=True,
        alibi_slopes=self.alibi_slopes,
        window_size=self.sliding_window,
        block_table=block_table,
        softcap=self.logits_soft_cap,
        fa_version=2,
    )
    return output


def _find(candidates):
    for mod, name in candidates:
        try:
            return getattr(importlib.import_module(mod), name)
        except Exception:
            continue
    return None


def apply_gems_patches_to_vllm(verbose=True):
    """Monkey-patch vLLM's RMSNorm / RotaryEmbedding / SiluAndMul / FlashAttentionImpl and
    ``torch.ops._C.silu_and_mul`` with this package's operators
    (patch_vllm_all.py:331-368).  Returns the list of patched targets."""
    import vllm  # noqa: F401

    patched = []
    targets = [
        ([("vllm.model_executor.layers.layernorm", "RMSNorm")], "forward_cuda", custom_gems_rms_forward_cuda),
        ([("vllm.model_executor.layers.rotary_embedding", "RotaryEmbedding"),
          ("vllm.model_executor.layers.rotary_embedding.base", "RotaryEmbedding")],
         "forward_cuda", custom_gems_rope_forward_cuda),
        ([("vllm.model_executor.layers.activation", "SiluAndMul")], "forward_cuda", custom_gems_silu_and_mul),
        ([("vllm.v1.attention.backends.flash_attn", "FlashAttentionImpl")], "forward",
         custom_gems_flash_attention_impl_forward),
        ([("vllm.attention.ops.paged_attn", "PagedAttention")], "write_to_paged_cache",
         custom_gems_write_to_paged_cache),
    ]
    for candidates, method, fn in targets:
        cls = _find(candidates)
        if cls is None:
            if verbose:
                print(f"FLAGGEMS: {candidates[0][1]} not found in this vLLM, skipped")
            continue
        patch_module_method(cls, method, fn, verbose)
        patched.append(f"{cls.__name__}.{method}")
    for lib_name, fn_name, fn in (("_C", "silu_and_mul", custom_silu_and_mul),
                                  ("_vllm_fa3_C", "get_scheduler_metadata", custom_get_scheduler_metadata)):
        try:
            patch_vllm_lib(lib_name, fn_name, fn, "CUDA", verbose)
            patched.append(f"{lib_name}.{fn_name}")
        except Exception as e:  # the op namespace exists only once vLLM's extension is loaded
            if verbose:
                print(f"FLAGGEMS: torch.ops.{lib_name}.{fn_name} not patched ({e})")
    return patched
