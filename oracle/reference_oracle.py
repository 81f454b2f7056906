"""CPU oracle of the inference operator path -- TEST INFRASTRUCTURE, NOT PRODUCT.

A restatement, in plain torch on the CPU, of the computations FlagGems' own tests use
as ground truth for the path's operators.  Only ``tests/``, the smoke check and the
CPU-baseline legs of ``bench.py`` may import this module; no operator of
``flaggems_b200`` calls into it, and the product has no CPU path at all.

Pinning: the FlagGems tree stores no golden vectors for these operators (each test
draws random inputs and compares with a torch expression).  The functions below are
therefore pinned against the reference's own test oracles *executed from the reference
checkout*: ``tests/golden/make_golden.py`` extracts those oracle functions from the
reference's test files, runs them on seeded inputs and stores inputs and outputs as
fixtures; ``tests/test_oracle_golden.py`` replays the fixtures through this module.
The two cache scatters are in addition accepted by the reference's own test functions, executed
with these functions standing in for the operators (``tests/golden/make_golden_cache_tests.py``).
``get_scheduler_metadata`` is pinned against results of the reference function itself
(``tests/golden/make_golden_scheduler.py`` runs it under Triton's interpreter).

Every function cites the reference file:line it follows (paths inside the FlagGems tree).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

__all__ = [
    "sdpa_causal",
    "paged_attention",
    "varlen_attention",
    "alibi_bias",
    "reshape_and_cache_flash",
    "fused_add_rms_norm",
    "rms_norm",
    "rope_cos_sin",
    "apply_rotary_pos_emb",
    "silu_and_mul",
    "mm",
    "addmm",
]


# --------------------------------------------------------------------------- attention
def sdpa_causal(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                is_causal: bool = True) -> torch.Tensor:
    """Dense scaled-dot-product attention ``[B, H, S, D]`` written out as masked softmax.

    Follows ``torch_sdpa`` (tests/test_attention_ops.py:200-229), i.e.
    ``F.scaled_dot_product_attention(q, k, v, scale=scale, is_causal=True)``; the
    top-left causal mask of SDPA equals the bottom-right one when Sq == Sk."""
    s = torch.einsum("bhqd,bhkd->bhqk", q.float(), k.float()) * scale
    if is_causal:
        sq, sk = q.shape[-2], k.shape[-2]
        mask = torch.ones(sq, sk, dtype=torch.bool).tril(diagonal=0)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhqk,bhkd->bhqd", p, v.float()).to(q.dtype)


def alibi_bias(slopes: torch.Tensor, seqlen_q: int, seqlen_k: int, causal: bool) -> torch.Tensor:
    """ALiBi bias ``[batch, heads, 1|seqlen_q, seqlen_k]`` from per-(batch, head) slopes.

    Follows ``attn_bias_from_alibi_slopes`` (tests/test_attention_ops.py:804-816)."""
    slopes = slopes.float().unsqueeze(-1).unsqueeze(-1)
    if causal:
        return torch.arange(-seqlen_k + 1, 1, dtype=torch.float32) * slopes
    row = torch.arange(seqlen_q, dtype=torch.long).unsqueeze(-1)
    col = torch.arange(seqlen_k, dtype=torch.long)
    rel = torch.abs(row + seqlen_k - seqlen_q - col)
    return -slopes * rel.to(slopes.dtype)


def paged_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    query_lens: Sequence[int],
    kv_lens: Sequence[int],
    block_tables: torch.Tensor,
    scale: float,
    attn_bias: Optional[torch.Tensor] = None,
    sliding_window: Optional[int] = None,
    soft_cap: Optional[float] = None,
    causal: bool = True,
    compute_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Varlen attention over a paged KV cache, one sequence at a time.

    Follows ``ref_paged_attn`` (tests/test_attention_ops.py:819-881): gather the pages
    named by ``block_tables[i]``, repeat KV heads for GQA, scale q, bottom-right causal
    mask ``triu(diagonal=kv_len - query_len + 1)``, optional sliding window and soft cap
    ``cap * tanh(s / cap)``, optional additive bias, softmax, cast to the value dtype,
    then PV.  ``compute_dtype`` (default: the input dtype, as the reference test does
    on the device) lets the caller evaluate the same formula in fp32."""
    num_seqs = len(query_lens)
    bt = block_tables.cpu().numpy()
    _, block_size, num_kv_heads, head_size = key_cache.shape
    cd = compute_dtype or query.dtype
    outputs: List[torch.Tensor] = []
    start = 0
    for i in range(num_seqs):
        ql, kl = int(query_lens[i]), int(kv_lens[i])
        q = query[start:start + ql].to(cd) * scale
        nblk = (kl + block_size - 1) // block_size
        idx = bt[i, :nblk]
        k = key_cache[idx].view(-1, num_kv_heads, head_size)[:kl].to(cd)
        v = value_cache[idx].view(-1, num_kv_heads, head_size)[:kl].to(cd)
        if q.shape[1] != k.shape[1]:
            rep = q.shape[1] // k.shape[1]
            k = torch.repeat_interleave(k, rep, dim=1)
            v = torch.repeat_interleave(v, rep, dim=1)
        attn = torch.einsum("qhd,khd->hqk", q, k)
        ones = torch.ones(ql, kl)
        mask = torch.triu(ones, diagonal=kl - ql + 1).bool() if causal else torch.zeros(ql, kl).bool()
        if sliding_window is not None:
            mask |= torch.triu(ones, diagonal=kl - (ql + sliding_window) + 1).bool().logical_not()
        if soft_cap is not None:
            attn = soft_cap * torch.tanh(attn / soft_cap)
        attn = attn.masked_fill(mask, float("-inf"))
        if attn_bias is not None:
            attn = attn + attn_bias[i, :, :ql, :kl]
        p = torch.softmax(attn, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)  # rows with no visible key -> zeros (kernel contract)
        out = torch.einsum("hqk,khd->qhd", p.to(v.dtype), v)
        outputs.append(out.to(query.dtype))
        start += ql
    return torch.cat(outputs, dim=0)


def varlen_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
    cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor, scale: float, causal: bool = True,
    soft_cap: Optional[float] = None, compute_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Contiguous varlen form: sequence i owns rows ``cu_seqlens[i]:cu_seqlens[i+1]``.

    Same per-sequence formula as :func:`paged_attention`; expressed by viewing the
    packed K/V as a one-token-per-page cache with an identity block table."""
    cq = cu_seqlens_q.tolist()
    ck = cu_seqlens_k.tolist()
    qlens = [cq[i + 1] - cq[i] for i in range(len(cq) - 1)]
    klens = [ck[i + 1] - ck[i] for i in range(len(ck) - 1)]
    maxk = max(klens) if klens else 0
    bt = torch.zeros((len(klens), max(maxk, 1)), dtype=torch.int32)
    for i, kl in enumerate(klens):
        bt[i, :kl] = torch.arange(ck[i], ck[i] + kl, dtype=torch.int32)
    return paged_attention(q, k.unsqueeze(1), v.unsqueeze(1), qlens, klens, bt, scale,
                           soft_cap=soft_cap, causal=causal, compute_dtype=compute_dtype)


# --------------------------------------------------------------------------- KV cache
def reshape_and_cache_flash(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                            value_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """``cache[slot // block_size, slot % block_size] = key[i]`` for every token, in place.

    Follows the loop of tests/test_attention_ops.py:1459-1467; negative slots are
    skipped as in the kernel (src/flag_gems/fused/reshape_and_cache_flash.py:33-35)."""
    block_size = key_cache.shape[1]
    blk = torch.div(slot_mapping, block_size, rounding_mode="floor").tolist()
    off = (slot_mapping % block_size).tolist()
    slots = slot_mapping.tolist()
    for i in range(slot_mapping.numel()):
        if slots[i] < 0:
            continue
        key_cache[blk[i], off[i], :, :] = key[i]
        value_cache[blk[i], off[i], :, :] = value[i]


def reshape_and_cache(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor,
                      value_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """vLLM v0 layout, in place: ``key_cache[blk, :, :, off, :] = key[i].reshape(H, D/x, x)`` and
    ``value_cache[blk, :, :, off] = value[i]`` (the loop of tests/test_attention_ops.py:1311-1321);
    negative slots are skipped as in the kernel (src/flag_gems/fused/reshape_and_cache.py:30-32)."""
    block_size = key_cache.shape[3]
    reshaped_key = key.reshape(key.shape[0], *key_cache[0, :, :, 0, :].shape)
    blk = torch.div(slot_mapping, block_size, rounding_mode="floor").tolist()
    off = (slot_mapping % block_size).tolist()
    slots = slot_mapping.tolist()
    for i in range(slot_mapping.numel()):
        if slots[i] < 0:
            continue
        key_cache[blk[i], :, :, off[i], :] = reshaped_key[i]
        value_cache[blk[i], :, :, off[i]] = value[i]


# --------------------------------------------------------------------------- norms
def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                       upcast: torch.dtype = torch.float64):
    """Returns ``(normed, new_residual)`` in the upcast dtype.

    Follows ``_torch_fused_add_rms_norm`` (tests/test_norm_ops.py:614-618) on inputs
    upcast as ``to_reference(..., True)`` does (tests/accuracy_utils.py:175-186)."""
    x = x.to(upcast) + residual.to(upcast)
    variance = x.pow(2).mean(-1, keepdim=True)
    hidden = x * torch.rsqrt(variance + eps)
    return weight.to(upcast) * hidden, x


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, upcast: torch.dtype = torch.float64):
    """``x * rsqrt(mean(x^2) + eps) * weight`` (tests/test_norm_ops.py, rms_norm oracle;
    kernel src/flag_gems/ops/rms_norm.py:17-51)."""
    x = x.to(upcast)
    variance = x.pow(2).mean(-1, keepdim=True)
    return weight.to(upcast) * (x * torch.rsqrt(variance + eps))


# --------------------------------------------------------------------------- rope
def rope_cos_sin(max_seq_len: int, dim: int, dtype: torch.dtype, base: float = 10000.0):
    """cos/sin tables ``[max_seq_len, dim // 2]`` computed in fp32, then cast to ``dtype``.

    Follows ``get_rope_cos_sin`` (tests/test_special_ops.py:106-112)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim))
    t = torch.arange(max_seq_len, dtype=inv_freq.dtype)
    freqs = torch.outer(t, inv_freq)
    return freqs.cos().to(dtype), freqs.sin().to(dtype)


def _rotate_half(x):
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def _rotate_interleave(x):
    x1 = x[..., ::2]
    x2 = x[..., 1::2]
    return torch.stack((-x2, x1), dim=-1).flatten(-2)


def apply_rotary_pos_emb(q, k, cos, sin, position_ids: Optional[torch.Tensor] = None,
                         rotary_interleaved: bool = False, upcast: torch.dtype = torch.float32):
    """Rotary embedding of q ``(..., seq, heads, dim)`` / k; returns upcast tensors.

    Follows ``torch_apply_rotary_pos_emb`` (tests/test_special_ops.py:133-161)."""
    q = q.to(upcast)
    k = k.to(upcast)
    cos = cos.to(upcast)
    sin = sin.to(upcast)
    if position_ids is None:
        cos = cos[None, : q.size(-3), None, :]
        sin = sin[None, : q.size(-3), None, :]
    else:
        cos = cos[position_ids].unsqueeze(-2)
        sin = sin[position_ids].unsqueeze(-2)
    if rotary_interleaved:
        cos = torch.repeat_interleave(cos, 2, dim=-1)
        sin = torch.repeat_interleave(sin, 2, dim=-1)
        rot = _rotate_interleave
    else:
        cos = torch.cat([cos, cos], dim=-1)
        sin = torch.cat([sin, sin], dim=-1)
        rot = _rotate_half
    return (q * cos) + (rot(q) * sin), (k * cos) + (rot(k) * sin)


# --------------------------------------------------------------------------- pointwise / blas
def silu_and_mul(x: torch.Tensor, y: torch.Tensor, upcast: torch.dtype = torch.float64) -> torch.Tensor:
    """``silu(x) * y`` on upcast inputs (tests/test_binary_pointwise_ops.py:1386)."""
    return torch.mul(torch.nn.functional.silu(x.to(upcast)), y.to(upcast))


def gelu_and_mul(x: torch.Tensor, y: torch.Tensor, approximate: str = "none",
                 upcast: torch.dtype = torch.float64) -> torch.Tensor:
    """``gelu(x, approximate) * y`` on upcast inputs (tests/test_binary_pointwise_ops.py:962-978)."""
    return torch.mul(torch.nn.functional.gelu(x.to(upcast), approximate=approximate), y.to(upcast))


def mm(a: torch.Tensor, b: torch.Tensor, upcast: torch.dtype = torch.float64) -> torch.Tensor:
    """``torch.mm`` on upcast inputs (tests/test_blas_ops.py:129-132)."""
    return torch.mm(a.to(upcast), b.to(upcast))


def bmm(a: torch.Tensor, b: torch.Tensor, upcast: torch.dtype = torch.float64) -> torch.Tensor:
    """``torch.bmm`` on upcast inputs (tests/test_blas_ops.py:95-111)."""
    return torch.bmm(a.to(upcast), b.to(upcast))


def addmm(bias, mat1, mat2, alpha=1.0, beta=1.0, upcast: torch.dtype = torch.float64) -> torch.Tensor:
    """``torch.addmm`` on upcast inputs (tests/test_blas_ops.py:38-44)."""
    return torch.addmm(bias.to(upcast), mat1.to(upcast), mat2.to(upcast), alpha=alpha, beta=beta)


# ---------------------------------------------------------------------------------------
# get_scheduler_metadata (split-KV scheduling of the FlashAttention-3 style decode),
# ops/get_scheduler_metadata.py.  Restated for compute capability >= 9.0 only (the
# sm8x tile table, :12-88, is not reachable on a B200); integer work, bit-exact.
# Pinned by tests/golden/golden_scheduler_metadata.pt, produced by running the reference
# function itself under Triton's interpreter with the device queries answered
# (10, 0) / 148 SMs.
# ---------------------------------------------------------------------------------------

def _round_head_dim(d: int, last: int) -> int:
    """ops/get_scheduler_metadata.py:191-216 (``last`` = 256 for qk, 512 for v)."""
    for step in (64, 96, 128, 192, 256):
        if d <= step:
            return step
    return last


def _tile_mn_sm90(d: int, dv: int, causal: bool, local: bool, paged_non_tma: bool, one_wg: bool):
    """(kBlockM, kBlockN) for 16-bit inputs, ops/get_scheduler_metadata.py:91-127."""
    if d <= 64:
        if dv == 512:
            return 64, 64
        if dv == 256:
            return 128, 112
        return 192, (128 if (causal or local) else 192)
    if d <= 96:
        return 192, (128 if (local or paged_non_tma) else 144)
    if d <= 128:
        return (64 if one_wg else 128), (128 if (causal or local or paged_non_tma) else 176)
    if d <= 192:
        return 128, (96 if (paged_non_tma or local) else (128 if dv <= 128 else 112))
    return 128, (64 if local else 80)


def _one_mma_warpgroup(headdim: int, seqlen_q: int, pack_gqa: bool, hq: int, hk: int) -> bool:
    """ops/get_scheduler_metadata.py:261-275."""
    return headdim == 128 and seqlen_q * ((hq // hk) if pack_gqa else 1) <= 64


def _split_heuristic(total_mblocks: int, num_sm: int, n_blocks: int, m_blocks: int, bytes_one_kv_head: int,
                     causal_or_local: bool, max_splits: int) -> int:
    """ops/get_scheduler_metadata.py:393-426 (double-precision efficiencies, as Python floats)."""
    import math
    if total_mblocks >= 0.8 * num_sm:
        l2 = 50 * 1024 * 1024
        if bytes_one_kv_head > l2 and m_blocks >= num_sm * 2 and not causal_or_local:
            return min(-(-bytes_one_kv_head // l2), max_splits)
        return 1
    if n_blocks <= 4:
        return 1
    max_splits = min(max_splits, num_sm, n_blocks)
    eff = []
    for s in range(1, max_splits + 1):
        waves = float(total_mblocks * s) / num_sm
        eff.append(waves / math.ceil(waves))
    best = max(eff) if eff else 0.0
    for s, e in enumerate(eff, start=1):
        if e >= 0.85 * best:
            return s
    return 1


def scheduler_plan(batch_size: int, max_seqlen_q: int, max_seqlen_k: int, num_heads: int, num_heads_k: int,
                   headdim: int, headdim_v: int, *, page_size: Optional[int] = None, has_leftpad: bool = False,
                   varlen_q: bool = False, max_seqlen_k_new: int = 0, is_causal: bool = False,
                   window_size_left: int = -1, window_size_right: int = -1, has_softcap: bool = False,
                   num_splits: int = 0, pack_gqa: Optional[bool] = None, num_sm: int = 148) -> dict:
    """The host half of get_scheduler_metadata, ops/get_scheduler_metadata.py:592-769:
    mask normalisation, pack-GQA choice, static split count and the tile the block counts
    are taken in."""
    elem = 2
    wl = window_size_left if window_size_left >= 0 else -1
    wr = window_size_right
    if wl >= max_seqlen_k - 1:
        wl = -1
    if wr >= max_seqlen_q - 1:
        wr = -1
    causal = bool(is_causal)
    if max_seqlen_q == 1 and wl == -1 and wr == -1 and ((headdim <= 64 or headdim > 128) or page_size is None):
        causal = False
    if causal:
        wr = 0
    causal = wl < 0 and wr == 0
    local = (wl >= 0 or wr >= 0) and not causal
    paged = page_size is not None
    d_r, dv_r = _round_head_dim(headdim, 256), _round_head_dim(headdim_v, 512)
    group = num_heads // num_heads_k

    # paged K/V through TMA: whole pages per key tile and more than one query tile (:219-258)
    paged_tma = False
    if paged and not has_leftpad and max_seqlen_k_new == 0:
        bm, bn = _tile_mn_sm90(d_r, dv_r, causal, local, False, False)
        paged_tma = page_size % bn == 0 and max_seqlen_q * group > bm

    if pack_gqa is None:  # :535-564, :278-293
        if (paged and not paged_tma) or num_splits > 1:
            pack_gqa = True
        elif num_heads == num_heads_k:
            pack_gqa = False
        elif varlen_q:
            pack_gqa = True
        else:
            bm, _ = _tile_mn_sm90(d_r, dv_r, causal, local, paged and not paged_tma, False)
            up = lambda a: -(-a // bm) * bm
            pack_gqa = float(max_seqlen_q) / up(max_seqlen_q) < 0.9 * (float(max_seqlen_q * group) / up(max_seqlen_q * group))

    dynamic = batch_size <= 992
    if num_splits <= 0:  # :296-390; inside, paged K/V always counts as the non-TMA form
        bm, bn = _tile_mn_sm90(d_r, dv_r, causal, local, paged, _one_mma_warpgroup(headdim, max_seqlen_q, pack_gqa,
                                                                                     num_heads, num_heads_k))
        k_loaded = max(0, min(max_seqlen_k, wl + wr + 1 + bm)) if local else max_seqlen_k
        n_blocks, m_blocks = -(-k_loaded // bn), -(-(max_seqlen_q * group) // bm)
        splits = _split_heuristic((1 if dynamic else batch_size) * num_heads_k * m_blocks, num_sm, n_blocks, m_blocks,
                                  max_seqlen_k * (headdim + headdim_v) * elem, causal or local, 128)
    else:
        splits = num_splits
    splits = min(splits, 256, num_sm)
    if splits > 1:
        pack_gqa = True
    bm, bn = _tile_mn_sm90(d_r, dv_r, causal, local, paged and not paged_tma,
                           _one_mma_warpgroup(headdim, max_seqlen_q, pack_gqa, num_heads, num_heads_k))
    return dict(num_splits=splits, pack_gqa=bool(pack_gqa), block_m=bm, block_n=bn, dynamic=dynamic, causal=causal,
                local=local, q_per_kv=(-(-num_heads // num_heads_k)) if pack_gqa else 1,
                heads=num_heads_k if pack_gqa else num_heads)


def get_scheduler_metadata(batch_size: int, max_seqlen_q: int, max_seqlen_k: int, num_heads: int, num_heads_k: int,
                           headdim: int, headdim_v: int, seqused_k: torch.Tensor,
                           cu_seqlens_q: Optional[torch.Tensor] = None, cu_seqlens_k_new: Optional[torch.Tensor] = None,
                           seqused_q: Optional[torch.Tensor] = None, leftpad_k: Optional[torch.Tensor] = None,
                           page_size: Optional[int] = None, max_seqlen_k_new: int = 0, is_causal: bool = False,
                           window_size_left: int = -1, window_size_right: int = -1, has_softcap: bool = False,
                           num_splits: int = 0, pack_gqa: Optional[bool] = None, sm_margin: int = 0,
                           sm_count: int = 148) -> torch.Tensor:
    """int32 ``[semaphore = 0, splits of sequence 0, 1, ...]`` (the per-sequence part only for
    batches of at most 992), ops/get_scheduler_metadata.py:567-894; the two device passes
    are :430-532 (per-sequence tile counts and their sum; then KV tiles per SM in fp32)."""
    import numpy as np
    num_sm = sm_count - sm_margin
    plan = scheduler_plan(batch_size, max_seqlen_q, max_seqlen_k, num_heads, num_heads_k, headdim, headdim_v,
                          page_size=page_size, has_leftpad=leftpad_k is not None,
                          varlen_q=cu_seqlens_q is not None or seqused_q is not None,
                          max_seqlen_k_new=max_seqlen_k_new, is_causal=is_causal, window_size_left=window_size_left,
                          window_size_right=window_size_right, has_softcap=has_softcap, num_splits=num_splits,
                          pack_gqa=pack_gqa, num_sm=num_sm)
    if not plan["dynamic"]:
        return torch.zeros(1, dtype=torch.int32)
    as_np = lambda t: t.detach().cpu().numpy().astype(np.int64)
    if seqused_q is not None:
        q_len = as_np(seqused_q)[:batch_size]
    elif cu_seqlens_q is not None:
        q_len = np.diff(as_np(cu_seqlens_q)[:batch_size + 1])
    else:
        q_len = np.full(batch_size, max_seqlen_q, dtype=np.int64)
    m_blocks = (q_len * plan["q_per_kv"] + plan["block_m"] - 1) // plan["block_m"]
    k_len = as_np(seqused_k)[:batch_size]
    if max_seqlen_k_new > 0:
        k_len = k_len + (np.diff(as_np(cu_seqlens_k_new)[:batch_size + 1]) if cu_seqlens_k_new is not None
                         else max_seqlen_k_new)
    if leftpad_k is not None:
        k_len = k_len - as_np(leftpad_k)[:batch_size]
    n_blocks = (k_len + plan["block_n"] - 1) // plan["block_n"]
    total = int((m_blocks * n_blocks).sum())
    if max_seqlen_k_new > 0 and cu_seqlens_k_new is None and seqused_q is None and cu_seqlens_q is None:
        # The first pass works in programs of 128 sequences (:467-506) and its sum is not masked: a lane past
        # the batch reads 0 keys but still gets the constant query length and the constant appended length,
        # so every padding lane adds one sequence of max_seqlen_q queries and max_seqlen_k_new keys.
        pad = -batch_size % 128
        total += pad * int(-(-(max_seqlen_q * plan["q_per_kv"]) // plan["block_m"])) * int(-(-max_seqlen_k_new // plan["block_n"]))
    f = np.float32
    per_sm = max(1, int(np.ceil(f(f(f(total) * f(1.1)) * f(plan["heads"])) / f(num_sm))))
    splits = np.maximum(1, np.minimum((n_blocks + per_sm - 1) // per_sm, plan["num_splits"]))
    return torch.from_numpy(np.concatenate([[0], splits]).astype(np.int32))
