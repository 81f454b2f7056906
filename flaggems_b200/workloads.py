"""Seeded synthetic inputs of the benchmark configurations.

Each builder returns plain tensors on the requested device, drawn from a
``torch.Generator`` seeded by the caller, with the shapes, dtypes and value
distributions of the five configurations the operator path is measured on:

1. dense causal SDPA, fp32, B=2 H=8 S=512 D=64 (CPU-runnable oracle case)
2. Llama-style elementwise block, bf16, T=4096, hidden 4096: fused_add_rms_norm,
   rotary_embedding (32 q heads, 8 kv heads, head 128), silu_and_mul on [T, 22016]
3. varlen causal GQA prefill: 16 sequences, lengths uniform in [128, 4096]
4. paged decode: batch 256, contexts uniform in [512, 8192], block 16, one new token
5. mm/addmm at Llama-3-8B projection shapes, M=8192

Lengths, block tables and slot mappings are drawn from a seeded CPU generator; tensor
values from a generator on the target device seeded from it.  Size arguments shrink a
configuration for tests while keeping its structure.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

GEMM_SHAPES: Dict[str, Tuple[int, int]] = {  # name -> (K, N) at M = 8192
    "qkv": (4096, 6144),
    "o": (4096, 4096),
    "gate_up": (4096, 28672),
    "down": (14336, 4096),
}


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def _randn(g, shape, dtype, device, std=1.0, mean=0.0):
    """N(mean, std) tensor.  On a CUDA device the numbers come from a device generator
    whose seed is drawn from ``g`` (multi-GB caches would take minutes on the host);
    comparisons against a CPU oracle always copy these very tensors, so both sides see
    the same values."""
    dev = torch.device(device)
    out = torch.empty(shape, dtype=dtype, device=dev)
    flat = out.view(-1)
    n = flat.numel()
    sub_seed = int(torch.randint(0, 2 ** 62, (1,), generator=g))
    gd = torch.Generator(device=dev)
    gd.manual_seed(sub_seed)
    step = 1 << 26
    for i in range(0, n, step):
        c = torch.randn(min(step, n - i), generator=gd, dtype=torch.float32, device=dev)
        if std != 1.0:
            c.mul_(std)
        if mean != 0.0:
            c.add_(mean)
        flat[i:i + c.numel()] = c.to(dtype)
    return out


# --------------------------------------------------------------------------- config 1
def sdpa_inputs(seed=0, B=2, H=8, S=512, D=64, device="cpu"):
    g = _gen(seed)
    q, k, v = (_randn(g, (B, H, S, D), torch.float32, device) for _ in range(3))
    return q, k, v, 1.0 / math.sqrt(D)


# --------------------------------------------------------------------------- config 2
def norm_inputs(seed=0, T=4096, hidden=4096, dtype=torch.bfloat16, device="cuda"):
    g = _gen(seed)
    x = _randn(g, (T, hidden), dtype, device)
    residual = _randn(g, (T, hidden), dtype, device)
    w = _randn(g, (hidden,), dtype, device, std=0.1, mean=1.0)
    return x, residual, w, 1e-6


def rope_tables(max_pos: int, dim: int, dtype, device, theta: float = 10000.0):
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq)
    return freqs.cos().to(dtype).to(device), freqs.sin().to(dtype).to(device)


def rope_inputs(seed=0, T=4096, q_heads=32, k_heads=8, head_dim=128, dtype=torch.bfloat16, device="cuda"):
    g = _gen(seed)
    q = _randn(g, (T, q_heads, head_dim), dtype, device)
    k = _randn(g, (T, k_heads, head_dim), dtype, device)
    cos, sin = rope_tables(T, head_dim, dtype, device)
    positions = torch.arange(T, dtype=torch.int64, device=device)
    return q, k, cos, sin, positions


def silu_inputs(seed=0, T=4096, width=22016, dtype=torch.bfloat16, device="cuda"):
    g = _gen(seed)
    return _randn(g, (T, width), dtype, device)


# --------------------------------------------------------------------------- configs 3 / 4
@dataclass
class PagedBatch:
    """A batch laid out for the paged form of flash_attn_varlen_func."""
    q: torch.Tensor             # [total_q, Hq, D]
    key_cache: torch.Tensor     # [num_blocks, block_size, Hk, D]
    value_cache: torch.Tensor
    cu_seqlens_q: torch.Tensor  # int32 [B+1]
    seqused_k: torch.Tensor     # int32 [B]
    block_table: torch.Tensor   # int32 [B, max_blocks]
    query_lens: List[int]
    kv_lens: List[int]
    max_seqlen_q: int
    max_seqlen_k: int
    scale: float
    # contiguous form of the same K/V (prefill only)
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    cu_seqlens_k: Optional[torch.Tensor] = None
    # decode only
    new_key: Optional[torch.Tensor] = None
    new_value: Optional[torch.Tensor] = None
    # int64 cache slot of every new token (decode), or of every packed K/V row (prefill)
    slot_mapping: Optional[torch.Tensor] = None


def _block_table(g, kv_lens, block_size, slack_blocks=0):
    blocks = [(n + block_size - 1) // block_size for n in kv_lens]
    num_blocks = sum(blocks) + slack_blocks
    perm = torch.randperm(num_blocks, generator=g)
    bt = torch.zeros((len(kv_lens), max(max(blocks), 1)), dtype=torch.int32)
    o = 0
    for i, nb in enumerate(blocks):
        bt[i, :nb] = perm[o:o + nb].to(torch.int32)
        o += nb
    return bt, num_blocks


def prefill_batch(seed=0, num_seqs=16, min_len=128, max_len=4096, q_heads=32, kv_heads=8, head_dim=128,
                  block_size=16, dtype=torch.bfloat16, device="cuda") -> PagedBatch:
    """Config 3: every sequence has q_len == k_len; K/V are provided both packed
    (``k``, ``v``, ``cu_seqlens_k``) and scattered into a paged cache through a random
    permutation of the physical blocks."""
    g = _gen(seed)
    lens = torch.randint(min_len, max_len + 1, (num_seqs,), generator=g).tolist()
    total = sum(lens)
    q = _randn(g, (total, q_heads, head_dim), dtype, device)
    k = _randn(g, (total, kv_heads, head_dim), dtype, device)
    v = _randn(g, (total, kv_heads, head_dim), dtype, device)
    cu = torch.zeros(num_seqs + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
    bt, num_blocks = _block_table(g, lens, block_size)
    kc = torch.zeros((num_blocks, block_size, kv_heads, head_dim), dtype=dtype, device=device)
    vc = torch.zeros_like(kc)
    # scatter the packed rows into their pages (slot = page * block_size + offset)
    slots = torch.empty(total, dtype=torch.int64)
    for i, n in enumerate(lens):
        t = torch.arange(n)
        slots[cu[i]:cu[i] + n] = bt[i, t // block_size].to(torch.int64) * block_size + (t % block_size)
    slots = slots.to(device)
    kc.view(-1, kv_heads, head_dim)[slots] = k
    vc.view(-1, kv_heads, head_dim)[slots] = v
    return PagedBatch(q=q, key_cache=kc, value_cache=vc, cu_seqlens_q=cu.to(device),
                      seqused_k=torch.tensor(lens, dtype=torch.int32, device=device),
                      block_table=bt.to(device), query_lens=lens, kv_lens=lens, max_seqlen_q=max(lens),
                      max_seqlen_k=max(lens), scale=head_dim ** -0.5, k=k, v=v, cu_seqlens_k=cu.to(device),
                      slot_mapping=slots)


def decode_batch(seed=0, batch=256, min_ctx=512, max_ctx=8192, q_heads=32, kv_heads=8, head_dim=128,
                 block_size=16, dtype=torch.bfloat16, device="cuda", fill_cache=True) -> PagedBatch:
    """Config 4: one query token per sequence; the new K/V token is the last position of
    each context and ``slot_mapping`` points at it through the permuted block table."""
    g = _gen(seed)
    ctx = torch.randint(min_ctx, max_ctx + 1, (batch,), generator=g).tolist()
    bt, num_blocks = _block_table(g, ctx, block_size)
    shape = (num_blocks, block_size, kv_heads, head_dim)
    if fill_cache:
        kc = _randn(g, shape, dtype, device)
        vc = _randn(g, shape, dtype, device)
    else:
        kc = torch.zeros(shape, dtype=dtype, device=device)
        vc = torch.zeros(shape, dtype=dtype, device=device)
    q = _randn(g, (batch, q_heads, head_dim), dtype, device)
    new_k = _randn(g, (batch, kv_heads, head_dim), dtype, device)
    new_v = _randn(g, (batch, kv_heads, head_dim), dtype, device)
    last = torch.tensor(ctx) - 1
    slot = bt[torch.arange(batch), last // block_size].to(torch.int64) * block_size + (last % block_size)
    return PagedBatch(q=q, key_cache=kc, value_cache=vc,
                      cu_seqlens_q=torch.arange(batch + 1, dtype=torch.int32, device=device),
                      seqused_k=torch.tensor(ctx, dtype=torch.int32, device=device),
                      block_table=bt.to(device), query_lens=[1] * batch, kv_lens=ctx, max_seqlen_q=1,
                      max_seqlen_k=max(ctx), scale=head_dim ** -0.5, new_key=new_k, new_value=new_v,
                      slot_mapping=slot.to(device))


def prefill_flops(lens, q_heads=32, head_dim=128) -> float:
    """Causal attention FLOPs: 4 * D * Hq * sum L(L+1)/2."""
    return float(sum(4 * head_dim * q_heads * (n * (n + 1) // 2) for n in lens))


def decode_bytes(ctx, batch, q_heads=32, kv_heads=8, head_dim=128, elem=2) -> float:
    """Algorithmic bytes of one decode step: K and V of every context once, q and out."""
    return float(2 * sum(ctx) * kv_heads * head_dim * elem + 2 * batch * q_heads * head_dim * elem
                 + batch * 4 + sum((c + 15) // 16 for c in ctx) * 4)


# --------------------------------------------------------------------------- config 5
def gemm_inputs(name: str, seed=0, M=8192, dtype=torch.bfloat16, device="cuda", b_column_major=False):
    K, N = GEMM_SHAPES[name]
    g = _gen(seed)
    a = _randn(g, (M, K), dtype, device)
    if b_column_major:
        b = _randn(g, (N, K), dtype, device, std=1.0 / math.sqrt(K)).t()
    else:
        b = _randn(g, (K, N), dtype, device, std=1.0 / math.sqrt(K))
    bias = _randn(g, (N,), dtype, device, std=0.02)
    return a, b, bias
