"""Multi-GPU partitioning of the path, one process per GPU (``torch.distributed``).

FlagGems itself has no distributed code.  The path shards where it is independent:
attention, cache writes and rope by KV head (no communication; outputs stay sharded
by head as in tensor-parallel serving), and the projections column-parallel with an
all-gather of the output shards (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open slice of ``total`` items owned by ``rank`` (remainder spread over the
    first ranks)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def kv_head_shard(num_heads: int, num_kv_heads: int, rank: int, world: int):
    """(q_head slice, kv_head slice) of a rank when attention is split by KV head."""
    if num_heads % num_kv_heads:
        raise ValueError("num_heads must be a multiple of num_kv_heads")
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} KV heads do not split over {world} ranks")
    group = num_heads // num_kv_heads
    k0, k1 = shard_range(num_kv_heads, rank, world)
    return slice(k0 * group, k1 * group), slice(k0, k1)


def column_shard(weight: torch.Tensor, bias, rank: int, world: int):
    """Column shard of B ``[K, N]`` (and bias ``[N]``) for column-parallel mm/addmm.
    N must split into 8-element multiples so every shard keeps 16-byte aligned rows."""
    N = weight.shape[1]
    if N % (8 * world):
        raise ValueError(f"N={N} does not split into {world} shards of 8-element multiples")
    c0, c1 = shard_range(N, rank, world)
    w = weight[:, c0:c1].contiguous()
    b = None if bias is None else bias[c0:c1].contiguous()
    return w, b


def all_gather_columns(local: torch.Tensor, world: int, group=None, out: torch.Tensor = None) -> torch.Tensor:
    """Assemble ``[M, N]`` from per-rank column shards ``[M, N/world]``.

    The collective gathers whole shards (``[world, M, N/world]``, one contiguous
    message per peer); a strided copy then lays them side by side.  ``out`` may be
    given to reuse the gather buffer across steps."""
    if world == 1:
        return local
    M, n = local.shape
    buf = out if out is not None else torch.empty((world * M, n), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf.view(world * M, n), local.contiguous(), group=group)
    return buf.view(world, M, n).permute(1, 0, 2).reshape(M, world * n)
