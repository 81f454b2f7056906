"""Multi-GPU partitioning of the path, one process per GPU (``torch.distributed``).

FlagGems itself has no distributed code.  The path shards where it is independent:
attention, cache writes and rope by KV head (no communication; outputs stay sharded
by head as in tensor-parallel serving), and the projections column-parallel with an
all-gather of the output shards (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

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


class PeerGather:
    """All-gather of equally shaped shards by copy-engine pushes over NVLink.

    NCCL's all-gather runs on SMs and competes with the compute kernels it is meant to
    overlap (a persistent GEMM loses whole waves when some SMs are taken).  Here every
    rank owns a gather buffer ``[world, *shard_shape]`` in symmetric memory
    (``torch.distributed._symmetric_memory``: the same allocation on every rank, mapped
    into every peer's address space); ``push`` copies the local shard into slot ``rank``
    of every peer's buffer with plain device-to-device copies (DMA engines, no SM; about
    760 GB/s per direction on B200), and ``finish`` closes the round with one tiny NCCL
    all-reduce on the same stream: when it completes on a rank, every rank has passed
    its own copies, so all slots of the local buffer are filled.

    On CPU tensors (gloo tests) it degrades to ``all_gather_into_tensor``.
    The caller must not start the next round of pushes before the consumers of the
    previous result are done with it.
    """

    def __init__(self, shard_shape, dtype, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.shard_shape = tuple(shard_shape)
        self.peer_slots: List[Optional[torch.Tensor]] = [None] * self.world
        self.use_p2p = self.device.type == "cuda" and self.world > 1
        full = (self.world, *self.shard_shape)
        if self.use_p2p:
            import torch.distributed._symmetric_memory as symm_mem

            self.buf = symm_mem.empty(full, dtype=dtype, device=self.device)
            self._handle = symm_mem.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
            for p in range(self.world):
                if p != self.rank:
                    self.peer_slots[p] = self._handle.get_buffer(p, full, dtype)[self.rank]
            self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
            dist.barrier(group=group)
        else:
            self.buf = torch.empty(full, dtype=dtype, device=self.device)

    def local_slot(self) -> torch.Tensor:
        """This rank's own slot of the gather buffer: a producer that writes its shard here
        saves the local copy ``push`` would otherwise make."""
        return self.buf[self.rank]

    def push(self, local: torch.Tensor, rows: Optional[Tuple[int, int]] = None) -> None:
        """Enqueue, on the current stream, the copies of ``local`` (or of its rows
        ``[rows[0], rows[1])``) into every rank's slot.  Pushing a shard in row blocks as
        they are produced lets the transfer start before the producer has finished."""
        r0, r1 = rows if rows is not None else (0, self.shard_shape[0])
        if not self.use_p2p:
            if r1 < self.shard_shape[0]:
                return  # the collective form moves the whole shard with its last block
            if self.world == 1:
                self.buf[0].copy_(local)
            else:
                dist.all_gather_into_tensor(self.buf.view(self.world * self.shard_shape[0], *self.shard_shape[1:]),
                                            local.contiguous(), group=self.group)
            return
        src = local[r0:r1]
        if local.data_ptr() != self.buf[self.rank].data_ptr():
            self.buf[self.rank][r0:r1].copy_(src, non_blocking=True)
        # One stream: copies to the peers follow each other.  Spreading them over one stream per
        # peer was measured and changes nothing (the rank's total egress stays near 680 GB/s).
        for i in range(1, self.world):  # staggered so that no peer is hit by everyone at once
            p = (self.rank + i) % self.world
            self.peer_slots[p][r0:r1].copy_(src, non_blocking=True)

    def finish(self) -> None:
        """Close a round of pushes (current stream): afterwards ``buf`` holds every shard."""
        if self.use_p2p:
            dist.all_reduce(self._token, group=self.group)

    def columns(self) -> torch.Tensor:
        """The gathered ``[M, world * n]`` matrix (a strided view of the buffer)."""
        M, n = self.shard_shape
        return self.buf.permute(1, 0, 2).reshape(M, self.world * n)
