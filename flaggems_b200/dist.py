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
    """Assemble the row-major ``[M, N]`` from per-rank column shards ``[M, N/world]`` with the
    library collective (NCCL on GPUs, gloo on CPU).

    The collective gathers whole shards (``[world, M, N/world]``, one contiguous message per
    peer); a transposing copy (``M x N`` elements, an SM kernel on GPUs) then lays them side by
    side, into ``out`` when given.  :class:`PeerGather` produces the same matrix without that
    copy."""
    if world == 1:
        return local
    M, n = local.shape
    tmp = torch.empty((world, M, n), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(tmp.view(world * M, n), local.contiguous(), group=group)
    if out is None:
        out = torch.empty((M, world * n), dtype=local.dtype, device=local.device)
    out.view(M, world, n).copy_(tmp.permute(1, 0, 2))
    return out


class PeerGather:
    """All-gather of column shards ``[M, n]`` into the row-major ``[M, world * n]`` matrix by
    copy-engine pushes over NVLink.

    NCCL's all-gather runs on SMs and competes with the compute kernels it is meant to
    overlap (a persistent GEMM loses whole waves when some SMs are taken), and it delivers
    ``[world, M, n]``, which still has to be transposed into the matrix the unsharded operator
    returns.  Here every rank owns the result matrix itself, ``[M, world * n]`` in symmetric
    memory (``torch.distributed._symmetric_memory``: the same allocation on every rank, mapped
    into every peer's address space).  The producer writes its shard straight into columns
    ``[rank * n, (rank + 1) * n)`` of its own matrix (``local_slot``: a strided view, which the
    GEMM takes as its output), ``push`` copies those columns into the same columns of every
    peer's matrix with strided device-to-device copies (``fg_copy_2d``: DMA engines, no SM, no
    multicast; about 760 GB/s per direction on B200), and ``finish`` closes the round with one
    tiny NCCL all-reduce on the same stream: when it completes on a rank, every rank has passed
    its own copies, so every column block of the local matrix is filled.  ``columns()`` is that
    matrix: no copy.

    ``buffers=2`` keeps two result matrices, so that the pushes of one round may still be in
    flight while the producer already writes the next round into the other matrix.

    On CPU tensors (gloo tests) it degrades to ``all_gather_into_tensor`` plus the transposing copy.
    The caller must not reuse a matrix before the consumers of its previous contents, and the
    ``finish`` of the round that filled it, are done.
    """

    def __init__(self, shard_shape, dtype, device, group=None, buffers: int = 1, push_streams: int = 1):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.shard_shape = tuple(shard_shape)
        if len(self.shard_shape) != 2:
            raise ValueError("PeerGather gathers two-dimensional column shards")
        M, n = self.shard_shape
        self.use_p2p = self.device.type == "cuda" and self.world > 1
        full = (M, self.world * n)
        self.bufs: List[torch.Tensor] = []
        self.peer_bufs: List[List[Optional[torch.Tensor]]] = []
        if self.use_p2p:
            import torch.distributed._symmetric_memory as symm_mem

            from . import _lib

            self._copy_2d = _lib.load().fg_copy_2d
            self._check = _lib.check
            self._handles = []
            for _ in range(buffers):
                buf = symm_mem.empty(full, dtype=dtype, device=self.device)
                handle = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
                self.bufs.append(buf)
                self._handles.append(handle)
                self.peer_bufs.append([None if p == self.rank else handle.get_buffer(p, full, dtype)
                                       for p in range(self.world)])
            self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
            # push_streams > 1: the copies to different peers are issued on that many side streams, so
            # that a rank sends to several peers at once and a peer that is momentarily busy with
            # another sender does not hold up the rank's whole queue
            self._side = [torch.cuda.Stream(device=self.device) for _ in range(push_streams)] \
                if push_streams > 1 else []
            dist.barrier(group=group)
        else:
            self.bufs = [torch.empty(full, dtype=dtype, device=self.device) for _ in range(buffers)]
        self.buf = self.bufs[0]

    def local_slot(self, b: int = 0) -> torch.Tensor:
        """This rank's own columns of result matrix ``b``: a producer that writes its shard
        here saves the local copy ``push`` would otherwise make."""
        n = self.shard_shape[1]
        return self.bufs[b][:, self.rank * n:(self.rank + 1) * n]

    def push(self, local: torch.Tensor, rows: Optional[Tuple[int, int]] = None, b: int = 0) -> None:
        """Enqueue, on the current stream, the copies of ``local`` (or of its rows
        ``[rows[0], rows[1])``) into this rank's columns of every rank's matrix ``b``."""
        M, n = self.shard_shape
        r0, r1 = rows if rows is not None else (0, M)
        if not self.use_p2p:
            if r1 < M:
                return  # the collective form moves the whole shard with its last block
            if self.world == 1:
                if local.data_ptr() != self.bufs[b].data_ptr():
                    self.bufs[b].copy_(local)
            else:
                all_gather_columns(local, self.world, self.group, out=self.bufs[b])
            return
        mine = self.local_slot(b)
        if local.data_ptr() != mine.data_ptr():
            mine[r0:r1].copy_(local[r0:r1], non_blocking=True)
        es = mine.element_size()
        pitch = mine.stride(0) * es
        cur = torch.cuda.current_stream(self.device)
        ready = None
        if self._side:
            ready = torch.cuda.Event()
            ready.record(cur)
            for st in self._side:
                st.wait_event(ready)
        # The peers are taken in staggered order (rank + 1, rank + 2, ...), so that ranks in step send to
        # different peers at any one time.
        for i in range(1, self.world):
            p = (self.rank + i) % self.world
            dst = self.peer_bufs[b][p]
            st = self._side[(i - 1) % len(self._side)] if self._side else cur
            self._check(self._copy_2d(dst.data_ptr() + r0 * pitch + self.rank * n * es, pitch,
                                      mine.data_ptr() + r0 * pitch, pitch, n * es, r1 - r0, st.cuda_stream))
        for st in self._side:   # what follows on the current stream (finish) comes after every copy
            done = torch.cuda.Event()
            done.record(st)
            cur.wait_event(done)

    def finish(self) -> None:
        """Close a round of pushes (current stream): afterwards the matrix holds every shard."""
        if self.use_p2p:
            dist.all_reduce(self._token, group=self.group)

    def columns(self, b: int = 0) -> torch.Tensor:
        """The gathered row-major ``[M, world * n]`` matrix (the buffer itself, no copy)."""
        return self.bufs[b]


class PeerGatherSlots:
    """All-gather of equally shaped shards into ``[world, *shard_shape]`` (one contiguous slot per
    rank) by copy-engine pushes over NVLink: the form with plain one-dimensional copies.

    Same protocol as :class:`PeerGather` (symmetric-memory buffers, the producer writes into
    ``local_slot``, ``push`` copies it into slot ``rank`` of every peer's buffer, ``finish`` closes
    the round with one tiny NCCL all-reduce on the same stream), but what a rank receives from a
    peer is one contiguous block.  On eight B200s stepping through the benchmark, contiguous
    pushes run at 700-720 GB/s per rank beside the compute kernels where the strided ones of
    :class:`PeerGather` reach 500-560 GB/s (in isolation both reach 750 GB/s); the price is
    the layout: the row-major ``[M, world * n]`` matrix takes one more, transposing copy
    (``columns()``).  ``buffers=2`` keeps two gather buffers for rounds that overlap.

    On CPU tensors (gloo tests) it degrades to ``all_gather_into_tensor``.
    The caller must not reuse a buffer before the consumers of its previous contents, and the
    ``finish`` of the round that filled it, are done.
    """

    def __init__(self, shard_shape, dtype, device, group=None, buffers: int = 1):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.shard_shape = tuple(shard_shape)
        self.use_p2p = self.device.type == "cuda" and self.world > 1
        full = (self.world, *self.shard_shape)
        self.bufs: List[torch.Tensor] = []
        self.peer_slots: List[List[Optional[torch.Tensor]]] = []
        if self.use_p2p:
            import torch.distributed._symmetric_memory as symm_mem

            self._handles = []
            for _ in range(buffers):
                buf = symm_mem.empty(full, dtype=dtype, device=self.device)
                handle = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
                self.bufs.append(buf)
                self._handles.append(handle)
                self.peer_slots.append([None if p == self.rank else handle.get_buffer(p, full, dtype)[self.rank]
                                        for p in range(self.world)])
            self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
            dist.barrier(group=group)
        else:
            self.bufs = [torch.empty(full, dtype=dtype, device=self.device) for _ in range(buffers)]
        self.buf = self.bufs[0]

    def local_slot(self, b: int = 0) -> torch.Tensor:
        """This rank's own slot of gather buffer ``b``: a producer that writes its shard here
        saves the local copy ``push`` would otherwise make."""
        return self.bufs[b][self.rank]

    def push(self, local: torch.Tensor, rows: Optional[Tuple[int, int]] = None, b: int = 0) -> None:
        """Enqueue, on the current stream, the copies of ``local`` (or of its rows
        ``[rows[0], rows[1])``) into slot ``rank`` of every rank's buffer ``b``."""
        r0, r1 = rows if rows is not None else (0, self.shard_shape[0])
        buf = self.bufs[b]
        if not self.use_p2p:
            if r1 < self.shard_shape[0]:
                return  # the collective form moves the whole shard with its last block
            if self.world == 1:
                if local.data_ptr() != buf[0].data_ptr():
                    buf[0].copy_(local)
            else:
                dist.all_gather_into_tensor(buf.view(self.world * self.shard_shape[0], *self.shard_shape[1:]),
                                            local.contiguous(), group=self.group)
            return
        src = local[r0:r1]
        if local.data_ptr() != buf[self.rank].data_ptr():
            buf[self.rank][r0:r1].copy_(src, non_blocking=True)
        # One stream: the copies to the peers follow each other, staggered so that ranks in step send
        # to different peers at any one time.
        for i in range(1, self.world):
            p = (self.rank + i) % self.world
            self.peer_slots[b][p][r0:r1].copy_(src, non_blocking=True)

    def finish(self) -> None:
        """Close a round of pushes (current stream): afterwards the buffer holds every shard."""
        if self.use_p2p:
            dist.all_reduce(self._token, group=self.group)

    def columns(self, b: int = 0) -> torch.Tensor:
        """The gathered ``[M, world * n]`` matrix: a transposing copy of the slots (M x world x n
        elements, an SM kernel on GPUs)."""
        M, n = self.shard_shape
        return self.bufs[b].permute(1, 0, 2).reshape(M, self.world * n)
