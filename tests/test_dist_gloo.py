"""World-size-2 CPU (gloo) test of the multi-GPU host logic: column-parallel GEMM shards
gathered into the full output, and KV-head sharding of attention with no exchange.  The
per-rank arithmetic is done with torch CPU ops here (the CUDA kernels need a GPU); what
is under test is the partitioning, the collective and the layout of the gathered result."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flaggems_b200 import dist as fdist


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)  # same data on every rank
        a = torch.randn(12, 32, generator=g)
        w = torch.randn(32, 48, generator=g)
        bias = torch.randn(48, generator=g)
        ws, bs = fdist.column_shard(w, bias, rank, world)
        local = torch.addmm(bs, a, ws)
        full = fdist.all_gather_columns(local, world)
        ok_gemm = torch.allclose(full, torch.addmm(bias, a, w), atol=1e-5)
        # the same through the gather object the GPU benchmark uses (collective fallback on CPU)
        pg = fdist.PeerGather(local.shape, local.dtype, "cpu")
        pg.push(local)
        pg.finish()
        ok_gemm = ok_gemm and torch.allclose(pg.columns(), torch.addmm(bias, a, w), atol=1e-5)
        ok_gemm = ok_gemm and pg.columns().is_contiguous() and pg.columns().data_ptr() == pg.bufs[0].data_ptr()
        # the contiguous-slot form, two buffers: [world, M, n] per buffer, columns() transposes
        ps = fdist.PeerGatherSlots(local.shape, local.dtype, "cpu", buffers=2)
        for b in (0, 1):
            ps.push(local * (b + 1), b=b)
            ps.finish()
            ok_gemm = ok_gemm and torch.allclose(ps.columns(b), (b + 1) * torch.addmm(bias, a, w), atol=1e-5)
            ok_gemm = ok_gemm and torch.allclose(ps.bufs[b][rank], (b + 1) * local)
        # attention by KV head: each rank's output slice equals the same slice of the full result
        q = torch.randn(5, 8, 16, generator=g)
        k = torch.randn(5, 4, 16, generator=g)
        v = torch.randn(5, 4, 16, generator=g)
        def attn(q, k, v):
            k = k.repeat_interleave(q.shape[1] // k.shape[1], dim=1)
            v = v.repeat_interleave(q.shape[1] // v.shape[1], dim=1)
            p = torch.softmax(torch.einsum("qhd,khd->hqk", q, k) * 0.25, dim=-1)
            return torch.einsum("hqk,khd->qhd", p, v)
        qs, ks = fdist.kv_head_shard(8, 4, rank, world)
        ok_attn = torch.allclose(attn(q[:, qs], k[:, ks], v[:, ks]), attn(q, k, v)[:, qs], atol=1e-6)
        flag = torch.tensor([int(ok_gemm and ok_attn)])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            ret["ok"] = bool(flag.item())
    finally:
        dist.destroy_process_group()


def test_column_parallel_and_head_sharding_world2():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret.get("ok") is True
