"""Decode attention without any allocation at call time (fg_flash_attn_decode_static).

Serving runtimes that pre-reserve all device memory, and hosts that use the C ABI
without an allocator of their own, cannot hand the split-KV kernel a workspace; this
entry point keeps that scratch in a fixed array inside the library.  Here it is called
straight through the C ABI, twice in a row (a large batch, then a smaller one, so the
second call runs over the leftovers of the first), and each result is compared with the
regular entry point fed a caller-allocated workspace -- the same kernels on the same chunk
plan, so the comparison is bit for bit -- and once with the CPU oracle.  A further call must
change neither the free device memory nor launch anything beyond its two kernels.
Collected last on purpose.
"""
import ctypes as C

import pytest
import torch

from flaggems_b200 import _lib, workloads
from oracle import reference_oracle as O  # checker only

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 1e-2  # the tolerance of the attention parity tests (used against the oracle)


def _params(b, out, lse):
    p = _lib.AttnParams()
    p.q, p.k, p.v, p.out, p.lse = b.q.data_ptr(), b.key_cache.data_ptr(), b.value_cache.data_ptr(), out.data_ptr(), \
        lse.data_ptr()
    p.cu_seqlens_q, p.seqused_k, p.block_table = b.cu_seqlens_q.data_ptr(), b.seqused_k.data_ptr(), \
        b.block_table.data_ptr()
    p.q_row_stride, p.q_head_stride = b.q.stride(0), b.q.stride(1)
    p.o_row_stride, p.o_head_stride = out.stride(0), out.stride(1)
    p.k_block_stride, p.k_row_stride, p.k_head_stride = b.key_cache.stride()[:3]
    p.v_block_stride, p.v_row_stride, p.v_head_stride = b.value_cache.stride()[:3]
    p.block_table_stride = b.block_table.stride(0)
    p.total_q, p.batch = b.q.shape[0], b.q.shape[0]
    p.num_heads, p.head_dim, p.num_heads_k = b.q.shape[1], b.q.shape[2], b.key_cache.shape[2]
    p.max_seqlen_q, p.max_seqlen_k = 1, b.max_seqlen_k
    p.block_size, p.num_blocks = b.key_cache.shape[1], b.key_cache.shape[0]
    p.window_left = p.window_right = -1
    p.softmax_scale, p.softcap = b.scale, 0.0
    p.causal, p.dtype = 1, _lib.dtype_code(b.q.dtype)
    return p


def _run_both(lib, b):
    dev = b.q.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    out_s, out_w = torch.empty_like(b.q), torch.empty_like(b.q)
    lse_s = torch.empty((b.q.shape[1], b.q.shape[0]), dtype=torch.float32, device=dev)
    lse_w = torch.empty_like(lse_s)
    # regular entry point with a workspace the caller allocated
    nbytes = lib.fg_flash_attn_workspace_bytes(b.q.shape[0], b.q.shape[1], b.q.shape[2], 1, b.max_seqlen_k)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    pw = _params(b, out_w, lse_w)
    pw.workspace, pw.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(lib.fg_flash_attn_varlen(C.byref(pw), stream))
    # the entry point under test: no workspace is passed at all
    ps = _params(b, out_s, lse_s)
    _lib.check(lib.fg_flash_attn_decode_static(C.byref(ps), stream))
    torch.cuda.synchronize()
    return out_s, lse_s, out_w, lse_w


def test_decode_static_matches_workspace_entry_point_twice_in_a_row():
    lib = _lib.load()
    assert lib.fg_flash_attn_decode_static_capacity() == 64 << 20
    first = workloads.decode_batch(seed=31, batch=48, min_ctx=200, max_ctx=6000, device="cuda")
    second = workloads.decode_batch(seed=32, batch=5, min_ctx=10, max_ctx=3000, device="cuda")
    for b in (first, second):
        out_s, lse_s, out_w, lse_w = _run_both(lib, b)
        assert torch.isfinite(out_s).all()
        # same kernels, same chunk plan, only the scratch differs: identical bits
        assert torch.equal(out_s, out_w)
        assert torch.equal(lse_s, lse_w)
    # the second (smaller) batch also against the CPU oracle
    ref = O.paged_attention(second.q.cpu(), second.key_cache.cpu(), second.value_cache.cpu(), second.query_lens,
                            second.kv_lens, second.block_table.cpu(), second.scale, compute_dtype=torch.float32)
    torch.testing.assert_close(out_s.cpu().float(), ref.float(), atol=ATOL, rtol=RTOL)


def test_decode_static_call_allocates_nothing_and_launches_two_kernels():
    lib = _lib.load()
    b = workloads.decode_batch(seed=34, batch=32, min_ctx=300, max_ctx=5000, device="cuda")
    out = torch.empty_like(b.q)
    lse = torch.empty((b.q.shape[1], b.q.shape[0]), dtype=torch.float32, device="cuda")
    p = _params(b, out, lse)
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.fg_flash_attn_decode_static(C.byref(p), stream))   # first touch on this device, if it is
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    launches0 = lib.fg_launch_count()
    _lib.check(lib.fg_flash_attn_decode_static(C.byref(p), stream))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "the call changed the free device memory"
    assert lib.fg_launch_count() - launches0 == 2   # the split-KV kernel and the combine kernel


def test_decode_static_rejects_what_does_not_fit_or_is_not_decode():
    lib = _lib.load()
    b = workloads.decode_batch(seed=33, batch=4, min_ctx=64, max_ctx=300, device="cuda")
    out = torch.empty_like(b.q)
    lse = torch.empty((b.q.shape[1], b.q.shape[0]), dtype=torch.float32, device="cuda")
    p = _params(b, out, lse)
    # a plan far beyond the built-in array: 4096 sequences x 64 heads x 8 chunks of 1024 tokens
    p.batch = p.total_q = 4096
    p.num_heads, p.num_heads_k = 64, 8
    p.max_seqlen_k = 8192
    assert lib.fg_flash_attn_decode_static(C.byref(p), None) == -4
    assert b"built-in array" in lib.fg_last_error()
    # more than one query token per sequence is not a decode batch
    p = _params(b, out, lse)
    p.max_seqlen_q = 2
    assert lib.fg_flash_attn_decode_static(C.byref(p), None) == -1
