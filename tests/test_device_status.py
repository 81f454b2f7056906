"""The device status word: a kernel whose bounded wait gave up must be impossible to miss.

CPU part: with the word set through the test hook, every launching entry point of the C
ABI refuses to launch (FG_ERR_DEVICE) and the Python wrappers raise; clearing restores
them.  GPU part: a single-thread kernel waits with the library's own bounded wait (limit
5 ms) on an mbarrier nothing arrives at -- no copy or MMA in flight, nothing faults or
hangs -- and the host sees the code without a synchronising read.
"""
import ctypes as C

import pytest
import torch

from flaggems_b200 import _lib

FG_ERR_DEVICE = -5


def test_every_launching_entry_point_refuses_while_the_word_is_set():
    lib = _lib.load()
    assert lib.fg_device_status_nosync() == 0
    lib.fg_debug_set_status(102)
    try:
        assert lib.fg_device_status_nosync() == 102
        z = C.c_int64(0)
        calls = {
            "fg_gemm": lambda: lib.fg_gemm(C.byref(_lib.GemmParams()), None),
            "fg_gemm_f32_split": lambda: lib.fg_gemm_f32_split(C.byref(_lib.GemmParams()), None, 0, None),
            "fg_gemm_batched": lambda: lib.fg_gemm_batched(C.byref(_lib.GemmParams()), 1, 0, 0, 0, 0, None),
            "fg_flash_attn_varlen": lambda: lib.fg_flash_attn_varlen(C.byref(_lib.AttnParams()), None),
            "fg_flash_attn_decode_static": lambda: lib.fg_flash_attn_decode_static(C.byref(_lib.AttnParams()), None),
            "fg_fused_add_rms_norm": lambda: lib.fg_fused_add_rms_norm(None, None, None, 1, 1, 1, 1, 1e-6, 2, None),
            "fg_rms_norm": lambda: lib.fg_rms_norm(None, None, None, 1, 1, 1, 1, 1e-6, 2, None),
            "fg_silu_and_mul": lambda: lib.fg_silu_and_mul(None, None, None, 0, None, None, None, None, 2, None),
            "fg_gelu_and_mul": lambda: lib.fg_gelu_and_mul(None, None, None, 0, None, None, None, None, 0, 2, None),
            "fg_rotary_embedding": lambda: lib.fg_rotary_embedding(C.byref(_lib.RopeParams()), None),
            "fg_reshape_and_cache_flash": lambda: lib.fg_reshape_and_cache_flash(
                None, None, None, None, None, 1, 1, 8, 16, 1, 8, 8, 128, 8, 8, 2, None),
            "fg_reshape_and_cache": lambda: lib.fg_reshape_and_cache(
                None, None, None, None, None, 1, 1, 8, 16, 1, 8, 8, 8, 2, None),
            "fg_get_scheduler_metadata": lambda: lib.fg_get_scheduler_metadata(
                C.byref(_lib.SchedulerParams()), None, None),
        }
        del z
        for name, call in calls.items():
            assert call() == FG_ERR_DEVICE, name
            assert b"status 102" in lib.fg_last_error(), name
        with pytest.raises(RuntimeError, match="gave up a bounded wait"):
            _lib.check(calls["fg_gemm"]())
        # host-only queries keep working
        assert lib.fg_flash_attn_workspace_bytes(4, 32, 128, 1, 4096) > 0
    finally:
        lib.fg_device_status(1)
    assert lib.fg_device_status_nosync() == 0
    # cleared: the same call now gets as far as its own argument checks
    assert lib.fg_gemm(C.byref(_lib.GemmParams()), None) == 0          # M = N = 0: nothing to do
    p = _lib.GemmParams()
    p.M = p.N = p.K = -1
    assert lib.fg_gemm(C.byref(p), None) == -1


@pytest.mark.gpu
def test_a_timed_out_wait_reaches_the_host_and_blocks_further_launches(fg):
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    a = torch.randn(256, 512, dtype=torch.bfloat16, device=dev)
    b = torch.randn(512, 256, dtype=torch.bfloat16, device=dev)
    good = fg.mm(a, b)                      # also sets up the host-visible word on this device
    torch.cuda.synchronize()
    assert _lib.device_status(reset=True) == 0
    outcome = torch.zeros(1, dtype=torch.int32, device=dev)
    try:
        _lib.check(lib.fg_debug_wait_timeout(5_000_000, outcome.data_ptr(), _lib.stream_ptr(dev)))
        torch.cuda.synchronize()            # the kernel returns by itself after ~5 ms
        assert int(outcome.item()) == 2     # the wait gave up (it did not see a phase that never came)
        assert _lib.device_status_nosync() == 103          # read from pinned host memory, no device read
        with pytest.raises(RuntimeError, match="gave up a bounded wait"):
            fg.mm(a, b)
        with pytest.raises(RuntimeError, match="gave up a bounded wait"):
            with fg.use_gems():
                torch.mm(a, b)
        assert _lib.device_status() == 103                 # the device word agrees
    finally:
        _lib.device_status(reset=True)
    assert _lib.device_status_nosync() == 0 and _lib.device_status() == 0
    assert torch.equal(fg.mm(a, b), good)                  # the context is intact and the kernels run again
    # A launch that is already queued behind the wait when it gives up: the host word was still clear
    # when it was enqueued, so it is launched; its CTAs read the device word on entry and return
    # without touching the output (the launch drains instead of running into the same timeout).
    out = torch.full((256, 256), 7.0, dtype=torch.bfloat16, device=dev)
    queued = False
    for _ in range(5):                                         # a host hiccup may make the enqueue come too late
        try:
            _lib.check(lib.fg_debug_wait_timeout(100_000_000, outcome.data_ptr(), _lib.stream_ptr(dev)))
            try:
                fg.mm_out(a, b, out=out)                       # enqueued within the 100 ms the wait lasts
                queued = True
            except RuntimeError:
                pass                                           # the wait had already given up: refused, try again
            torch.cuda.synchronize()
            assert _lib.device_status_nosync() == 103
            assert bool((out == 7.0).all()), "a drained (or refused) launch must not write its output"
        finally:
            _lib.device_status(reset=True)
        if queued:
            break
    if not queued:
        pytest.skip("the host never enqueued the second launch within 100 ms of the first")
    fg.mm_out(a, b, out=out)
    assert torch.equal(out, good)
