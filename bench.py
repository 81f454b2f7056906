#!/usr/bin/env python
"""Benchmark of the inference operator path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One *step* is one pass of the operator path over one batch of seeded synthetic input at
the benchmark configuration sizes: fused_add_rms_norm, rotary_embedding and silu_and_mul
on the T=4096 Llama block, varlen causal GQA prefill (16 sequences, 128..4096 tokens),
reshape_and_cache_flash + paged decode (batch 256, contexts 512..8192), and mm / addmm at
the four Llama-3-8B projection shapes with M=8192.  The headline value is operator
invocations per second; every operator's own figure (TFLOP/s or GB/s against the measured
B200 roofline) is in ``per_op``.

Under ``torchrun`` (N > 1) every rank runs the same step on its own batch of sequences
(no exchange), and the projections become column-parallel: each rank multiplies by its
own column shard and the shards are all-gathered over NVLink with NCCL on a side stream
(weak scaling: fixed work per GPU).

``--impl reference`` times the CPU oracle (torch CPU restatement of the reference's test
oracles) on the host cores on a bounded sample of the same step.

Rank 0 prints exactly one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "inference operator-path throughput (fused_add_rms_norm, rope, silu_and_mul, varlen prefill, " \
         "cache write + paged decode, mm/addmm at the benchmark configs)"
UNIT = "ops/s"
NCCL_CTAS = 16  # SMs left to NCCL's copy kernels when N > 1
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons while the timed region runs:
    an NVML polling thread (every ~5 ms, read-only queries), or `nvidia-smi -lms` when the
    NVML bindings are missing.  The timed region of the default run is only ~50 ms long, too
    short for nvidia-smi's own sampling loop to be sure to hit it."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []      # nvidia-smi form: (time, csv line)
        self.samples = []    # NVML form: (time, sm_mhz, reason names)
        self.thread = None
        self.stop_flag = False
        self.smax = None
        self.nvml = None

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            pr = torch.cuda.get_device_properties(self.index)
            bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
            h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:  # noqa: BLE001
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        return pynvml, h

    def start(self):
        try:
            self.nvml, self.handle = self._nvml_handle()
            self.smax = float(self.nvml.nvmlDeviceGetMaxClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _poll(self):
        n = self.nvml
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons")
        bits = {
            "hw_slowdown": getattr(n, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(n, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self.stop_flag:
            try:
                clk = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = int(get_reasons(self.handle))
                self.samples.append((time.time(), clk, [k for k, b in bits.items() if mask & b]))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.004)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=1)
            inside = [x for x in self.samples if t0 <= x[0] <= t1] or \
                [x for x in self.samples if t0 - 0.05 <= x[0] <= t1 + 0.05] or self.samples
            sm = [x[1] for x in inside]
            reasons = sorted({r for x in inside for r in x[2]})
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.smax, "reasons": reasons,
                    "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML bindings and no nvidia-smi"], "samples": 0}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        for ts, line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                clk, mx = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            smax = mx
            if t0 - 0.05 <= ts <= t1 + 0.25:
                sm.append(clk)
                for n, v in zip(self.NAMES, parts[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        if not sm:  # region shorter than one sample: use whatever was seen
            sm = [float(l.split(",")[0]) for _, l in self.lines if l and l[0].isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi"}


# --------------------------------------------------------------------------- workload
class Step:
    """The operators of one step with their inputs resident on ``device``."""

    def __init__(self, device, rank: int, world: int, seed: int = 0, small: bool = False, only: str = "",
                 gather: str = "p2p", row_blocks: int = 1, op_order: str = "spread"):
        import flaggems_b200 as fg
        from flaggems_b200 import dist as fdist
        from flaggems_b200 import workloads as W

        self.gather = gather
        self.row_blocks = row_blocks
        self.op_order = op_order
        self.skip_gather = False   # N > 1: second timing of the step without the all-gathers

        self.fg, self.W, self.fdist = fg, W, fdist
        self.device, self.rank, self.world = device, rank, world
        self.only = only
        s = seed + 1000 * rank  # every rank owns a different batch of sequences
        self.x, self.res, self.w, self.eps = W.norm_inputs(seed=s + 1, device=device)
        self.q, self.k, self.cos, self.sin, self.pos = W.rope_inputs(seed=s + 2, device=device)
        self.act = W.silu_inputs(seed=s + 3, device=device)
        self.half = self.act.shape[1] // 2
        self.silu_out = torch.empty((self.act.shape[0], self.half), dtype=self.act.dtype, device=device)
        # --small: reduced attention/GEMM sizes for profiler captures (operands still exceed L2)
        pre_kw = dict(num_seqs=8, min_len=1024, max_len=3072) if small else {}
        dec_kw = dict(batch=64, min_ctx=1024, max_ctx=4096) if small else {}
        self.pre = W.prefill_batch(seed=s + 4, device=device, **pre_kw)
        self.pre_out = torch.empty_like(self.pre.q)
        self.dec = W.decode_batch(seed=s + 5, device=device, **dec_kw)
        self.dec_out = torch.empty_like(self.dec.q)
        # projections: A replicated (same seed on every rank), B/bias = this rank's column shard
        self.gemm = {}
        for i, name in enumerate(W.GEMM_SHAPES):
            a, b, bias = W.gemm_inputs(name, seed=seed + 10 + i, device=device, M=2048 if small else 8192)
            if world > 1:  # the shard of a [K, N * world] weight owned by this rank
                _, b, bias = W.gemm_inputs(name, seed=seed + 10 + i + 100 * (rank + 1), device=device,
                                           M=2048 if small else 8192)
            gathered = None
            if world > 1 and gather != "nccl":
                # the GEMM writes its shard straight into this rank's slot of the gather buffer
                gathered = fdist.PeerGather((a.shape[0], b.shape[1]), a.dtype, device)
                c = gathered.local_slot()
            else:
                c = torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device=device)
                if world > 1:
                    gathered = torch.empty((world * a.shape[0], b.shape[1]), dtype=a.dtype, device=device)
            self.gemm[name] = (a, b, bias, c, gathered)
        self.comm_stream = torch.cuda.Stream(device=device) if world > 1 else None
        self.comm_events = {}  # name -> (start, end) events of the last all-gather of that projection
        self.ops = self._build_ops()

    # each entry: (name, callable, work, kind) with kind "hbm" (bytes) or "tensor" (flops)
    def _build_ops(self):
        fg, W = self.fg, self.W
        T, H = self.x.shape
        ops = []
        # The projections come first: with N > 1 their output shards are all-gathered on a side
        # stream while the rest of the step runs.  There a small projection leads so that NVLink is
        # already busy while the largest one (gate_up) computes; gate_up follows at once because
        # its gather is the longest transfer of the step.  (On one GPU the projections are tensor-bound and their
        # order among themselves is immaterial.)
        for name in (("qkv", "gate_up", "down", "o") if self.world > 1 else ("gate_up", "qkv", "down", "o")):
            a, b, bias, c, gathered = self.gemm[name]
            M, K = a.shape
            N = b.shape[1]
            if name in ("qkv", "gate_up"):  # qkv and gate_up carry a bias in the benchmark (addmm), o/down are mm
                ops.append((f"addmm[{name}]", self._gemm_call(name, True), M * N * (2 * K + 1), "tensor"))
            else:
                ops.append((f"mm[{name}]", self._gemm_call(name, False), 2 * M * N * K, "tensor"))
        rest = {}
        rest["fused_add_rms_norm"] = (("fused_add_rms_norm", lambda: fg.fused_add_rms_norm(self.x, self.res, [H], self.w, self.eps),
                    4 * T * H * 2 + H * 2, "hbm"))
        tq, hq, d = self.q.shape
        hk = self.k.shape[1]
        rest["rotary_embedding"] = (("rotary_embedding",
                    lambda: fg.apply_rotary_pos_emb(self.q, self.k, self.cos, self.sin, self.pos, False, True),
                    2 * (tq * hq * d + tq * hk * d) * 2 + tq * 2 * (d // 2) * 2 + tq * 8, "hbm"))
        a1, a2 = self.act[:, :self.half], self.act[:, self.half:]
        rest["silu_and_mul"] = (("silu_and_mul", lambda: fg.silu_and_mul_out(a1, a2, self.silu_out),
                    self.act.numel() * 2 + self.silu_out.numel() * 2, "hbm"))
        p = self.pre
        rest["prefill"] = (("flash_attn_varlen_func[prefill]",
                    lambda: fg.flash_attn_varlen_func(p.q, p.key_cache, p.value_cache, p.max_seqlen_q, p.cu_seqlens_q,
                                                      p.max_seqlen_k, seqused_k=p.seqused_k, causal=True,
                                                      block_table=p.block_table, out=self.pre_out),
                    W.prefill_flops(p.query_lens), "tensor"))
        dd = self.dec
        nk = dd.new_key.numel() * 2
        rest["cache"] = (("reshape_and_cache_flash",
                    lambda: fg.reshape_and_cache_flash(dd.new_key, dd.new_value, dd.key_cache, dd.value_cache,
                                                       dd.slot_mapping, "auto", None, None),
                    4 * nk + dd.slot_mapping.numel() * 8, "hbm"))
        rest["decode"] = (("flash_attn_varlen_func[decode]",
                    lambda: fg.flash_attn_varlen_func(dd.q, dd.key_cache, dd.value_cache, 1, dd.cu_seqlens_q,
                                                      dd.max_seqlen_k, seqused_k=dd.seqused_k, causal=True,
                                                      block_table=dd.block_table, out=self.dec_out),
                    W.decode_bytes(dd.kv_lens, len(dd.kv_lens)), "hbm"))
        # Order of the remaining operators.  The calls are independent (own buffers), so any order computes
        # the same; what the order changes is whose time the write-back of an operator's output is counted
        # in: up to 126 MB of dirty L2 lines leave for DRAM while the NEXT operator runs.  A tensor-bound
        # operator absorbs that, a 20 us streaming kernel doubles its DRAM traffic.  The short memory-bound
        # operators therefore follow the operators that leave the L2 cleanest (--op-order grouped restores the
        # order by operator family that earlier lines of this benchmark used).
        order = (["prefill", "fused_add_rms_norm", "cache", "decode", "rotary_embedding", "silu_and_mul"]
                 if self.op_order == "spread" else
                 ["fused_add_rms_norm", "rotary_embedding", "silu_and_mul", "prefill", "cache", "decode"])
        ops += [rest[k] for k in order]
        if self.only:
            ops = [o for o in ops if self.only in o[0]]
            if not ops:
                raise SystemExit(f"--only {self.only!r} matches no operator")
        return ops

    def _gemm_call(self, name, with_bias):
        fg = self.fg
        a, b, bias, c, gathered = self.gemm[name]

        # With N > 1 and the copy-engine gather, the first and largest projection is computed in
        # row blocks and every block is pushed to the peers as soon as it exists, so the NVLink
        # transfers start a fraction of a GEMM after the step begins instead of a whole one.
        # Measured at N=4: no gain (5.64 ms per step with 2 blocks against 5.39 ms with 1): the
        # GEMM and the copies slow each other down when they overlap, so the default is 1 block.
        blocks = self.row_blocks if (self.world > 1 and self.gather != "nccl" and name == "gate_up") else 1
        M = a.shape[0]
        bounds = [(i * M // blocks, (i + 1) * M // blocks) for i in range(blocks)]

        def run():
            cur = torch.cuda.current_stream(self.device)
            ev = None
            if self.world > 1:
                ev = self.comm_events.setdefault(
                    name, (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
            for bi, (r0, r1) in enumerate(bounds):
                if with_bias:
                    fg.addmm_out(bias, a[r0:r1], b, out=c[r0:r1])
                else:
                    fg.mm_out(a[r0:r1], b, out=c[r0:r1])
                if self.world > 1 and not self.skip_gather:
                    # column-parallel: gather the shards on the side stream; the next operators
                    # of the step overlap with the transfer, the step ends when all gathers have landed
                    self.comm_stream.wait_stream(cur)
                    with torch.cuda.stream(self.comm_stream):
                        if bi == 0:
                            ev[0].record()
                        if self.gather == "nccl":
                            torch.distributed.all_gather_into_tensor(gathered, c)
                        else:
                            gathered.push(c, rows=(r0, r1))
                        if bi == len(bounds) - 1:
                            ev[1].record()
        return run

    def run(self, events=None, before=None, after=None):
        """One step.  `before(i)` / `after(i)` run around operator i on the host (the
        end-to-end form uses them to order the PCIe copies of that operator)."""
        for i, (_, fn, _, _) in enumerate(self.ops):
            if before is not None:
                before(i)
            if events is not None:
                events[i][0].record()
            fn()
            if events is not None:
                events[i][1].record()
            if after is not None:
                after(i)
        if self.comm_stream is not None and not self.skip_gather:
            if self.gather != "nccl":
                with torch.cuda.stream(self.comm_stream):
                    next(iter(self.gemm.values()))[4].finish()  # one tiny all-reduce closes all pushes
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)

    # ---------------- end-to-end form: host buffers in, host buffers out
    def make_e2e(self):
        """Pinned host copies of the per-step activations and host buffers for the results.
        Weights, cos/sin tables and the paged KV cache are resident state (they are not
        inputs of a step in serving); everything a step consumes or produces crosses PCIe.
        Each operator gets the list of tensors it consumes and produces, so that its uploads
        can run on one copy engine and its downloads on the other while other operators
        compute."""
        dd, p = self.dec, self.pre
        io = {
            "fused_add_rms_norm": ([self.x, self.res], [self.x, self.res]),
            "rotary_embedding": ([self.q, self.k, self.pos], [self.q, self.k]),
            "silu_and_mul": ([self.act], [self.silu_out]),
            "flash_attn_varlen_func[prefill]": ([p.q], [self.pre_out]),
            "reshape_and_cache_flash": ([dd.new_key, dd.new_value, dd.slot_mapping], []),
            "flash_attn_varlen_func[decode]": ([dd.q], [self.dec_out]),
        }
        for n in self.gemm:
            a, _, _, c, _ = self.gemm[n]
            io[("addmm" if n in ("qkv", "gate_up") else "mm") + f"[{n}]"] = ([a], [c])
        pin = lambda t, fill: (torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) if fill
                               else torch.empty(t.shape, dtype=t.dtype, pin_memory=True))
        self.e2e_plan = []
        h2d = d2h = 0
        for name, _, _, _ in self.ops:
            ins, outs = io[name]
            self.e2e_plan.append(([(pin(t, True), t) for t in ins], [(pin(t, False), t) for t in outs]))
            h2d += sum(t.numel() * t.element_size() for t in ins)
            d2h += sum(t.numel() * t.element_size() for t in outs)
        self.h2d_stream = torch.cuda.Stream(device=self.device)
        self.d2h_stream = torch.cuda.Stream(device=self.device)
        self.e2e_in_ev = [torch.cuda.Event() for _ in self.ops]
        self.e2e_out_ev = [torch.cuda.Event() for _ in self.ops]
        return h2d, d2h

    def run_e2e(self):
        """Host buffers -> step -> host buffers.  Uploads are queued operator by operator on
        one stream, downloads on another, the operators on the current stream: operator i
        starts when its inputs have landed and its results leave while later operators run."""
        cur = torch.cuda.current_stream(self.device)
        self.h2d_stream.wait_stream(cur)   # the previous step has consumed / downloaded its buffers
        self.d2h_stream.wait_stream(cur)
        with torch.cuda.stream(self.h2d_stream):
            for i, (ins, _) in enumerate(self.e2e_plan):
                for h, d in ins:
                    d.copy_(h, non_blocking=True)
                self.e2e_in_ev[i].record(self.h2d_stream)

        def before(i):
            cur.wait_event(self.e2e_in_ev[i])

        def after(i):
            outs = self.e2e_plan[i][1]
            if not outs:
                return
            self.e2e_out_ev[i].record(cur)
            with torch.cuda.stream(self.d2h_stream):
                self.d2h_stream.wait_event(self.e2e_out_ev[i])
                for h, d in outs:
                    h.copy_(d, non_blocking=True)

        self.run(before=before, after=after)
        cur.wait_stream(self.d2h_stream)
        cur.wait_stream(self.h2d_stream)


# dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch under ncu
# (profiles/gemm_tcgen05_kernel_gate_up_m2048.md, section "Full-size launch"): 762,320,128 + 444,165,376
NCU_DRAM_BYTES_PER_LAUNCH = {"addmm[gate_up]": 1206485504}


# --------------------------------------------------------------------------- operators beyond the step
def extra_op_times(device, peaks, reps=10):
    """Operators of the next scope rows, timed on their own (not part of `value`):
    aten::_flash_attention_forward on a dense causal GQA batch (8 x 4096 tokens, 32/8 heads,
    d=128, bf16) in the packed layout and as the transposed views SDPA passes."""
    import flaggems_b200 as fg

    g = torch.Generator(device="cpu").manual_seed(77)
    B, S, H, Hk, D = 8, 4096, 32, 8, 128
    mk = lambda h: torch.randn((B, S, h, D), generator=g, dtype=torch.float32).to(device=device, dtype=torch.bfloat16)
    q, k, v = mk(H), mk(Hk), mk(Hk)
    flops = 4 * B * H * D * S * (S + 1) // 2
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    out = []
    for label, args in (("packed (batch, seq, heads, dim)", (q, k, v)),
                        ("transposed views of (batch, heads, seq, dim)",
                         tuple(x.transpose(1, 2).contiguous().transpose(1, 2) for x in (q, k, v)))):
        fn = lambda: fg.flash_attention_forward(*args, None, None, S, S, 0.0, True, False)
        for _ in range(3):
            fn()
        times = []
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        out.append({"op": f"_flash_attention_forward dense causal B{B} S{S} H{H}/{Hk} d{D}, {label}", "ms": round(ms, 4),
                    "bound": "tensor", "achieved": round(flops / ms / 1e9, 1), "unit": "TFLOP/s",
                    "peak": peaks["bf16_tflops"], "frac": round(flops / ms / 1e9 / peaks["bf16_tflops"], 3)})
    # bmm: 32 problems of 1024 x 1024 x 1024, bf16 (one launch)
    a3 = torch.randn((32, 1024, 1024), generator=g, dtype=torch.float32).to(device=device, dtype=torch.bfloat16)
    b3 = torch.randn((32, 1024, 1024), generator=g, dtype=torch.float32).to(device=device, dtype=torch.bfloat16)
    fn = lambda: fg.bmm(a3, b3)
    for _ in range(3):
        fn()
    times = []
    for _ in range(reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    fl = 2 * 32 * 1024 ** 3
    out.append({"op": "bmm 32 x [1024, 1024] x [1024, 1024] bf16 (incl. output allocation)", "ms": round(ms, 4),
                "bound": "tensor", "achieved": round(fl / ms / 1e9, 1), "unit": "TFLOP/s",
                "peak": peaks["bf16_tflops"], "frac": round(fl / ms / 1e9 / peaks["bf16_tflops"], 3)})
    # gelu_and_mul on the silu_and_mul benchmark shape: halves of [4096, 22016], bf16
    x = torch.randn((4096, 22016), generator=g, dtype=torch.float32).to(device=device, dtype=torch.bfloat16)
    half = x.shape[1] // 2
    nbytes = x.numel() * 2 + x.shape[0] * half * 2
    for approximate in ("none", "tanh"):
        fn = lambda: fg.gelu_and_mul(x[:, :half], x[:, half:], approximate)
        with torch.no_grad():
            for _ in range(3):
                fn()
            times = []
            for _ in range(reps):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        out.append({"op": f"gelu_and_mul[{approximate}] halves of [4096, 22016] (incl. output allocation)",
                    "ms": round(ms, 4), "bound": "hbm", "achieved": round(nbytes / ms / 1e6, 1), "unit": "GB/s",
                    "peak": peaks["hbm_gbs"], "frac": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 3)})
    return out


# --------------------------------------------------------------------------- reference GPU path
def triton_reference_times(step, reps=5):
    """Per-operator times of the unmodified reference (its Triton kernels, installed under
    baseline/_ref) on the same device buffers; informational, only with --triton-ref.
    Returns a list of {"op", "ms"} or a one-line reason why it could not run."""
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "flag_gems")):
        return "reference install baseline/_ref is not present"
    sys.path.insert(0, ref_dir)
    try:
        import flag_gems as ref
    except Exception as e:  # noqa: BLE001
        return f"reference does not import: {type(e).__name__}: {e}"
    finally:
        sys.path.remove(ref_dir)
    import importlib

    # (the packages re-export functions under the names of their modules, so fetch the modules by path)
    silu_out = importlib.import_module("flag_gems.fused.silu_and_mul").silu_and_mul_out
    mm_out = importlib.import_module("flag_gems.ops.mm").mm_out
    addmm_out = importlib.import_module("flag_gems.ops.addmm").addmm_out
    p, dd = step.pre, step.dec
    H = step.x.shape[1]
    a1, a2 = step.act[:, :step.half], step.act[:, step.half:]
    calls = {
        "fused_add_rms_norm": lambda: ref.fused_add_rms_norm(step.x, step.res, [H], step.w, step.eps),
        "rotary_embedding": lambda: ref.apply_rotary_pos_emb(step.q, step.k, step.cos, step.sin, step.pos, False, True),
        "silu_and_mul": lambda: silu_out(a1, a2, step.silu_out),
        "flash_attn_varlen_func[prefill]": lambda: ref.flash_attn_varlen_func(
            p.q, p.key_cache, p.value_cache, p.max_seqlen_q, p.cu_seqlens_q, p.max_seqlen_k, seqused_k=p.seqused_k,
            causal=True, block_table=p.block_table, out=step.pre_out),
        "reshape_and_cache_flash": lambda: ref.reshape_and_cache_flash(
            dd.new_key, dd.new_value, dd.key_cache, dd.value_cache, dd.slot_mapping, "auto", None, None),
        "flash_attn_varlen_func[decode]": lambda: ref.flash_attn_varlen_func(
            dd.q, dd.key_cache, dd.value_cache, 1, dd.cu_seqlens_q, dd.max_seqlen_k, seqused_k=dd.seqused_k,
            causal=True, block_table=dd.block_table, out=step.dec_out),
    }
    for n in step.gemm:
        a, b, bias, c, _ = step.gemm[n]
        if n in ("qkv", "gate_up"):
            calls[f"addmm[{n}]"] = (lambda a=a, b=b, bias=bias, c=c: addmm_out(bias, a, b, out=c))
        else:
            calls[f"mm[{n}]"] = (lambda a=a, b=b, c=c: mm_out(a, b, out=c))
    # The reference's launcher (utils/libentry.py:883-903) passes the argument list of Triton
    # 3.3-3.5 when it re-launches a kernel from its own cache; with the Triton 3.6 of this image
    # every second call of an operator fails with "function takes exactly N arguments".  The
    # first call of a process (Triton's own JIT path) works, so its caches are emptied before
    # each call -- run-time state only, the installed package is untouched.  That path has
    # more host overhead; a short device-side sleep in front of the timed call lets the host
    # run ahead, so the events bracket the reference's kernels and not its Python.
    import gc

    lib_entry_cls = importlib.import_module("flag_gems.utils.libentry").LibEntry

    def forget():
        for obj in gc.get_objects():
            if isinstance(obj, lib_entry_cls):
                for dev_cache in obj.kernel_cache:
                    dev_cache.clear()

    flush = torch.empty(512 << 20, dtype=torch.uint8, device=step.device)
    out = []
    for name, _, _, _ in step.ops:
        fn = calls.get(name)
        if fn is None:
            continue
        try:
            for _ in range(2):   # includes the JIT build and the reference's autotuning
                forget()
                fn()
            torch.cuda.synchronize()
            times = []
            for _ in range(reps):
                forget()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                flush.zero_()                  # 512 MB written: the operator's operands leave the 126 MB L2
                torch.cuda._sleep(4_000_000)   # ~2 ms of device time for the host to get ahead
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            out.append({"op": name, "ms": round(statistics.median(times), 4)})
        except Exception as e:  # noqa: BLE001
            out.append({"op": name, "error": f"{type(e).__name__}: {str(e)[:120]}"})
    return out


# --------------------------------------------------------------------------- CPU arm
def cpu_step_sample(seed=0):
    """Time the CPU oracle on a bounded sample of one step; returns (scaled seconds for a
    full step, number of ops, description).  Each operator is timed on a slice and scaled
    by its algorithmic work."""
    from flaggems_b200 import workloads as W
    from oracle import reference_oracle as O  # CPU baseline leg

    total = 0.0
    detail = {}

    def timed(fn):
        t0 = time.perf_counter()
        fn()
        return time.perf_counter() - t0

    x, r, w, eps = W.norm_inputs(seed=seed + 1, T=4096, device="cpu")
    t = timed(lambda: O.fused_add_rms_norm(x, r, w, eps, upcast=torch.float32))
    detail["fused_add_rms_norm"] = t
    q, k, cos, sin, pos = W.rope_inputs(seed=seed + 2, T=4096, device="cpu")
    cos4, sin4 = W.rope_tables(4096, 128, torch.bfloat16, "cpu")
    t = timed(lambda: O.apply_rotary_pos_emb(q, k, cos4, sin4, pos))
    detail["rotary_embedding"] = t
    act = W.silu_inputs(seed=seed + 3, T=2048, device="cpu")
    h = act.shape[1] // 2
    t = timed(lambda: O.silu_and_mul(act[:, :h], act[:, h:], upcast=torch.float32)) * 2
    detail["silu_and_mul"] = t
    # prefill: one 1024-token sequence, scaled by FLOPs to the 16-sequence batch
    g = torch.Generator().manual_seed(seed + 4)
    lens = torch.randint(128, 4097, (16,), generator=g).tolist()
    pb = W.prefill_batch(seed=seed + 4, num_seqs=1, min_len=1024, max_len=1024, device="cpu")
    t1 = timed(lambda: O.paged_attention(pb.q, pb.key_cache, pb.value_cache, pb.query_lens, pb.kv_lens, pb.block_table,
                                         pb.scale, compute_dtype=torch.float32))
    detail["flash_attn_varlen_func[prefill]"] = t1 * W.prefill_flops(lens) / W.prefill_flops([1024])
    # decode: 16 sequences with 2048-token contexts, scaled by context tokens
    db = W.decode_batch(seed=seed + 5, batch=16, min_ctx=2048, max_ctx=2048, device="cpu")
    g = torch.Generator().manual_seed(seed + 5)
    ctx = torch.randint(512, 8193, (256,), generator=g).tolist()
    kc, vc = db.key_cache.clone(), db.value_cache.clone()
    t0 = timed(lambda: O.reshape_and_cache_flash(db.new_key, db.new_value, kc, vc, db.slot_mapping))
    detail["reshape_and_cache_flash"] = t0 * 256 / 16
    t1 = timed(lambda: O.paged_attention(db.q, db.key_cache, db.value_cache, db.query_lens, db.kv_lens,
                                         db.block_table, db.scale, compute_dtype=torch.float32))
    detail["flash_attn_varlen_func[decode]"] = t1 * sum(ctx) / (16 * 2048)
    # projections: 512 of the 8192 rows
    for i, name in enumerate(W.GEMM_SHAPES):
        a, b, bias = W.gemm_inputs(name, seed=seed + 10 + i, M=512, device="cpu")
        # operands upcast beforehand, as the reference's harness does before it calls torch on the CPU
        # (the weight's conversion does not grow with the rows and must not be scaled with them)
        a, b, bias = a.float(), b.float(), bias.float()
        if name in ("qkv", "gate_up"):
            t = timed(lambda: O.addmm(bias, a, b, upcast=torch.float32))
        else:
            t = timed(lambda: O.mm(a, b, upcast=torch.float32))
        detail[f"gemm[{name}]"] = t * 16
    total = sum(detail.values())
    sample = ("per operator: norm/rope all 4096 tokens, silu_and_mul 2048 of 4096 rows, prefill one 1024-token "
              "sequence (scaled by FLOPs), decode 16 sequences x 2048 context (scaled by context tokens), GEMMs 512 "
              "of 8192 rows; fp32 torch CPU")
    return total, len(detail), sample, detail


def run_reference_arm(args, rank):
    if rank != 0:
        return
    cores = torch.get_num_threads()
    for _ in range(max(1, min(args.warmup, 1))):   # one untimed pass: page faults, thread pool start-up
        cpu_step_sample()
    times = []
    n_ops = 10
    sample = ""
    for _ in range(args.steps):
        t, n_ops, sample, _ = cpu_step_sample()
        times.append(t)
    step_s = statistics.mean(times)
    val = n_ops / step_s
    out = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out))


def workload_config(n_gpus, n_ops=10, small=False, only=""):
    cfg = _workload_config(n_gpus)
    cfg["ops_per_step"] = n_ops
    if small or only:
        cfg["workload"] = f"PROFILING SUBSET (small={small}, only={only!r}) of: " + cfg["workload"]
    return cfg


def _workload_config(n_gpus):
    return {
        "workload": "operator-path step at configs 2-5: T=4096 hidden=4096 elementwise block; 16-seq varlen causal "
                    "GQA prefill (32/8 heads, d=128, len 128..4096); batch-256 paged decode (ctx 512..8192, block 16)"
                    " with cache write; mm/addmm M=8192 at qkv/o/gate_up/down",
        "ops_per_step": 10,
        "parallelism": "single GPU" if n_gpus == 1 else
                       f"{n_gpus} ranks: sequences sharded with no exchange; projections column-parallel, shards "
                       "all-gathered over NVLink beside the compute (copy-engine pushes + one NCCL all-reduce per step, "
                       "or ncclAllGather with --gather nccl)",
        "l2": "no explicit flush: the step cycles through ~8 GB of operands, every operator's inputs are evicted "
              "from the 126 MB L2 between its consecutive invocations",
    }


# --------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer (PCIe) leg")
    ap.add_argument("--only", default="", help="run only the operators whose name contains this string")
    ap.add_argument("--extra", action="store_true",
                    help="N=1: also time the operators built beyond the benchmark step (dense _flash_attention_forward, "
                         "gelu_and_mul, bmm)")
    ap.add_argument("--triton-ref", action="store_true",
                    help="N=1: also time the unmodified reference's Triton kernels (baseline/_ref) per operator; "
                         "adds the reference's JIT and autotuning time to the run")
    ap.add_argument("--gather", default="p2p", choices=["p2p", "nccl"],
                    help="N > 1: how the projection shards are gathered (copy-engine pushes into peer-mapped "
                         "buffers closed by one NCCL all-reduce, or ncclAllGather)")
    ap.add_argument("--row-blocks", type=int, default=1,
                    help="N > 1 with --gather p2p: row blocks a projection is computed and pushed in")
    ap.add_argument("--op-order", default="spread", choices=["spread", "grouped"],
                    help="order of the operators inside a step: 'spread' puts the short memory-bound operators "
                         "behind the ones that leave little dirty data in L2, 'grouped' runs them by family")
    ap.add_argument("--small", action="store_true",
                    help="reduced attention / GEMM sizes (for profiler captures); not a benchmark configuration")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3  # timing rule: at least three warm-up steps

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    saved_stdout = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        if args.gather == "nccl":
            # NCCL's all-gather kernels run beside the compute kernels: cap their CTAs and keep
            # the persistent GEMM off the SMs they occupy
            os.environ.setdefault("NCCL_MAX_CTAS", str(NCCL_CTAS))
        # NCCL writes its banner to stdout; the contract is ONE JSON line there, so stdout is
        # pointed at stderr until the result is printed
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        torch.distributed.init_process_group("nccl", device_id=device)

    from flaggems_b200 import _lib

    peaks, peak_kind = load_peaks()
    if world > 1 and args.gather == "nccl":
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        _lib.set_num_sms(sms - NCCL_CTAS)
    step = Step(device, rank, world, small=args.small, only=args.only, gather=args.gather, row_blocks=args.row_blocks,
                op_order=args.op_order)
    n_ops = len(step.ops)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step.run()
    barrier()

    events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_ops)]
              for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    launches0 = _lib.launch_count()
    barrier()
    t0 = time.time()
    e0.record()
    for s in range(args.steps):
        step.run(events[s])
    e1.record()
    barrier()
    t1 = time.time()
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop(t0, t1)
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * n_ops / (ms_step * 1e-3)

    per_op = []
    for i, (name, _, work, kind) in enumerate(step.ops):
        ms = statistics.mean(events[s][i][0].elapsed_time(events[s][i][1]) for s in range(args.steps))
        if kind == "hbm":
            ach, peak, unit = work / ms / 1e6, peaks["hbm_gbs"], "GB/s"
        else:
            # every operator is timed on its own (a 0.2-1.4 ms kernel): the burst cuBLAS figure is the
            # denominator; the sustained one (power cap) is carried along in the roofline object
            ach, peak, unit = work / ms / 1e9, peaks["bf16_tflops"], "TFLOP/s"
        per_op.append({"op": name, "ms": round(ms, 4), "bound": kind, "achieved": round(ach, 1), "unit": unit,
                       "peak": peak, "frac": round(ach / peak, 3)})
    dom = max(per_op, key=lambda o: o["ms"])
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel
    # from one ncu capture of the same launch; the captures are summarised under profiles/.
    # Only full-size launches of the default workload have a figure.
    traffic = None if args.small else NCU_DRAM_BYTES_PER_LAUNCH.get(dom["op"])
    roofline = {"bound": dom["bound"], "kernel": dom["op"], "achieved": dom["achieved"], "peak": dom["peak"],
                "unit": dom["unit"], "frac": dom["frac"], "peak_source": peak_kind,
                "traffic": traffic}
    if dom["bound"] == "tensor":
        roofline["peak_kind"] = "burst (kernel timed alone)"
        roofline["peak_sustained"] = peaks["bf16_tflops_sustained"]

    # ---- end to end: pinned host buffers in and out, copies inside the timed region
    h2d = d2h = 0
    ms_e2e = float("nan")
    e2e_val = None
    if not args.no_e2e:
        h2d, d2h = step.make_e2e()
        for _ in range(2):
            step.run_e2e()
        barrier()
        e0.record()
        for _ in range(args.steps):
            step.run_e2e()
        e1.record()
        barrier()
        ms_e2e = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms_e2e], device=device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms_e2e = float(t.item())
        e2e_val = world * n_ops / (ms_e2e / args.steps * 1e-3)
    status = _lib.device_status(reset=True)

    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": dict(workload_config(world, n_ops, args.small, args.only),
                                            op_order=[o[0] for o in step.ops]), "roofline": roofline,
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches), "clocks": clocks, "per_op": per_op, "device_status": status,
    }
    if rank == 0 and world == 1 and args.extra:
        out["extra_ops"] = extra_op_times(device, peaks)
    if rank == 0 and world == 1 and args.triton_ref:
        out["triton_ref"] = triton_reference_times(step)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_step_sample()   # untimed: first-touch page faults and the thread pool's start-up
        t, n, sample, detail = cpu_step_sample()
        out["cpu_baseline"] = {"value": n / t, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                               "sample": sample + "; second of two passes", "step_seconds_scaled": t}
    if world > 1:
        # the same K steps without the all-gathers: what the sharded operators alone scale like
        step.skip_gather = True
        for _ in range(2):
            step.run()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        g0.record()
        for _ in range(args.steps):
            step.run()
        g1.record()
        barrier()
        step.skip_gather = False
        ms_ng = g0.elapsed_time(g1)
        t = torch.tensor([ms_ng], device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_ng = float(t.item())
        out["no_gather"] = {"value": world * n_ops / (ms_ng / args.steps * 1e-3), "unit": UNIT,
                            "ms_per_step": ms_ng / args.steps,
                            "note": "same step with the projection outputs left sharded (no NVLink traffic)"}
        gathers = []
        for name, (g0, g1) in step.comm_events.items():
            ms = g0.elapsed_time(g1)
            g = step.gemm[name][4]
            nbytes = (g.buf.numel() if hasattr(g, "buf") else g.numel()) * 2
            gathers.append({"op": f"all_gather[{name}]", "ms": round(ms, 4), "bytes": nbytes,
                            "busbw_GBs": round(nbytes * (world - 1) / world / ms / 1e6, 1)})
        out["all_gather"] = gathers
    if saved_stdout is not None:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        os.dup2(2, 1)  # anything NCCL prints while shutting down goes to stderr
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
