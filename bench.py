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
own column shard and the shards are gathered over NVLink into the row-major result on
every rank (weak scaling: fixed work per GPU; the gathers of one step overlap the next
step's operators).  The same run also times the ``tp`` leg -- the single-GPU step itself
partitioned over the ranks (attention, rope and the cache write by KV head, norm and
silu_and_mul by token rows, the projections by N/G columns + gather; fixed total work) --
and checks every sharded result against the unsharded one (``shard_check``).

At N = 1 the line also carries ``triton_ref`` (the unmodified reference's Triton kernels
timed on the same buffers in the same run), ``extra_ops`` (operator forms beyond the step)
and ``cpu_baseline``.

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
    """The operators of one step with their inputs resident on ``device``.

    ``mode`` "weak": every rank owns a full-size step (its own sequences and tokens; the
    projections multiply the replicated A by this rank's own full-size column shard of a weight
    that is ``world`` times wider, and the shards are gathered into the row-major result on every
    rank).  ``mode`` "tp": the single-GPU step itself partitioned over the ranks -- the same
    seeded batch on every rank; attention, the cache write and rope by KV head, norm and
    silu_and_mul by token rows, the projections by N/world columns plus the gather.
    Only the operators that ``only`` selects get buffers."""

    def __init__(self, device, rank: int, world: int, seed: int = 0, small: bool = False, only: str = "",
                 gather: str = "p2p", op_order: str = "spread", mode: str = "weak", pipeline: bool = True,
                 push_streams: int = 1):
        import flaggems_b200 as fg
        from flaggems_b200 import dist as fdist
        from flaggems_b200 import workloads as W

        self.gather = gather
        self.op_order = op_order
        self.mode = mode
        self.skip_gather = False   # N > 1: second timing of the step without the gathers
        # N > 1: the gathers of step s may still be in flight while step s + 1 computes (two
        # result matrices per projection); a step then waits for the gathers of the step before it
        self.can_pipeline = world > 1 and gather != "nccl"    # two result buffers per projection exist
        self.pipeline = bool(pipeline) and self.can_pipeline
        self.step_no = 0
        self.fg, self.W, self.fdist = fg, W, fdist
        self.device, self.rank, self.world = device, rank, world
        self.only = only
        tp = mode == "tp" and world > 1
        self.tp = tp
        s = seed if tp else seed + 1000 * rank  # weak: every rank owns a different batch of sequences
        want = lambda name: (not only) or (only in name)
        self.names = {
            "norm": "fused_add_rms_norm", "rope": "rotary_embedding", "silu": "silu_and_mul",
            "prefill": "flash_attn_varlen_func[prefill]", "cache": "reshape_and_cache_flash",
            "decode": "flash_attn_varlen_func[decode]",
        }
        hq_all, hk_all = 32, 8
        qs, ks = (fdist.kv_head_shard(hq_all, hk_all, rank, world) if tp else (slice(None), slice(None)))
        self.qs, self.ks = qs, ks
        rows = lambda T: fdist.shard_range(T, rank, world) if tp else (0, T)
        if want(self.names["norm"]):
            x, res, self.w, self.eps = W.norm_inputs(seed=s + 1, device=device)
            r0, r1 = rows(x.shape[0])
            self.x, self.res = x[r0:r1], res[r0:r1]
        if want(self.names["rope"]):
            q, k, self.cos, self.sin, self.pos = W.rope_inputs(seed=s + 2, device=device)
            self.q, self.k = q[:, qs], k[:, ks]
        if want(self.names["silu"]):
            act = W.silu_inputs(seed=s + 3, device=device)
            r0, r1 = rows(act.shape[0])
            self.act = act[r0:r1]
            self.half = self.act.shape[1] // 2
            self.silu_out = torch.empty((self.act.shape[0], self.half), dtype=self.act.dtype, device=device)
        # --small: reduced attention/GEMM sizes for profiler captures (operands still exceed L2)
        pre_kw = dict(num_seqs=8, min_len=1024, max_len=3072) if small else {}
        dec_kw = dict(batch=64, min_ctx=1024, max_ctx=4096) if small else {}
        if want(self.names["prefill"]):
            self.pre = W.prefill_batch(seed=s + 4, device=device, **pre_kw)
            self.pre_out = torch.empty_like(self.pre.q)
        if want(self.names["cache"]) or want(self.names["decode"]):
            self.dec = W.decode_batch(seed=s + 5, device=device, **dec_kw)
            self.dec_out = torch.empty_like(self.dec.q)
        # projections: A replicated (same seed on every rank), B/bias = this rank's column shard
        self.gemm = {}
        Mg = 2048 if small else 8192
        for i, name in enumerate(W.GEMM_SHAPES):
            op_name = ("addmm" if name in ("qkv", "gate_up") else "mm") + f"[{name}]"
            if not want(op_name):
                continue
            a, b, bias = W.gemm_inputs(name, seed=seed + 10 + i, device=device, M=Mg)
            if tp:      # this rank's N / world columns of the one weight
                b, bias = fdist.column_shard(b, bias, rank, world)
            elif world > 1:  # the full-size shard of a [K, N * world] weight owned by this rank
                _, b, bias = W.gemm_inputs(name, seed=seed + 10 + i + 100 * (rank + 1), device=device, M=Mg)
            gathered = None
            if world > 1 and gather == "p2p-slots":
                # contiguous slot per rank, [world, M, n]: one-dimensional copies, no row-major result
                gathered = fdist.PeerGatherSlots((a.shape[0], b.shape[1]), a.dtype, device,
                                                 buffers=2 if self.can_pipeline else 1)
                c = [gathered.local_slot(i) for i in range(len(gathered.bufs))]
            elif world > 1 and gather != "nccl":
                # the GEMM writes its shard straight into its columns of the row-major result
                gathered = fdist.PeerGather((a.shape[0], b.shape[1]), a.dtype, device,
                                            buffers=2 if self.can_pipeline else 1, push_streams=push_streams)
                c = [gathered.local_slot(i) for i in range(len(gathered.bufs))]
            else:
                c = [torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device=device)]
                if world > 1:
                    gathered = torch.empty((a.shape[0], world * b.shape[1]), dtype=a.dtype, device=device)
            self.gemm[name] = (a, b, bias, c, gathered)
        self.comm_stream = torch.cuda.Stream(device=device) if world > 1 else None
        self.comm_events = {}  # name -> (start, end) events of the last gather of that projection
        self.gather_done = [None, None]   # per result matrix: event behind the finish() of its last round
        self.ops = self._build_ops()

    # each entry: (name, callable, work, kind) with kind "hbm" (bytes) or "tensor" (flops)
    def _build_ops(self):
        fg, W = self.fg, self.W
        share = self.world if self.tp else 1     # tp: a rank does 1/world of every operator's work
        ops = []
        # The projections come first: with N > 1 their output shards are gathered on a side
        # stream while the rest of the step runs.  There a small projection leads so that NVLink is
        # already busy while the largest one (gate_up) computes; gate_up follows at once because
        # its gather is the longest transfer of the step.  (On one GPU the projections are tensor-bound and their
        # order among themselves is immaterial.)
        for name in (("qkv", "gate_up", "down", "o") if self.world > 1 else ("gate_up", "qkv", "down", "o")):
            if name not in self.gemm:
                continue
            a, b, bias, c, gathered = self.gemm[name]
            M, K = a.shape
            N = b.shape[1]
            if name in ("qkv", "gate_up"):  # qkv and gate_up carry a bias in the benchmark (addmm), o/down are mm
                ops.append((f"addmm[{name}]", self._gemm_call(name, True), M * N * (2 * K + 1), "tensor"))
            else:
                ops.append((f"mm[{name}]", self._gemm_call(name, False), 2 * M * N * K, "tensor"))
        rest = {}
        nm = self.names
        if hasattr(self, "x"):
            T, H = self.x.shape
            rest["norm"] = ((nm["norm"], lambda: fg.fused_add_rms_norm(self.x, self.res, [H], self.w, self.eps),
                             4 * T * H * 2 + H * 2, "hbm"))
        if hasattr(self, "q"):
            tq, hq, d = self.q.shape
            hk = self.k.shape[1]
            rest["rope"] = ((nm["rope"],
                             lambda: fg.apply_rotary_pos_emb(self.q, self.k, self.cos, self.sin, self.pos, False, True),
                             2 * (tq * hq * d + tq * hk * d) * 2 + tq * 2 * (d // 2) * 2 + tq * 8, "hbm"))
        if hasattr(self, "act"):
            a1, a2 = self.act[:, :self.half], self.act[:, self.half:]
            rest["silu"] = ((nm["silu"], lambda: fg.silu_and_mul_out(a1, a2, self.silu_out),
                             self.act.numel() * 2 + self.silu_out.numel() * 2, "hbm"))
        qs, ks = self.qs, self.ks
        if hasattr(self, "pre"):
            p = self.pre
            pq, pk, pv, po = p.q[:, qs], p.key_cache[:, :, ks], p.value_cache[:, :, ks], self.pre_out[:, qs]
            rest["prefill"] = ((nm["prefill"],
                                lambda: fg.flash_attn_varlen_func(pq, pk, pv, p.max_seqlen_q, p.cu_seqlens_q,
                                                                  p.max_seqlen_k, seqused_k=p.seqused_k, causal=True,
                                                                  block_table=p.block_table, out=po),
                                W.prefill_flops(p.query_lens) / share, "tensor"))
        if hasattr(self, "dec"):
            dd = self.dec
            nk_, nv_ = dd.new_key[:, ks], dd.new_value[:, ks]
            dk, dv = dd.key_cache[:, :, ks], dd.value_cache[:, :, ks]
            dq, do = dd.q[:, qs], self.dec_out[:, qs]
            nk = nk_.numel() * 2
            if not self.only or self.only in nm["cache"]:
                rest["cache"] = ((nm["cache"],
                                  lambda: fg.reshape_and_cache_flash(nk_, nv_, dk, dv, dd.slot_mapping, "auto", None, None),
                                  4 * nk + dd.slot_mapping.numel() * 8, "hbm"))
            if not self.only or self.only in nm["decode"]:
                rest["decode"] = ((nm["decode"],
                                   lambda: fg.flash_attn_varlen_func(dq, dk, dv, 1, dd.cu_seqlens_q, dd.max_seqlen_k,
                                                                     seqused_k=dd.seqused_k, causal=True,
                                                                     block_table=dd.block_table, out=do),
                                   W.decode_bytes(dd.kv_lens, len(dd.kv_lens), q_heads=dq.shape[1], kv_heads=dk.shape[2]),
                                   "hbm"))
        # Order of the remaining operators.  The calls are independent (own buffers), so any order computes
        # the same; what the order changes is whose time the write-back of an operator's output is counted
        # in: up to 126 MB of dirty L2 lines leave for DRAM while the NEXT operator runs.  A tensor-bound
        # operator absorbs that, a 20 us streaming kernel doubles its DRAM traffic.  The short memory-bound
        # operators therefore follow the operators that leave the L2 cleanest (--op-order grouped restores the
        # order by operator family that earlier lines of this benchmark used).
        order = (["prefill", "norm", "cache", "decode", "rope", "silu"] if self.op_order == "spread" else
                 ["norm", "rope", "silu", "prefill", "cache", "decode"])
        ops += [rest[k] for k in order if k in rest]
        if not ops:
            raise SystemExit(f"--only {self.only!r} matches no operator")
        return ops

    def _gemm_call(self, name, with_bias):
        fg = self.fg
        a, b, bias, c, gathered = self.gemm[name]

        def run():
            cur = torch.cuda.current_stream(self.device)
            buf = (self.step_no & 1) if self.pipeline else 0
            out = c[buf]
            if with_bias:
                fg.addmm_out(bias, a, b, out=out)
            else:
                fg.mm_out(a, b, out=out)
            if self.world > 1 and not self.skip_gather:
                ev = self.comm_events.setdefault(
                    name, (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
                # column-parallel: gather the shards on the side stream; the next operators
                # overlap with the transfer
                self.comm_stream.wait_stream(cur)
                with torch.cuda.stream(self.comm_stream):
                    ev[0].record()
                    if self.gather == "nccl":
                        self.fdist.all_gather_columns(out, self.world, out=gathered)
                    else:
                        gathered.push(out, b=buf)
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
        if self.comm_stream is not None and not self.skip_gather and self.gemm:
            cur = torch.cuda.current_stream(self.device)
            buf = (self.step_no & 1) if self.pipeline else 0
            with torch.cuda.stream(self.comm_stream):
                if self.gather != "nccl":
                    next(iter(self.gemm.values()))[4].finish()  # one tiny all-reduce closes all pushes of the step
                done = torch.cuda.Event()
                done.record()
                self.gather_done[buf] = done
            if self.pipeline:
                # this step's gathers go on beside the next step; before the step after that writes
                # into the same result matrices again, the gathers of the step BEFORE this one must be
                # over on every rank, which its closing all-reduce has established
                prev = self.gather_done[buf ^ 1]
                if prev is not None:
                    cur.wait_event(prev)
            else:
                cur.wait_stream(self.comm_stream)
        self.step_no += 1

    def drain(self):
        """Wait (on the current stream) for every gather still in flight."""
        if self.comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)

    def gathered_result(self, name):
        """The row-major [M, world * n] result of projection `name` of the last step run."""
        g = self.gemm[name][4]
        if g is None:
            return self.gemm[name][3][0]
        if hasattr(g, "bufs"):
            return g.bufs[((self.step_no - 1) & 1) if self.pipeline else 0]
        return g

    # ---------------- end-to-end form: host buffers in, host buffers out
    def make_e2e(self):
        """Pinned host copies of the per-step activations and host buffers for the results.
        Weights, cos/sin tables and the paged KV cache are resident state (they are not
        inputs of a step in serving); everything a step consumes or produces crosses PCIe.
        Each operator gets the list of tensors it consumes and produces, so that its uploads
        can run on one copy engine and its downloads on the other while other operators
        compute."""
        io = {}
        if hasattr(self, "x"):
            io[self.names["norm"]] = ([self.x, self.res], [self.x, self.res])
        if hasattr(self, "q"):
            io[self.names["rope"]] = ([self.q, self.k, self.pos], [self.q, self.k])
        if hasattr(self, "act"):
            io[self.names["silu"]] = ([self.act], [self.silu_out])
        if hasattr(self, "pre"):
            io[self.names["prefill"]] = ([self.pre.q], [self.pre_out])
        if hasattr(self, "dec"):
            dd = self.dec
            io[self.names["cache"]] = ([dd.new_key, dd.new_value, dd.slot_mapping], [])
            io[self.names["decode"]] = ([dd.q], [self.dec_out])
        for n in self.gemm:
            a, _, _, c, _ = self.gemm[n]
            io[("addmm" if n in ("qkv", "gate_up") else "mm") + f"[{n}]"] = ([a], [c[0]])
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


def ncu_dram_bytes_per_launch():
    """DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one full-size launch of an
    operator's kernel, from ncu captures of `bench.py --only <operator>`; the figures and the
    commands that made them are kept in profiles/dram_traffic.json."""
    p = ROOT / "profiles" / "dram_traffic.json"
    try:
        return {k: int(v["dram_bytes_per_launch"]) for k, v in json.loads(p.read_text()).items()
                if isinstance(v, dict) and "dram_bytes_per_launch" in v}
    except Exception:  # noqa: BLE001
        return {}


def timed_median(fn, flush, reps=10, warm=3):
    """Median CUDA-event time (ms) of `fn()` with the L2 emptied (a 256 MB write) before every call."""
    for _ in range(warm):
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
    return statistics.median(times)


# --------------------------------------------------------------------------- operators beyond the step
def extra_op_times(device, peaks, reps=10, full=False):
    """Operator forms that are not part of `value`, each timed on its own (L2 emptied before every call):
    reshape_and_cache_flash on all K/V rows of the prefill batch (the size at which a GB/s figure
    means something), rotary_embedding out of place, and the four projections with a column-major
    B, and a 4096^3 fp32 mm (the tensor-core form from bf16 pieces).  With `full` also the operators of the
    next scope rows: aten::_flash_attention_forward on a dense causal GQA batch (packed and as the
    transposed views SDPA passes), bmm, gelu_and_mul."""
    import flaggems_b200 as fg
    from flaggems_b200 import workloads as W

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    out = []

    def entry(op, ms, work, kind):
        if kind == "hbm":
            ach, peak, unit = work / ms / 1e6, peaks["hbm_gbs"], "GB/s"
        else:
            ach, peak, unit = work / ms / 1e9, peaks["bf16_tflops"], "TFLOP/s"
        out.append({"op": op, "ms": round(ms, 4), "bound": kind, "achieved": round(ach, 1), "unit": unit,
                    "peak": peak, "frac": round(ach / peak, 3)})

    # cache write of every K/V row of the 16-sequence prefill batch (~33.8 k tokens, ~277 MB)
    p = W.prefill_batch(seed=4, device=device)
    T, hk, d = p.k.shape
    ms = timed_median(lambda: fg.reshape_and_cache_flash(p.k, p.v, p.key_cache, p.value_cache, p.slot_mapping, "auto",
                                                         None, None), flush, reps)
    entry(f"reshape_and_cache_flash, {T} tokens x {hk} heads x {d} (all K/V rows of the prefill batch)", ms,
          4 * T * hk * d * 2 + T * 8, "hbm")
    del p
    # rotary_embedding out of place (the benchmark step times the in-place form vLLM uses)
    q, k, cos, sin, pos = W.rope_inputs(seed=2, device=device)
    tq, hq, d = q.shape
    hk = k.shape[1]
    ms = timed_median(lambda: fg.apply_rotary_pos_emb(q, k, cos, sin, pos, False, False), flush, reps)
    entry("rotary_embedding out of place, q [4096,32,128] k [4096,8,128] (incl. output allocation)", ms,
          2 * (tq * hq * d + tq * hk * d) * 2 + tq * 2 * (d // 2) * 2 + tq * 8, "hbm")
    del q, k
    # projections with a column-major B (the reference's tests run both layouts)
    for i, name in enumerate(W.GEMM_SHAPES):
        a, b, bias = W.gemm_inputs(name, seed=10 + i, device=device, b_column_major=True)
        c = torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device=device)
        M, K = a.shape
        N = b.shape[1]
        if name in ("qkv", "gate_up"):
            ms = timed_median(lambda: fg.addmm_out(bias, a, b, out=c), flush, reps)
            entry(f"addmm[{name}] with column-major B", ms, M * N * (2 * K + 1), "tensor")
        else:
            ms = timed_median(lambda: fg.mm_out(a, b, out=c), flush, reps)
            entry(f"mm[{name}] with column-major B", ms, 2 * M * N * K, "tensor")
        del a, b, c
    # fp32 mm (never TF32): at this size three bf16 pieces per operand on the tensor cores, chunked accumulation
    g32 = torch.Generator(device=device).manual_seed(78)
    a32 = torch.randn((4096, 4096), generator=g32, dtype=torch.float32, device=device)
    b32 = torch.randn((4096, 4096), generator=g32, dtype=torch.float32, device=device)
    ms = timed_median(lambda: fg.mm(a32, b32), flush, max(3, reps // 3), warm=1)
    out.append({"op": "mm fp32 4096 x 4096 x 4096 (no TF32; incl. output and scratch allocation)", "ms": round(ms, 4),
                "bound": "tensor (six bf16 piece products per fp32 product)", "achieved": round(2 * 4096 ** 3 / ms / 1e9, 1),
                "unit": "TFLOP/s"})
    del a32, b32
    if not full:
        return out
    g = torch.Generator(device="cpu").manual_seed(77)
    B, S, H, Hk, D = 8, 4096, 32, 8, 128
    mk = lambda h: torch.randn((B, S, h, D), generator=g, dtype=torch.float32).to(device=device, dtype=torch.bfloat16)
    q, k, v = mk(H), mk(Hk), mk(Hk)
    flops = 4 * B * H * D * S * (S + 1) // 2
    for label, args in (("packed (batch, seq, heads, dim)", (q, k, v)),
                        ("transposed views of (batch, heads, seq, dim)",
                         tuple(x.transpose(1, 2).contiguous().transpose(1, 2) for x in (q, k, v)))):
        ms = timed_median(lambda: fg.flash_attention_forward(*args, None, None, S, S, 0.0, True, False), flush, reps)
        entry(f"_flash_attention_forward dense causal B{B} S{S} H{H}/{Hk} d{D}, {label}", ms, flops, "tensor")
    # bmm: 32 problems of 1024 x 1024 x 1024, bf16 (one launch)
    a3 = torch.randn((32, 1024, 1024), generator=g, dtype=torch.float32).to(device=device, dtype=torch.bfloat16)
    b3 = torch.randn((32, 1024, 1024), generator=g, dtype=torch.float32).to(device=device, dtype=torch.bfloat16)
    ms = timed_median(lambda: fg.bmm(a3, b3), flush, reps)
    entry("bmm 32 x [1024, 1024] x [1024, 1024] bf16 (incl. output allocation)", ms, 2 * 32 * 1024 ** 3, "tensor")
    # gelu_and_mul on the silu_and_mul benchmark shape: halves of [4096, 22016], bf16
    x = torch.randn((4096, 22016), generator=g, dtype=torch.float32).to(device=device, dtype=torch.bfloat16)
    half = x.shape[1] // 2
    nbytes = x.numel() * 2 + x.shape[0] * half * 2
    for approximate in ("none", "tanh"):
        with torch.no_grad():
            ms = timed_median(lambda: fg.gelu_and_mul(x[:, :half], x[:, half:], approximate), flush, reps)
        entry(f"gelu_and_mul[{approximate}] halves of [4096, 22016] (incl. output allocation)", ms, nbytes, "hbm")
    return out


# --------------------------------------------------------------------------- reference GPU path
def triton_reference_times(step, reps=5):
    """Per-operator times of the unmodified reference (its Triton kernels, installed under
    baseline/_ref) on the same device buffers, in the same run.  Returns
    {"ops": [{"op", "ms"}...], "step_ms": sum} or {"unavailable": reason}."""
    from baseline import triton_reference as tref

    t_start = time.time()
    try:
        ref = tref.load()
    except tref.ReferenceUnavailable as e:
        return {"unavailable": str(e)}
    silu_out = tref.module_attr("flag_gems.fused.silu_and_mul", "silu_and_mul_out")
    mm_out = tref.module_attr("flag_gems.ops.mm", "mm_out")
    addmm_out = tref.module_attr("flag_gems.ops.addmm", "addmm_out")
    nm = step.names
    calls = {}
    if hasattr(step, "x"):
        H = step.x.shape[1]
        calls[nm["norm"]] = lambda: ref.fused_add_rms_norm(step.x, step.res, [H], step.w, step.eps)
    if hasattr(step, "q"):
        calls[nm["rope"]] = lambda: ref.apply_rotary_pos_emb(step.q, step.k, step.cos, step.sin, step.pos, False, True)
    if hasattr(step, "act"):
        a1, a2 = step.act[:, :step.half], step.act[:, step.half:]
        calls[nm["silu"]] = lambda: silu_out(a1, a2, step.silu_out)
    if hasattr(step, "pre"):
        p = step.pre
        calls[nm["prefill"]] = lambda: ref.flash_attn_varlen_func(
            p.q, p.key_cache, p.value_cache, p.max_seqlen_q, p.cu_seqlens_q, p.max_seqlen_k, seqused_k=p.seqused_k,
            causal=True, block_table=p.block_table, out=step.pre_out)
    if hasattr(step, "dec"):
        dd = step.dec
        calls[nm["cache"]] = lambda: ref.reshape_and_cache_flash(
            dd.new_key, dd.new_value, dd.key_cache, dd.value_cache, dd.slot_mapping, "auto", None, None)
        calls[nm["decode"]] = lambda: ref.flash_attn_varlen_func(
            dd.q, dd.key_cache, dd.value_cache, 1, dd.cu_seqlens_q, dd.max_seqlen_k, seqused_k=dd.seqused_k,
            causal=True, block_table=dd.block_table, out=step.dec_out)
    for n in step.gemm:
        a, b, bias, c, _ = step.gemm[n]
        if n in ("qkv", "gate_up"):
            calls[f"addmm[{n}]"] = (lambda a=a, b=b, bias=bias, c=c[0]: addmm_out(bias, a, b, out=c))
        else:
            calls[f"mm[{n}]"] = (lambda a=a, b=b, c=c[0]: mm_out(a, b, out=c))
    # The reference's launcher cannot re-launch a kernel from its own cache under this image's Triton
    # (see baseline/triton_reference.py), so the cache is emptied before each call.  That path has
    # more host overhead; a short device-side sleep in front of the timed call lets the host
    # run ahead, so the events bracket the reference's kernels and not its Python.
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=step.device)
    out = []
    for name, _, _, _ in step.ops:
        fn = calls.get(name)
        if fn is None:
            continue
        try:
            for _ in range(2):   # includes the JIT build and the reference's autotuning
                tref.forget()
                fn()
            torch.cuda.synchronize()
            times = []
            for _ in range(reps):
                tref.forget(rescan=False)
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
    ok = [o["ms"] for o in out if "ms" in o]
    return {"ops": out, "step_ms": round(sum(ok), 4) if len(ok) == len(out) else None,
            "how": "unmodified reference package (Triton kernels as compiled by this image's Triton) on the same device "
                   "buffers; per operator: median of %d calls, L2 emptied by a 512 MB write before each, CUDA events "
                   "around the call with the host run ahead" % reps,
            "seconds_spent": round(time.time() - t_start, 1)}


# --------------------------------------------------------------------------- CPU arm
def host_threads():
    """Threads the CPU arm uses: every core this process may run on.  torchrun exports
    OMP_NUM_THREADS=1 to its workers, which would leave the arm on one core."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, n)


_CPU_INPUTS: dict = {}


def cpu_step_sample(seed=0):
    """Time the CPU oracle on a bounded sample of one step; returns (scaled seconds for a
    full step, number of ops, description, per-operator scaled seconds, seconds really spent).
    Each operator is timed on a slice and scaled by its algorithmic work."""
    from flaggems_b200 import workloads as W
    from oracle import reference_oracle as O  # CPU baseline leg

    detail = {}
    spent = [0.0]

    def timed(fn):
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        spent[0] += dt
        return dt

    # the sample's inputs are drawn once per process and reused by every pass
    inp = _CPU_INPUTS.get(seed)
    if inp is None:
        g = torch.Generator().manual_seed(seed + 4)
        lens = torch.randint(128, 4097, (16,), generator=g).tolist()
        g = torch.Generator().manual_seed(seed + 5)
        ctx = torch.randint(512, 8193, (256,), generator=g).tolist()
        inp = _CPU_INPUTS[seed] = {
            "norm": W.norm_inputs(seed=seed + 1, T=4096, device="cpu"),
            "rope": W.rope_inputs(seed=seed + 2, T=4096, device="cpu"),
            "tables": W.rope_tables(4096, 128, torch.bfloat16, "cpu"),
            "act": W.silu_inputs(seed=seed + 3, T=4096, device="cpu"),
            "lens": lens, "ctx": ctx,
            # prefill: one 2048-token sequence, scaled by FLOPs to the 16-sequence batch
            "pb": W.prefill_batch(seed=seed + 4, num_seqs=1, min_len=2048, max_len=2048, device="cpu"),
            # decode: 32 sequences with 2048-token contexts, scaled by context tokens
            "db": W.decode_batch(seed=seed + 5, batch=32, min_ctx=2048, max_ctx=2048, device="cpu"),
            # projections: 1024 of the 8192 rows; operands upcast beforehand, as the reference's harness does
            # before it calls torch on the CPU (the weight's conversion does not grow with the rows and must
            # not be scaled with them)
            "gemm": {name: tuple(t.float() for t in W.gemm_inputs(name, seed=seed + 10 + i, M=1024, device="cpu"))
                     for i, name in enumerate(W.GEMM_SHAPES)},
        }
    x, r, w, eps = inp["norm"]
    detail["fused_add_rms_norm"] = timed(lambda: O.fused_add_rms_norm(x, r, w, eps, upcast=torch.float32))
    q, k, _, _, pos = inp["rope"]
    cos4, sin4 = inp["tables"]
    detail["rotary_embedding"] = timed(lambda: O.apply_rotary_pos_emb(q, k, cos4, sin4, pos))
    act = inp["act"]
    h = act.shape[1] // 2
    detail["silu_and_mul"] = timed(lambda: O.silu_and_mul(act[:, :h], act[:, h:], upcast=torch.float32))
    pb, lens = inp["pb"], inp["lens"]
    t1 = timed(lambda: O.paged_attention(pb.q, pb.key_cache, pb.value_cache, pb.query_lens, pb.kv_lens, pb.block_table,
                                         pb.scale, compute_dtype=torch.float32))
    detail["flash_attn_varlen_func[prefill]"] = t1 * W.prefill_flops(lens) / W.prefill_flops([2048])
    db, ctx = inp["db"], inp["ctx"]
    kc, vc = db.key_cache.clone(), db.value_cache.clone()
    t0 = timed(lambda: O.reshape_and_cache_flash(db.new_key, db.new_value, kc, vc, db.slot_mapping))
    detail["reshape_and_cache_flash"] = t0 * 256 / 32
    t1 = timed(lambda: O.paged_attention(db.q, db.key_cache, db.value_cache, db.query_lens, db.kv_lens,
                                         db.block_table, db.scale, compute_dtype=torch.float32))
    detail["flash_attn_varlen_func[decode]"] = t1 * sum(ctx) / (32 * 2048)
    for name, (a, b, bias) in inp["gemm"].items():
        if name in ("qkv", "gate_up"):
            t = timed(lambda: O.addmm(bias, a, b, upcast=torch.float32))
        else:
            t = timed(lambda: O.mm(a, b, upcast=torch.float32))
        detail[f"gemm[{name}]"] = t * 8
    total = sum(detail.values())
    sample = ("per operator: norm/rope/silu_and_mul all 4096 tokens, prefill one 2048-token "
              "sequence (scaled by FLOPs), decode 32 sequences x 2048 context (scaled by context tokens), GEMMs 1024 "
              "of 8192 rows; fp32 torch CPU; every operator's time scaled by its algorithmic work to the full step")
    return total, len(detail), sample, detail, spent[0]


def run_reference_arm(args, rank):
    if rank != 0:
        return
    cores = host_threads()
    torch.set_num_threads(cores)
    for _ in range(max(1, min(args.warmup, 1))):   # one untimed pass: page faults, thread pool start-up
        cpu_step_sample()
    times, spent = [], []
    n_ops = 10
    sample = ""
    for _ in range(args.steps):
        t, n_ops, sample, _, sp = cpu_step_sample()
        times.append(t)
        spent.append(sp)
    step_s = statistics.mean(times)
    val = n_ops / step_s
    out = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        # ms_per_step is a full step EXTRAPOLATED from the sample: each timed step really ran
        # sample_seconds of CPU work
        "extrapolated": True, "sample_seconds": round(statistics.mean(spent), 3),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                         "extrapolated": True, "sample_seconds": round(statistics.mean(spent), 3)},
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
                       f"{n_gpus} ranks, weak scaling: every rank runs the full-size step on its own sequences (no "
                       "exchange); the projections multiply the replicated A by the rank's own full-size column shard "
                       "and the shards are gathered over NVLink onto every rank (copy-engine pushes into peer-mapped "
                       "buffers + one NCCL all-reduce per step, overlapping the next step's operators; --gather picks "
                       "contiguous slots [ranks, M, N] (default), the row-major [M, ranks x N] written directly, or "
                       "ncclAllGather).  The 'tp' key holds the fixed-size step partitioned over the ranks, gathered "
                       "into the row-major [M, N]",
        "l2": "no explicit flush: the step cycles through ~8 GB of operands, every operator's inputs are evicted "
              "from the 126 MB L2 between its consecutive invocations",
    }


# --------------------------------------------------------------------------- N > 1: sharded == unsharded
def shard_check(device, rank, world):
    """Untimed: the single-GPU operators partitioned over the ranks (attention, cache write and
    rope by KV head; norm and silu_and_mul by token rows; projections by N / world columns,
    gathered) give the unsharded results.  Every rank builds the same seeded inputs at the
    benchmark's sizes, computes its shard, the shards are collected on every rank and rank 0
    compares them with its own unsharded run: bit-equal for the cache write, atol = rtol = 1e-2
    otherwise.  Returns {"status": "ok" | "FAILED", "ops": {...}}."""
    import flaggems_b200 as fg
    from flaggems_b200 import dist as fdist
    from flaggems_b200 import workloads as W

    dist = torch.distributed
    res = {}

    def compare(name, got, want, exact=False):
        g, w = got.float(), want.float()
        err = (g - w).abs()
        ok = bool(torch.equal(got, want)) if exact else bool((err <= 1e-2 + 1e-2 * w.abs()).all().item())
        res[name] = {"ok": ok, "max_abs": float(err.max().item()), "bit_equal": bool(torch.equal(got, want))}

    def gather_cat(local, dim):
        local = local.contiguous()
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local)
        return torch.cat(parts, dim=dim)

    qs, ks = fdist.kv_head_shard(32, 8, rank, world)
    # ---- projections: B [K, N / world] -> C_g [M, N / world] -> row-major [M, N] on every rank
    for i, name in enumerate(W.GEMM_SHAPES):
        a, b, bias = W.gemm_inputs(name, seed=10 + i, device=device)
        bs, zs = fdist.column_shard(b, bias, rank, world)
        pg = fdist.PeerGather((a.shape[0], bs.shape[1]), a.dtype, device)
        if name in ("qkv", "gate_up"):
            fg.addmm_out(zs, a, bs, out=pg.local_slot())
            want = fg.addmm(bias, a, b) if rank == 0 else None
        else:
            fg.mm_out(a, bs, out=pg.local_slot())
            want = fg.mm(a, b) if rank == 0 else None
        pg.push(pg.local_slot())
        pg.finish()
        torch.cuda.synchronize()
        if rank == 0:
            compare(f"gemm[{name}] columns gathered", pg.columns(), want)
        del a, b, bias, bs, zs, want
        dist.barrier()
        del pg
    # ---- prefill by KV head on the same batch
    p = W.prefill_batch(seed=4, device=device)
    kw = dict(max_seqlen_q=p.max_seqlen_q, cu_seqlens_q=p.cu_seqlens_q, max_seqlen_k=p.max_seqlen_k,
              seqused_k=p.seqused_k, causal=True, block_table=p.block_table)
    out = torch.empty_like(p.q)
    fg.flash_attn_varlen_func(p.q[:, qs], p.key_cache[:, :, ks], p.value_cache[:, :, ks], out=out[:, qs], **kw)
    got = gather_cat(out[:, qs], 1)
    if rank == 0:
        compare("prefill by KV head", got, fg.flash_attn_varlen_func(p.q, p.key_cache, p.value_cache, **kw))
    del p, out, got
    # ---- cache write and decode by KV head on the same batch
    d = W.decode_batch(seed=5, device=device)
    hk, hd = d.key_cache.shape[2], d.key_cache.shape[3]
    fg.reshape_and_cache_flash(d.new_key[:, ks], d.new_value[:, ks], d.key_cache[:, :, ks], d.value_cache[:, :, ks],
                               d.slot_mapping, "auto", None, None)
    wrote_k = gather_cat(d.key_cache.view(-1, hk, hd)[d.slot_mapping][:, ks], 1)
    wrote_v = gather_cat(d.value_cache.view(-1, hk, hd)[d.slot_mapping][:, ks], 1)
    if rank == 0:
        compare("cache write by KV head (K)", wrote_k, d.new_key, exact=True)
        compare("cache write by KV head (V)", wrote_v, d.new_value, exact=True)
        # rank 0 completes its own cache for the unsharded decode
        fg.reshape_and_cache_flash(d.new_key, d.new_value, d.key_cache, d.value_cache, d.slot_mapping, "auto", None, None)
    kw = dict(max_seqlen_q=1, cu_seqlens_q=d.cu_seqlens_q, max_seqlen_k=d.max_seqlen_k, seqused_k=d.seqused_k,
              causal=True, block_table=d.block_table)
    out = torch.empty_like(d.q)
    fg.flash_attn_varlen_func(d.q[:, qs], d.key_cache[:, :, ks], d.value_cache[:, :, ks], out=out[:, qs], **kw)
    got = gather_cat(out[:, qs], 1)
    if rank == 0:
        compare("decode by KV head", got, fg.flash_attn_varlen_func(d.q, d.key_cache, d.value_cache, **kw))
    del d, out, got
    # ---- rope by head, norm and silu_and_mul by token rows
    q, k, cos, sin, pos = W.rope_inputs(seed=2, device=device)
    oq, ok_ = fg.apply_rotary_pos_emb(q[:, qs], k[:, ks], cos, sin, pos, False, False)
    gq, gk = gather_cat(oq, 1), gather_cat(ok_, 1)
    if rank == 0:
        wq, wk = fg.apply_rotary_pos_emb(q, k, cos, sin, pos, False, False)
        compare("rotary_embedding by head (q)", gq, wq)
        compare("rotary_embedding by head (k)", gk, wk)
    x, r, w, eps = W.norm_inputs(seed=1, device=device)
    r0, r1 = fdist.shard_range(x.shape[0], rank, world)
    xs, rs = x[r0:r1].clone(), r[r0:r1].clone()
    fg.fused_add_rms_norm(xs, rs, [x.shape[1]], w, eps)
    if x.shape[0] % world == 0:
        gx, gr = gather_cat(xs, 0), gather_cat(rs, 0)
        if rank == 0:
            fg.fused_add_rms_norm(x, r, [x.shape[1]], w, eps)
            compare("fused_add_rms_norm by rows (out)", gx, x)
            compare("fused_add_rms_norm by rows (residual)", gr, r)
    act = W.silu_inputs(seed=3, device=device)
    half = act.shape[1] // 2
    r0, r1 = fdist.shard_range(act.shape[0], rank, world)
    so = fg.silu_and_mul(act[r0:r1, :half], act[r0:r1, half:])
    if act.shape[0] % world == 0:
        gs = gather_cat(so, 0)
        if rank == 0:
            compare("silu_and_mul by rows", gs, fg.silu_and_mul(act[:, :half], act[:, half:]))
    torch.cuda.synchronize()
    dist.barrier()
    if rank != 0:
        return None
    return {"status": "ok" if all(v["ok"] for v in res.values()) else "FAILED", "ops": res}


def time_steps(step, steps, barrier, events=None):
    """K steps between barriers; returns the CUDA-event time in ms (this rank)."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for s in range(steps):
        step.run(events[s] if events is not None else None)
    step.drain()
    e1.record()
    barrier()
    return e0.elapsed_time(e1)


def max_over_ranks(ms, device, world):
    if world > 1:
        t = torch.tensor([ms], device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())
    return ms


def per_op_table(step, events, steps, peaks):
    per_op = []
    for i, (name, _, work, kind) in enumerate(step.ops):
        ms = statistics.mean(events[s][i][0].elapsed_time(events[s][i][1]) for s in range(steps))
        if kind == "hbm":
            ach, peak, unit = work / ms / 1e6, peaks["hbm_gbs"], "GB/s"
        else:
            # every operator is timed on its own (a 0.2-1.4 ms kernel): the burst cuBLAS figure is the
            # denominator; the sustained one (power cap) is carried along in the roofline object
            ach, peak, unit = work / ms / 1e9, peaks["bf16_tflops"], "TFLOP/s"
        per_op.append({"op": name, "ms": round(ms, 4), "bound": kind, "achieved": round(ach, 1), "unit": unit,
                       "peak": peak, "frac": round(ach / peak, 3)})
    return per_op


def numa_note(local_rank):
    """Where the GPU and this process's host memory sit (read-only sysfs queries)."""
    note = {}
    try:
        pr = torch.cuda.get_device_properties(local_rank)
        bus = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        note["gpu_numa_node"] = int(Path(f"/sys/bus/pci/devices/{bus}/numa_node").read_text())
    except Exception:  # noqa: BLE001
        note["gpu_numa_node"] = None
    try:
        nodes = sorted(int(p.name[4:]) for p in Path("/sys/devices/system/node").glob("node[0-9]*"))
        note["host_numa_nodes"] = len(nodes)
    except Exception:  # noqa: BLE001
        note["host_numa_nodes"] = None
    note["cpus_allowed"] = host_threads()
    return note


# --------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer (PCIe) leg")
    ap.add_argument("--only", default="", help="run (and allocate) only the operators whose name contains this string")
    ap.add_argument("--extra", action="store_true",
                    help="N=1: extra_ops also covers the operators built beyond the benchmark step (dense "
                         "_flash_attention_forward, gelu_and_mul, bmm)")
    ap.add_argument("--no-extra", action="store_true", help="N=1: skip extra_ops altogether")
    ap.add_argument("--no-triton-ref", action="store_true",
                    help="N=1: do not time the unmodified reference's Triton kernels (baseline/_ref) beside ours; "
                         "the leg adds the reference's JIT and autotuning time to the run")
    ap.add_argument("--triton-ref", action="store_true", help="accepted for compatibility: the leg is on by default")
    ap.add_argument("--no-tp", action="store_true", help="N>1: skip the tp leg and the shard check")
    ap.add_argument("--pipeline", default="auto", choices=["auto", "on", "off"],
                    help="N>1: whether the gathers of a step may overlap the next step's operators.  auto: only when "
                         "the gathers cannot hide inside their own step (their bytes at 700 GB/s take longer than "
                         "0.8 x the step without gathers, measured after warm-up): at 8 ranks, not at 2 or 4, where "
                         "the overlap gains nothing and the copies slow the next step's projections")
    ap.add_argument("--no-pipeline", action="store_true", help="same as --pipeline off")
    ap.add_argument("--push-streams", type=int, default=1,
                    help="N>1 with --gather p2p: side streams the copies to the peers are spread over")
    ap.add_argument("--gather", default="p2p-slots", choices=["p2p", "p2p-slots", "nccl"],
                    help="N > 1, weak-scaling step: how the projection shards are gathered.  p2p-slots: contiguous "
                         "copy-engine pushes into one slot per rank ([ranks, M, N]); p2p: strided copy-engine pushes "
                         "straight into the row-major [M, ranks x N] (what the tp leg always uses; slower beside the "
                         "compute kernels at 8 ranks); nccl: ncclAllGather + transposing copy")
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
    if args.no_pipeline:
        args.pipeline = "off"
    step = Step(device, rank, world, small=args.small, only=args.only, gather=args.gather, op_order=args.op_order,
                pipeline=args.pipeline == "on", push_streams=args.push_streams)
    n_ops = len(step.ops)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step.run()
    step.drain()
    barrier()
    pipeline_why = None
    if world > 1 and args.pipeline == "auto" and step.can_pipeline and step.gemm:
        # can the gathers hide inside their own step?  compare their bytes at 700 GB/s with the step without gathers
        step.skip_gather = True
        step.run()
        ms_c = max_over_ranks(time_steps(step, 2, barrier), device, world) / 2
        step.skip_gather = False
        ingress = sum(step.gemm[n][3][0].numel() * 2 for n in step.gemm) * (world - 1)
        ms_g = ingress / 700e9 * 1e3
        step.pipeline = ms_g > 0.8 * ms_c
        pipeline_why = f"gathers {ms_g:.2f} ms at 700 GB/s against {ms_c:.2f} ms of operators per step"
        for _ in range(2):
            step.run()
        step.drain()
        barrier()

    events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_ops)]
              for _ in range(args.steps)]
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    launches0 = _lib.launch_count()
    t0 = time.time()
    ms_total = time_steps(step, args.steps, barrier, events)
    t1 = time.time()
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop(t0, t1)
    ms_total = max_over_ranks(ms_total, device, world)
    ms_step = ms_total / args.steps
    value = world * n_ops / (ms_step * 1e-3)

    per_op = per_op_table(step, events, args.steps, peaks)
    dom = max(per_op, key=lambda o: o["ms"])
    # DRAM bytes per launch of the dominant kernel from one ncu capture of the same launch;
    # only full-size launches of the default workload have a figure.
    traffic = None if args.small else ncu_dram_bytes_per_launch().get(dom["op"])
    roofline = {"bound": dom["bound"], "kernel": dom["op"], "achieved": dom["achieved"], "peak": dom["peak"],
                "unit": dom["unit"], "frac": dom["frac"], "peak_source": peak_kind,
                "traffic": traffic}
    if dom["bound"] == "tensor":
        roofline["peak_kind"] = "burst (kernel timed alone)"
        roofline["peak_sustained"] = peaks["bf16_tflops_sustained"]

    # ---- N > 1: the same K steps without the gathers (what the sharded operators alone scale like)
    no_gather = gathers = None
    if world > 1:
        gathers = []
        for name, (g0, g1) in step.comm_events.items():
            ms = g0.elapsed_time(g1)
            nbytes = step.gathered_result(name).numel() * 2
            gathers.append({"op": f"all_gather[{name}]", "ms": round(ms, 4), "bytes": nbytes,
                            "busbw_GBs": round(nbytes * (world - 1) / world / ms / 1e6, 1)})
        ingress = sum(g["bytes"] for g in gathers) * (world - 1) / world
        step.skip_gather = True
        for _ in range(2):
            step.run()
        ms_ng = max_over_ranks(time_steps(step, args.steps, barrier), device, world)
        step.skip_gather = False
        no_gather = {"value": world * n_ops / (ms_ng / args.steps * 1e-3), "unit": UNIT,
                     "ms_per_step": ms_ng / args.steps,
                     "note": "same step with the projection outputs left sharded (no NVLink traffic)",
                     "nvlink_ingress_bytes_per_rank_per_step": int(ingress),
                     "ingress_GBs_in_the_headline_step": round(ingress / ms_step / 1e6, 1)}

    # ---- end to end: pinned host buffers in and out, copies inside the timed region
    h2d = d2h = 0
    ms_e2e = float("nan")
    e2e_val = None
    if not args.no_e2e:
        step.drain()
        pipelined = step.pipeline
        step.pipeline = False          # the results that leave for the host are those of the step itself
        h2d, d2h = step.make_e2e()
        for _ in range(2):
            step.run_e2e()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step.run_e2e()
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1), device, world)
        e2e_val = world * n_ops / (ms_e2e / args.steps * 1e-3)
        step.pipeline = pipelined
    status = _lib.device_status(reset=True)

    e2e = {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": ms_e2e / args.steps}
    if e2e_val is not None:
        # both directions run at the same time on the two copy engines: each moves its bytes within the step
        e2e["h2d_GBs_per_rank"] = round(h2d / (ms_e2e / args.steps) / 1e6, 2)
        e2e["d2h_GBs_per_rank"] = round(d2h / (ms_e2e / args.steps) / 1e6, 2)
        e2e["host"] = numa_note(local_rank)
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": dict(workload_config(world, n_ops, args.small, args.only),
                                            op_order=[o[0] for o in step.ops]), "roofline": roofline,
        "e2e": e2e,
        "gpu_launches": int(launches), "clocks": clocks, "per_op": per_op, "device_status": status,
    }
    if world > 1:
        out["no_gather"] = no_gather
        out["all_gather"] = gathers
        out["config"]["gather"] = args.gather
        out["config"]["gather_pipeline"] = ("the gathers of step s overlap the operators of step s+1 (two result "
                                            "buffers per projection); all K steps' gathers land inside the timed region"
                                            if step.pipeline else "every step waits for its own gathers")
        if pipeline_why:
            out["config"]["gather_pipeline"] += f" (chosen after warm-up: {pipeline_why})"
    if world == 1 and not args.small and not args.only:
        if not args.no_triton_ref:
            tr = triton_reference_times(step)
            if tr.get("step_ms"):
                tr["ours_step_ms"] = round(ms_step, 4)
                tr["reference_step_over_ours"] = round(tr["step_ms"] / ms_step, 3)
                ours = {o["op"]: o["ms"] for o in per_op}
                for o in tr["ops"]:
                    if "ms" in o and o["op"] in ours:
                        o["ours_ms"] = ours[o["op"]]
                        o["reference_over_ours"] = round(o["ms"] / ours[o["op"]], 2)
            out["triton_ref"] = tr
    del step
    torch.cuda.empty_cache()
    if world == 1 and not args.small and not args.only:
        if not args.no_extra:
            out["extra_ops"] = extra_op_times(device, peaks, full=args.extra)
        if not args.no_cpu_baseline:
            torch.set_num_threads(host_threads())
            cpu_step_sample()   # untimed: first-touch page faults and the thread pool's start-up
            t, n, sample, detail, spent = cpu_step_sample()
            out["cpu_baseline"] = {"value": n / t, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                   "sample": sample + "; second of two passes", "step_seconds_scaled": t,
                                   "extrapolated": True, "sample_seconds": round(spent, 3)}
    if world > 1 and not args.no_tp and not args.small and not args.only:
        # ---- the fixed-size step partitioned over the ranks (strong scaling), under its own key
        chk = shard_check(device, rank, world)
        torch.cuda.empty_cache()
        tp = Step(device, rank, world, gather="p2p", op_order=args.op_order, mode="tp", pipeline=False,
                  push_streams=args.push_streams)
        for _ in range(args.warmup):
            tp.run()
        tp.drain()
        tp_events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                      for _ in range(len(tp.ops))] for _ in range(args.steps)]
        ms_tp = max_over_ranks(time_steps(tp, args.steps, barrier, tp_events), device, world) / args.steps
        tp_gathers = []
        for name, (g0, g1) in tp.comm_events.items():
            ms = g0.elapsed_time(g1)
            nbytes = tp.gathered_result(name).numel() * 2
            tp_gathers.append({"op": f"all_gather[{name}]", "ms": round(ms, 4), "bytes": nbytes,
                               "busbw_GBs": round(nbytes * (world - 1) / world / ms / 1e6, 1)})
        tp.skip_gather = True
        for _ in range(2):
            tp.run()
        ms_tp_ng = max_over_ranks(time_steps(tp, args.steps, barrier), device, world) / args.steps
        out["tp"] = {
            "what": "the single-GPU step (fixed total work) partitioned over the ranks: attention, cache write and rope "
                    "by KV head, norm and silu_and_mul by token rows, projections B [K, N/ranks] -> C [M, N/ranks] "
                    "gathered into the row-major [M, N] on every rank; every step waits for its own gathers",
            "scaling": "strong", "ms_per_step": ms_tp, "value": len(tp.ops) / (ms_tp * 1e-3), "unit": "steps' ops/s",
            "ms_per_step_without_gather": ms_tp_ng, "per_op_rank0": per_op_table(tp, tp_events, args.steps, peaks),
            "all_gather": tp_gathers,
            "nvlink_ingress_bytes_per_rank_per_step": int(sum(g["bytes"] for g in tp_gathers) * (world - 1) / world),
        }
        out["shard_check"] = chk["status"] if chk else None
        out["shard_check_detail"] = chk["ops"] if chk else None
        del tp
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
