#!/usr/bin/env python
"""Benchmark of the fused-kernel hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c5|c3|c3f|c2|c1|c4g|gemm|pw] [--impl ours|reference]

Default workload "c4": the transformer MLP block forward + backward, bf16, 8192 tokens per GPU, d 4096,
ff 16384 -- six fused GEMMs per step, metric fused-GEMM TFLOP/s.  With N > 1 (launched under
torch.distributed.run, one process per GPU) tokens are sharded over the ranks and the weight / bias
gradients are averaged with NCCL through the library's own communicator (he_allreduce_grads), overlapped
with the remaining backward GEMMs; the value is N x per-GPU work / max-over-ranks device time.
At N = 1 the default run also times the other single-GPU configurations in the same process and reports
them under "configs": the README fused matmul 4096^3 as planned ("c3") and with the in-kernel mainloop
rewrite forced ("c3f"), the fused affine + layout change and the f32 permutation ("c2"), the f32 MLP
training step ("c1").  Other workloads: c4g = the MLP block as one op graph through the host runtime,
gemm = a plain 8192^3 bf16 matmul, pw = stand-alone pointwise programs on 64 Mi-element tensors.

Rank 0 prints exactly one JSON line.  c1-c3 have no cross-GPU dependency: with N > 1 they run an independent
replica per rank.  `--impl reference` times the CPU restatement of the same work (oracle/) on the host
cores; it loads neither the CUDA library nor the package initialiser.
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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)



def host_configs():
    """helium_b200/configs.py (graphs + seeded inputs, pure numpy) WITHOUT running the package initialiser, so
    that the CPU legs -- above all `--impl reference` -- never map libhelium_b200.so: the modules are imported
    under a stand-in package whose path is the package directory."""
    import importlib
    import types
    name = "helium_b200_hostonly"
    if name not in sys.modules:
        pkg = types.ModuleType(name)
        pkg.__path__ = [os.path.join(ROOT, "helium_b200")]
        sys.modules[name] = pkg
    return importlib.import_module(name + ".configs")


C2A_SHAPE = (64, 256, 56, 56)
C2B_SHAPE = (4096, 4096, 8)
C2A_BYTES = 2 * 64 * 256 * 56 * 56 * 2 + 2 * 256 * 4      # x in + y out (bf16) + s, b (f32)
C2B_BYTES = 2 * 4096 * 4096 * 8 * 4                       # in + out (f32)
C3_MNK = (4096, 4096, 4096)
C3_FLOPS = 2 * 4096 ** 3
NCCL_CTAS_DEFAULT = 32


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


TRAFFIC_SOURCE = "profiles/dram_traffic.txt (ncu capture of this kernel and shape, committed; not measured by this run)"


def load_traffic(name: str):
    """Per-launch DRAM traffic (bytes) of the dominant kernel, read from the committed ncu summary
    profiles/dram_traffic.txt (lines `key bytes  # comment`), or None when the kernel has no capture.  The
    JSON line labels it with `traffic_source`: it is a recorded figure, not a measurement of the run."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    if not os.path.exists(path):
        return None
    for ln in open(path):
        f = ln.split("#")[0].split()
        if len(f) >= 2 and f[0] == name:
            return int(float(f[1]))
    return None


# ---- clock sampling during the timed region ----------------------------------------------------------
class ClockSampler:
    FIELDS = ("utilization.gpu,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str):
        self.gpu = gpu_id  # "GPU-<uuid>" (CUDA ordinals and nvidia-smi indices need not agree)
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        total = 0
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                util, clk, cmax = float(f[0]), float(f[1]), float(f[2])
            except ValueError:
                continue
            total += 1
            if util <= 0:
                continue  # idle sample (before the first launch / between legs)
            sm.append(clk); mx.append(cmax)
            try:
                power.append(float(f[3]))
            except ValueError:
                pass
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples_under_load": len(sm), "samples": total,
                "power_w_max": max(power) if power else None}


# ---- workloads ---------------------------------------------------------------------------------------
# A workload object owns its device buffers and exposes:
#   step(record)   one pass over resident inputs; when `record` is a list, CUDA events bracketing the
#                  dominant kernel are appended to it as (name, start, end)
#   step_e2e()     the same pass fed from pinned host buffers, results read back to the host
#   cpu_sample()   (static) a bounded sample of the same work on the host cores -> (value, cores, text)
def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


class _E2EPipeline:
    """End-to-end leg: two sets of device buffers and three streams, so that the upload of step i+1, the
    kernels of step i and the download of step i-1 overlap (PCIe is full duplex).  This is the
    host-to-device pipelining helium's executor does per stream (helium/src/cuda.rs:192-222).
    `upload(k)`, `run(k)`, `download(k)` enqueue the work of one step on buffer set k; the caller
    synchronises the device after the last step."""
    note = "three streams, two device buffer sets: upload of step i+1, kernels of step i, download of step i-1 overlap"

    def __init__(self, torch, dev):
        self.torch = torch
        self.st_up, self.st_run, self.st_down = (torch.cuda.Stream(device=dev) for _ in range(3))
        self.ev_up = [torch.cuda.Event() for _ in range(2)]
        self.ev_run = [torch.cuda.Event() for _ in range(2)]
        self.ev_down = [torch.cuda.Event() for _ in range(2)]
        self.i = 0

    def step(self, upload, run, download):
        torch = self.torch
        k = self.i & 1
        first_use = self.i < 2
        self.i += 1
        with torch.cuda.stream(self.st_up):
            if not first_use:
                self.st_up.wait_event(self.ev_run[k])      # the kernels that last read this input set are done
            upload(k)
            self.ev_up[k].record(self.st_up)
        with torch.cuda.stream(self.st_run):
            self.st_run.wait_event(self.ev_up[k])
            if not first_use:
                self.st_run.wait_event(self.ev_down[k])   # the previous results of this set have left the device
            run(k)
            self.ev_run[k].record(self.st_run)
        with torch.cuda.stream(self.st_down):
            self.st_down.wait_event(self.ev_run[k])
            download(k)
            self.ev_down[k].record(self.st_down)


class WorkloadC2:
    key = "c2"
    metric, unit = "pointwise_permute_hbm_gbs", "GB/s"
    dtype = "bf16 (f32 fma) + f32 bit moves"
    description = ("configs[1]: y=relu(x*s_c+b_c) bf16 [64,256,56,56] NCHW->NHWC fused in one kernel; "
                   "permute f32 [4096,4096,8] axes (2,0,1)")
    l2_note = "inputs exceed L2 (512 MiB permute input; the 103 MB pointwise input is evicted by the 1 GiB permute between its uses)"
    launches_per_step = 2
    work_per_step = C2A_BYTES + C2B_BYTES
    work_scale = 1e9
    e2e_note = _E2EPipeline.note

    def __init__(self, ctx, dev, world, rank, peaks, reducer):
        import torch
        import helium_b200 as hb
        from helium_b200 import ir
        from helium_b200.configs import c2_inputs, graph_affine_relu_permute
        self.torch = torch
        x_h, s_h, b_h, p_h = c2_inputs(1)
        self.plan_a = hb.Plan.pointwise(ctx, graph_affine_relu_permute(*C2A_SHAPE))
        st = hb.permute_output_strides(list(C2B_SHAPE), [(1, 2), (0, 1)])
        self.plan_b = hb.Plan.permute(ctx, list(C2B_SHAPE), st, ir.F32)
        self.x_pin = torch.from_numpy(x_h.view(np.int16)).pin_memory()
        self.p_pin = torch.from_numpy(p_h).pin_memory()
        self.s_pin = torch.from_numpy(s_h).pin_memory(); self.b_pin = torch.from_numpy(b_h).pin_memory()
        self.x_d = self.x_pin.to(dev).view(torch.bfloat16); self.s_d = self.s_pin.to(dev); self.b_d = self.b_pin.to(dev)
        self.p_d = self.p_pin.to(dev)
        self.y_d = torch.empty((64, 56, 56, 256), dtype=torch.bfloat16, device=dev)
        self.q_d = torch.empty((8, 4096, 4096), dtype=torch.float32, device=dev)
        self.y_pin = torch.empty((64, 56, 56, 256), dtype=torch.int16).pin_memory()
        self.q_pin = torch.empty((8, 4096, 4096), dtype=torch.float32).pin_memory()
        self.h2d = self.x_pin.numel() * 2 + self.p_pin.numel() * 4 + 2 * 256 * 4
        self.d2h = self.y_pin.numel() * 2 + self.q_pin.numel() * 4
        self.bufs = [dict(x=self.x_d, s=self.s_d, b=self.b_d, p=self.p_d, y=self.y_d, q=self.q_d),
                     dict(x=torch.empty_like(self.x_d), s=torch.empty_like(self.s_d), b=torch.empty_like(self.b_d),
                          p=torch.empty_like(self.p_d), y=torch.empty_like(self.y_d), q=torch.empty_like(self.q_d))]
        self.pipe = _E2EPipeline(torch, dev)
        self.dominant = {"permute_c2b": ("permute_tile_vec<4> on [4096,4096,8] f32", C2B_BYTES, "hbm", peaks["hbm_gbs"], "GB/s"),
                         "pointwise_c2a": ("affine+relu+NCHW->NHWC tile kernel on bf16 [64,256,56,56]", C2A_BYTES, "hbm", peaks["hbm_gbs"], "GB/s")}
        self.dominant_key = "permute_c2b"

    def step(self, record=None):
        torch = self.torch
        st = torch.cuda.current_stream()
        if record is None:
            self.plan_a.launch([self.x_d, self.s_d, self.b_d], [self.y_d])
            self.plan_b.launch([self.p_d], [self.q_d])
            return
        a0, a1 = _events(torch); b0, b1 = _events(torch)
        a0.record(st); self.plan_a.launch([self.x_d, self.s_d, self.b_d], [self.y_d]); a1.record(st)
        b0.record(st); self.plan_b.launch([self.p_d], [self.q_d]); b1.record(st)
        record.append(("pointwise_c2a", a0, a1)); record.append(("permute_c2b", b0, b1))

    def step_e2e(self):
        torch = self.torch

        def upload(k):
            B = self.bufs[k]
            B["x"].view(torch.int16).copy_(self.x_pin, non_blocking=True)
            B["s"].copy_(self.s_pin, non_blocking=True); B["b"].copy_(self.b_pin, non_blocking=True)
            B["p"].copy_(self.p_pin, non_blocking=True)

        def run(k):
            B = self.bufs[k]
            self.plan_a.launch([B["x"], B["s"], B["b"]], [B["y"]])
            self.plan_b.launch([B["p"]], [B["q"]])

        def download(k):
            B = self.bufs[k]
            self.y_pin.copy_(B["y"].view(torch.int16), non_blocking=True)
            self.q_pin.copy_(B["q"], non_blocking=True)

        self.pipe.step(upload, run, download)

    @staticmethod
    def cpu_sample(steps=3, warmup=1):
        """Every timed step is one full pass of both kernels' work on the host cores."""
        cfg = host_configs()
        from oracle import oracle_c as OC
        x, s, b, p = cfg.c2_inputs(1)
        st = [4096, 1, 4096 * 4096]
        for _ in range(max(1, warmup)):                           # the first call also builds / loads the C object
            OC.affine_relu_nchw_nhwc(x, s, b); OC.permute(p, st)
        t0 = time.perf_counter()
        for _ in range(steps):
            OC.affine_relu_nchw_nhwc(x, s, b)
            OC.permute(p, st)
        dt = (time.perf_counter() - t0) / steps
        return (C2A_BYTES + C2B_BYTES) / dt / 1e9, OC.num_threads(), \
            f"{steps} full steps (both kernels' work) of the C+OpenMP restatement (oracle/oracle_c.c); the reference has no CPU path", dt


class _GemmBase:
    """Shared pieces of the tensor-core workloads: L2 flush buffer, TFLOP/s bookkeeping."""
    work_scale = 1e12
    l2_note = "256 MiB buffer written between iterations to flush L2 (inside the timed region; its ~40 us are included)"

    def _flush_buffer(self, dev):
        return self.torch.empty(256 << 20, dtype=self.torch.uint8, device=dev)

    @staticmethod
    def _cpu_gemm_sample(m, n, k, rows, masked, seed, steps=1, warmup=1):
        """`rows` output rows of an [m,k]x[k,n] bf16 GEMM on the host cores per timed step, scaled linearly to m
        rows; returns (seconds per full GEMM, threads)."""
        cfg = host_configs()
        from oracle import oracle_c as OC
        r = cfg.rng(seed)
        a = cfg.bf16_normal(r, (rows, k)); b = cfg.bf16_normal(r, (k, n), 1.0 / np.sqrt(k))
        mk = cfg.bf16_bernoulli(r, (rows, k)) if masked else None
        for _ in range(max(1, warmup)):                           # builds / loads the C object, warms the caches
            OC.gemm_bf16(a[:8], b, None if mk is None else mk[:8], 0, 8)
        t0 = time.perf_counter()
        for _ in range(steps):
            OC.gemm_bf16(a, b, mk, 0, rows)
        dt = (time.perf_counter() - t0) / steps * (m / rows)
        return dt, OC.num_threads()


class WorkloadGemm(_GemmBase):
    key = "gemm"
    metric, unit = "gemm_tflops", "TFLOP/s"
    dtype = "bf16 x bf16 -> f32 accumulate"
    description = "plain matmul 8192^3 bf16 (Op::Matmul contract, no fusion), bf16 output"
    launches_per_step = 1
    M = N = K = 8192
    work_per_step = 2.0 * 8192 ** 3

    def __init__(self, ctx, dev, world, rank, peaks, reducer):
        import torch
        import helium_b200 as hb
        from helium_b200.configs import graph_linear
        self.torch = torch
        m, n, k = self.M, self.N, self.K
        self.plan = hb.Plan.fused_matmul(ctx, graph_linear(m, n, k, bias=False, precision=self.precision()))
        gen = torch.Generator(device=dev).manual_seed(2)
        self.a_d = torch.randn((m, k), generator=gen, device=dev).to(torch.bfloat16)
        self.b_d = (torch.randn((k, n), generator=gen, device=dev) / 90.0).to(torch.bfloat16)
        self.a_pin = self.a_d.cpu().pin_memory(); self.b_pin = self.b_d.cpu().pin_memory()
        self.outs_d = self.plan.alloc_outputs(dev)
        self.out_pin = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
        self.flush = self._flush_buffer(dev)
        self.sets = [(self.a_d, self.b_d, self.outs_d), (torch.empty_like(self.a_d), torch.empty_like(self.b_d), self.plan.alloc_outputs(dev))]
        self.pipe = _E2EPipeline(torch, dev)
        self.h2d, self.d2h = 2 * m * k * 2, m * n * 2
        self.dominant = {"gemm_plain": (self.plan.description, self.work_per_step, "tensor", peaks["bf16_tflops"] * self.peak_factor, "TFLOP/s")}
        self.dominant_key = "gemm_plain"

    peak_factor = 1.0

    @staticmethod
    def precision():
        return None

    def step(self, record=None):
        self.flush.zero_()
        if record is None:
            self.plan.launch([self.a_d, self.b_d], self.outs_d)
            return
        st = self.torch.cuda.current_stream()
        e0, e1 = _events(self.torch)
        e0.record(st); self.plan.launch([self.a_d, self.b_d], self.outs_d); e1.record(st)
        record.append(("gemm_plain", e0, e1))

    e2e_note = _E2EPipeline.note

    def step_e2e(self):
        def upload(k):
            self.sets[k][0].copy_(self.a_pin, non_blocking=True); self.sets[k][1].copy_(self.b_pin, non_blocking=True)

        def run(k):
            self.plan.launch([self.sets[k][0], self.sets[k][1]], self.sets[k][2])

        def download(k):
            self.out_pin.copy_(self.sets[k][2][0], non_blocking=True)

        self.pipe.step(upload, run, download)

    @staticmethod
    def cpu_sample(steps=1, warmup=1):
        rows = 256
        dt, cores = _GemmBase._cpu_gemm_sample(8192, 8192, 8192, rows, False, 2, steps, warmup)
        return 2.0 * 8192 ** 3 / dt / 1e12, cores, \
            f"{steps} timed steps of {rows} of 8192 output rows each, C+OpenMP restatement (oracle/oracle_c.c), scaled linearly", dt


class WorkloadC3(_GemmBase):
    key = "c3"
    metric, unit = "fused_gemm_tflops", "TFLOP/s"
    dtype = "bf16 x bf16 -> f32 accumulate, f32 epilogue"
    description = ("configs[2]: fused matmul 4096^3 bf16, mainloop relu(A)*M, epilogue bias/relu/tanh/gate/MSE + "
                   "Sum over Batch and Columns + two backward tiles (README graph)")
    work_per_step = float(C3_FLOPS)

    def __init__(self, ctx, dev, world, rank, peaks, reducer):
        import torch
        import helium_b200 as hb
        from helium_b200.configs import c3_inputs, graph_c3
        self.torch = torch
        m, n, k = C3_MNK
        ins_h = c3_inputs(m, n, k, False)
        self.plan = hb.Plan.fused_matmul(ctx, graph_c3(m, n, k, False))
        self.pins = [torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).pin_memory() for a in ins_h]
        self.ins_d = [p.to(dev).view(torch.bfloat16) for p in self.pins]
        self.ins_d[5] = self.ins_d[1]  # the epilogue mask is the mainloop mask (k == n)
        self.outs_d = self.plan.alloc_outputs(dev)
        self.outs_pin = [torch.empty(o.shape, dtype=torch.int16 if o.dtype == torch.bfloat16 else torch.float32).pin_memory()
                         for o in self.outs_d]
        self.flush = self._flush_buffer(dev)
        ins2 = [torch.empty_like(t) for t in self.ins_d]
        ins2[5] = ins2[1]
        self.sets = [(self.ins_d, self.outs_d), (ins2, self.plan.alloc_outputs(dev))]
        self.pipe = _E2EPipeline(torch, dev)
        self.h2d = sum(p.numel() * 2 for i, p in enumerate(self.pins) if i != 5)
        self.d2h = sum(p.numel() * p.element_size() for p in self.outs_pin)
        self.plan.launch(self.ins_d, self.outs_d)
        self.launches_per_step = self.plan.last_launch_count
        self.dominant = {"gemm_c3": (self.plan.description, self.work_per_step, "tensor", peaks["bf16_tflops"], "TFLOP/s")}
        self.dominant_key = "gemm_c3"

    def step(self, record=None):
        self.flush.zero_()  # operands (201 MB) partly fit the 126 MB L2: evict between iterations
        if record is None:
            self.plan.launch(self.ins_d, self.outs_d)
            return
        st = self.torch.cuda.current_stream()
        e0, e1 = _events(self.torch)
        e0.record(st); self.plan.launch(self.ins_d, self.outs_d); e1.record(st)
        record.append(("gemm_c3", e0, e1))

    e2e_note = _E2EPipeline.note

    def step_e2e(self):
        torch = self.torch

        def upload(k):
            for i, (d, p) in enumerate(zip(self.sets[k][0], self.pins)):
                if i != 5:
                    d.view(torch.int16).copy_(p, non_blocking=True)

        def run(k):
            self.plan.launch(self.sets[k][0], self.sets[k][1])

        def download(k):
            for o, p in zip(self.sets[k][1], self.outs_pin):
                p.copy_(o.view(torch.int16) if o.dtype == torch.bfloat16 else o, non_blocking=True)

        self.pipe.step(upload, run, download)

    @staticmethod
    def cpu_sample(steps=1, warmup=1):
        rows = 1024
        dt, cores = _GemmBase._cpu_gemm_sample(4096, 4096, 4096, rows, True, 2, steps, warmup)
        return C3_FLOPS / dt / 1e12, cores, \
            (f"{steps} timed steps of {rows} of 4096 output rows each of the mainloop-fused GEMM (epilogue not included), "
             "C+OpenMP restatement (oracle/oracle_c.c), scaled linearly"), dt


class WorkloadC4(_GemmBase):
    key = "c4"
    metric, unit = "fused_gemm_tflops", "TFLOP/s"
    dtype = "bf16 x bf16 -> f32 accumulate, f32 epilogue"
    TOKENS, D, FF = 8192, 4096, 16384
    description = ("configs[3]: transformer MLP block forward+backward, 8192 tokens per GPU, d=4096, ff=16384, bf16; six fused GEMMs "
                   "(bias+GELU, bias+residual, dgelu-gate+colsum, two weight-gradient GEMMs, residual+colsum); "
                   "weight/bias gradients averaged over ranks with NCCL, overlapped with the remaining GEMMs")
    l2_note = "every GEMM streams operands larger than L2 (W1/W2/H/Z are 128-256 MiB each); no flush needed"
    work_per_step = 6 * 2.0 * 8192 * 4096 * 16384

    def __init__(self, ctx, dev, world, rank, peaks, reducer, overlap_sms=0):
        import torch
        from helium_b200.mlp_block import MlpBlock, mlp_block_inputs
        self.torch = torch
        self.reducer = reducer
        T, d, ff = self.TOKENS, self.D, self.FF
        self.blk = MlpBlock(ctx, T, d, ff, dev, overlap_sms=overlap_sms)
        host = mlp_block_inputs(T, d, ff, seed=3, shard=rank)       # same weights on every rank, a different token shard each
        self.blk.load(host)
        as_pin = lambda v: torch.from_numpy(np.ascontiguousarray(v).view(np.int16)).pin_memory()
        self.x_pin, self.do_pin = as_pin(host["X"]), as_pin(host["dO"])
        self.dx_pin = torch.empty((T, d), dtype=torch.int16).pin_memory()
        self.db_pin = torch.empty(ff + d, dtype=torch.float32).pin_memory()
        self.h2d = 2 * T * d * 2
        self.d2h = T * d * 2 + (ff + d) * 4
        blk = self.blk
        self.io = [(blk.X, blk.dO, blk.dX, blk.db_flat),
                   (torch.empty_like(blk.X), torch.empty_like(blk.dO), torch.empty_like(blk.dX), torch.empty_like(blk.db_flat))]
        self.pipe = _E2EPipeline(torch, dev)
        self.blk.step(self.reducer)
        self.launches_per_step = self.blk.launch_count()
        peak = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
        gemm_flops = self.work_per_step / 6
        self.dominant = {k: (f"{k}: {self.blk.plans[k].description}", gemm_flops, "tensor", peak, "TFLOP/s") for k in self.blk.plans}
        self.dominant_key = None       # chosen after timing: the GEMM with the largest share of the step
        self.peak_note = "sustained cuBLAS bf16 figure (the kernels run inside a multi-millisecond step under the power cap)"

    def step(self, record=None):
        blk, red = self.blk, self.reducer
        if record is None:
            blk.step(red)
            return
        torch = self.torch
        st = torch.cuda.current_stream()
        p = blk.plans

        def timed(name, ins, outs):
            e0, e1 = _events(torch)
            e0.record(st); p[name].launch(ins, outs); e1.record(st)
            record.append((name, e0, e1))

        timed("H", [blk.X, blk.W1, blk.b1], [blk.H, blk.Z])
        timed("O", [blk.H, blk.W2, blk.b2, blk.X], [blk.O])
        timed("dZ", [blk.dO, blk.W2, blk.Z], [blk.dZ, blk.db1])
        timed("dW1", [blk.X, blk.dZ], [blk.dW1])
        if red is not None:
            red.reduce_bucket([blk.dW1])
        timed("dW2", [blk.H, blk.dO], [blk.dW2])
        if red is not None:
            red.reduce_bucket([blk.dW2])
        timed("dX", [blk.dZ, blk.W1, blk.dO], [blk.dX, blk.db2])
        if red is not None:
            red.reduce_bucket([blk.db_flat])
            red.finish()

    e2e_note = _E2EPipeline.note + "; the gradient all-reduce runs on its own stream behind the kernels of the same step"

    def _bind_io(self, k):
        blk = self.blk
        blk.X, blk.dO, blk.dX, blk.db_flat = self.io[k]
        blk.db1 = blk.db_flat[:blk.ff].view(1, blk.ff)
        blk.db2 = blk.db_flat[blk.ff:].view(1, blk.d)

    def step_e2e(self):
        torch = self.torch

        def upload(k):
            self.io[k][0].view(torch.int16).copy_(self.x_pin, non_blocking=True)
            self.io[k][1].view(torch.int16).copy_(self.do_pin, non_blocking=True)

        def run(k):
            self._bind_io(k)
            self.blk.step(self.reducer)

        def download(k):
            self.dx_pin.copy_(self.io[k][2].view(torch.int16), non_blocking=True)
            self.db_pin.copy_(self.io[k][3], non_blocking=True)

        self.pipe.step(upload, run, download)

    @staticmethod
    def cpu_sample(steps=1, warmup=1):
        rows = 256
        dt, cores = _GemmBase._cpu_gemm_sample(8192, 16384, 4096, rows, False, 3, steps, warmup)
        dt *= 6     # six GEMMs of equal flop count per step
        return WorkloadC4.work_per_step / dt / 1e12, cores, \
            (f"{steps} timed steps of {rows} of 8192 rows of the X*W1 GEMM each, C+OpenMP restatement (oracle/oracle_c.c), scaled "
             "linearly to the six equal-sized GEMMs of a step (epilogues not included)"), dt


class WorkloadC4Graph(_GemmBase):
    """configs[3] again, but handed to the C++ host runtime as ONE helium-style op graph (casts after every
    matmul, explicit transposes, swap_dims -> reduce -> reshape bias gradients) instead of six hand-built
    subgraphs: what the drop-in path behind helium's planner produces.  Single GPU (no gradient exchange)."""
    key = "c4g"
    metric, unit = "fused_gemm_tflops", "TFLOP/s"
    dtype = "bf16 x bf16 -> f32 accumulate, f32 epilogue"
    TOKENS, D, FF = 8192, 4096, 16384
    description = ("configs[3] as one op graph through the host runtime: transformer MLP block forward+backward, 8192 tokens, d=4096, "
                   "ff=16384, bf16; the planner fuses it into six matmul instructions and one column-sum kernel, replayed as a CUDA graph")
    l2_note = "every GEMM streams operands larger than L2; no flush needed"
    work_per_step = 6 * 2.0 * 8192 * 4096 * 16384

    def __init__(self, ctx, dev, world, rank, peaks, reducer):
        import torch
        import helium_b200 as hb
        from helium_b200 import configs
        from helium_b200.mlp_block import mlp_block_inputs
        self.torch = torch
        T, d, ff = self.TOKENS, self.D, self.FF
        g = configs.graph_mlp_block_train(T, d, ff)
        host = mlp_block_inputs(T, d, ff, seed=3, shard=rank)
        as_pin = lambda v: torch.from_numpy(np.ascontiguousarray(v).view(np.int16)).pin_memory()
        order = ("X", "W1", "b1", "W2", "b2", "dO")
        self.pins = {k: as_pin(host[k]) for k in order}
        self.ins = [self.pins[k].to(dev).view(torch.bfloat16) for k in order]
        bf, f32 = torch.bfloat16, torch.float32
        self.outs = [torch.empty((T, d), dtype=bf, device=dev), torch.empty((T, d), dtype=bf, device=dev),
                     torch.empty((d, ff), dtype=bf, device=dev), torch.empty(ff, dtype=f32, device=dev),
                     torch.empty((ff, d), dtype=bf, device=dev), torch.empty(d, dtype=f32, device=dev)]
        hg = hb.HostGraph(g)
        self.ex = hb.Executor(ctx, hg, self.ins, self.outs, capture=True)
        self._keep = hg
        st = self.ex.stats()
        self.launches_per_step = st["launches"]
        self.dx_pin = torch.empty((T, d), dtype=torch.int16).pin_memory()
        self.h2d = 2 * T * d * 2
        self.d2h = T * d * 2
        peak = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
        self.dominant = {"mlp_block_graph": (f"CUDA graph of {st['launches']} kernels ({st['instrs']} fused instructions, {st['steps']} plan steps)",
                                             self.work_per_step, "tensor", peak, "TFLOP/s")}
        self.dominant_key = "mlp_block_graph"
        self.peak_note = "sustained cuBLAS bf16 figure (multi-millisecond step under the power cap)"

    def step(self, record=None):
        if record is None:
            self.ex.run()
            return
        st = self.torch.cuda.current_stream()
        e0, e1 = _events(self.torch)
        e0.record(st); self.ex.run(); e1.record(st)
        record.append(("mlp_block_graph", e0, e1))

    def step_e2e(self):
        torch = self.torch
        self.ins[0].view(torch.int16).copy_(self.pins["X"], non_blocking=True)
        self.ins[5].view(torch.int16).copy_(self.pins["dO"], non_blocking=True)
        self.ex.run()
        self.dx_pin.copy_(self.outs[1].view(torch.int16), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    cpu_sample = staticmethod(lambda steps=1, warmup=1: WorkloadC4.cpu_sample(steps, warmup))


class WorkloadGemmF8(WorkloadGemm):
    """The same product requested as MulF8AccumF32 (E4M3 x E4M3): bf16 operands in HBM, rounded once per launch into
    8-bit copies (two extra launches inside the timed step), tcgen05 kind::f8f6f4."""
    key = "gemm8"
    dtype = "e4m3 x e4m3 -> f32 accumulate (bf16 operands rounded to 8 bits inside the step)"
    description = "plain matmul 8192^3, bf16 operands, MulF8AccumF32 { E4M3, E4M3 }, bf16 output"
    launches_per_step = 3
    peak_factor = 2.0
    peak_note = "no measured 8-bit peak on this pool: twice the measured bf16 burst figure (the nominal ratio)"

    @staticmethod
    def precision():
        from helium_b200 import ir
        return ir.prec_f8(ir.PREC_F8_F32, ir.F8_E4M3, ir.F8_E4M3)


class WorkloadPointwise:
    """Stand-alone pointwise programs on tensors larger than L2 (the P1 row of the hot path): three short dense
    programs served by hand-written kernels, two longer programs served by kernels specialised at plan time (one
    with a row-vector broadcast), and the first of those again on the register-program interpreter."""
    key = "pw"
    metric, unit = "pointwise_hbm_gbs", "GB/s"
    dtype = "bf16 / f32 storage, f32 arithmetic"
    N = 8192 * 8192
    description = ("stand-alone pointwise programs on 64 Mi-element tensors: relu(a)*m (bf16), a+b (f32), w-0.01*g (f32) on the dense "
                   "elementwise kernels; gelu(a+b)*c (bf16) and tanh(x+bias[col]) (f32, [8192,8192]) on plan-time specialised kernels; "
                   "gelu(a+b)*c once more on the interpreter")
    l2_note = "every tensor is 128 MiB (bf16) or 256 MiB (f32): larger than L2"
    work_scale = 1e9

    def __init__(self, ctx, dev, world, rank, peaks, reducer):
        import torch
        import helium_b200 as hb
        from helium_b200 import ir
        self.torch = torch
        n = self.N
        td = {ir.BF16: torch.bfloat16, ir.F32: torch.float32}
        gen = torch.Generator(device=dev).manual_seed(6)

        def case(name, dts, build, shapes=None, interpreter=False):
            g = ir.Graph()
            shapes = shapes or [[n]] * len(dts)
            ins = [g.new_input(list(sh), d) for sh, d in zip(shapes, dts)]
            g.new_output(build(g, ins))
            saved = os.environ.get("HE_PW_JIT")
            if interpreter:
                os.environ["HE_PW_JIT"] = "0"     # read when the plan is made
            try:
                plan = hb.Plan.pointwise(ctx, g)
            finally:
                if interpreter:
                    if saved is None:
                        del os.environ["HE_PW_JIT"]
                    else:
                        os.environ["HE_PW_JIT"] = saved
            tin = [torch.randn(*sh, generator=gen, device=dev).to(td[d]) for sh, d in zip(shapes, dts)]
            tout = plan.alloc_outputs(dev)
            nbytes = sum(t.numel() * t.element_size() for t in tin + tout)
            return name, plan, tin, tout, nbytes

        self.cases = [
            case("relu_mul_bf16", [ir.BF16, ir.BF16], lambda g, i: g.binary(ir.BIN_MUL, g.unary(ir.UN_RELU, i[0]), i[1])),
            case("add_f32", [ir.F32, ir.F32], lambda g, i: g.binary(ir.BIN_ADD, i[0], i[1])),
            case("sgd_f32", [ir.F32, ir.F32], lambda g, i: g.binary(ir.BIN_ADD, i[0], g.unary(ir.UN_NEG, g.binary(ir.BIN_MUL, i[1], g.constant(0.01, [n]))))),
            case("gelu_add_mul_bf16_specialised", [ir.BF16, ir.BF16, ir.BF16],
                 lambda g, i: g.binary(ir.BIN_MUL, g.unary(ir.UN_GELU, g.binary(ir.BIN_ADD, i[0], i[1])), i[2])),
            case("bias_tanh_f32_specialised", [ir.F32, ir.F32],
                 lambda g, i: g.unary(ir.UN_TANH, g.binary(ir.BIN_ADD, i[0], g.broadcast_to(i[1], [8192, 8192]))), shapes=[[8192, 8192], [8192]]),
            case("gelu_add_mul_bf16_interpreter", [ir.BF16, ir.BF16, ir.BF16],
                 lambda g, i: g.binary(ir.BIN_MUL, g.unary(ir.UN_GELU, g.binary(ir.BIN_ADD, i[0], i[1])), i[2]), interpreter=True),
            case("sum_sq_diff_f32_specialised", [ir.F32, ir.F32],
                 lambda g, i: g.reduce(ir.RED_SUM, g.unary(ir.UN_POW_CONST, g.binary(ir.BIN_SUB, i[0], i[1]), 2.0), 1)),
            case("sum_sq_diff_f32_interpreter", [ir.F32, ir.F32],
                 lambda g, i: g.reduce(ir.RED_SUM, g.unary(ir.UN_POW_CONST, g.binary(ir.BIN_SUB, i[0], i[1]), 2.0), 1), interpreter=True),
        ]
        # the allocation-free trailing-dims Sum (he_reduce_sum_f32_noalloc): 16 groups of 4 Mi f32 elements
        from helium_b200._lib import check, lib as _lib
        self._lib, self._check = _lib, check
        self.red_in = torch.randn(16 * (1 << 22), generator=gen, device=dev)
        self.red_out = torch.empty(16, dtype=torch.float32, device=dev)
        self.red_bytes = self.red_in.numel() * 4
        self.work_per_step = float(sum(c[4] for c in self.cases)) + self.red_bytes
        n_launch = 0
        for _, plan, tin, tout, _ in self.cases:     # one untimed launch each: the plans report how many kernels they enqueue
            plan.launch(tin, tout)
            n_launch += plan.last_launch_count
        self.launches_per_step = n_launch + 2
        self.dominant = {c[0]: (c[1].description, c[4], "hbm", peaks["hbm_gbs"], "GB/s") for c in self.cases}
        self.dominant["reduce_sum_noalloc_f32"] = ("he_reduce_sum_f32_noalloc on [16, 4 Mi] f32", self.red_bytes, "hbm", peaks["hbm_gbs"], "GB/s")
        self.dominant_key = "relu_mul_bf16"
        self.e2e_work_per_step = float(self.cases[0][4])   # the end-to-end leg runs the first program only
        self.pin_in = self.cases[0][2][0].cpu().pin_memory(); self.pin_m = self.cases[0][2][1].cpu().pin_memory()
        self.pin_out = torch.empty_like(self.pin_in).pin_memory()
        self.h2d = 2 * self.pin_in.numel() * 2
        self.d2h = self.pin_in.numel() * 2

    def step(self, record=None):
        st = self.torch.cuda.current_stream()
        for name, plan, tin, tout, _ in self.cases:
            if record is None:
                plan.launch(tin, tout)
            else:
                e0, e1 = _events(self.torch)
                e0.record(st); plan.launch(tin, tout); e1.record(st)
                record.append((name, e0, e1))
        import ctypes as C
        call = lambda: self._check(self._lib.he_reduce_sum_f32_noalloc(self.red_in.data_ptr(), self.red_out.data_ptr(), 16, 1 << 22,
                                                                        C.c_void_p(st.cuda_stream)))
        if record is None:
            call()
        else:
            e0, e1 = _events(self.torch)
            e0.record(st); call(); e1.record(st)
            record.append(("reduce_sum_noalloc_f32", e0, e1))

    def step_e2e(self):
        # the first program only, fed from and read back to pinned host memory
        name, plan, tin, tout, _ = self.cases[0]
        tin[0].copy_(self.pin_in, non_blocking=True); tin[1].copy_(self.pin_m, non_blocking=True)
        plan.launch(tin, tout)
        self.pin_out.copy_(tout[0], non_blocking=True)
        self.torch.cuda.current_stream().synchronize()

    @staticmethod
    def cpu_sample(steps=1, warmup=1):
        cfg = host_configs()
        from oracle import oracle as O
        n = 1 << 22
        r = cfg.rng(6)
        a, m = cfg.bf16_normal(r, (n,)), cfg.bf16_normal(r, (n,))
        run = lambda: O.encode(np.maximum(O.decode(a, O.BF16, (n,)), 0) * O.decode(m, O.BF16, (n,)), O.BF16)
        for _ in range(warmup):
            run()
        t0 = time.perf_counter()
        for _ in range(steps):
            run()
        dt = (time.perf_counter() - t0) / steps
        return 3 * n * 2 / dt / 1e9, 1, f"{steps} timed steps of relu(a)*m on {n} bf16 elements with the numpy oracle (single thread)", dt


class WorkloadC1:
    key = "c1"
    metric, unit = "train_steps_per_s", "step/s"
    dtype = "f32 (SIMT FFMA products, f32 accumulate)"
    description = ("configs[0]: MLP 784->512->10 training step, batch 256, f32: forward, softmax cross-entropy, backward, SGD lr 0.01; "
                   "the whole op graph planned (fusion + steps) by the C++ host runtime and replayed as one CUDA graph")
    l2_note = "working set 4.1 MB is L2-resident by construction (weights are re-read every step, as in training)"
    work_per_step = 1.0
    work_scale = 1.0
    COMPULSORY_BYTES = 4.1e6

    def __init__(self, ctx, dev, world, rank, peaks, reducer):
        import torch
        import helium_b200 as hb
        from helium_b200 import configs
        self.torch = torch
        g = configs.graph_mlp_train_step()
        ins = configs.mlp_inputs()
        self.x_pin = torch.from_numpy(ins[0]).pin_memory(); self.t_pin = torch.from_numpy(ins[1]).pin_memory()
        self.x_d, self.t_d = self.x_pin.to(dev), self.t_pin.to(dev)
        w_a = [torch.from_numpy(a).to(dev) for a in ins[2:]]
        w_b = [torch.empty_like(w) for w in w_a]
        self.loss_d = torch.zeros(1, dtype=torch.float32, device=dev)
        self.loss_pin = torch.zeros(1, dtype=torch.float32).pin_memory()
        hg = hb.HostGraph(g)
        # two executors that ping-pong the parameters, so consecutive steps really train: A reads w_a and
        # writes w_b, B reads w_b and writes w_a
        self.ex = [hb.Executor(ctx, hg, [self.x_d, self.t_d] + w_a, [self.loss_d] + w_b, capture=True),
                   hb.Executor(ctx, hg, [self.x_d, self.t_d] + w_b, [self.loss_d] + w_a, capture=True)]
        self._keep = (hg, w_a, w_b)
        self.parity = 0
        st = self.ex[0].stats()
        self.launches_per_step = st["launches"]
        self.plan_stats = st
        self.h2d = self.x_pin.numel() * 4 + self.t_pin.numel() * 4
        self.d2h = 4
        self.dominant = {"mlp_step_graph": (f"CUDA graph of {st['launches']} kernels ({st['instrs']} fused instructions, {st['steps']} plan steps)",
                                            self.COMPULSORY_BYTES, "hbm", peaks["hbm_gbs"], "GB/s")}
        self.dominant_key = "mlp_step_graph"

    def step(self, record=None):
        ex = self.ex[self.parity]
        self.parity ^= 1
        if record is None:
            ex.run()
            return
        st = self.torch.cuda.current_stream()
        e0, e1 = _events(self.torch)
        e0.record(st); ex.run(); e1.record(st)
        record.append(("mlp_step_graph", e0, e1))

    e2e_note = "one stream, no host synchronisation between steps: batch upload, graph replay and loss download are queued back to back"

    def step_e2e(self):
        # every step uploads its batch and downloads its loss; the host does not wait in between
        # (a training loop reads the loss of step i while step i+1 is already queued)
        self.x_d.copy_(self.x_pin, non_blocking=True); self.t_d.copy_(self.t_pin, non_blocking=True)
        self.step()
        self.loss_pin.copy_(self.loss_d, non_blocking=True)

    @staticmethod
    def cpu_sample(steps=20, warmup=1):
        cfg = host_configs()
        from oracle import oracle as O
        g = cfg.graph_mlp_train_step()
        ins = cfg.mlp_inputs()
        for _ in range(max(1, warmup)):
            O.evaluate(g, ins)
        t0 = time.perf_counter()
        for _ in range(steps):
            O.evaluate(g, ins)
        dt = (time.perf_counter() - t0) / steps
        try:
            from threadpoolctl import threadpool_info
            cores = max([i.get("num_threads", 1) for i in threadpool_info()] or [1])
        except Exception:
            cores = 1
        return 1.0 / dt, cores, f"{steps} timed steps of the numpy f64 restatement (oracle/oracle.py) of the same op graph; the reference's CPU backend is a stub", dt


class WorkloadC5:
    """configs[4]: one training step of the convolutional network of resnet-train (the model the reference trains on
    ImageNet; the benchmark list calls it ResNet-50, the reference contains no 50-layer network), batch 128 per GPU of synthetic
    3 x 224 x 224 images, 1000 classes, bf16 activations / f32 master weights, SGD with helium's momentum 0.9."""
    key = "c5"
    metric, unit = "train_steps_per_s", "step/s"
    dtype = "bf16 x bf16 -> f32 accumulate (implicit-GEMM convolutions), f32 master weights"
    BATCH, HW, CLASSES = 128, 224, 1000
    description = ("configs[4]: resnet-train network (7x7/2 head, 4 x (downsample block + basic block), bn/relu, 1x1 to 1000 classes), "
                   "training step forward + backward + SGD momentum 0.9, batch 128 per GPU of synthetic 3x224x224 images, bf16 compute, f32 "
                   "master weights; implicit-GEMM convolutions with bias / residual / batch-statistics epilogues; the step's launches are "
                   "replayed from three CUDA graphs (forward, backward, optimiser)")
    l2_note = "activations of one step (several GB) exceed L2; every step re-reads them"
    work_per_step = 1.0
    work_scale = 1.0

    def __init__(self, ctx, dev, world, rank, peaks, reducer):
        import torch
        from helium_b200 import convnet
        self.torch, self.reducer = torch, reducer
        self.net = convnet.ConvNet(ctx, self.BATCH, self.HW, self.CLASSES, dev)
        self.net.load_params(convnet.init_params(4, self.CLASSES))
        bits, labels = convnet.synthetic_batch(self.BATCH, self.HW, self.CLASSES, seed=4, shard=rank)
        self.x_pin = torch.from_numpy(bits.view(np.int16)).pin_memory()
        self.l_pin = torch.from_numpy(labels).pin_memory()
        self.loss_pin = torch.zeros(self.BATCH, dtype=torch.float32).pin_memory()
        self.net.acts["x0"].view(torch.int16).copy_(self.x_pin)
        self.net.labels.copy_(self.l_pin)
        self.h2d = self.x_pin.numel() * 2 + self.l_pin.numel() * 4
        self.d2h = self.BATCH * 4
        self.net.step(0.01, self.reducer)
        self.launches_per_step = self.net.launches
        flops = 3.0 * convnet.flops_per_image(self.HW, self.CLASSES) * self.BATCH
        peak = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
        self.dominant = {"step": (f"whole step: {self.launches_per_step} launches, {flops / 1e12:.3f} TFLOP of convolution math "
                                  "(forward + data and filter gradients)", flops, "tensor", peak, "TFLOP/s"),
                         "forward": ("forward pass", flops / 3, "tensor", peak, "TFLOP/s"),
                         "backward": ("backward pass", 2 * flops / 3, "tensor", peak, "TFLOP/s")}
        self.dominant_key = "step"
        self.peak_note = "sustained cuBLAS bf16 figure; the step is a mix of tensor-core and HBM-bound kernels, so the fraction is informational"

    def step(self, record=None):
        net, torch = self.net, self.torch
        if record is None:
            net.step(0.01, self.reducer, graph=True)   # replayed from CUDA graphs after the first (eager) step
            return
        st = torch.cuda.current_stream()
        e = {}
        def mark(tag):
            e[tag] = torch.cuda.Event(enable_timing=True)
            e[tag].record(st)
        net.step(0.01, self.reducer, graph=True, mark=mark)
        record.append(("forward", e["start"], e["forward"])); record.append(("backward", e["forward"], e["backward"]))
        record.append(("step", e["start"], e["end"]))

    e2e_note = "one stream: image upload, step, loss download queued back to back without host synchronisation"

    def step_e2e(self):
        torch = self.torch
        self.net.acts["x0"].view(torch.int16).copy_(self.x_pin, non_blocking=True)
        self.net.labels.copy_(self.l_pin, non_blocking=True)
        self.net.step(0.01, self.reducer, graph=True)
        self.loss_pin.copy_(self.net.loss, non_blocking=True)

    @staticmethod
    def cpu_sample(steps=1, warmup=0):
        """The float64 torch restatement of the same step on 2 images per timed step, scaled linearly to 128."""
        import torch
        from oracle import convnet_torch as CT
        # parameters / images without the package (its initialiser would load the CUDA library)
        r = np.random.Generator(np.random.Philox(4))
        names = CT.parameter_shapes(WorkloadC5.CLASSES)
        params = {}
        for n, shape in names:
            if n.endswith(".w"):
                params[n] = (r.standard_normal(shape, dtype=np.float32) / np.float32(np.sqrt(shape[0] * shape[1] * shape[2]))).astype(np.float32)
            elif n.endswith(".g"):
                params[n] = np.ones(shape, dtype=np.float32)
            else:
                params[n] = np.zeros(shape, dtype=np.float32)
        n_img = 2
        img = r.standard_normal((n_img, WorkloadC5.HW, WorkloadC5.HW, 3), dtype=np.float32)
        bits = (img.view(np.uint32) >> 16).astype(np.uint16)
        labels = r.integers(0, WorkloadC5.CLASSES, size=n_img).astype(np.int32)
        for _ in range(warmup):
            CT.training_step(params, bits, labels, WorkloadC5.CLASSES, 0.01, 0.9, None)
        t0 = time.perf_counter()
        for _ in range(steps):
            CT.training_step(params, bits, labels, WorkloadC5.CLASSES, 0.01, 0.9, None)
        dt = (time.perf_counter() - t0) / steps * (WorkloadC5.BATCH / n_img)
        return 1.0 / dt, torch.get_num_threads(), \
            (f"{steps} timed steps of the float64 torch restatement (oracle/convnet_torch.py) on {n_img} images each, scaled linearly to "
             "a batch of 128; the reference's CPU backend is a stub"), dt


class WorkloadC3Fused(WorkloadC3):
    """configs[2] with the relu(A) * M rewrite forced into the GEMM's mainloop (one kernel plus the fold of its
    reductions), where the planner on its own materialises the operand first at this size."""
    key = "c3f"
    description = WorkloadC3.description + "; in-kernel mainloop rewrite forced (HE_GEMM_MAINLOOP=fused)"

    def __init__(self, *a, **kw):
        prev = os.environ.get("HE_GEMM_MAINLOOP")
        os.environ["HE_GEMM_MAINLOOP"] = "fused"      # read at plan time
        try:
            super().__init__(*a, **kw)
        finally:
            if prev is None:
                os.environ.pop("HE_GEMM_MAINLOOP", None)
            else:
                os.environ["HE_GEMM_MAINLOOP"] = prev


WORKLOADS = {w.key: w for w in (WorkloadC1, WorkloadC2, WorkloadC3, WorkloadC3Fused, WorkloadC4, WorkloadC4Graph, WorkloadC5, WorkloadGemm,
                                WorkloadGemmF8, WorkloadPointwise)}
DEFAULT_STEPS = {"c1": 2000, "c2": 200, "c3": 200, "c3f": 200, "c4": 30, "c4g": 30, "c5": 10, "gemm": 100, "gemm8": 100, "pw": 50}
# what the default N = 1 run times beside its own workload, and the steps each gets
SUB_RECORDS = (("configs[2] fused matmul 4096^3 (as planned)", "c3", 100), ("configs[2] with the in-kernel mainloop rewrite", "c3f", 100),
               ("configs[1] pointwise + permute", "c2", 100), ("configs[0] MLP training step f32", "c1", 1000),
               ("configs[4] conv-net training step", "c5", 10),
               ("plain matmul 8192^3 requested as MulF8AccumF32 (8-bit copies, tcgen05 kind::f8f6f4)", "gemm8", 30),
               ("stand-alone pointwise programs on 64 Mi-element tensors", "pw", 30))


def config_for(key: str, world: int) -> dict:
    """The `config` object of the JSON line: a function of the workload and the rank count only, so that the
    product arm and `--impl reference` print the same one."""
    wl = WORKLOADS[key]
    config = {"workload": wl.description, "l2": wl.l2_note}
    if os.environ.get("HE_PLANNER"):
        config["planner"] = os.environ["HE_PLANNER"]
    if key == "c5":
        config.update({"images_per_gpu": wl.BATCH, "sharding": "batch",
                       "grad_allreduce": "NCCL mean through he_allreduce_grads, 2 buckets (filters bf16, vectors f32) after the backward pass; "
                                         "batch-norm statistics stay per GPU" if world > 1 else "none (1 rank)"})
    elif key == "c4":
        n_grads = 2 * wl.D * wl.FF * 2 + (wl.FF + wl.D) * 4
        config.update({"tokens_per_gpu": wl.TOKENS, "sharding": "tokens",
                       "grad_allreduce": "NCCL mean through he_allreduce_grads, 3 buckets (dW1, dW2, biases), overlapped with the "
                                         "remaining backward GEMMs" if world > 1 else "none (1 rank)",
                       "allreduce_bytes_per_step": n_grads if world > 1 else 0})
    else:
        config["replicas"] = world
    return config


def _use_all_host_threads():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to every rank; the CPU legs run on one rank only and
    are meant to use every host core the process may run on, so undo that before the OpenMP library loads."""
    if os.environ.get("OMP_NUM_THREADS") == "1" and "TORCHELASTIC_RUN_ID" in os.environ:
        try:
            os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
        except AttributeError:
            os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)


def run_reference_arm(args):
    """`--impl reference`: the reference is Rust + run-time generated CUDA, has no CPU implementation of
    this path and cannot be built in this image, so the arm times the CPU restatement of the same work
    (oracle/) on all host cores.  Every one of the `--steps` timed steps (after `--warmup` untimed ones) is a
    bounded sample of the workload (the `sample` text says which), scaled to a full step.  Neither the CUDA
    library nor the package initialiser is loaded."""
    _use_all_host_threads()
    wl = WORKLOADS[args.workload]
    value, cores, sample, dt = wl.cpu_sample(max(1, args.steps), max(0, args.warmup))
    line = {"impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": max(1, args.steps), "warmup": max(0, args.warmup), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": config_for(args.workload, args.gpus),
            "cpu_baseline": {"value": value, "unit": wl.unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    assert not any("libhelium_b200" in ln for ln in open("/proc/self/maps")), "the reference arm must not map the CUDA library"
    print(json.dumps(line))


def measure(wl, key, steps, warmup, world, dev, barrier, brief, peaks, busy_s=0.6):
    """Times one workload: `warmup` untimed steps, a short busy loop (so that clock samples cover the timed
    region), `steps` timed steps between CUDA events bracketed by barrier + synchronize, then the end-to-end
    leg from pinned host buffers.  Returns the fields of a JSON record (without clocks / cpu_baseline)."""
    import torch
    import torch.distributed as dist
    barrier()
    t_warm = time.perf_counter()
    for _ in range(warmup):
        wl.step()
    barrier()
    # Keep the device busy for ~busy_s more, so that the clock samples cover the timed region.  The number of
    # steps must be the SAME on every rank (a step of a sharded workload contains collectives: a rank that ran one
    # step more than its peer would wait for ever), so it is derived from the slowest rank's warm-up time and
    # agreed on before the loop, not from each rank's own clock inside it.
    per_step = (time.perf_counter() - t_warm) / max(1, warmup)
    if world > 1:
        t = torch.tensor([per_step], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        per_step = float(t.item())
    n_busy = 0 if brief else int(min(200, max(1, busy_s / max(per_step, 1e-6))))
    for _ in range(n_busy):
        wl.step()
    torch.cuda.synchronize()
    records = []
    t_start = torch.cuda.Event(enable_timing=True); t_end = torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record()
    for _ in range(steps):
        wl.step(records)
    t_end.record()
    barrier()
    elapsed_ms = t_start.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / steps
    per_kernel = {}
    for name, a, b in records:
        per_kernel.setdefault(name, []).append(a.elapsed_time(b))
    kernel_ms = {k: statistics.mean(v) for k, v in per_kernel.items()}

    # ---- end-to-end leg: host buffers in, host buffers out, copies inside the timed region ----------
    e2e_steps = {"c1": min(steps, 500), "c2": max(3, min(steps, 40))}.get(key, max(3, min(steps, 10)))
    if brief:
        e2e_steps = 0
    for _ in range(2 if e2e_steps else 0):
        wl.step_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        wl.step_e2e()
    barrier()
    e2e_sec = (time.perf_counter() - t0) / e2e_steps if e2e_steps else float("nan")
    if world > 1:
        t = torch.tensor([e2e_sec], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_sec = float(t.item())

    to_value = lambda sec: wl.work_per_step * world / sec / wl.work_scale
    dom_key = wl.dominant_key or max(kernel_ms, key=kernel_ms.get)
    name, work, bound, peak, punit = wl.dominant[dom_key]
    k_ms = kernel_ms[dom_key]
    achieved = work / (k_ms * 1e-3) / (1e9 if bound == "hbm" else 1e12)
    traffic = load_traffic(dom_key)
    roofline = {"bound": bound, "kernel": name, "achieved": achieved, "peak": peak, "unit": punit, "frac": achieved / peak,
                "peak_source": peaks["source"] + (": " + wl.peak_note if hasattr(wl, "peak_note") else ""),
                "kernel_ms": k_ms, "traffic": traffic, "traffic_source": TRAFFIC_SOURCE if traffic is not None else None}
    if len(kernel_ms) > 1:
        roofline["kernels"] = {}
        for k, ms in kernel_ms.items():
            _, w_k, b_k, p_k, _ = wl.dominant[k]
            a_k = w_k / (ms * 1e-3) / (1e9 if b_k == "hbm" else 1e12)
            roofline["kernels"][k] = {"ms": ms, "achieved": a_k, "frac": a_k / p_k, "share_of_step": ms / ms_per_step}
    rec = {
        "metric": wl.metric, "value": to_value(ms_per_step * 1e-3), "unit": wl.unit, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic", "config": config_for(key, world), "roofline": roofline,
        "e2e": None if brief else {"value": getattr(wl, "e2e_work_per_step", wl.work_per_step) * world / e2e_sec / wl.work_scale,
                                   "unit": wl.unit, "h2d_bytes_per_step": wl.h2d,
                                   "d2h_bytes_per_step": wl.d2h, "ms_per_step": e2e_sec * 1e3, "steps": e2e_steps,
                                   "pipelining": getattr(wl, "e2e_note", "one stream: upload, kernels, download in order")},
        "gpu_launches": wl.launches_per_step * steps,
    }
    return rec


def _parse_cpulist(text: str):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_to_gpu_numa_node(torch, local_rank: int, sysfs: str = "/sys"):
    """With several ranks on one host every rank stages its inputs through pinned host memory; pages pinned on the
    other socket cross the inter-socket link on every copy.  Before any pinned buffer exists the process is moved
    to the CPUs of the NUMA node its GPU hangs off (first touch then places the buffers there).  Nothing happens
    when the host shows one node, the GPU's node is unknown, or those CPUs are outside the process's CPU set.
    Returns a note for the bench line, or None."""
    try:
        nodes = [d for d in os.listdir(os.path.join(sysfs, "devices/system/node")) if d.startswith("node") and d[4:].isdigit()]
        if len(nodes) < 2:
            return None
        pr = torch.cuda.get_device_properties(local_rank)
        addr = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        with open(os.path.join(sysfs, "bus/pci/devices", addr, "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            cpus = _parse_cpulist(f.read()) & os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return f"rank bound to the {len(cpus)} CPUs of NUMA node {node} (GPU {addr}) before pinned buffers were allocated"
    except (OSError, ValueError, AttributeError):
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub", action="store_true", help="default workload at N = 1: do not time the other configurations as well")
    ap.add_argument("--reducer", default="comm", choices=["comm", "torch"],
                    help="gradient exchange of c4 at N > 1: the library's communicator (he_allreduce_grads) or torch.distributed")
    ap.add_argument("--nccl-ctas", type=int, default=NCCL_CTAS_DEFAULT,
                    help="c4 at N > 1: CTAs the gradient all-reduce may occupy (ncclConfig maxCTAs); the two GEMMs it overlaps are "
                         "planned for that many fewer SMs.  0 = NCCL's default and full-device GEMM grids")
    ap.add_argument("--planner", default=None, choices=["pairwise", "search"],
                    help="c1 / c4g (whole graphs through the host runtime): how instructions are formed, the reference's pairwise "
                         "merging (default) or the fusion search")
    ap.add_argument("--brief", action="store_true",
                    help="profiler captures only: no busy loop before the timed region, no end-to-end leg, no CPU baseline "
                         "(the printed line is then not a bench value)")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = DEFAULT_STEPS[args.workload] if args.impl == "ours" else 20
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            run_reference_arm(args)
        return 0
    if args.warmup < 3:
        args.warmup = 3
    if args.planner:
        os.environ["HE_PLANNER"] = args.planner   # read by heh_graph_create

    import torch
    import torch.distributed as dist

    import helium_b200 as hb
    from helium_b200.grad_sync import CommReducer, GradReducer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: helium_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    numa_note = bind_to_gpu_numa_node(torch, local_rank) if world > 1 else None
    if world > 1:
        import datetime
        # a short collective timeout: a rank that falls out of step must end the run in minutes, not hold the GPUs
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=90))
    ctx = hb.Context(local_rank)
    peaks = load_peaks()
    dev = torch.device("cuda", local_rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    reducer, comm = None, None
    if world > 1 and args.workload in ("c4", "c5"):
        if args.reducer == "comm":
            def exchange(b: bytes) -> bytes:
                t = torch.tensor(list(b), dtype=torch.uint8, device=dev)
                dist.broadcast(t, src=0)
                return bytes(t.cpu().tolist())
            comm = hb.Comm(ctx, rank, world, exchange, max_ctas=args.nccl_ctas)
            reducer = CommReducer(comm)
        else:
            reducer = GradReducer()
    wl_kwargs = {"overlap_sms": args.nccl_ctas} if (world > 1 and args.workload == "c4") else {}
    wl = WORKLOADS[args.workload](ctx, dev, world, rank, peaks, reducer, **wl_kwargs)

    try:
        gpu_id = "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:
        gpu_id = str(local_rank)
    # nvidia-smi needs ~0.2 s to deliver its first sample, so it is started before the warm-up and
    # read until the last leg finishes; only samples taken while the GPU was busy are used
    sampler = ClockSampler(gpu_id)
    if rank == 0:
        sampler.start()
    line = measure(wl, args.workload, args.steps, args.warmup, world, dev, barrier, args.brief, peaks)
    ctx.poll()
    if numa_note:
        line["host_affinity"] = numa_note
    if comm is not None:
        comm.poll()
        line["config"]["nccl_max_ctas"] = args.nccl_ctas
        line["config"]["gemm_sms_reserved_under_allreduce"] = args.nccl_ctas
    elif reducer is not None:
        line["config"]["grad_allreduce"] = "NCCL mean through torch.distributed, 3 buckets, overlapped"
    if rank == 0 and not args.no_cpu_baseline and not args.brief and world == 1:
        value, cores, sample, _ = WORKLOADS[args.workload].cpu_sample(3, 1)
        line["cpu_baseline"] = {"value": value, "unit": wl.unit, "cores": cores, "kind": "port", "sample": sample}

    # ---- the other single-GPU configurations, timed in the same run ---------------------------------
    if world == 1 and args.workload == "c4" and not args.no_sub and not args.brief:
        del wl
        torch.cuda.empty_cache()
        subs = {}
        for label, key, sub_steps in SUB_RECORDS:
            sub = WORKLOADS[key](ctx, dev, 1, 0, peaks, None)
            rec = measure(sub, key, sub_steps, max(3, args.warmup), 1, dev, barrier, False, peaks, busy_s=0.3)
            ctx.poll()
            keep = {k: rec[k] for k in ("metric", "value", "unit", "steps", "ms_per_step", "dtype", "roofline", "e2e", "gpu_launches")}
            keep["workload"] = rec["config"]["workload"]
            if not args.no_cpu_baseline:
                value, cores, sample, _ = WORKLOADS[key].cpu_sample(2, 1)
                keep["cpu_baseline"] = {"value": value, "unit": rec["unit"], "cores": cores, "kind": "port", "sample": sample}
            subs[label] = keep
            line["gpu_launches"] += rec["gpu_launches"]
            del sub
            torch.cuda.empty_cache()
        line["configs"] = subs

    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        line["clocks"] = clocks
        if args.brief:
            line["note"] = "--brief run for a profiler capture: not a bench value"
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        if comm is not None:
            comm.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
