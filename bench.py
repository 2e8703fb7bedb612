#!/usr/bin/env python
"""Benchmark of the fused-kernel hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3] [--impl ours|reference]

Default workload = BASELINE.json configs[1] ("c2"): one step is
  (a) y = relu(x * s_c + b_c) on bf16 [64,256,56,56] NCHW written as NHWC, one fused kernel, and
  (b) the f32 permutation [4096,4096,8] -> axes (2,0,1),
on synthetic seeded inputs; the metric is algorithmic HBM bytes moved per second.
`--workload c3` times the fused 4096^3 GEMM of configs[2] (TFLOP/s).

Rank 0 prints exactly one JSON line.  With N > 1 (launched under torch.distributed.run) every rank
runs an independent replica of the step (the path has no cross-GPU dependency) and the whole-job
value is N x bytes / max-over-ranks time.
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

C2A_SHAPE = (64, 256, 56, 56)
C2B_SHAPE = (4096, 4096, 8)
C2A_BYTES = 2 * 64 * 256 * 56 * 56 * 2 + 2 * 256 * 4      # x in + y out (bf16) + s, b (f32)
C2B_BYTES = 2 * 4096 * 4096 * 8 * 4                       # in + out (f32)
C3_MNK = (4096, 4096, 4096)
C3_FLOPS = 2 * 4096 ** 3


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_traffic(name: str):
    """Per-launch DRAM traffic (bytes) of the dominant kernel from the committed ncu summary, or None."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        return json.load(open(path)).get(name)
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
def make_c2_inputs(seed=1):
    """Seeded synthetic inputs of configs[1] as host (numpy) storage arrays."""
    from helium_b200.configs import c2_inputs
    return c2_inputs(seed)


def run_reference_arm(args):
    """`--impl reference`: the reference has no CPU (or runnable GPU) implementation of this path here,
    so the arm times the C restatement of its kernels (oracle/oracle_c.c) on all host cores."""
    from oracle import oracle_c as OC
    x, s, b, p = make_c2_inputs()
    st = [4096, 1, 4096 * 4096]
    threads = OC.num_threads()
    for _ in range(max(1, min(args.warmup, 1))):
        OC.affine_relu_nchw_nhwc(x, s, b); OC.permute(p, st)
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        OC.affine_relu_nchw_nhwc(x, s, b)
        OC.permute(p, st)
    dt = (time.perf_counter() - t0) / steps
    val = (C2A_BYTES + C2B_BYTES) / dt / 1e9
    line = {"impl": "reference", "metric": "pointwise_permute_hbm_gbs", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16+f32 (bit moves, f32 fma)", "data": "synthetic",
            "config": {"workload": "configs[1]: affine+relu+NCHW->NHWC bf16 [64,256,56,56]; permute f32 [4096,4096,8] axes (2,0,1)"},
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port",
                             "sample": f"full configs[1] step, {steps} steps, C+OpenMP restatement (the reference has no CPU path)"},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "gemm"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            run_reference_arm(args)
        return 0
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    import helium_b200 as hb
    from helium_b200 import ir
    from helium_b200.configs import c3_inputs, graph_affine_relu_permute, graph_c3

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: helium_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = hb.Context(local_rank)
    peaks = load_peaks()
    dev = torch.device("cuda", local_rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.workload == "c2":
        x_h, s_h, b_h, p_h = make_c2_inputs()
        plan_a = hb.Plan.pointwise(ctx, graph_affine_relu_permute(*C2A_SHAPE))
        st = hb.permute_output_strides(list(C2B_SHAPE), [(1, 2), (0, 1)])
        plan_b = hb.Plan.permute(ctx, list(C2B_SHAPE), st, ir.F32)
        # pinned host buffers for the end-to-end leg
        x_pin = torch.from_numpy(x_h.view(np.int16)).pin_memory()
        p_pin = torch.from_numpy(p_h).pin_memory()
        s_pin = torch.from_numpy(s_h).pin_memory(); b_pin = torch.from_numpy(b_h).pin_memory()
        x_d = x_pin.to(dev).view(torch.bfloat16); s_d = s_pin.to(dev); b_d = b_pin.to(dev); p_d = p_pin.to(dev)
        y_d = torch.empty((64, 56, 56, 256), dtype=torch.bfloat16, device=dev)
        q_d = torch.empty((8, 4096, 4096), dtype=torch.float32, device=dev)
        y_pin = torch.empty((64, 56, 56, 256), dtype=torch.int16).pin_memory()
        q_pin = torch.empty((8, 4096, 4096), dtype=torch.float32).pin_memory()
        step_bytes = C2A_BYTES + C2B_BYTES
        stream = torch.cuda.current_stream()

        def step(record=None):
            plan_a.launch([x_d, s_d, b_d], [y_d])
            if record is not None:
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                plan_b.launch([p_d], [q_d])
                e1.record(stream)
                record.append((e0, e1))
            else:
                plan_b.launch([p_d], [q_d])

        def step_e2e():
            x_d.view(torch.int16).copy_(x_pin, non_blocking=True)
            s_d.copy_(s_pin, non_blocking=True); b_d.copy_(b_pin, non_blocking=True)
            p_d.copy_(p_pin, non_blocking=True)
            plan_a.launch([x_d, s_d, b_d], [y_d])
            plan_b.launch([p_d], [q_d])
            y_pin.copy_(y_d.view(torch.int16), non_blocking=True)
            q_pin.copy_(q_d, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        launches_per_step = 2
        h2d = x_pin.numel() * 2 + p_pin.numel() * 4 + 2 * 256 * 4
        d2h = y_pin.numel() * 2 + q_pin.numel() * 4
        metric, unit, dtype = "pointwise_permute_hbm_gbs", "GB/s", "bf16 (f32 fma) + f32 bit moves"
        workload = ("configs[1]: y=relu(x*s_c+b_c) bf16 [64,256,56,56] NCHW->NHWC fused in one kernel; "
                    "permute f32 [4096,4096,8] axes (2,0,1)")
        to_value = lambda sec_per_step: step_bytes * world / sec_per_step / 1e9
        dominant = ("permute_tile_vec<4> on [4096,4096,8] f32", C2B_BYTES, "hbm", peaks["hbm_gbs"], "GB/s", "permute_c2b")
        l2_note = "inputs exceed L2 (512 MiB permute input; the 103 MB pointwise input is evicted by the 1 GiB permute between its uses)"
    elif args.workload == "gemm":
        # plain bf16 matmul (the G0 contract): A [8192,8192] K-major, B [8192,8192] N-major, bf16 out
        from helium_b200.configs import graph_linear
        m = n = k = 8192
        g = graph_linear(m, n, k, bias=False)
        plan = hb.Plan.fused_matmul(ctx, g)
        gen = torch.Generator(device=dev).manual_seed(2)
        a_d = torch.randn((m, k), generator=gen, device=dev).to(torch.bfloat16)
        b_d = (torch.randn((k, n), generator=gen, device=dev) / 90.0).to(torch.bfloat16)
        a_pin = a_d.cpu().pin_memory(); b_pin = b_d.cpu().pin_memory()
        outs_d = plan.alloc_outputs(dev)
        out_pin = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        stream = torch.cuda.current_stream()
        plan_desc = plan.description

        def step(record=None):
            flush.zero_()
            if record is not None:
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                plan.launch([a_d, b_d], outs_d)
                e1.record(stream)
                record.append((e0, e1))
            else:
                plan.launch([a_d, b_d], outs_d)

        def step_e2e():
            a_d.copy_(a_pin, non_blocking=True); b_d.copy_(b_pin, non_blocking=True)
            plan.launch([a_d, b_d], outs_d)
            out_pin.copy_(outs_d[0], non_blocking=True)
            torch.cuda.current_stream().synchronize()

        launches_per_step = 1
        h2d = 2 * m * k * 2
        d2h = m * n * 2
        flops = 2.0 * m * n * k
        metric, unit, dtype = "gemm_tflops", "TFLOP/s", "bf16 x bf16 -> f32 accumulate"
        workload = "plain matmul 8192^3 bf16 (Op::Matmul contract, no fusion), bf16 output"
        to_value = lambda sec_per_step: flops * world / sec_per_step / 1e12
        dominant = (plan_desc, flops, "tensor", peaks["bf16_tflops"], "TFLOP/s", "gemm_plain")
        l2_note = "256 MiB buffer written between iterations to flush L2 (inside the timed region)"
    else:
        m, n, k = C3_MNK
        g = graph_c3(m, n, k, False)
        ins_h = c3_inputs(m, n, k, False)
        plan = hb.Plan.fused_matmul(ctx, g)
        pins = [torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).pin_memory() for a in ins_h]
        ins_d = [p.to(dev).view(torch.bfloat16) for p in pins]
        ins_d[5] = ins_d[1]  # the epilogue mask is the mainloop mask (k == n)
        outs_d = plan.alloc_outputs(dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        stream = torch.cuda.current_stream()

        def step(record=None):
            flush.zero_()  # operands fit L2 (201 MB vs 126 MB partly): evict between iterations
            if record is not None:
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                plan.launch(ins_d, outs_d)
                e1.record(stream)
                record.append((e0, e1))
            else:
                plan.launch(ins_d, outs_d)

        outs_pin = [torch.empty(o.shape, dtype=torch.int16 if o.dtype == torch.bfloat16 else torch.float32).pin_memory() for o in outs_d]

        def step_e2e():
            for d, p in zip(ins_d[:1] + ins_d[2:5] + ins_d[6:], pins[:1] + pins[2:5] + pins[6:]):
                d.view(torch.int16).copy_(p, non_blocking=True)
            ins_d[1].view(torch.int16).copy_(pins[1], non_blocking=True)
            plan.launch(ins_d, outs_d)
            for o, p in zip(outs_d, outs_pin):
                p.copy_(o.view(torch.int16) if o.dtype == torch.bfloat16 else o, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        launches_per_step = 4
        h2d = sum(p.numel() * 2 for i, p in enumerate(pins) if i != 5)
        d2h = sum(p.numel() * p.element_size() for p in outs_pin)
        metric, unit, dtype = "fused_gemm_tflops", "TFLOP/s", "bf16 x bf16 -> f32 accumulate, f32 epilogue"
        workload = ("configs[2]: fused matmul 4096^3 bf16, mainloop relu(A)*M, epilogue bias/relu/tanh/gate/MSE + "
                    "Sum over Batch and Columns + two backward tiles (README graph)")
        to_value = lambda sec_per_step: C3_FLOPS * world / sec_per_step / 1e12
        dominant = (plan.description, C3_FLOPS, "tensor", peaks["bf16_tflops"], "TFLOP/s", "gemm_c3")
        l2_note = "256 MiB buffer written between iterations to flush L2 (inside the timed region; its ~40 us are included)"

    # ---- warm-up, then the timed region ------------------------------------------------------------
    try:
        gpu_id = "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:
        gpu_id = str(local_rank)
    # nvidia-smi needs ~0.2 s to deliver its first sample, so it is started before the warm-up and
    # read until the end-to-end leg finishes; only samples taken while the GPU was busy are used
    sampler = ClockSampler(gpu_id)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    # keep the device busy long enough for the clock record to cover the measurement
    t_busy = time.perf_counter()
    while time.perf_counter() - t_busy < 0.6:
        step()
        torch.cuda.synchronize()
    records = []
    t_start = torch.cuda.Event(enable_timing=True); t_end = torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record()
    for _ in range(args.steps):
        step(records)
    t_end.record()
    barrier()
    elapsed_ms = t_start.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in records)
    ctx.poll()

    # ---- end-to-end leg: host buffers in, host buffers out, copies inside the timed region ----------
    for _ in range(2):
        step_e2e()
    barrier()
    e2e_steps = max(3, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    barrier()
    e2e_sec = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_sec], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_sec = float(t.item())

    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        name, work, bound, peak, punit, traffic_key = dominant
        achieved = work / (kernel_ms * 1e-3) / (1e9 if bound == "hbm" else 1e12)
        line = {
            "metric": metric, "value": to_value(ms_per_step * 1e-3), "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": dtype, "data": "synthetic",
            "config": {"workload": workload, "l2": l2_note, "replicas": world},
            "roofline": {"bound": bound, "kernel": name, "achieved": achieved, "peak": peak, "unit": punit, "frac": achieved / peak,
                         "peak_source": peaks["source"], "kernel_ms": kernel_ms, "traffic": load_traffic(traffic_key)},
            "e2e": {"value": to_value(e2e_sec), "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_sec * 1e3},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if args.workload == "c2" and not args.no_cpu_baseline:
            from oracle import oracle_c as OC
            x, s, b, p = x_h, s_h, b_h, p_h
            OC.affine_relu_nchw_nhwc(x, s, b)  # first call also builds / loads the C object
            reps = 3
            t0 = time.perf_counter()
            for _ in range(reps):
                OC.affine_relu_nchw_nhwc(x, s, b)
                OC.permute(p, [4096, 1, 4096 * 4096])
            cpu_sec = (time.perf_counter() - t0) / reps
            line["cpu_baseline"] = {"value": (C2A_BYTES + C2B_BYTES) / cpu_sec / 1e9, "unit": "GB/s", "cores": OC.num_threads(),
                                    "kind": "port", "sample": f"{reps} full configs[1] steps of the C+OpenMP restatement (oracle/oracle_c.c); the reference has no CPU path"}
        elif args.workload == "c3" and not args.no_cpu_baseline:
            from oracle import oracle_c as OC
            a, mk, bm = (np.ascontiguousarray(v).reshape(4096, 4096) for v in (ins_h[0], ins_h[1], ins_h[2]))
            rows = 256
            t0 = time.perf_counter()
            OC.gemm_bf16(a, bm, mk, 0, rows)
            cpu_sec = (time.perf_counter() - t0) * (4096 / rows)
            line["cpu_baseline"] = {"value": C3_FLOPS / cpu_sec / 1e12, "unit": "TFLOP/s", "cores": OC.num_threads(), "kind": "port",
                                    "sample": f"{rows} of 4096 output rows of the mainloop-fused GEMM, C+OpenMP restatement, scaled linearly"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
