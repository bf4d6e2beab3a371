#!/usr/bin/env python
"""Benchmark of the matmul / conv2d hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

Prints ONE JSON line.  The headline workload is the broadcast-rhs (Linear-layer) matmul of dfdx's
`MatMatBrKernel`: X[64,256,1024] f32 x W^T with W stored [4096,1024], forward + both gradients.  One "step" =
forward GEMM + grad_rhs GEMM + grad_lhs GEMM (three kernel launches, 412.3 GFLOP) on one batch of synthetic
input.  `value` is the whole-job logical TFLOP/s with inputs resident in HBM; `e2e` is the same metric through
`dfdx_b200.Cuda.matmul` + backward with the step's inputs copied from pinned host memory and the weight gradient
read back, inside the timed region.  With N > 1 (launched under torchrun) every rank runs its own 64-item batch
(weak scaling) and the weight gradient is all-reduced over NCCL each step, on a side stream under the grad_lhs
GEMM; `strong` in the same line holds the fixed problem partitioned over the N ranks.

The same line carries, under `configs`, the other configurations of the path (single 1024^3 matmul, rank-4
attention matmuls, conv2d, the attention matmuls through the fused kernels, the encoder training step), each a
few steps with its own roofline figures, and under `cublas_as_dfdx` the cuBLAS calls dfdx makes today on the
same shapes (through torch), measured beside them outside the timed regions.

`--workload c1|c3|c4|c5|attn` times one configuration alone (for profiling); `--headline-only` skips the
`configs`, `strong` and cuBLAS legs.

`--impl reference` times the CPU stand-in of dfdx's `Cpu` device (oracle/cpu_baseline.c) on all host
threads over a bounded sub-batch per step.
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

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

B, S, K, N = 64, 256, 1024, 4096
FLOP_PER_ITEM = 6 * S * K * N              # fwd + two backward GEMMs for one batch item
FLOP_PER_STEP = B * FLOP_PER_ITEM          # 412.3 GFLOP
FLOP_PER_LAUNCH = FLOP_PER_STEP / 3.0      # each of the three GEMMs: 137.4 GFLOP
METRIC = "gemm_fwd_bwd_tflops"
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the headline workload from one ncu capture
# (forward 303.2 MB, grad_rhs 357.4 MB, grad_lhs 438.5 MB); it is not re-measured by a bench run.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 366.4e6
WORKLOAD = f"config[1]: MatMatBr f32 X[{B},{S},{K}] x W^T, W stored [{N},{K}], fwd + grad_lhs + grad_rhs"
MIB = 1024.0 * 1024.0
# SMs left to the NCCL kernel that runs beside the grad_lhs GEMM, and that kernel's CTA bound
OVERLAP_SMS = 8


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timed regions run."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []          # (host arrival time, csv line)

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()

    def summary(self, t0=None, t1=None):
        """Summary over the samples that arrived in [t0, t1] (all samples if that window caught none)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = list(self.lines)
        window = [ln for (t, ln) in lines if t0 is not None and t0 <= t <= t1 + 0.05]
        scope = "timed region"
        if not window:
            window, scope = [ln for (_, ln) in lines], "whole run (timed region shorter than one sample)"
        for ln in window:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "scope": scope,
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_baseline_run(items: int, repeats: int):
    """Times forward + backward of `items` batch items of the workload on the CPU port.  Returns
    (seconds per repeat, threads)."""
    import numpy as np
    from oracle import oracle
    oracle.build()
    L = oracle.baseline_lib()
    if not L.cpu_baseline_supported():
        raise RuntimeError("host CPU lacks AVX2/FMA")
    import ctypes as C
    rng = np.random.default_rng(0xD0FD + 2)
    x = rng.standard_normal((items, S, K), dtype=np.float32)
    w = ((rng.random((N, K), dtype=np.float32) * 2 - 1) / 32).astype(np.float32)
    dy = rng.standard_normal((items, S, N), dtype=np.float32)
    y = np.empty((items, S, N), dtype=np.float32)
    gx = np.zeros_like(x)
    gw = np.zeros_like(w)
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    st = lambda *v: (C.c_size_t * len(v))(*v)
    ls, rs = st(S * K, K, 1), st(1, K)         # weight consumed as the (K, N) view with strides [1, K]
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        L.cpu_matmat_br_forward(items, S, K, N, fp(x), ls, fp(w), rs, fp(y))
        L.cpu_matmat_br_backward(items, S, K, N, fp(x), ls, fp(gx), fp(w), rs, fp(gw), fp(dy))
        times.append(time.perf_counter() - t0)
    return times, int(L.cpu_baseline_threads())


def cpu_baseline_block():
    """Bounded (~10-20 s) CPU sample: one item first, then as many items as fit that time."""
    t1, threads = cpu_baseline_run(1, 1)
    items = max(1, min(B, int(12.0 / max(t1[0], 1e-3))))
    t, threads = cpu_baseline_run(items, 1)
    tflops = items * FLOP_PER_ITEM / t[0] / 1e12
    return {"value": round(tflops, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{items} of {B} batch items of the workload, fwd+bwd, {t[0]:.2f} s; "
                      "stand-in for dfdx's gemm-crate Cpu path (not buildable here)"}


def run_reference(args, rank: int):
    if rank != 0:
        return
    t1, threads = cpu_baseline_run(1, 1)
    items = max(1, min(B, int(4.0 / max(t1[0], 1e-3))))
    times, threads = cpu_baseline_run(items, args.warmup + args.steps)
    timed = times[args.warmup:]
    total = sum(timed)
    tflops = items * FLOP_PER_ITEM * len(timed) / total / 1e12
    sample = f"{items} of {B} batch items per step, fwd+bwd, CPU port of dfdx's Cpu path on {threads} threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(tflops, 4), "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * total / len(timed), 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": round(tflops, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(tflops, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------------ GPU harness
class Harness:
    """Device, ranks, timing with CUDA events on the launching stream (max over ranks), clocks."""

    def __init__(self, dev, rank, world, local_rank):
        import torch
        self.torch = torch
        self.dev, self.lib, self.device = dev, dev.lib, dev.device
        self.rank, self.world = rank, world
        self.stream = torch.cuda.current_stream(self.device)
        self.peaks, self.peaks_kind = measured_peaks()
        self.sampler = ClockSampler(local_rank)
        self.flush_buf = None
        self.tf32 = None                       # cuBLAS TF32 rates measured in this run (burst, sustained)

    def barrier(self):
        self.torch.cuda.synchronize(self.device)
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
            self.torch.cuda.synchronize(self.device)

    def max_over_ranks(self, ms: float) -> float:
        if self.world == 1:
            return ms
        import torch.distributed as dist
        t = self.torch.tensor([ms], device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def region(self, fn, steps, warmup):
        """`steps` back-to-back calls of fn between two events.  Returns a dict: ms (max over ranks), launches,
        tensor launches and the host-time window of the region."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0, t0 = self.lib.b200_launch_count(), self.lib.b200_tensor_launch_count()
        h0 = time.time()
        e0.record(self.stream)
        for _ in range(steps):
            fn()
        e1.record(self.stream)
        torch.cuda.synchronize(self.device)
        h1 = time.time()
        self.barrier()
        return {"ms": self.max_over_ranks(e0.elapsed_time(e1)), "launches": int(self.lib.b200_launch_count() - l0),
                "tc_launches": int(self.lib.b200_tensor_launch_count() - t0), "window": (h0, h1), "steps": steps}

    def region_for(self, fn, seconds, warmup):
        """The same, for at least `seconds` of device time (step count from a short probe; every rank uses rank 0's)."""
        probe = self.region(fn, 5, warmup)
        steps = max(5, int(seconds * 1e3 / max(probe["ms"] / 5, 1e-3)) + 1)
        return self.region(fn, steps, 0)

    def region_flushed(self, fn, steps, warmup):
        """Per-step events with a write larger than L2 between steps (for workloads whose data fits L2)."""
        torch = self.torch
        if self.flush_buf is None:
            self.flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=self.device)
        for _ in range(warmup):
            fn()
        self.barrier()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        l0, t0 = self.lib.b200_launch_count(), self.lib.b200_tensor_launch_count()
        h0 = time.time()
        for i in range(steps):
            self.flush_buf.fill_(i & 1)
            ev[i][0].record(self.stream)
            fn()
            ev[i][1].record(self.stream)
        torch.cuda.synchronize(self.device)
        h1 = time.time()
        self.barrier()
        ms = sum(a.elapsed_time(b) for a, b in ev)
        return {"ms": self.max_over_ranks(ms), "launches": int(self.lib.b200_launch_count() - l0),
                "tc_launches": int(self.lib.b200_tensor_launch_count() - t0), "window": (h0, h1), "steps": steps}

    def check_status(self, where):
        import dfdx_b200
        dfdx_b200._lib.check(self.dev.device_status(), f"device status after {where}")

    # -- roofline denominators -------------------------------------------------------------------
    def tensor_peak(self, kind: str, region_s: float):
        """(peak TFLOP/s, basis) for logical flops of `kind` ('f16' or 'f32' = 3xTF32).  A region shorter than a
        second runs at boost clocks and is held against the burst figure, a longer one against the sustained one."""
        burst = region_s < 1.0
        tag = "burst" if burst else "sustained"
        if kind == "f16":
            p = self.peaks["bf16_tflops"] if burst else self.peaks["bf16_tflops_sustained"]
            return p, f"{self.peaks_kind} bf16_tflops{'' if burst else '_sustained'} ({tag}; f16 runs at the bf16 rate)"
        half = (self.peaks["bf16_tflops"] if burst else self.peaks["bf16_tflops_sustained"]) / 2.0
        if self.tf32:
            t = self.tf32["burst"] if burst else self.tf32["sustained"]
            # the denominator is the larger of the two estimates of the dense tf32 rate, so that it never flatters
            rate, how = (t, f"cuBLAS TF32 8192^3 measured in this run ({tag})") if t >= half else \
                        (half, f"{self.peaks_kind} bf16 ({tag}) / 2, above this run's cuBLAS TF32 {t:.0f}")
        else:
            rate, how = half, f"{self.peaks_kind} bf16 ({tag}) / 2 (tf32 rate assumed)"
        return rate / 3.0, f"{how} / 3 (3xTF32: three tensor MACs per logical MAC)"

    def roofline(self, bound, kind, flops, algo_bytes, ms_per_unit, region_s, kernel=None, traffic=None):
        if bound == "hbm":
            achieved = algo_bytes / (ms_per_unit * 1e-3) / 1e9
            peak, unit, basis = self.peaks["hbm_gbs"], "GB/s", f"{self.peaks_kind} hbm_gbs (device copy)"
        else:
            achieved = flops / (ms_per_unit * 1e-3) / 1e12
            (peak, basis), unit = self.tensor_peak(kind, region_s), "TFLOP/s"
        out = {"bound": bound, "achieved": round(achieved, 2), "peak": round(peak, 2), "unit": unit,
               "frac": round(achieved / peak, 4), "traffic": traffic, "peak_basis": basis,
               "region_s": round(region_s, 4)}
        if kernel:
            out["kernel"] = kernel
        return out


# ------------------------------------------------------------------------------------------------ workloads
def make_c2(h, items=B, overlap=True, group=None, overlap_sms=OVERLAP_SMS):
    """The headline workload on `items` batch items.  Returns (step, tensors)."""
    import torch
    import dfdx_b200
    from dfdx_b200.parallel import OverlappedReducer, allreduce_shared_grads
    lib, device, st = h.lib, h.device, dfdx_b200._lib.strides
    g = torch.Generator(device="cpu").manual_seed(0xD0FD + 2 + 1000 * h.rank)
    x_h = torch.randn(items, S, K, generator=g, dtype=torch.float32).pin_memory()
    w_h = ((torch.rand(N, K, generator=g, dtype=torch.float32) * 2 - 1) / (K ** 0.5))
    dy_h = torch.randn(items, S, N, generator=g, dtype=torch.float32).pin_memory()
    x, w, dy = x_h.to(device), w_h.to(device), dy_h.to(device)
    w_view = w.permute(1, 0)                                  # Linear's zero-copy (K, N) view of (N, K)
    y = torch.empty(items, S, N, device=device)
    gx = torch.zeros(items * S * K, device=device)
    gw = torch.zeros(N * K, device=device)
    reducer = OverlappedReducer(device, group) if (h.world > 1 and overlap) else None
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    F32, check = dfdx_b200.F32, dfdx_b200._lib.check
    xs, ws = st(x.stride()), st(w_view.stride())

    def step():
        # `MatMatBrKernel::forward` + `::backward` through the C ABI on buffers already in HBM.  The shared weight's
        # gradient buffer starts from zero (dfdx zero-fills gradients, tensor/cuda/device.rs:259-266) and is summed
        # over ranks while the grad_lhs GEMM runs.
        s = h.stream.cuda_stream
        check(lib.b200_matmat_br_forward(F32, items, S, K, N, x.data_ptr(), xs, w_view.data_ptr(), ws, y.data_ptr(), s),
              "forward")
        gw.zero_()
        if reducer is None:
            check(lib.b200_matmat_br_backward(F32, items, S, K, N, x.data_ptr(), xs, gx.data_ptr(), w_view.data_ptr(),
                                              ws, gw.data_ptr(), dy.data_ptr(), s, None), "backward")
            if h.world > 1:
                allreduce_shared_grads([gw])
            return
        check(lib.b200_matmat_br_backward(F32, items, S, K, N, x.data_ptr(), xs, None, w_view.data_ptr(), ws,
                                          gw.data_ptr(), dy.data_ptr(), s, None), "backward (grad_rhs)")
        reducer.start([gw])
        lib.b200_set_max_ctas(sms - overlap_sms)
        try:
            check(lib.b200_matmat_br_backward(F32, items, S, K, N, x.data_ptr(), xs, gx.data_ptr(), w_view.data_ptr(),
                                              ws, None, dy.data_ptr(), s, None), "backward (grad_lhs)")
        finally:
            lib.b200_set_max_ctas(0)
        reducer.finish()

    return step, {"x_h": x_h, "dy_h": dy_h, "x": x, "dy": dy, "w_view": w_view, "gw": gw, "reducer": reducer}


def make_c2_e2e(h, t):
    """End-to-end step.  The inputs cross PCIe every step (320 MiB, about 6 ms) and that copy is longer than the
    GEMMs (about 2 ms), so the upload of step i+1 is issued on a copy stream into the other of two device
    buffer sets while step i computes; the weight gradient goes back on the compute stream."""
    import torch
    from dfdx_b200.parallel import allreduce_shared_grads
    dev, device, stream = h.dev, h.device, h.stream
    x_h, dy_h, w_view = t["x_h"], t["dy_h"], t["w_view"]
    gw_h = torch.empty(N * K, dtype=torch.float32).pin_memory()
    copy_stream = torch.cuda.Stream(device)
    sets = [{"x": torch.empty_like(t["x"]), "dy": torch.empty_like(t["dy"]),
             "ready": torch.cuda.Event(), "free": torch.cuda.Event()} for _ in range(2)]
    for st in sets:
        st["free"].record(stream)
    i = [0]

    def step():
        st = sets[i[0] & 1]
        i[0] += 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(st["free"])               # the step that last used this set has finished
            st["x"].copy_(x_h, non_blocking=True)
            st["dy"].copy_(dy_h, non_blocking=True)
            st["ready"].record(copy_stream)
        stream.wait_event(st["ready"])
        out, bwd = dev.matmul(st["x"], w_view)
        _, gw_view = bwd(st["dy"])
        gwb = gw_view.permute(1, 0)
        if h.world > 1:
            allreduce_shared_grads([gwb])
        st["free"].record(stream)
        gw_h.copy_(gwb.reshape(-1), non_blocking=True)

    return step, {"h2d": int(x_h.numel() * 4 + dy_h.numel() * 4), "d2h": int(gw_h.numel() * 4)}


def make_c1(h, rows=1024, strong=False, group=None):
    """Configuration 1: A[1024,1024] x B[1024,1024] f32, forward + both gradients.  `strong`: this rank holds
    `rows` rows of A / C / dC (the M-partition); the shared B's gradient is all-reduced."""
    import torch
    from dfdx_b200.parallel import allreduce_shared_grads
    import dfdx_b200
    device = h.device
    # dfdx's device carries a second stream on which the grad_lhs GEMM of every backward runs beside the grad_rhs GEMM
    # (matmul/cuda_kernel.rs:282-310); with GEMMs this small the two share the machine
    dev = dfdx_b200.Cuda(device.index, par_stream=True)
    g = torch.Generator(device="cpu").manual_seed(0xD0FD + 1 + 1000 * h.rank)
    a = (torch.rand(rows, 1024, generator=g) * 2 - 1).to(device)
    b = (torch.rand(1024, 1024, generator=g) * 2 - 1).to(device)
    dc = torch.randn(rows, 1024, generator=g).to(device)
    ga, gb = torch.zeros_like(a), torch.zeros_like(b)

    def step():
        dev.matmat_forward(a, b)
        dev.matmat_backward(a, ga, b, gb, dc)
        if strong and h.world > 1:
            allreduce_shared_grads([gb], group)

    return step


def make_c3(h):
    import torch
    dev, device = h.dev, h.device
    g = torch.Generator(device="cpu").manual_seed(0xD0FD + 3 + 1000 * h.rank)
    q, k, v = (torch.randn(16, 16, 512, 64, generator=g).half().to(device) for _ in range(3))
    kt = k.permute(0, 1, 3, 2)
    p = torch.softmax(torch.randn(16, 16, 512, 512, generator=g), -1).half().to(device)
    do = torch.randn(16, 16, 512, 64, generator=g).half().to(device)
    ds = torch.randn(16, 16, 512, 512, generator=g).half().to(device)
    gq, gk, gv, gp = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v), torch.zeros_like(p)

    def step():
        dev.matmat_batch4_forward(q, kt)                 # scores = Q K^T
        dev.matmat_batch4_forward(p, v)                  # out = P V   (softmax is not on the path)
        dev.matmat_batch4_backward(p, gp, v, gv, do)     # dP, dV
        dev.matmat_batch4_backward(q, gq, kt, gk, ds)    # dQ, dK
    return step


def make_attn(h):
    """Configuration 3's tensors through the fused kernels: softmax(Q K^T / sqrt(d)) V, forward + backward."""
    import torch
    dev, device = h.dev, h.device
    g = torch.Generator(device="cpu").manual_seed(0xD0FD + 9 + 1000 * h.rank)
    q = torch.randn(16, 512, 16, 64, generator=g).half().to(device).permute(0, 2, 1, 3)
    k = torch.randn(16, 512, 16, 64, generator=g).half().to(device).permute(0, 2, 3, 1)
    v = torch.randn(16, 512, 16, 64, generator=g).half().to(device).permute(0, 2, 1, 3)
    do = torch.randn(16, 512, 16, 64, generator=g).half().to(device).permute(0, 2, 1, 3)
    bufs = (dev.alloc_grad(q), dev.alloc_grad(k), dev.alloc_grad(v))

    def step():
        out, lse = dev.attention_forward(q, k, v, 0.125, want_lse=True)
        dev.attention_backward(q, k, v, 0.125, out, lse, do, accumulate_into=bufs)
    return step


def make_f16(h):
    """One f16 GEMM of 8192^3 (the shape the measured cuBLAS bf16 peak of this pool is quoted on)."""
    import torch
    dev, device = h.dev, h.device
    g = torch.Generator(device="cpu").manual_seed(0xD0FD + 16 + 1000 * h.rank)
    a = torch.randn(8192, 8192, generator=g).half().to(device)
    b = torch.randn(8192, 8192, generator=g).half().to(device)
    c = torch.empty(8192, 8192, dtype=torch.float16, device=device)

    def step():
        dev.gemm((8192, 8192, 8192), a, a.stride(), b, b.stride(), 0.0, c, c.stride())
    return step


def make_c4(h, group=None):
    import torch
    from dfdx_b200.parallel import allreduce_shared_grads
    dev, device = h.dev, h.device
    g = torch.Generator(device="cpu").manual_seed(0xD0FD + 4 + 1000 * h.rank)
    x = torch.randn(32, 64, 56, 56, generator=g).to(device)
    w = ((torch.rand(128, 64, 3, 3, generator=g) * 2 - 1) / 24.0).to(device)
    dy = torch.randn(32, 128, 56, 56, generator=g).to(device)
    op = dev.conv2d_op(x, w, 1, 1, 1, 1)
    y, gx, gw = torch.empty(32, 128, 56, 56, device=device), torch.zeros_like(x), torch.zeros_like(w)

    def step():
        dev.conv2d_forward(op, x, w, y)
        dev.conv2d_backward(op, x, gx, w, gw, dy)
        if h.world > 1:
            allreduce_shared_grads([gw], group)
    return step


OTHER = {
    # name: (builder, flops per step per GPU, algorithmic bytes, bound, arithmetic, description)
    "c1": (make_c1, 6 * 1024 ** 3, 44 * MIB, "tensor", "f32",
           "config[0]: MatMat f32 A[1024,1024] x B[1024,1024], fwd + grad_lhs + grad_rhs (the two gradient GEMMs on "
           "dfdx's two streams)"),
    "c3": (make_c3, 2 * 6 * 256 * 512 * 512 * 64, 1136 * MIB, "hbm", "f16",
           "config[2]: MatMatBatch4 f16 Q,K,V[16,16,512,64]: QK^T and PV, forward + backward (6 GEMM groups; the "
           "score-sized tensors cross HBM, so the bound is memory)"),
    "attn": (make_attn, 2 * 6 * 256 * 512 * 512 * 64, 9 * 16 * MIB, "tensor", "f16",
             "config[2] shapes, fused: softmax(Q K^T / 8) V for f16 Q,K,V[16,16,512,64], forward + backward "
             "(b200_attention_forward / _backward; flops of the six GEMM groups, recomputation not counted)"),
    "f16": (make_f16, 2 * 8192 ** 3, 3 * 128 * MIB, "tensor", "f16",
            "one f16 GEMM 8192^3, f32 accumulate (not a BASELINE configuration: the shape the pool's cuBLAS peak is measured on)"),
    "c4": (make_c4, 3 * 2 * 32 * 128 * 576 * 3136, 246 * MIB, "tensor", "f32",
           "config[3]: conv2d f32 x[32,64,56,56] * w[128,64,3,3], stride 1, padding 1, fwd + both gradients"),
}


def run_other(h, name, steps, warmup):
    builder, flops, algo_bytes, bound, kind, desc = OTHER[name]
    step = builder(h)
    r = h.region_flushed(step, steps, max(warmup, 3))
    h.check_status(name)
    per_step = r["ms"] / steps
    return {
        "workload": desc, "dtype": kind, "tflops": round(h.world * flops / (per_step * 1e-3) / 1e12, 3),
        "ms_per_step": round(per_step, 4), "steps": steps, "gpu_launches": r["launches"],
        "tensor_core_launches": r["tc_launches"], "l2": "256 MiB flush buffer written between timed steps",
        "roofline": h.roofline(bound, kind, flops, algo_bytes, per_step, r["ms"] * 1e-3),
    }


def run_transformer(h, args, steps, warmup):
    """Configuration 5: data-parallel training step of a 6-layer encoder (d_model 512, 8 heads, ffn 2048),
    batch 64 per GPU, sequence 256, MSE loss, Adam; all matmuls on this library (dfdx_b200/encoder.py)."""
    import torch
    from dfdx_b200.encoder import Trainer
    dev, device, lib = h.dev, h.device, h.lib
    BATCH, SEQ, MODEL = 64, 256, 512
    trainer = Trainer(dev, h.world, layers=6, model=MODEL, heads=8, ff=2048, seed=0,       # same init on every rank
                      fused=False if args.unfused_epilogues else (True if args.unfused_attention else "attention"))
    g = torch.Generator(device="cpu").manual_seed(0xD0FD + 5 + 1000 * h.rank)             # different data per rank
    x_h = torch.randn(BATCH, SEQ, MODEL, generator=g).half().pin_memory()
    t_h = torch.randn(BATCH, SEQ, MODEL, generator=g).half().pin_memory()
    x, t = x_h.to(device), t_h.to(device)
    l_before = lib.b200_launch_count()
    captured = trainer.capture(x, t)                            # 3 eager warm-up steps + 1 recorded step
    launches_per_step = (lib.b200_launch_count() - l_before) // 4 if captured else None
    losses = []

    def step_e2e():
        xd, td = x_h.to(device, non_blocking=True), t_h.to(device, non_blocking=True)
        losses.append(float(trainer.step(xd, td).detach()))          # the loss crosses back to the host every step

    r = h.region(lambda: trainer.step(x, t), steps, max(warmup, 3))
    h.check_status("the encoder step")
    e2e_steps = max(3, min(steps, 10))
    r2 = h.region(step_e2e, e2e_steps, 3)
    gemm_flop = 2.010e12                                     # matmul flops per step per GPU (forward + backward)
    per_step = r["ms"] / steps
    sps, sps_e2e = 1e3 / per_step, e2e_steps / (r2["ms"] * 1e-3)
    return {
        "workload": "config[4]: encoder 6 x (d_model 512, 8 heads, ffn 2048), batch 64/GPU, seq 256, MSE, Adam",
        "dtype": "f16 compute, f32 accumulate, f32 master weights",
        "steps_per_s": round(sps, 3), "tokens_per_s": round(h.world * BATCH * SEQ * sps, 1),
        "ms_per_step": round(per_step, 3), "steps": steps,
        "parameters": sum(p.numel() for p in trainer.model.parameters()),
        "parallelism": f"dp{h.world}: one NCCL all-reduce of the flat f32 gradient buffer per step, inside the step's CUDA graph",
        "matmuls": "all on libdfdx_b200 (MatMatBr + MatMatBatch4, forward and backward); w_q, w_k and w_v, stored next "
                   "to each other, run as one (model -> 3 * model) MatMatBr each way; weight gradients are added in f32 "
                   "into the f32 gradient buffer (b200_matmat_br_grad_rhs_f32); casts, "
                   "loss and Adam are torch ops (separate non-matmul kernels in dfdx too)",
        "rowwise": "torch LayerNorm / sum" if args.unfused_epilogues else
                   "LayerNorm forward + backward and the bias gradients on libdfdx_b200",
        "attention": "two batched GEMMs + softmax" if (args.unfused_epilogues or args.unfused_attention)
                     else "fused attention kernels (b200_attention_forward / _backward)",
        "gpu_launches": int(launches_per_step * steps) if captured else r["launches"],
        "cuda_graph": bool(captured), "cuda_graph_error": getattr(trainer, "capture_error", None),
        "gemm_tflops_per_gpu": round(gemm_flop * sps / 1e12, 2),
        "roofline": h.roofline("tensor", "f16", gemm_flop, None, per_step, r["ms"] * 1e-3),
        "e2e": {"tokens_per_s": round(h.world * BATCH * SEQ * sps_e2e, 1), "steps_per_s": round(sps_e2e, 3),
                "steps": e2e_steps, "h2d_bytes_per_step": int(2 * x_h.numel() * 2), "d2h_bytes_per_step": 4,
                "last_loss": losses[-1] if losses else None},
    }


def cublas_as_dfdx(h):
    """The GPU comparator: cuBLAS driven the way dfdx drives it (matmul/cuda_kernel.rs:62-135,177-179,226-236), through
    torch: default-math sgemm (`allow_tf32 = False`) for f32, f16 in / out with f32 compute for f16.  Also the
    TF32 rate of this GPU (the dense rate the 3xTF32 kernel is held against).  CUDA events, best of several."""
    import torch
    device = h.device
    res = {}

    def best(fn, reps=8, inner=1):
        fn(); torch.cuda.synchronize(device)
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(inner):
                fn()
            e1.record()
            torch.cuda.synchronize(device)
            ts.append(e0.elapsed_time(e1) / inner)
        return min(ts)

    old = torch.backends.cuda.matmul.allow_tf32
    try:
        a = torch.randn(8192, 8192, device=device)
        b = torch.randn(8192, 8192, device=device)
        c = torch.empty(8192, 8192, device=device)
        torch.backends.cuda.matmul.allow_tf32 = True
        ms = best(lambda: torch.matmul(a, b, out=c))
        burst = 2 * 8192 ** 3 / (ms * 1e-3) / 1e12
        n_loop = max(10, int(2000.0 / ms))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_loop):
            torch.matmul(a, b, out=c)
        e1.record()
        torch.cuda.synchronize(device)
        sustained = 2 * 8192 ** 3 * n_loop / (e0.elapsed_time(e1) * 1e-3) / 1e12
        res["tf32_8192"] = {"tflops_burst": round(burst, 1), "tflops_sustained": round(sustained, 1),
                            "seconds_sustained": round(e0.elapsed_time(e1) * 1e-3, 2)}
        h.tf32 = {"burst": burst, "sustained": sustained}
        del a, b, c
        # config 2's forward: X[16384,1024] x W^T[1024,4096], weight stored (4096,1024)
        x = torch.randn(B * S, K, device=device)
        w = torch.randn(N, K, device=device)
        y = torch.empty(B * S, N, device=device)
        fl = 2.0 * B * S * K * N
        torch.backends.cuda.matmul.allow_tf32 = False
        ms = best(lambda: torch.matmul(x, w.t(), out=y), reps=4)
        res["c2_forward_sgemm"] = {"ms": round(ms, 4), "tflops": round(fl / (ms * 1e-3) / 1e12, 1),
                                   "note": "what dfdx calls for f32: cublasSgemm, default math"}
        torch.backends.cuda.matmul.allow_tf32 = True
        ms = best(lambda: torch.matmul(x, w.t(), out=y))
        res["c2_forward_tf32"] = {"ms": round(ms, 4), "tflops": round(fl / (ms * 1e-3) / 1e12, 1),
                                  "note": "1xTF32 (lower precision than the f32 path here): one tensor MAC per logical MAC"}
        del x, w, y
        # config 1: 1024^3 sgemm
        torch.backends.cuda.matmul.allow_tf32 = False
        a = torch.randn(1024, 1024, device=device); b = torch.randn(1024, 1024, device=device)
        c = torch.empty(1024, 1024, device=device)
        ms = best(lambda: torch.matmul(a, b, out=c), inner=10)
        res["c1_forward_sgemm"] = {"ms": round(ms, 4), "tflops": round(2 * 1024 ** 3 / (ms * 1e-3) / 1e12, 1)}
        del a, b, c
        # f16: 8192^3, the encoder's Linear shape with bias, config 3's score GEMM
        a = torch.randn(8192, 8192, device=device).half(); b = torch.randn(8192, 8192, device=device).half()
        c = torch.empty(8192, 8192, device=device, dtype=torch.float16)
        ms = best(lambda: torch.matmul(a, b, out=c))
        res["f16_8192"] = {"ms": round(ms, 4), "tflops": round(2 * 8192 ** 3 / (ms * 1e-3) / 1e12, 1)}
        del a, b, c
        x = torch.randn(16384, 512, device=device).half(); w = torch.randn(2048, 512, device=device).half()
        bias = torch.randn(2048, device=device).half(); y = torch.empty(16384, 2048, device=device, dtype=torch.float16)
        ms = best(lambda: torch.addmm(bias, x, w.t(), out=y), inner=10)
        res["f16_linear_16384x512x2048_addmm"] = {"ms": round(ms, 4), "tflops": round(2 * 16384 * 512 * 2048 / (ms * 1e-3) / 1e12, 1)}
        del x, w, bias, y
        q = torch.randn(256, 512, 64, device=device).half(); k = torch.randn(256, 512, 64, device=device).half()
        s = torch.empty(256, 512, 512, device=device, dtype=torch.float16)
        ms = best(lambda: torch.bmm(q, k.transpose(1, 2), out=s), inner=4)
        res["c3_scores_hgemm_batched"] = {"ms": round(ms, 4), "gbs": round((2 * 16 + 128) * MIB / (ms * 1e-3) / 1e9, 1)}
        del q, k, s
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    torch.cuda.empty_cache()
    return res


def ours_on_cublas_shapes(h):
    """This library on the shapes of `cublas_as_dfdx` (same timing method), so the two can be read side by side."""
    import torch
    dev, device = h.dev, h.device
    res = {}

    def best(fn, reps=8, inner=1):
        fn(); torch.cuda.synchronize(device)
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(inner):
                fn()
            e1.record()
            torch.cuda.synchronize(device)
            ts.append(e0.elapsed_time(e1) / inner)
        return min(ts)

    x = torch.randn(B * S, K, device=device); w = torch.randn(N, K, device=device)
    y = torch.empty(B * S, N, device=device)
    wv = w.t()
    ms = best(lambda: dev.gemm((B * S, K, N), x, x.stride(), wv, wv.stride(), 0.0, y, y.stride()))
    res["c2_forward_f32"] = {"ms": round(ms, 4), "tflops": round(2.0 * B * S * K * N / (ms * 1e-3) / 1e12, 1)}
    del x, w, y, wv
    a = torch.randn(1024, 1024, device=device); b = torch.randn(1024, 1024, device=device)
    c = torch.empty(1024, 1024, device=device)
    ms = best(lambda: dev.gemm((1024, 1024, 1024), a, a.stride(), b, b.stride(), 0.0, c, c.stride()), inner=10)
    res["c1_forward_f32"] = {"ms": round(ms, 4), "tflops": round(2 * 1024 ** 3 / (ms * 1e-3) / 1e12, 1)}
    del a, b, c
    a = torch.randn(8192, 8192, device=device).half(); b = torch.randn(8192, 8192, device=device).half()
    c = torch.empty(8192, 8192, device=device, dtype=torch.float16)
    ms = best(lambda: dev.gemm((8192, 8192, 8192), a, a.stride(), b, b.stride(), 0.0, c, c.stride()))
    res["f16_8192"] = {"ms": round(ms, 4), "tflops": round(2 * 8192 ** 3 / (ms * 1e-3) / 1e12, 1)}
    del a, b, c
    x = torch.randn(1, 16384, 512, device=device).half(); w = torch.randn(2048, 512, device=device).half()
    bias = torch.randn(2048, device=device).half()
    ms = best(lambda: dev.linear_forward(x, w.t(), bias), inner=10)
    res["f16_linear_16384x512x2048_bias"] = {"ms": round(ms, 4), "tflops": round(2 * 16384 * 512 * 2048 / (ms * 1e-3) / 1e12, 1)}
    del x, w, bias
    q = torch.randn(16, 16, 512, 64, device=device).half(); k = torch.randn(16, 16, 512, 64, device=device).half()
    kt = k.permute(0, 1, 3, 2)
    ms = best(lambda: dev.matmat_batch4_forward(q, kt), inner=4)
    res["c3_scores_f16"] = {"ms": round(ms, 4), "gbs": round((2 * 16 + 128) * MIB / (ms * 1e-3) / 1e9, 1)}
    torch.cuda.empty_cache()
    h.check_status("the comparator shapes")
    return res


# ------------------------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--headline-only", action="store_true",
                    help="only the headline workload: no `configs`, `strong`, sustained or cuBLAS legs (profiling)")
    ap.add_argument("--unfused-attention", action="store_true",
                    help="workload c5: scores / softmax / weighted sum as two batched GEMMs and a softmax instead of "
                         "the fused attention kernels")
    ap.add_argument("--unfused-epilogues", action="store_true",
                    help="workload c5: bias / ReLU / score scale as separate ops after the GEMMs (the reference's op sequence)")
    ap.add_argument("--allreduce", default="overlap", choices=["overlap", "inline"],
                    help="N > 1: the weight gradient's all-reduce on a side stream under the grad_lhs GEMM (default), or "
                         "in line on the compute stream after both gradient GEMMs")
    ap.add_argument("--overlap-sms", type=int, default=OVERLAP_SMS,
                    help="SMs the grad_lhs GEMM leaves to the overlapped all-reduce (and that collective's CTA bound)")
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5", "attn", "f16"],
                    help="c2 (default) is the benchmark line with every configuration inside; the others time one "
                         "configuration alone (device-resident; used for profiling)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import dfdx_b200
    from dfdx_b200.parallel import nccl_group

    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = dfdx_b200.Cuda(local_rank)
    h = Harness(dev, rank, world, local_rank)
    warmup = max(args.warmup, 3)

    def finish(out):
        if rank == 0:
            print(json.dumps(out))
        if world > 1:
            dist.destroy_process_group()

    if args.workload != "c2":
        # one configuration alone
        if rank == 0:
            h.sampler.start()
            time.sleep(0.3)
        res = run_transformer(h, args, args.steps, warmup) if args.workload == "c5" else \
            run_other(h, args.workload, args.steps, warmup)
        h.sampler.stop()
        if args.workload == "c5":
            metric, value, unit = "transformer_train_tokens_per_s", res["tokens_per_s"], "token/s"
        else:
            metric, value, unit = METRIC, res["tflops"], "TFLOP/s"
        finish({"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": warmup,
                "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": res["dtype"], "data": "synthetic", "config": {"workload": res["workload"]},
                "gpu_launches": res["gpu_launches"], "e2e": res.get("e2e"), "roofline": res["roofline"],
                "clocks": h.sampler.summary() if rank == 0 else None, "detail": res})
        return

    # ---- the headline workload -------------------------------------------------------------------------
    overlap = args.allreduce == "overlap"
    side_group = nccl_group(max(args.overlap_sms, 1)) if (world > 1 and overlap and args.overlap_sms > 0) else None
    step, t = make_c2(h, B, overlap=overlap, group=side_group, overlap_sms=args.overlap_sms)
    if rank == 0:
        h.sampler.start()
        time.sleep(0.3)          # let nvidia-smi come up before the GPU work starts
    r = h.region(step, args.steps, warmup)
    h.check_status("the timed region")
    clocks = h.sampler.summary(*r["window"]) if rank == 0 else None
    region_s = r["ms"] * 1e-3

    sustained = None
    if not args.headline_only:
        rs = h.region_for(step, 2.0, 0)
        h.check_status("the sustained region")
        sustained = (rs, h.sampler.summary(*rs["window"]) if rank == 0 else None)

    step_e2e, io = make_c2_e2e(h, t)
    e2e_steps = max(3, min(args.steps, 10))
    r_e2e = h.region(step_e2e, e2e_steps, 3)
    h.check_status("the e2e region")

    strong = None
    if world > 1 and not args.headline_only:
        # the same fixed problem (B = 64) partitioned over the ranks along the batch; config 1 along M
        per = B // world
        sstep, _ = make_c2(h, per, overlap=overlap, group=side_group, overlap_sms=args.overlap_sms)
        r_s = h.region(sstep, args.steps, warmup)
        rows = 1024 // world
        c1s = make_c1(h, rows=rows, strong=True)
        r_c1 = h.region_flushed(c1s, max(10, min(args.steps, 30)), warmup)
        h.check_status("the strong-scaling regions")
        strong = {
            "c2": {"partition": f"batch {B} -> {per} items per GPU, W replicated, grad_rhs (16 MiB) all-reduced under the grad_lhs GEMM",
                   "value": round(FLOP_PER_STEP * per * world / B * args.steps / (r_s["ms"] * 1e-3) / 1e12, 3),
                   "unit": "TFLOP/s", "ms_per_step": round(r_s["ms"] / args.steps, 4)},
            "c1": {"partition": f"M 1024 -> {rows} rows of A, C, dC per GPU, B replicated, grad_rhs (4 MiB) all-reduced",
                   "value": round(6 * rows * world * 1024 * 1024 * r_c1["steps"] / (r_c1["ms"] * 1e-3) / 1e12, 3),
                   "unit": "TFLOP/s", "ms_per_step": round(r_c1["ms"] / r_c1["steps"], 4)},
        }

    comparator = ours_shapes = None
    if not args.headline_only:
        comparator = cublas_as_dfdx(h)          # also measures the TF32 rate the f32 roofline uses
        ours_shapes = ours_on_cublas_shapes(h)

    configs = None
    if not args.headline_only:
        small = max(10, min(args.steps, 30))
        configs = {name: run_other(h, name, small, warmup) for name in ("c1", "c3", "c4", "attn", "f16")}
        configs["c5"] = run_transformer(h, args, max(10, min(args.steps, 30)), warmup)
    h.sampler.stop()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    tflops = world * FLOP_PER_STEP * args.steps / (r["ms"] * 1e-3) / 1e12
    e2e_tflops = world * FLOP_PER_STEP * e2e_steps / (r_e2e["ms"] * 1e-3) / 1e12
    # Dominant kernel: gemm_tf32x3_kernel<256>; every tensor launch of the step is one 137.4-GFLOP GEMM.
    per_launch_ms = r["ms"] / max(r["tc_launches"], 1)
    roof = h.roofline("tensor", "f32", FLOP_PER_LAUNCH, None, per_launch_ms, region_s,
                      kernel="gemm_tf32x3_kernel<256> (logical f32 flops; 3 tf32 MMAs per logical MAC)",
                      traffic=NCU_TRAFFIC_BYTES_PER_LAUNCH)
    roof["traffic_note"] = ("dram read+write bytes per launch, mean of the 3 launches of a step, from one ncu capture "
                            "of this workload (not re-measured by this run); algorithmic mean 380 MB")
    roof["avg_launch_ms"] = round(per_launch_ms, 4)
    roof["sm_mhz_median"] = clocks["sm_mhz"] if clocks else None
    out = {
        "metric": METRIC, "value": round(tflops, 3), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(r["ms"] / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "arithmetic": "3xTF32 tcgen05 (kind::tf32), f32 accumulate in TMEM",
                   "l2": "inputs+outputs per step 672 MiB > 126 MB L2 (no flush needed)",
                   "parallelism": "1 GPU" if world == 1 else
                                  f"weak scaling: each of the {world} ranks runs its own {B}-item batch; the shared weight's "
                                  f"gradient (16 MiB) is all-reduced over NCCL " +
                                  (f"on a side stream under the grad_lhs GEMM ({args.overlap_sms} SMs left to it)" if overlap
                                   else "in line after the gradient GEMMs")},
        "gpu_launches": r["launches"], "tensor_core_launches": r["tc_launches"],
        "clocks": clocks,
        "e2e": {"value": round(e2e_tflops, 3), "unit": "TFLOP/s", "steps": e2e_steps,
                "h2d_bytes_per_step": io["h2d"], "d2h_bytes_per_step": io["d2h"],
                "api": "dfdx_b200.Cuda.matmul + backward, pinned host inputs (X, dY) in, grad_rhs out; "
                       "the next step's upload overlaps this step's GEMMs (two buffer sets, copy stream)"},
        "roofline": roof,
    }
    if sustained:
        rs, cl = sustained
        v = world * FLOP_PER_STEP * rs["steps"] / (rs["ms"] * 1e-3) / 1e12
        ms_l = rs["ms"] / max(rs["tc_launches"], 1)
        out["value_sustained"] = {
            "value": round(v, 3), "unit": "TFLOP/s", "steps": rs["steps"], "seconds": round(rs["ms"] * 1e-3, 3),
            "clocks": cl, "roofline": h.roofline("tensor", "f32", FLOP_PER_LAUNCH, None, ms_l, rs["ms"] * 1e-3)}
    if strong:
        out["strong"] = strong
    if configs:
        out["configs"] = configs
    if comparator:
        out["cublas_as_dfdx"] = comparator
        out["this_library_same_shapes"] = ours_shapes
    if world == 1 and not args.no_cpu_baseline:
        try:
            out["cpu_baseline"] = cpu_baseline_block()
        except Exception as exc:  # the baseline is a reported side number, never the product
            out["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port",
                                   "sample": f"failed: {exc}"}
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
