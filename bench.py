#!/usr/bin/env python
"""Benchmark of the fused-operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3] [--impl ours|reference]

A step is one launch of the fused graph of the chosen workload on synthetic, seeded inputs that are already
resident in HBM.  The headline workload is the BatchNorm training-forward graph (fp16 [64,256,56,56]);
``--workload`` selects the fused elementwise chain (c1) or the residual+RMSNorm+SwiGLU graph (c3) instead,
and the default run also reports those in ``other_workloads``.  With N > 1 (torchrun, one rank per GPU) every
rank runs the same-sized shard of a batch N times larger (weak scaling, no collective on the data path); the
timed region is bracketed by a barrier + synchronize and the maximum over ranks is reported.

Output: one JSON line (rank 0) with the whole-job throughput in GB/s of algorithmic bytes, the roofline of
the dominant kernel against the measured HBM peak, the end-to-end figure through the public API with host
buffers, and the NumPy evaluation of the same graph on the host cores as the CPU baseline.
``--impl reference`` times only that NumPy evaluation (the reference has no CPU executor of its own; its
tests evaluate every graph with NumPy).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c1": "fused elementwise exp(x)*y+0.5, fp32 [8192,8192]",
    "c2": "BatchNorm training-forward, fp16 NCHW [64,256,56,56], fp32 statistics",
    "c3": "residual-add + RMSNorm + SwiGLU, bf16 [16384,4096]",
}
ALGO_BYTES = {"c1": 805306368, "c2": 205524992, "c3": 805314560}
DTYPE = {"c1": "f32", "c2": "f16 storage / f32 math", "c3": "bf16 storage / f32 math"}


def make_inputs(name, seed_offset=0, scale=1.0):
    """Seeded synthetic inputs of the workload's shapes and distributions (host arrays)."""
    import ml_dtypes
    if name == "c1":
        rng = np.random.default_rng(0 + seed_offset)
        rows = max(1, int(8192 * scale))
        return [rng.uniform(-1, 1, (rows, 8192)).astype(np.float32) for _ in range(2)]
    if name == "c2":
        rng = np.random.default_rng(2 + seed_offset)
        n = max(1, int(64 * scale))
        x = rng.standard_normal((n, 256, 56, 56), dtype=np.float32).astype(np.float16)
        gamma = rng.normal(1, 0.1, (1, 256, 1, 1)).astype(np.float32)
        beta = rng.normal(0, 0.1, (1, 256, 1, 1)).astype(np.float32)
        return [x, gamma, beta]
    if name == "c3":
        rng = np.random.default_rng(3 + seed_offset)
        t = max(1, int(16384 * scale))
        bf = ml_dtypes.bfloat16
        h, r, g, u = (rng.standard_normal((t, 4096), dtype=np.float32).astype(bf) for _ in range(4))
        w = rng.normal(1, 0.02, (4096,)).astype(np.float32).astype(bf)
        return [h, r, w, g, u]
    raise ValueError(name)


def build_graph(k, name, loaded, arrays):
    from dvm_b200 import workloads as W
    if name == "c1":
        return [W.fused_elementwise(k, *loaded)]
    if name == "c2":
        n, _, h, w = arrays[0].shape
        return list(W.batchnorm_train(k, *loaded, n * h * w))
    if name == "c3":
        return list(W.rmsnorm_swiglu(k, *loaded, 4096))
    raise ValueError(name)


def algo_bytes(name, arrays, outputs):
    return int(sum(a.nbytes for a in arrays) + sum(o.nbytes for o in outputs))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [s.strip() for s in out.strip().split(",")]
                self.samples.append(float(f[0]))
                self.max_mhz = float(f[1])
                for n, v in zip(names, f[2:]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def cpu_eval(name, arrays):
    """NumPy evaluation of the workload's graph (the oracle), returning the outputs."""
    from oracle.dvm_oracle import OracleKernel
    o = OracleKernel()
    loaded = [o.load(a) for a in arrays]
    return [o.store(v) for v in build_graph(o, name, loaded, arrays)]


def cpu_baseline(name, budget_s=12.0):
    """Time the NumPy graph evaluation on a bounded sample of the workload (fraction of the leading dim)."""
    scale = {"c1": 1.0 / 32, "c2": 1.0 / 16, "c3": 1.0 / 64}[name]
    arrays = make_inputs(name, scale=scale)
    t0 = time.perf_counter()
    outs = cpu_eval(name, arrays)
    dt = time.perf_counter() - t0
    reps = 1
    best = dt
    while dt * (reps + 1) < budget_s and reps < 3:
        t0 = time.perf_counter()
        cpu_eval(name, arrays)
        best = min(best, time.perf_counter() - t0)
        reps += 1
    nbytes = algo_bytes(name, arrays, outs)
    return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
            "sample": "%s of the leading dimension of %s (%d algorithmic bytes), best of %d NumPy evaluations"
                      % ("1/%d" % round(1 / scale), name, nbytes, reps)}


def run_reference(args, rank):
    if rank != 0:
        return
    name = args.workload
    scale = {"c1": 1.0 / 32, "c2": 1.0 / 16, "c3": 1.0 / 64}[name]
    arrays = make_inputs(name, scale=scale)
    outs = None
    for _ in range(args.warmup):
        outs = cpu_eval(name, arrays)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        outs = cpu_eval(name, arrays)
    dt = time.perf_counter() - t0
    nbytes = algo_bytes(name, arrays, outs)
    v = nbytes * args.steps / dt / 1e9
    sample = "1/%d of the leading dimension per step (%d algorithmic bytes)" % (round(1 / scale), nbytes)
    print(json.dumps({
        "impl": "reference", "metric": "fused_op_hbm_throughput", "value": v, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE[name], "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "note": "NumPy evaluation of the same graph on host cores; the "
                   "reference ships no CPU executor and its tests use NumPy as the evaluator"},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


class DeviceWorkload:
    """One compiled fused graph with its inputs resident on the device."""

    def __init__(self, name, seed_offset=0, scale=1.0):
        import dvm_b200 as dvm
        self.name = name
        self.arrays = make_inputs(name, seed_offset, scale)
        ktype = "vector:spec,dyn" if name == "c3" else "vector"
        self.k = dvm.PyKernel(ktype, "dev", int(os.environ.get("LOCAL_RANK", "0")))
        self.loads = [self.k.load(list(a.shape), dvm.frontend.dvm_dtype_of(a.dtype)) for a in self.arrays]
        for op, a in zip(self.loads, self.arrays):
            self.k.input(op, a)
        vals = build_graph(self.k, name, self.loads, self.arrays)
        self.stores = [self.k.store(v) for v in vals]
        self.k.codegen()
        self.jit_us = self.k.jit_us()
        self.launches_per_step = self.k.das().count("vmain")

    def outputs(self):
        return [self.k.output(s) for s in self.stores]


def time_steps(wl, steps, warmup, dist):
    import torch
    for _ in range(warmup):
        wl.k.launch()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        wl.k.launch()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def time_e2e(wl, steps, warmup, dist):
    """Public-API path with host buffers: H2D of every input, launch, D2H of every output, per step."""
    import torch
    lib = wl.k._lib
    pinned = []
    for a in wl.arrays:
        t = torch.from_numpy(a.view(np.uint8).reshape(-1)).pin_memory()
        pinned.append(t)
    outs = [torch.empty(int(np.prod(s.shape(), dtype=np.int64)) * wl.k.output(s).dtype.itemsize, dtype=torch.uint8).pin_memory()
            for s in wl.stores]

    def step():
        for op, t in zip(wl.loads, pinned):
            lib.dvm_rt_memcpy_h2d(wl.k.device_ptr(op), t.data_ptr(), t.numel(), None)
        wl.k.launch()
        for s, t in zip(wl.stores, outs):
            lib.dvm_rt_memcpy_d2h(t.data_ptr(), wl.k.device_ptr(s), t.numel(), None)
        lib.dvm_rt_sync(None)

    for _ in range(max(1, warmup)):
        step()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([dt], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    h2d = int(sum(t.numel() for t in pinned))
    d2h = int(sum(t.numel() for t in outs))
    return dt, h2d, d2h


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (earlier measurement on this pool)"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the other workloads, e2e and the CPU baseline")
    ap.add_argument("--scale", type=float, default=1.0,
                    help="fraction of the workload's leading dimension (profiling captures use a small case)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as td
        td.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = td

    name = args.workload
    wl = DeviceWorkload(name, seed_offset=1000 * rank, scale=args.scale)
    nbytes = algo_bytes(name, wl.arrays, [np.empty(s.shape(), wl.k.output(s).dtype) for s in wl.stores])

    with ClockSampler(local_rank) as clocks:
        ms = time_steps(wl, args.steps, args.warmup, dist)
        # per-launch duration of the dominant kernel, device events on the launch stream
        lo, hi, mean = wl.k.perf(warmup=3, reps=max(20, min(args.steps, 200)))
    value = nbytes * args.steps * world / (ms * 1e-3) / 1e9
    peak, peak_src = measured_peak()
    achieved = nbytes / (mean * 1e-6) / 1e9
    line = {
        "metric": "fused_op_hbm_throughput", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE[name], "data": "synthetic",
        "config": {"workload": WORKLOADS[name], "algorithmic_bytes_per_step_per_gpu": nbytes,
                   "l2": "inputs larger than L2 (no flush)", "sharding": "each rank runs a full-size shard (batch x N)",
                   "scale": args.scale},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": peak_src, "kernel": "dvm_b200_vm_vector",
                     "us_per_launch": {"min": lo, "mean": mean, "max": hi},
                     "frac_of_nominal_8TBs": achieved / 8000.0},
        "gpu_launches": args.steps * wl.launches_per_step,
        "jit_us": wl.jit_us,
        "clocks": clocks.summary(),
    }
    if not args.no_extras:
        dt, h2d, d2h = time_e2e(wl, max(3, min(args.steps, 10)), 1, dist)
        e2e_steps = max(3, min(args.steps, 10))
        line["e2e"] = {"value": nbytes * e2e_steps * world / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": d2h, "ms_per_step": dt / e2e_steps * 1e3}
        if rank == 0 and world == 1:
            line["cpu_baseline"] = cpu_baseline(name)
            others = {}
            del wl
            for other in sorted(WORKLOADS):
                if other == name:
                    continue
                w2 = DeviceWorkload(other)
                nb = algo_bytes(other, w2.arrays, [np.empty(s.shape(), w2.k.output(s).dtype) for s in w2.stores])
                lo2, hi2, mean2 = w2.k.perf(warmup=3, reps=30)
                others[other] = {"workload": WORKLOADS[other], "us_per_launch": mean2, "GBs": nb / (mean2 * 1e-6) / 1e9,
                                 "frac_of_measured_peak": nb / (mean2 * 1e-6) / 1e9 / peak, "jit_us": w2.jit_us}
                del w2
            line["other_workloads"] = others
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
