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
``--impl reference`` runs the unmodified reference instead: its own CUDA backend (built from the reference tree into
oracle/_ref) through its own Python module for c1-c3, with `value` = its kernels on resident inputs and `e2e` = its own
host-buffer path (input / run / output per step); for c4/c5, which its GPU backend cannot run, and when no GPU or module
is there, the NumPy evaluation of the same graph on the host cores (the evaluator of the reference's own tests).
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
    "c4": "fused attention, bf16 Q/K/V [8,32,2048,128], fp32 softmax",
    "c5": "MatMul + bias + tanh-GeLU post-fusion, bf16 [16384,8192]x[8192,8192], fp32 accumulate",
}
ALGO_BYTES = {"c1": 805306368, "c2": 205524992, "c3": 805314560, "c4": 536870912, "c5": 671105024}
ALGO_FLOPS = {"c4": 549755813888, "c5": 2199023255552}
DTYPE = {"c1": "f32", "c2": "f16 storage / f32 math", "c3": "bf16 storage / f32 math", "c4": "bf16 operands / f32 accumulate",
         "c5": "bf16 operands / f32 accumulate"}
KTYPE = {"c1": "vector", "c2": "vector", "c3": "vector:spec,dyn", "c4": "split", "c5": "mix"}


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
    if name == "c4":
        rng = np.random.default_rng(4 + seed_offset)
        b = max(1, int(8 * scale))
        return [rng.standard_normal((b, 32, 2048, 128), dtype=np.float32).astype(ml_dtypes.bfloat16) for _ in range(3)]
    if name == "c5":
        rng = np.random.default_rng(5 + seed_offset)
        m = max(128, int(16384 * scale))
        bf = ml_dtypes.bfloat16
        a = (rng.standard_normal((m, 8192), dtype=np.float32) * 0.02).astype(bf)
        b = (rng.standard_normal((8192, 8192), dtype=np.float32) * 0.02).astype(bf)
        bias = (rng.standard_normal((8192,), dtype=np.float32) * 0.02).astype(bf)
        return [a, b, bias]
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
    if name == "c4":
        return [W.attention(k, *loaded, 1.0 / np.sqrt(128.0))]
    if name == "c5":
        return [W.matmul_bias_gelu(k, *loaded)]
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


def cpu_sample(name):
    """A bounded sample of the workload for the host-side evaluation: (arrays, description)."""
    if name == "c4":
        arrays = [a[:1, :2] for a in make_inputs("c4", scale=1.0 / 8)]
        return arrays, "2 of the 256 (batch, head) slices of c4"
    if name == "c5":
        arrays = make_inputs("c5", scale=1.0 / 64)
        return arrays, "256 of the 16384 rows of A (1/64 of c5)"
    scale = {"c1": 1.0 / 32, "c2": 1.0 / 16, "c3": 1.0 / 64}[name]
    return make_inputs(name, scale=scale), "1/%d of the leading dimension of %s" % (round(1 / scale), name)


def work_of(name, arrays, outs):
    """Units of the workload's metric in one evaluation: algorithmic bytes, or flops for the tensor-core graphs."""
    if name == "c4":
        b, h, s, d = arrays[0].shape
        return 4.0 * b * h * s * s * d
    if name == "c5":
        return 2.0 * arrays[0].shape[0] * arrays[1].shape[0] * arrays[1].shape[1]
    return float(algo_bytes(name, arrays, outs))


def unit_of(name):
    return "TFLOP/s" if name in ("c4", "c5") else "GB/s"


def unit_scale(name):
    return 1e12 if name in ("c4", "c5") else 1e9


def metric_of(name):
    return {"c4": "attention_tflops", "c5": "matmul_post_fusion_tflops"}.get(name, "fused_op_hbm_throughput")


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_baseline(name, budget_s=12.0):
    """Time the NumPy graph evaluation (the oracle) on a bounded sample of the workload."""
    arrays, what = cpu_sample(name)
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
    work = work_of(name, arrays, outs)
    # NumPy's elementwise and reduction loops are single-threaded; its fp32 matmul uses the BLAS threads
    cores = host_threads() if name in ("c4", "c5") else 1
    return {"value": work / best / unit_scale(name), "unit": unit_of(name), "cores": cores, "kind": "port",
            "sample": "%s, best of %d NumPy evaluations" % (what, reps)}


def reference_cuda(name, scale=1.0):
    """The same graph on the reference's own CUDA backend (oracle/_ref, built from the reference tree by
    oracle/build_ref.py): returns (kernel builder, arrays, outputs) or None when the module is absent, no device is
    usable, or the graph needs an op the reference's GPU backend lacks (MatMul, ReduceMax: src/system.cc:290-294)."""
    if name not in ("c1", "c2", "c3"):
        return None
    try:
        from oracle import ref_backend
        if ref_backend.module() is None:
            return None
        arrays = make_inputs(name, scale=scale)
        k = ref_backend.RefKernel("vector" if name == "c1" else "split")
        loads = [k.load(a) for a in arrays]
        stores = [k.store(v) for v in build_graph(k, name, loads, arrays)]
        k.run()
        outs = [k.output(s) for s in stores]
        return k, arrays, outs
    except Exception as e:   # an unusable reference must not take the benchmark down
        sys.stderr.write("reference CUDA backend unavailable for %s: %s\n" % (name, e))
        return None


def config_of(name, **extra):
    """The `config` object of a bench line: both arms fill the same keys."""
    cfg = {"workload": WORKLOADS[name], "algorithmic_bytes_per_step_per_gpu": ALGO_BYTES[name],
           "l2": "inputs larger than L2 (no flush)", "sharding": "each rank runs a full-size shard (batch x N)", "scale": 1.0}
    if name in ALGO_FLOPS:
        cfg["algorithmic_flops_per_step_per_gpu"] = float(ALGO_FLOPS[name])
    cfg.update(extra)
    return cfg


def run_reference_cuda(args, name):
    """Reference arm on the reference's own CUDA backend.  `value`: K runs of its kernels with the inputs resident
    (its run() launches every kernel of the split graph and waits for the stream).  `e2e`: the same K steps through
    its own host-buffer path - input() of every load, run(), output() of every store - which is what a user of its
    Python module executes per call."""
    import torch
    got = reference_cuda(name)
    if got is None:
        return False
    k, arrays, outs = got
    for _ in range(args.warmup):
        k.k.run()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        k.k.run()   # launches every kernel of the split graph and waits for the stream
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    work = work_of(name, arrays, outs)
    v = work * args.steps / dt / unit_scale(name)
    lo, hi, mean = k.perf()
    e2e_steps = max(2, min(args.steps, 5))
    k.step_from_host()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        up, down = k.step_from_host()
    torch.cuda.synchronize()
    dt_e2e = time.perf_counter() - t0
    print(json.dumps({
        "impl": "reference", "metric": metric_of(name), "value": v, "unit": unit_of(name), "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE[name], "data": "synthetic",
        "config": config_of(name),
        "note": "the reference's own CUDA backend (src/vm_gpu.cu compiled for sm_100a from the reference tree), same graph "
                "through its Python module; value = inputs resident, wall clock around K run() calls; kernel time by its "
                "perf(): %.1f us mean (device events)" % mean,
        "kernel_us_by_perf": {"min": lo, "max": hi, "mean": mean},
        "cpu_baseline": {"value": v, "unit": unit_of(name), "cores": 0, "kind": "reference",
                         "sample": "not a CPU run: the full workload on the GPU through the reference's CUDA backend "
                                   "(the reference has no CPU executor)"},
        "e2e": {"value": work * e2e_steps / dt_e2e / unit_scale(name), "unit": unit_of(name), "h2d_bytes_per_step": int(up),
                "d2h_bytes_per_step": int(down), "ms_per_step": dt_e2e / e2e_steps * 1e3,
                "how": "the reference's own host-buffer path per step: input() of every load (device allocation + synchronous "
                       "upload from pageable NumPy memory), run(), output() of every store"},
    }))
    return True


def run_reference(args, rank):
    if rank != 0:
        return
    name = args.workload
    try:
        import torch
        if torch.cuda.is_available() and run_reference_cuda(args, name):
            return
    except Exception as e:
        sys.stderr.write("falling back to the NumPy evaluation: %s\n" % e)
    arrays, what = cpu_sample(name)
    outs = None
    for _ in range(args.warmup):
        outs = cpu_eval(name, arrays)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        outs = cpu_eval(name, arrays)
    dt = time.perf_counter() - t0
    v = work_of(name, arrays, outs) * args.steps / dt / unit_scale(name)
    cores = host_threads() if name in ("c4", "c5") else 1
    print(json.dumps({
        "impl": "reference", "metric": metric_of(name), "value": v, "unit": unit_of(name), "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE[name], "data": "synthetic",
        "config": config_of(name),
        "note": "NumPy evaluation of the same graph on host cores (a bounded sample per step); the reference ships no CPU "
                "executor and its tests use NumPy as the evaluator",
        "cpu_baseline": {"value": v, "unit": unit_of(name), "cores": cores, "kind": "port", "sample": what + " per step"},
        "e2e": {"value": v, "unit": unit_of(name), "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


class DeviceWorkload:
    """One compiled fused graph with its inputs resident on the device."""

    def __init__(self, name, seed_offset=0, scale=1.0):
        import dvm_b200 as dvm
        self.name = name
        self.arrays = make_inputs(name, seed_offset, scale)
        self.k = dvm.PyKernel(KTYPE[name], "dev", int(os.environ.get("LOCAL_RANK", "0")))
        self.loads = [self.k.load(list(a.shape), dvm.frontend.dvm_dtype_of(a.dtype)) for a in self.arrays]
        for op, a in zip(self.loads, self.arrays):
            self.k.input(op, a)
        vals = build_graph(self.k, name, self.loads, self.arrays)
        self.stores = [self.k.store(v) for v in vals]
        self.k.codegen()
        self.jit_us = self.k.jit_us()
        das = self.k.das()
        self.launches_per_step = das.count("vmain") + das.count("mmain") + das.count("amain")

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


def time_e2e_pipelined(wl, steps, warmup, dist):
    """The same per-step work as time_e2e (H2D of every input from pinned memory, launch, D2H of every output) for a caller
    that streams batches: two sets of device buffers, the copies in, the launches (`dvm_launch_reloc` with the set's
    addresses) and the copies out run on three streams ordered by events, so that the upload of step i + 1 and the download
    of step i - 1 overlap the kernel of step i.  Returns (seconds, h2d bytes per step, d2h bytes per step)."""
    import ctypes
    import torch
    from dvm_b200 import _capi
    lib = wl.k._lib
    pinned = [torch.from_numpy(a.view(np.uint8).reshape(-1)).pin_memory() for a in wl.arrays]
    out_bytes = [int(np.prod(s.shape(), dtype=np.int64)) * wl.k.output(s).dtype.itemsize for s in wl.stores]
    host_out = [[torch.empty(n, dtype=torch.uint8).pin_memory() for n in out_bytes] for _ in range(2)]
    dev_in = [[torch.empty(t.numel(), dtype=torch.uint8, device="cuda") for t in pinned] for _ in range(2)]
    dev_out = [[torch.empty(n, dtype=torch.uint8, device="cuda") for n in out_bytes] for _ in range(2)]
    relocs = []
    for b in range(2):
        arr = (_capi.Reloc * (len(wl.loads) + len(wl.stores)))()
        for i, (op, t) in enumerate(zip(wl.loads, dev_in[b])):
            arr[i].io, arr[i].addr = op._h, t.data_ptr()
        for i, (op, t) in enumerate(zip(wl.stores, dev_out[b])):
            arr[len(wl.loads) + i].io, arr[len(wl.loads) + i].addr = op._h, t.data_ptr()
        relocs.append(arr)
    ws = wl.k._ws.ptr if wl.k._ws is not None else None
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    in_done = [torch.cuda.Event() for _ in range(2)]
    run_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]

    def step(i):
        b = i & 1
        if i >= 2:
            s_in.wait_event(run_done[b])     # the kernel of step i - 2 has read this set's inputs
        for t, d in zip(pinned, dev_in[b]):
            lib.dvm_rt_memcpy_h2d(d.data_ptr(), t.data_ptr(), t.numel(), ctypes.c_void_p(s_in.cuda_stream))
        in_done[b].record(s_in)
        s_run.wait_event(in_done[b])
        if i >= 2:
            s_run.wait_event(out_done[b])    # the results of step i - 2 have left this set's outputs
        rc = lib.dvm_launch_reloc(wl.k._k, relocs[b], len(relocs[b]), ws, ctypes.c_void_p(s_run.cuda_stream))
        if rc != 0:
            raise RuntimeError("dvm_launch_reloc failed: %d" % rc)
        run_done[b].record(s_run)
        s_out.wait_event(run_done[b])
        for d, t in zip(dev_out[b], host_out[b]):
            lib.dvm_rt_memcpy_d2h(t.data_ptr(), d.data_ptr(), t.numel(), ctypes.c_void_p(s_out.cuda_stream))
        out_done[b].record(s_out)

    for i in range(2 * max(1, warmup)):
        step(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(steps):
        step(i + 2)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([dt], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    # leave the kernel bound to its own buffers again
    wl.k.codegen()
    return dt, int(sum(t.numel() for t in pinned)), int(sum(out_bytes))


def measured_peak(name):
    """Roofline denominator for the workload's dominant kernel: measured HBM copy bandwidth or bf16 GEMM rate."""
    key, fallback = ("bf16_tflops", 1590.0) if name in ("c4", "c5") else ("hbm_gbs", 6650.0)
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))[key]), "measured (MEASURED_PEAKS.json %s)" % key
        except Exception:
            pass
    return fallback, "fallback (earlier measurement on this pool)"


def measured_sustained():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["bf16_tflops_sustained"])
    except Exception:
        return None


KERNEL_NAME = {"c1": "dvm_b200_vm_vector_flat", "c2": "dvm_b200_vm_vector_nd_r128", "c3": "dvm_b200_vm_vector_group",
               "c4": "dvm_b200_attention_bf16_sf", "c5": "dvm_b200_mm_tcgen05_pair"}


def device_summary(name, reps=30):
    """Per-launch figures of one workload on the current device (inputs resident, device events)."""
    wl = DeviceWorkload(name)
    outs = [np.empty(s.shape(), wl.k.output(s).dtype) for s in wl.stores]
    work = work_of(name, wl.arrays, outs)
    lo, hi, mean = wl.k.perf(warmup=3, reps=reps)
    peak, _ = measured_peak(name)
    # K launches back to back between two events (what the headline workload's figure is, too); `us_single` is one event
    # pair per launch, which adds the launch latency
    single = mean
    mean = time_launches(wl.k, reps, 3, None) / reps * 1e3
    rate = work / (mean * 1e-6) / unit_scale(name)
    out = {"workload": WORKLOADS[name], "us_per_launch": mean, "us_single": single, "us_min": lo, "rate": rate, "unit": unit_of(name),
           "frac_of_measured_peak": rate / peak, "jit_us": wl.jit_us, "launches": wl.launches_per_step}
    if name in ("c4", "c5"):
        # back-to-back tensor-core launches run under the power cap: the sustained cuBLAS figure is their denominator, the
        # burst figure that of a launch timed alone
        sustained = measured_sustained()
        out["rate_single_launch"] = work / (single * 1e-6) / unit_scale(name)
        out["frac_of_measured_burst_single_launch"] = out["rate_single_launch"] / peak
        out["frac_back_to_back_of_burst"] = rate / peak
        # like with like: the launch timed alone against the burst figure, the launches back to back against the sustained one
        out["frac_of_measured_peak"] = out["frac_of_measured_burst_single_launch"]
        if sustained:
            out["frac_of_measured_sustained"] = rate / sustained
    wl.k.release_io()
    return out


def dynamic_shape_jit():
    """c3 as one dynamic-shape kernel stepped through its token counts in order: host microseconds from the new
    shape to the finished program (compile + bind), and the kernel time at that shape."""
    import ml_dtypes
    import dvm_b200 as dvm
    bf = ml_dtypes.bfloat16
    k = dvm.PyKernel("vector:spec,dyn", "dev", int(os.environ.get("LOCAL_RANK", "0")))
    t_ref = dvm.IntArrayRef([1, 4096])
    w_ref = dvm.IntArrayRef([4096])
    loads = [k.load(t_ref, dvm.bfloat16), k.load(t_ref, dvm.bfloat16), k.load(w_ref, dvm.bfloat16),
             k.load(t_ref, dvm.bfloat16), k.load(t_ref, dvm.bfloat16)]
    from dvm_b200 import workloads as W
    stores = [k.store(v) for v in W.rmsnorm_swiglu(k, *loads, 4096)]
    out = {}
    for t in (1, 7, 128, 1000, 4096, 16384):
        rng = np.random.default_rng(3 + 1000 * t)
        t_ref.update([t, 4096])
        arrs = [rng.standard_normal((t, 4096), dtype=np.float32).astype(bf) for _ in range(2)]
        arrs.append(rng.normal(1, 0.02, (4096,)).astype(np.float32).astype(bf))
        arrs += [rng.standard_normal((t, 4096), dtype=np.float32).astype(bf) for _ in range(2)]
        for op, a in zip(loads, arrs):
            k.input(op, a)
        k.codegen()
        jit = k.jit_us()
        # from "the shape is known" to "the kernel is enqueued", on the host: the shape update, then shape inference +
        # planning + emission + binding (every call plans from scratch) and the launch call, i.e. the C ABI calls a framework
        # makes for a new shape (dvm_int_array_update, dvm_codegen, dvm_launch); device buffers exist already
        lib_sync = k._lib.dvm_rt_sync
        lib_sync(None)
        t0 = time.perf_counter()
        t_ref.update([t, 4096])
        k.repeat_codegen_launch()
        enq = (time.perf_counter() - t0) * 1e6
        lib_sync(None)
        lo, hi, mean = k.perf(warmup=2, reps=10)
        b2b = time_launches(k, 20, 2, None) / 20 * 1e3
        nbytes = 49152 * t + 8192   # h, r, g, u in, two results out (bf16 [t, 4096] each) and the weight row
        out[str(t)] = {"jit_us": jit, "shape_to_enqueued_us": enq, "kernel_us": b2b, "kernel_us_single_launch": mean,
                       "gbs": nbytes / (b2b * 1e-6) / 1e9, "frac_of_measured_peak": nbytes / (b2b * 1e-6) / 1e9 / measured_peak("c3")[0]}
    k.release_io()
    return out


def init_product_comm(rank, world, dist):
    """The library's own NCCL communicator for this process: rank 0 makes the rendezvous id, torch.distributed carries it."""
    from dvm_b200 import frontend
    box = [frontend.comm_unique_id() if rank == 0 else None]
    if dist is not None:
        dist.broadcast_object_list(box, src=0)
    frontend.init_comm_with_id(rank, world, box[0])


def c5tp_workload(rank, world, local_rank, scale=1.0):
    """The K-split tensor-parallel MatMul as ONE kernel of the library: MatMul of the rank's K slice, all-reduce of the fp32
    partial products (Kernel::AllReduce on the library's NCCL communicator), bias + GeLU, bf16 result."""
    import dvm_b200 as dvm
    from dvm_b200 import sharding, workloads as W
    a, b, bias = make_inputs("c5", scale=scale)
    m, n, kdim = a.shape[0], b.shape[1], a.shape[1]
    ar, br = sharding.ksplit_operands(a, b, rank, world)
    del a, b
    k = dvm.PyKernel("mix", "dev", local_rank)
    la, lb, lbias = k.load(list(ar.shape), dvm.bfloat16), k.load(list(br.shape), dvm.bfloat16), k.load([n], dvm.bfloat16)
    k.input(la, ar)
    k.input(lb, br)
    k.input(lbias, bias)
    total = k.allreduce("sum", k.cast(k.matmul(la, lb, False, False), dvm.float32))
    out = k.store(k.cast(W.gelu_tanh(k, k.add(total, k.cast(lbias, dvm.float32))), dvm.bfloat16))
    k.codegen()
    return k, out, (m, n, kdim)


def time_launches(k, steps, warmup, dist):
    """Device milliseconds of `steps` launches of `k`, bracketed by barriers, maximum over the ranks."""
    import torch
    for _ in range(warmup):
        k.launch()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        k.launch()
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


def c5tp_record(args, rank, world, local_rank, dist, steps):
    """Figures of the K-split variant on `world` ranks (strong scaling: the whole product is one unit)."""
    k, out, (m, n, kdim) = c5tp_workload(rank, world, local_rank, args.scale)
    ms = time_launches(k, steps, max(args.warmup, 3), dist)
    stages = k.perf_stages(warmup=2, reps=5)
    das = k.das()
    names = [ln.split("(")[0] + ("(" + ln.split("(")[1].split(",")[0] + ")" if ln.startswith("cmain") else "")
             for ln in das.splitlines() if ln[:5] in ("mmain", "vmain", "cmain", "amain")]
    wire = sum(int(w) for w in __import__("re").findall(r"wire_bytes=(\d+)", das))
    coll_us = sum(us for nm, us in zip(names, stages) if nm.startswith("cmain"))
    flops = 2.0 * m * n * kdim
    rec = {"ms_per_step": ms / steps, "value": flops * steps / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
           "scaling": "strong", "stages": names, "stage_us_serialised": [round(float(u), 1) for u in stages],
           "collective_share_of_stage_time": coll_us / max(sum(stages), 1e-9), "wire_bytes_per_rank": wire,
           "workspace_bytes_per_rank": m * n * 4}
    k.release_io()
    return rec


def run_c5tp(args, rank, world, local_rank, dist):
    """`--workload c5tp`: the K-split tensor-parallel MatMul as the headline line."""
    init_product_comm(rank, world, dist)
    with ClockSampler(local_rank) as clocks:
        rec = c5tp_record(args, rank, world, local_rank, dist, args.steps)
    peak, peak_src = measured_peak("c5")
    per_gpu = rec["value"] / world
    if rank == 0:
        print(json.dumps({
            "metric": "matmul_post_fusion_tflops", "value": rec["value"], "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": rec["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE["c5"], "data": "synthetic",
            "config": config_of("c5", workload=WORKLOADS["c5"] + "; K split over %d ranks, fp32 partial products combined over NCCL "
                                "inside the kernel's plan" % world, sharding="K / N per rank, one product", scale=args.scale),
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
                         "traffic": None, "peak_source": peak_src, "kernel": "dvm_b200_mm_tcgen05_pair"},
            "c5tp": rec, "gpu_launches": args.steps * len(rec["stages"]), "clocks": clocks.summary(),
        }))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def c2_by_channels_record(rank, world, local_rank, dist, steps=10):
    """The BatchNorm workload cut by channels (each channel's statistics are independent, so no collective): every rank
    holds the full NCHW tensors and normalises its 256 / N channels through strided loads and stores."""
    import dvm_b200 as dvm
    from dvm_b200 import workloads as W
    x, gamma, beta = make_inputs("c2")
    n, c, h, w = x.shape
    per = c // world
    first = rank * per
    stride = [c * h * w, h * w, w, 1]
    k = dvm.PyKernel("vector", "dev", local_rank)
    lx = k.view_load([n, per, h, w], stride, dvm.float16)
    lg, lb = k.load([1, per, 1, 1], dvm.float32), k.load([1, per, 1, 1], dvm.float32)
    k.input(lx, x, offset=first * h * w)
    k.input(lg, np.ascontiguousarray(gamma[:, first:first + per]))
    k.input(lb, np.ascontiguousarray(beta[:, first:first + per]))
    y, mean, var = W.batchnorm_train(k, lx, lg, lb, n * h * w)
    sy = k.view_store(y, stride)
    k.set_output(sy, np.zeros_like(x), offset=first * h * w)
    k.store(mean)
    k.store(var)
    k.codegen()
    ms = time_launches(k, steps, 3, dist)
    peak, _ = measured_peak("c2")
    per_gpu = ALGO_BYTES["c2"] / world * steps / (ms * 1e-3) / 1e9
    rec = {"partition": "channels / %d per GPU (strided slab of NCHW)" % world, "us_per_step": ms / steps * 1e3,
           "value": per_gpu * world, "unit": "GB/s", "scaling": "strong", "per_gpu_frac_of_measured_peak": per_gpu / peak}
    k.release_io()
    return rec


def strong_scaling_record(name, rank, world, local_rank, dist, steps=10):
    """One BASELINE workload cut into `world` parts along its leading dimension (no collective): whole-job rate and the
    per-GPU roofline fraction."""
    wl = DeviceWorkload(name, seed_offset=1000 * rank, scale=1.0 / world)
    outs = [np.empty(s.shape(), wl.k.output(s).dtype) for s in wl.stores]
    work = work_of(name, wl.arrays, outs)
    ms = time_launches(wl.k, steps, 3, dist)
    peak, _ = measured_peak(name)
    per_gpu = work * steps / (ms * 1e-3) / unit_scale(name)
    rec = {"partition": {"c1": "rows", "c3": "tokens", "c4": "batch", "c5": "rows of A"}[name] + " / %d per GPU" % world,
           "us_per_step": ms / steps * 1e3, "value": per_gpu * world, "unit": unit_of(name), "scaling": "strong",
           "per_gpu_frac_of_measured_peak": per_gpu / peak}
    wl.k.release_io()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["c5tp"])
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
        if args.workload == "c5tp":
            args.workload = "c5"
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
    if name == "c5tp":
        run_c5tp(args, rank, world, local_rank, dist)
        return
    wl = DeviceWorkload(name, seed_offset=1000 * rank, scale=args.scale)
    outs = [np.empty(s.shape(), wl.k.output(s).dtype) for s in wl.stores]
    work = work_of(name, wl.arrays, outs)
    nbytes = algo_bytes(name, wl.arrays, outs)

    with ClockSampler(local_rank) as clocks:
        ms = time_steps(wl, args.steps, args.warmup, dist)
        # per-launch duration of the dominant kernel, device events on the launch stream; the loop runs for about 1.5 s so
        # that the clock sampler (one nvidia-smi query per ~0.1 s) sees the same kernel under load more than once
        reps = int(min(10000, max(20, 1500.0 / max(ms / args.steps, 1e-3))))
        if args.no_extras:
            reps = max(20, min(args.steps, 200))   # (profiling captures run the command under ncu: keep it short)
        lo, hi, mean = wl.k.perf(warmup=3, reps=reps)
    value = work * args.steps * world / (ms * 1e-3) / unit_scale(name)
    peak, peak_src = measured_peak(name)
    # the kernel's average launch duration over the timed region: K launches back to back between two events on the launch
    # stream (one launch per step); a pair of events around every single launch adds the launch latency to each (`us_per_launch`)
    kernel_us = ms / args.steps * 1e3 / max(1, wl.launches_per_step)
    achieved = work / (ms / args.steps * 1e-3) / unit_scale(name)
    tensor = name in ("c4", "c5")
    # DRAM bytes per full-size launch from the ncu captures summarised under profiles/ (dram__bytes_read + write; the
    # quarter-size captures of c1, c3, c4, c5 are scaled by 4: their traffic grows with the leading dimension)
    traffic = {"c1": 4 * (135.2e6 + 36.0e6), "c2": 195.7e6 + 55.8e6, "c3": 4 * (135.0e6 + 39.9e6),
               "c4": 4 * (101.0e6 + 13.0e6), "c5": 4 * (520.3e6 + 62.0e6)}.get(name)
    if traffic is not None and args.scale != 1.0:
        traffic *= args.scale
    line = {
        "metric": metric_of(name), "value": value, "unit": unit_of(name), "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE[name], "data": "synthetic",
        "config": config_of(name, algorithmic_bytes_per_step_per_gpu=nbytes, scale=args.scale),
        "roofline": {"bound": "tensor" if tensor else "hbm", "achieved": achieved, "peak": peak, "unit": unit_of(name),
                     "frac": achieved / peak, "traffic": traffic, "traffic_source": "ncu capture (profiles/), bytes per launch",
                     "peak_source": peak_src, "kernel": KERNEL_NAME[name],
                     "kernel_us": kernel_us, "us_per_launch": {"min": lo, "mean": mean, "max": hi,
                                                               "how": "one event pair per launch (includes the launch latency)"},
                     "frac_of_nominal": achieved / (2250.0 if tensor else 8000.0)},
        "gpu_launches": args.steps * wl.launches_per_step,
        "jit_us": wl.jit_us,
        "clocks": clocks.summary(),
    }
    if tensor:
        line["config"]["algorithmic_flops_per_step_per_gpu"] = float(work)
    if not args.no_extras:
        e2e_steps = max(3, min(args.steps, 10))
        dt, h2d, d2h = time_e2e(wl, e2e_steps, 1, dist)
        serial = {"value": work * e2e_steps * world / dt / unit_scale(name), "unit": unit_of(name),
                  "ms_per_step": dt / e2e_steps * 1e3}
        pipe_steps = max(6, min(args.steps, 20))
        dt, h2d, d2h = time_e2e_pipelined(wl, pipe_steps, 1, dist)
        line["e2e"] = {"value": work * pipe_steps * world / dt / unit_scale(name), "unit": unit_of(name),
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": dt / pipe_steps * 1e3,
                       "how": "host buffers in pinned memory; every step uploads its inputs, launches through dvm_launch_reloc "
                              "and downloads its outputs; two buffer sets on three streams overlap the copies of neighbouring "
                              "steps with the kernel",
                       "one_step_at_a_time": serial}
        if rank == 0 and world == 1:
            line["cpu_baseline"] = cpu_baseline(name)
            wl.k.release_io()
            del wl
            others = {}
            for other in sorted(WORKLOADS):
                if other != name:
                    others[other] = device_summary(other)
            line["other_workloads"] = others
            line["dynamic_shape_jit_c3"] = dynamic_shape_jit()
            # second comparison: the reference's own CUDA backend on the same GPU (kernel time by its perf())
            ref = {}
            for other in ("c1", "c2", "c3"):
                got = reference_cuda(other)
                if got is not None:
                    lo_r, hi_r, mean_r = got[0].perf()
                    ref[other] = {"us_per_run": mean_r, "rate": work_of(other, got[1], got[2]) / (mean_r * 1e-6) / unit_scale(other),
                                  "unit": unit_of(other), "kernels": got[0].k.das().count("vmain")}
                    try:
                        got[0].k.release_io()   # frees its device buffers now (its split kernels refuse and free on destruction)
                    except RuntimeError:
                        pass
                del got
            line["reference_cuda_backend"] = ref or "not available"
    if dist is not None and not args.no_extras:
        # what only exists on several GPUs: the K-split MatMul with its collective, and the BASELINE shapes cut N ways
        try:
            wl.k.release_io()
        except Exception:
            pass
        multi = {}
        try:
            init_product_comm(rank, world, dist)
            multi["c5tp"] = c5tp_record(args, rank, world, local_rank, dist, steps=10)
        except Exception as e:   # the headline line must survive a failure here
            multi["c5tp"] = {"error": str(e)[:300]}
        for other in ("c1", "c2", "c3", "c4", "c5"):
            try:
                multi[other] = (c2_by_channels_record(rank, world, local_rank, dist) if other == "c2"
                                else strong_scaling_record(other, rank, world, local_rank, dist))
            except Exception as e:
                multi[other] = {"error": str(e)[:300]}
        line["multi_gpu"] = multi
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
