#!/usr/bin/env python
"""Benchmark of the compiled-graph inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path (one Executable::run of the compiled graph) over one batch of
seeded synthetic input.  The default workload is the GEMM + fused-epilogue graph
C = GELU(A.B + bias), M=N=K=8192, bf16 with fp32 accumulation; the other compiled graphs (mlp,
conv_stack, transformer, mamba) are selectable with --workload.

`value`   throughput with inputs resident in HBM, timed with CUDA events on the launch stream,
          max over ranks; every rank runs the full workload (weak scaling, no collective).
`e2e`     the same metric through the plan's host-buffer entry point: pinned host inputs are copied
          to the device, the graph runs, the result is copied back, inside the timed region.
`roofline` the dominant kernel's algorithmic FLOPs (or bytes) per launch over its measured launch
          time, against the measured peaks of MEASURED_PEAKS.json.
`cpu_baseline` the reference's own CPU backend (oracle/_ref, built from the reference sources) on a
          bounded slab of the same workload, on this box's host cores.

`--impl reference` times only the reference CPU backend, on all host cores, and prints the same
line shape.
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

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["source"] = "fallback"
    return p


# ---- workloads ------------------------------------------------------------------------------------
def _bf16(x):
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return (((bits.astype(np.uint64) + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFFFFFF) >> 16).astype(np.uint16)


class GemmWorkload:
    """configs[1]: C = GELU(A.B + bias), square, bias replicated to a full tensor for the
    reference-native `add`; A, B ~ U(-1,1), bias ~ N(0,0.1), seed 1."""

    def __init__(self, n=8192, dtype="bf16"):
        self.n, self.dtype = n, dtype
        self.name = f"gemm_bias_gelu_{dtype}_{n}"
        self.plan = f"gemm_bias_gelu_{dtype}_{n}"
        self.metric, self.unit = "GEMM TFLOP/s", "TFLOP/s"
        self.flops = 2.0 * n ** 3
        self.units_per_step = self.flops / 1e12          # TFLOP per step
        self.allow_tf32 = dtype == "f32"
        self.bound = "tensor"
        self.arith = "bf16" if dtype == "bf16" else "tf32"

    def host_inputs(self, rank):
        rng = np.random.default_rng(1 + 1000 * rank)
        n = self.n
        conv = _bf16 if self.dtype == "bf16" else (lambda x: x)
        a = conv(rng.uniform(-1, 1, (n, n)).astype(np.float32))
        b = conv(rng.uniform(-1, 1, (n, n)).astype(np.float32))
        bias = rng.normal(0, 0.1, (n,)).astype(np.float32)
        return [a, b, conv(np.tile(bias[None, :], (n, 1)))]

    # the reference CPU backend on a slab of `rows` rows of A (rows are independent)
    def cpu_slab(self, rows):
        from frame_public_b200 import irtext
        dt = "bfloat16" if self.dtype == "bf16" else "float32"
        g = irtext.IrGraph("cpu")
        va, vb, vbias = g.input(dt, (rows, self.n)), g.input(dt, (self.n, self.n)), g.input(dt, (rows, self.n))
        g.output(g.unary("gelu", g.add(g.matmul(va, vb), vbias)))
        return g.text(), 2.0 * rows * self.n ** 2 / 1e12

    def cpu_slab_inputs(self, rows, full_inputs):
        a, b, bias = full_inputs
        return [a[:rows], b, bias[:rows]]

    def cpu_case(self, calib_seconds, host_inputs, target_seconds=12.0):
        """(ir text, inputs, units in the metric, description) of a bounded CPU sample."""
        rows = 1 if calib_seconds is None else int(max(1, min(64, target_seconds / max(calib_seconds, 1e-3))))
        text, units = self.cpu_slab(rows)
        return text, self.cpu_slab_inputs(rows, host_inputs), units, (
            f"first {rows} rows of A through the reference CPU backend's compiled graph (matmul, add, gelu)")


class GraphWorkload:
    """configs[0], [2], [3], [4]: a compiled model graph; metric = samples/s."""

    BUILDERS = {
        "mlp": ("mlp_f32_b64", "mlp", dict(), dict(), 1.0),
        "conv_stack": ("conv_stack_f32_b32_224", "conv_stack", dict(), dict(batch=1), 1.0),
        "transformer": ("transformer_bf16_b8_s512_d1024", "transformer_block", dict(), dict(batch=1, seq=128), None),
        "mamba": ("mamba_f32_b16_s2048_d768", "mamba_block", dict(), dict(batch=1, seq=256), None),
    }

    def __init__(self, key):
        from frame_public_b200 import configs
        self.key = key
        self.plan, builder, self.full_kw, self.cpu_kw, _ = self.BUILDERS[key]
        self.builder = getattr(configs, builder)
        self.name = self.plan
        self.metric, self.unit = "samples/s of compiled graph", "samples/s"
        self._wl0 = None
        # fp32 graphs run with CompileOptions::allow_tf32 (BASELINE's fp32 GEMM/conv bar is rel 1e-3)
        self.allow_tf32 = key in ("mlp", "conv_stack", "mamba")
        self.arith = {"mlp": "tf32", "conv_stack": "tf32", "transformer": "bf16", "mamba": "tf32"}[key]
        self.bound = None  # decided from the per-step profile

    def _full(self, rank):
        if self._wl0 is None or self._wl0[0] != rank:
            self._wl0 = (rank, self.builder(seed=10 + 1000 * rank, **self.full_kw))
        return self._wl0[1]

    def host_inputs(self, rank):
        wl = self._full(rank)
        self.units_per_step = float(wl.samples)
        self.flops = wl.flops
        return wl.inputs

    def cpu_case(self, calib_seconds, host_inputs, target_seconds=12.0):
        small = self.builder(seed=10, **{**self.full_kw, **self.cpu_kw})
        full = self._full(0)
        # samples/s of the full-size graph = small samples/s scaled by FLOPs per sample
        scale = (small.flops / small.samples) / (full.flops / full.samples)
        desc = (f"{small.name} through the reference CPU backend's compiled graph"
                + ("" if abs(scale - 1.0) < 1e-9 else f", scaled by FLOPs per sample ({scale:.4f})"))
        return small.ir_text, small.inputs, small.samples * scale, desc


def make_workload(name):
    if name.startswith("gemm_bias_gelu_"):
        _, _, _, dtype, n = name.split("_")
        return GemmWorkload(int(n), dtype)
    if name in GraphWorkload.BUILDERS:
        return GraphWorkload(name)
    raise SystemExit(f"unknown workload {name}; choose gemm_bias_gelu_<bf16|f32>_<n> or one of "
                     + ", ".join(GraphWorkload.BUILDERS))


# ---- clocks -----------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.proc = None
        self.lines = []
        self.nvml = None        # (module, handle) when NVML can be polled in-process
        self.samples = []       # (time, sm MHz, max sm MHz, reasons bitmask)
        self._stop = False

    def start(self):
        # NVML polled every 2 ms from a thread (read-only queries): a 20-step timed region lasts
        # tens of milliseconds, which a 100 ms nvidia-smi loop samples once or not at all.
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.device)
            pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
            self.nvml = (pynvml, handle)
            threading.Thread(target=self._poll, daemon=True).start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.device), "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _poll(self):
        pynvml, handle = self.nvml
        try:
            mx = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            mx = None
        while not self._stop:
            try:
                sm = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                try:
                    why = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except Exception:
                    why = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((time.time(), float(sm), float(mx) if mx else None, int(why)))
            except Exception:
                pass
            time.sleep(0.002)

    def _stop_nvml(self, t0, t1):
        self._stop = True
        names = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))
        inside = [x for x in self.samples if t0 <= x[0] <= t1] or self.samples[-3:]
        sm = [x[1] for x in inside]
        mx = [x[2] for x in inside if x[2] is not None]
        reasons = sorted({name for x in inside for bit, name in names if x[3] & bit})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "source": "nvml, 2 ms poll"}

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.nvml is not None:
            return self._stop_nvml(t0, t1)
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ts, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9 or not (t0 - 0.05 <= ts <= t1 + 0.2):
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            for ts, line in self.lines[-3:]:
                parts = [p.strip() for p in line.split(",")]
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except (ValueError, IndexError):
                    pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---- our arm ---------------------------------------------------------------------------------------
def run_ours(args):
    from frame_public_b200 import capi, runtime
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    device = local_rank
    lib = capi.load()
    if capi.device_count() <= device:
        raise SystemExit("bench.py: no CUDA device for this rank: the sm_100a library has no CPU fallback")

    wl = make_workload(args.workload)
    peaks = load_peaks()
    plan = runtime.CompiledPlan(runtime.load_plan_text(wl.plan), device, allow_tf32=wl.allow_tf32)
    host_inputs = wl.host_inputs(rank)

    # pinned host staging + resident device buffers
    def pinned_copy(arr):
        p = capi.c_void_p()
        capi.check(lib.fb200_host_alloc(arr.nbytes, capi.byref(p)))
        view = np.frombuffer((capi.ctypes.c_char * arr.nbytes).from_address(p.value), dtype=arr.dtype).reshape(arr.shape)
        view[...] = arr
        return p, view

    pinned_in = [pinned_copy(a) for a in host_inputs]
    out_specs = plan.outputs
    out_bytes = [int(np.prod(s, dtype=np.int64)) * capi.ITEMSIZE[dt] for dt, s in out_specs]
    pinned_out = []
    for nb in out_bytes:
        p = capi.c_void_p()
        capi.check(lib.fb200_host_alloc(nb, capi.byref(p)))
        pinned_out.append(p)
    dev_in = [capi.DeviceBuffer.from_numpy(a, device) for a in host_inputs]
    dev_out = [capi.DeviceBuffer(nb, device) for nb in out_bytes]
    stream = capi.c_void_p()
    capi.check(lib.fb200_stream_create(device, capi.byref(stream)))
    ev = [capi.c_void_p() for _ in range(4)]
    for e in ev:
        capi.check(lib.fb200_event_create(device, 1, capi.byref(e)))

    def barrier():
        capi.check(lib.fb200_stream_synchronize(device, stream))
        if dist is not None:
            dist.barrier()

    def elapsed(e0, e1):
        ms = capi.c_float(0)
        capi.check(lib.fb200_event_elapsed_ms(e0, e1, capi.byref(ms)))
        return float(ms.value)

    def max_over_ranks(ms):
        if dist is None:
            return ms
        import torch
        t = torch.tensor([ms], device=f"cuda:{local_rank}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    in_ptrs = [b.ptr for b in dev_in]
    out_ptrs = [b.ptr for b in dev_out]

    # Between timed iterations: either the step's working set exceeds the 126 MB L2, or a buffer
    # larger than L2 is rewritten before every step.
    working_set = sum(a.nbytes for a in host_inputs) + sum(out_bytes) + plan.arena_bytes
    flush = None
    if working_set <= 160 * 1024 * 1024:
        flush = capi.DeviceBuffer(256 * 1024 * 1024, device)
        l2_note = "256 MiB buffer rewritten before every timed step (L2 flush); flush time excluded"
    else:
        l2_note = f"working set {working_set / 2**20:.0f} MiB per step, larger than L2"

    # ---- device-resident timing ---------------------------------------------------------------
    for _ in range(max(3, args.warmup)):
        plan.run_device(in_ptrs, out_ptrs, stream)
    barrier()
    sampler = ClockSampler(device)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = capi.launch_count()
    t_wall0 = time.time()
    if flush is None:
        capi.check(lib.fb200_event_record(device, ev[0], stream))
        for _ in range(args.steps):
            plan.run_device(in_ptrs, out_ptrs, stream)
        capi.check(lib.fb200_event_record(device, ev[1], stream))
        barrier()
        ms_local = elapsed(ev[0], ev[1])
    else:
        ms_local = 0.0
        for i in range(args.steps):
            capi.check(lib.fb200_memset(device, flush.ptr, i & 0xFF, flush.nbytes, stream))
            capi.check(lib.fb200_event_record(device, ev[0], stream))
            plan.run_device(in_ptrs, out_ptrs, stream)
            capi.check(lib.fb200_event_record(device, ev[1], stream))
            capi.check(lib.fb200_stream_synchronize(device, stream))
            ms_local += elapsed(ev[0], ev[1])
        barrier()
    t_wall1 = time.time()
    launches = capi.launch_count() - launches0
    ms_total = max_over_ranks(ms_local)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    status = capi.kernel_status(device)
    if status != 0:
        raise SystemExit(f"bench.py: a bounded wait gave up inside a kernel (status {status}); no number reported")
    ms_per_step = ms_total / args.steps
    value = world * wl.units_per_step / (ms_per_step / 1e3)

    # ---- end to end: host buffers in, host buffers out ---------------------------------------------
    host_in_ptrs = [p.value for p, _ in pinned_in]
    host_out_ptrs = [p.value for p in pinned_out]
    e2e_steps = max(2, min(args.steps, 10))
    # end to end: every step copies its inputs from pinned host memory and its result back; the steps
    # are queued through the pipelined entry point (copy-in, run and copy-out of neighbouring steps
    # overlap) and the clock stops after the last result has reached the host
    for _ in range(3):
        plan.run_host_async_ptrs(host_in_ptrs, host_out_ptrs, stream)
    plan.host_sync()
    barrier()
    capi.check(lib.fb200_event_record(device, ev[2], stream))
    for _ in range(e2e_steps):
        plan.run_host_async_ptrs(host_in_ptrs, host_out_ptrs, stream)
    plan.host_sync()
    capi.check(lib.fb200_event_record(device, ev[3], stream))
    barrier()
    e2e_ms = max_over_ranks(elapsed(ev[2], ev[3])) / e2e_steps
    e2e_value = world * wl.units_per_step / (e2e_ms / 1e3)

    # ---- roofline of the dominant kernel: per-step device times of eager runs ---------------------------
    from frame_public_b200 import plantext
    ptext = plantext.parse(runtime.load_plan_text(wl.plan))
    prof = None
    for _ in range(3):
        cur = plan.profile(in_ptrs, out_ptrs, stream)
        prof = cur if prof is None else [(a[0], min(a[1], b[1])) for a, b in zip(prof, cur)]
    dom_index = max(range(len(prof)), key=lambda i: prof[i][1])
    dom_op, dom_ms = prof[dom_index]
    d_flops, d_bytes = plantext.step_work(ptext, dom_index)
    if dom_op == "attention_fan":   # one launch standing for every per-head chain of the plan
        d_flops, d_bytes = plantext.attention_fan_work(ptext)
    step_total = sum(ms for _, ms in prof)
    if d_flops > 0 and (wl.arith != "f32"):
        bound = "tensor"
        achieved = d_flops / 1e12 / (dom_ms / 1e3)
        peak = peaks.get("bf16_tflops")
        peak_note = peaks["source"] + " dense bf16 cuBLAS GEMM"
        if wl.arith == "tf32":
            peak = peak / 2.0
            peak_note += ", halved: TF32 runs at half the bf16 tensor rate"
        roof_unit = "TFLOP/s"
    else:
        bound = "hbm"
        achieved = d_bytes / 1e9 / (dom_ms / 1e3)
        peak = peaks.get("hbm_gbs")
        peak_note = peaks["source"] + " STREAM-style copy"
        roof_unit = "GB/s"
    roofline = {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": roof_unit,
                "frac": round(achieved / peak, 4) if peak else None, "traffic": TRAFFIC.get(wl.name),
                "kernel": dom_op, "kernel_ms": round(dom_ms, 4),
                "kernel_share_of_step": round(dom_ms / step_total, 3) if step_total else None,
                "peak_source": peak_note,
                "steps_ms": {f"{i}:{op}": round(ms, 4) for i, (op, ms) in enumerate(prof) if ms > 0}
                if sum(1 for _, ms in prof if ms > 0) <= 40 else None}

    # ---- reference CPU backend on a bounded slab (rank 0, N=1 only) -------------------------------------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = cpu_slab_baseline(wl, host_inputs, target_seconds=12.0)

    if rank == 0:
        line = {
            "metric": wl.metric, "value": round(value, 3), "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.arith,
            "data": "synthetic", "impl": "frame_b200",
            "config": {"workload": wl.name, "per_gpu": "one full workload per rank, no collective",
                       "l2": l2_note, "accumulate": "fp32", "launches_per_step": plan.launches_per_run,
                       "arena_bytes": plan.arena_bytes},
            "e2e": {"value": round(e2e_value, 3), "unit": wl.unit,
                    "h2d_bytes_per_step": int(sum(a.nbytes for a in host_inputs)),
                    "d2h_bytes_per_step": int(sum(out_bytes)), "ms_per_step": round(e2e_ms, 3)},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
            "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, in bytes, from the
# ncu captures summarised under profiles/ (null where no capture of that workload exists)
TRAFFIC = {
    "gemm_bias_gelu_bf16_8192": 1.31e9,   # profiles/gemm_tcgen05_bf16_dram_traffic_8192.md
}


def cpu_slab_baseline(wl, host_inputs, target_seconds):
    from oracle import ref_runtime
    if not ref_runtime.available():
        return {"value": None, "unit": wl.unit, "cores": 0, "kind": "reference",
                "sample": "oracle/_ref (the reference build) is not present on this box"}
    ref_runtime.load_b200_backend()   # registers the new ops' CPU kernels (gelu, ...) in the reference process

    def timed(case):
        text, ins, units, desc = case
        comp = ref_runtime.Compiled(text, "cpu")
        t0 = time.time()
        comp.run(ins)
        dt = time.time() - t0
        comp.close()
        return dt, units, desc

    dt, units, desc = timed(wl.cpu_case(None, host_inputs, target_seconds))
    if isinstance(wl, GemmWorkload):
        dt, units, desc = timed(wl.cpu_case(dt, host_inputs, target_seconds))
    return {"value": units / dt, "unit": wl.unit, "cores": 1, "kind": "reference",
            "sample": f"{desc}, {dt:.1f} s on one core (the reference CPU backend is single-threaded)"}


# ---- reference arm ------------------------------------------------------------------------------------
def _ref_worker(args_tuple):
    name, rows, steps, warmup, seed = args_tuple
    sys.path.insert(0, ROOT)
    from oracle import ref_runtime
    ref_runtime.load_b200_backend()
    wl = make_workload(name)
    text, units = wl.cpu_slab(rows)
    rng = np.random.default_rng(seed)
    n = wl.n
    conv = _bf16 if wl.dtype == "bf16" else (lambda x: x)
    ins = [conv(rng.uniform(-1, 1, (rows, n)).astype(np.float32)), conv(rng.uniform(-1, 1, (n, n)).astype(np.float32)),
           conv(rng.normal(0, 0.1, (rows, n)).astype(np.float32))]
    comp = ref_runtime.Compiled(text, "cpu")
    for _ in range(warmup):
        comp.run(ins)
    t0 = time.time()
    for _ in range(steps):
        comp.run(ins)
    return (time.time() - t0) / max(1, steps), units


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref_runtime
    wl = make_workload(args.workload)
    if not ref_runtime.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref (the reference CPU backend built from its sources) is not present"}))
        return
    import multiprocessing as mp
    cores = os.cpu_count() or 1
    procs = max(1, min(cores, 64))
    rows = 1   # one row of A per process per step: 2*N^2 FLOP, about a second of the reference's naive matmul
    warm = max(0, args.warmup)
    steps = max(1, args.steps)   # about 0.7 s per step: the default K and W finish in seconds
    ctx = mp.get_context("spawn")
    with ctx.Pool(procs) as pool:
        res = pool.map(_ref_worker, [(wl.name, rows, steps, warm, 100 + i) for i in range(procs)])
    t_step = max(r[0] for r in res)
    units = sum(r[1] for r in res)
    value = units / t_step
    line = {
        "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": steps, "warmup": warm, "ms_per_step": t_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": wl.arith, "data": "synthetic", "impl": "reference",
        "config": {"workload": wl.name},
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": procs, "kind": "reference",
                         "sample": f"{procs} processes x {rows} row(s) of A per step through the reference CPU backend's "
                                   f"compiled graph (matmul, add, gelu); the backend itself is single-threaded"},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="gemm_bias_gelu_bf16_8192")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
