#!/usr/bin/env python
"""Benchmark of the compiled-graph inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path (one Executable::run of the compiled graph) over one batch of
seeded synthetic input.  The default workload is the GEMM + fused-epilogue graph
C = GELU(A.B + bias), M=N=K=8192, bf16 with fp32 accumulation; the other compiled graphs (mlp,
conv_stack, transformer, mamba) are selectable with --workload.

With N > 1 (torchrun, one process per GPU) the ONE workload is partitioned: every rank takes a
contiguous range of the batch (rows of A and of the full-shape bias for the GEMM), runs its own plan
on its own device, and there is no data-path collective (strong scaling).

`value`    whole-job throughput with inputs resident in HBM, CUDA events on the launch stream, the
           slowest rank's time.
`e2e`      the same through the plan's host-buffer entry point: every step copies its activations
           from pinned host memory and its result back, inside the timed region; parameters
           (weights, the reference's full-shape biases) stay on the device, as in a Frame module.
`roofline` the dominant kernel's algorithmic FLOPs (or bytes) per launch over its measured launch
           time, against the measured peaks; `sustained` repeats it over two seconds of
           back-to-back steps against the sustained peak.
`cpu_baseline`, `parity`  the reference's own CPU backend (oracle/_ref) on a slab of the same
           seeded workload (rows and samples are independent), timed on one host core, and the
           comparison of that slab with the same rows of the GPU result.
`batch_sharded`, `colsplit`  (default workload only) the Mamba block batch-sharded over the ranks,
           and the column-split GEMM whose epilogue stores C into every rank over NVLink.

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
class Workload:
    """One of the five compiled graphs at its full size.  Every rank builds the same seeded full-size
    inputs and cuts its own batch range out of them."""

    GRAPHS = {
        # key: (configs.FULL_BUILDERS key, plan name for a batch of b, full batch, arithmetic on the GPU)
        "mlp": ("mlp", "mlp_f32_b{b}", 64, "tf32"),
        "conv_stack": ("conv_stack", "conv_stack_f32_b{b}_224", 32, "tf32"),
        "transformer": ("transformer", "transformer_bf16_b{b}_s512_d1024", 8, "bf16"),
        "mamba": ("mamba", "mamba_f32_b{b}_s2048_d768", 16, "tf32"),
    }

    def __init__(self, name):
        from frame_public_b200 import configs
        self.configs = configs
        if name.startswith("gemm_bias_gelu_"):
            _, _, _, dtype, n = name.split("_")
            self.n, self.gemm_dtype = int(n), dtype
            self.is_gemm = True
            self.key = "gemm_" + dtype
            self.name = name
            self.batch = self.n                      # rows of A
            self.metric, self.unit = "GEMM TFLOP/s", "TFLOP/s"
            self.arith = "bf16" if dtype == "bf16" else "tf32"
            self.units_total = 2.0 * self.n ** 3 / 1e12   # TFLOP per step, whole job
        elif name in self.GRAPHS:
            self.is_gemm = False
            self.key, self.plan_fmt, self.batch, self.arith = self.GRAPHS[name]
            self.name = self.plan_fmt.format(b=self.batch)
            self.metric, self.unit = "samples/s of compiled graph", "samples/s"
            self.units_total = float(self.batch)
        else:
            raise SystemExit(f"unknown workload {name}; choose gemm_bias_gelu_<bf16|f32>_<n> or one of "
                             + ", ".join(self.GRAPHS))
        # fp32 graphs run with CompileOptions::allow_tf32 (the fp32 GEMM/conv tier is rel 1e-3)
        self.allow_tf32 = self.arith == "tf32"
        self._full = None

    def plan_name(self, world):
        if self.batch % world != 0:
            raise SystemExit(f"bench.py: {self.batch} rows/samples do not split over {world} ranks")
        b = self.batch // world
        if self.is_gemm:
            return self.name if world == 1 else f"gemm_bias_gelu_{self.gemm_dtype}_{b}x{self.n}x{self.n}"
        return self.plan_fmt.format(b=b)

    def full(self):
        """The seeded full-size workload (frame_public_b200.configs): inputs, FLOPs, dtype."""
        if self._full is None:
            c = self.configs
            if self.is_gemm:
                self._full = c.gemm_epilogue(n=self.n, dtype=c.BF16 if self.gemm_dtype == "bf16" else c.F32)
            else:
                builder, kw = c.FULL_BUILDERS[self.key]
                self._full = builder(**kw)
        return self._full

    def shard_inputs(self, plan_inputs, rank, world):
        """This rank's inputs: every input whose leading dimension shrank with the batch is cut to the
        rank's contiguous range, the others (weights) are taken whole.  Returns (arrays, indices of
        the inputs that are per-step activations: input 0 only; the rest are parameters)."""
        from frame_public_b200 import sharding
        out = []
        for arr, (_, shape) in zip(self.full().inputs, plan_inputs):
            if tuple(arr.shape) == tuple(shape):
                out.append(arr)
                continue
            assert arr.shape[1:] == tuple(shape[1:]) and arr.shape[0] % shape[0] == 0, (arr.shape, shape)
            per = arr.shape[0] // self.batch      # rows per sample
            b0, b1 = sharding.shard_range(self.batch, rank, world)
            out.append(np.ascontiguousarray(arr[b0 * per:b1 * per]))
        return out, [0]

    def slab_available(self):
        return (not self.is_gemm) or self.n == 8192


# ---- clocks -----------------------------------------------------------------------------------------
class ClockSampler:
    """SM clock and throttle reasons of THIS rank's GPU during a timed region.  The GPU is looked up by
    its PCI bus id: NVML and nvidia-smi indices ignore CUDA_VISIBLE_DEVICES, CUDA ordinals do not."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, device):
        from frame_public_b200 import capi
        self.device = device
        buf = capi.ctypes.create_string_buffer(64)
        try:
            capi.check(capi.load().fb200_device_pci_bus_id(device, buf, 64))
            self.bus_id = buf.value.decode()
        except Exception:
            self.bus_id = None
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
            if self.bus_id is not None:
                handle = pynvml.nvmlDeviceGetHandleByPciBusId(self.bus_id.encode())
            else:
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
                 "-i", self.bus_id if self.bus_id else str(self.device), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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

    def window(self, t0, t1):
        """Summary of the samples taken in [t0, t1] (NVML polling only; the sampler keeps running)."""
        inside = [x for x in self.samples if t0 <= x[0] <= t1] or self.samples[-3:]
        sm = [x[1] for x in inside]
        mx = [x[2] for x in inside if x[2] is not None]
        reasons = sorted({name for x in inside for bit, name in self.REASONS if x[3] & bit})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "source": "nvml, 2 ms poll", "pci_bus_id": self.bus_id}

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.nvml is not None:
            out = self.window(t0, t1)
            self._stop = True
            return out
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
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi, 100 ms loop",
                "pci_bus_id": self.bus_id}


# ---- one workload shard on one device -------------------------------------------------------------------
class PlanBench:
    """This rank's shard of a workload: the compiled plan, resident device buffers, pinned host
    buffers for the activations and the result, and the timed loops."""

    def __init__(self, wl, rank, world, device, stream):
        from frame_public_b200 import capi, runtime
        self.capi, self.lib = capi, capi.load()
        self.wl, self.rank, self.world, self.device, self.stream = wl, rank, world, device, stream
        self.plan_name = wl.plan_name(world)
        self.plan = runtime.CompiledPlan(runtime.load_plan_text(self.plan_name), device, allow_tf32=wl.allow_tf32)
        self.host_inputs, self.activations = wl.shard_inputs(self.plan.inputs, rank, world)
        self.out_bytes = [int(np.prod(s, dtype=np.int64)) * capi.ITEMSIZE[dt] for dt, s in self.plan.outputs]
        self.dev_in = [capi.DeviceBuffer.from_numpy(a, device) for a in self.host_inputs]
        self.dev_out = [capi.DeviceBuffer(nb, device) for nb in self.out_bytes]
        self.in_ptrs = [b.ptr for b in self.dev_in]
        self.out_ptrs = [b.ptr for b in self.dev_out]
        self.events = [capi.c_void_p() for _ in range(2)]
        for e in self.events:
            capi.check(self.lib.fb200_event_create(device, 1, capi.byref(e)))
        # Between timed iterations: either the step's working set exceeds the 126 MB L2, or a buffer
        # larger than L2 is rewritten before every step.
        self.working_set = sum(a.nbytes for a in self.host_inputs) + sum(self.out_bytes) + self.plan.arena_bytes
        self.flush = None
        if self.working_set <= 160 * 1024 * 1024:
            self.flush = capi.DeviceBuffer(256 * 1024 * 1024, device)
            self.l2_note = "256 MiB buffer rewritten before every timed step (L2 flush); flush time excluded"
        else:
            self.l2_note = f"working set {self.working_set / 2**20:.0f} MiB per step, larger than L2"
        self._pinned = None

    def sync(self):
        self.capi.check(self.lib.fb200_stream_synchronize(self.device, self.stream))

    def elapsed(self, e0, e1):
        ms = self.capi.c_float(0)
        self.capi.check(self.lib.fb200_event_elapsed_ms(e0, e1, self.capi.byref(ms)))
        return float(ms.value)

    def run(self):
        self.plan.run_device(self.in_ptrs, self.out_ptrs, self.stream)

    def timed_steps(self, steps):
        """Device time of `steps` runs in ms (this rank), CUDA events on the launch stream."""
        capi, lib, ev = self.capi, self.lib, self.events
        if self.flush is None:
            capi.check(lib.fb200_event_record(self.device, ev[0], self.stream))
            for _ in range(steps):
                self.run()
            capi.check(lib.fb200_event_record(self.device, ev[1], self.stream))
            self.sync()
            return self.elapsed(ev[0], ev[1])
        total = 0.0
        for i in range(steps):
            capi.check(lib.fb200_memset(self.device, self.flush.ptr, i & 0xFF, self.flush.nbytes, self.stream))
            capi.check(lib.fb200_event_record(self.device, ev[0], self.stream))
            self.run()
            capi.check(lib.fb200_event_record(self.device, ev[1], self.stream))
            self.sync()
            total += self.elapsed(ev[0], ev[1])
        return total

    def _pin(self, nbytes):
        p = self.capi.c_void_p()
        self.capi.check(self.lib.fb200_host_alloc(nbytes, self.capi.byref(p)))
        return p

    def prepare_host_path(self):
        """Pinned host buffers for the activations and the outputs; parameters bound as resident."""
        if self._pinned is not None:
            return
        capi = self.capi
        host_in = [0] * len(self.host_inputs)
        self.h2d_bytes = 0
        for i, arr in enumerate(self.host_inputs):
            if i in self.activations:
                p = self._pin(arr.nbytes)
                view = np.frombuffer((capi.ctypes.c_char * arr.nbytes).from_address(p.value), dtype=arr.dtype).reshape(arr.shape)
                view[...] = arr
                host_in[i] = p.value
                self.h2d_bytes += arr.nbytes
            else:
                self.plan.bind_resident(i, self.dev_in[i].ptr)
        self.host_out = [self._pin(nb) for nb in self.out_bytes]
        self._pinned = (host_in, [p.value for p in self.host_out])

    def e2e_steps(self, steps):
        """ms for `steps` pipelined host-to-host runs; the clock stops when the last result is on the host."""
        capi, lib, ev = self.capi, self.lib, self.events
        self.prepare_host_path()
        host_in, host_out = self._pinned
        capi.check(lib.fb200_event_record(self.device, ev[0], self.stream))
        for _ in range(steps):
            self.plan.run_host_async_ptrs(host_in, host_out, self.stream)
        self.plan.host_sync()
        capi.check(lib.fb200_event_record(self.device, ev[1], self.stream))
        self.sync()
        return self.elapsed(ev[0], ev[1])

    def output_host(self, index=0):
        dt, shape = self.plan.outputs[index]
        return self.dev_out[index].download(self.capi.NP_STORAGE[dt], shape)


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, in bytes, from the
# ncu captures summarised under profiles/ (null where no capture of that workload exists)
TRAFFIC = {
    "gemm_bias_gelu_bf16_8192": 1.34e9,   # profiles/gemm_tcgen05_bf16_dram_traffic_8192.md
}


def dist_setup(local_rank, world):
    if world <= 1:
        return None
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return dist


def max_over_ranks(dist, local_rank, value):
    from frame_public_b200 import sharding
    return sharding.max_over_ranks(value, dist, f"cuda:{local_rank}")


# ---- our arm ---------------------------------------------------------------------------------------
def run_ours(args):
    from frame_public_b200 import capi, plantext, runtime, sharding
    rank, local_rank, world = sharding.env_rank()
    device = local_rank
    lib = capi.load()
    if capi.device_count() <= device:
        raise SystemExit("bench.py: no CUDA device for this rank: the sm_100a library has no CPU fallback")
    dist = dist_setup(local_rank, world)
    wl = Workload(args.workload)
    peaks = load_peaks()
    stream = capi.c_void_p()
    capi.check(lib.fb200_stream_create(device, capi.byref(stream)))
    pb = PlanBench(wl, rank, world, device, stream)
    warmup = max(3, args.warmup)

    def barrier():
        pb.sync()
        if dist is not None:
            dist.barrier()

    # ---- device-resident timing ---------------------------------------------------------------
    for _ in range(warmup):
        pb.run()
    barrier()
    sampler = ClockSampler(device)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = capi.launch_count()
    t_wall0 = time.time()
    ms_local = pb.timed_steps(args.steps)
    barrier()
    t_wall1 = time.time()
    launches = capi.launch_count() - launches0
    ms_total = max_over_ranks(dist, local_rank, ms_local)
    clocks = sampler.window(t_wall0, t_wall1) if rank == 0 and sampler.nvml is not None else None
    status = capi.kernel_status(device)
    if status != 0:
        raise SystemExit(f"bench.py: a bounded wait gave up inside a kernel (status {status}); no number reported")
    ms_per_step = ms_total / args.steps
    value = wl.units_total / (ms_per_step / 1e3)

    # ---- end to end: pinned host activations in, result out to the host, every step -------------------
    e2e_steps = max(2, min(args.steps, 10))
    pb.e2e_steps(3)
    barrier()
    e2e_ms = max_over_ranks(dist, local_rank, pb.e2e_steps(e2e_steps)) / e2e_steps
    barrier()
    e2e_value = wl.units_total / (e2e_ms / 1e3)
    h2d = int(sharding.sum_over_ranks(float(pb.h2d_bytes), dist, f"cuda:{local_rank}"))     # all ranks together
    d2h = int(sharding.sum_over_ranks(float(sum(pb.out_bytes)), dist, f"cuda:{local_rank}"))

    # ---- roofline of the dominant kernel: per-step device times of eager runs ---------------------------
    ptext = plantext.parse(runtime.load_plan_text(pb.plan_name))
    prof = None
    for _ in range(3):
        cur = pb.plan.profile(pb.in_ptrs, pb.out_ptrs, stream)
        prof = cur if prof is None else [(a[0], min(a[1], b[1])) for a, b in zip(prof, cur)]
    dom_index = max(range(len(prof)), key=lambda i: prof[i][1])
    dom_op, dom_ms = prof[dom_index]
    d_flops, d_bytes = plantext.step_work(ptext, dom_index)
    if dom_op == "attention_fan":   # one launch standing for every per-head chain of the plan
        d_flops, d_bytes = plantext.attention_fan_work(ptext)
    step_total = sum(ms for _, ms in prof)
    tensor_bound = d_flops > 0
    tensor_peak = peaks.get("bf16_tflops")
    tensor_note = peaks["source"] + " dense bf16 cuBLAS GEMM"
    if wl.arith == "tf32":
        tensor_peak = tensor_peak / 2.0
        tensor_note += ", halved: TF32 runs at half the bf16 tensor rate"
    if tensor_bound:
        bound, achieved, peak, peak_note, roof_unit = "tensor", d_flops / 1e12 / (dom_ms / 1e3), tensor_peak, tensor_note, "TFLOP/s"
    else:
        bound, achieved, peak, roof_unit = "hbm", d_bytes / 1e9 / (dom_ms / 1e3), peaks.get("hbm_gbs"), "GB/s"
        peak_note = peaks["source"] + " STREAM-style copy"
    roofline = {"bound": bound, "achieved": round(achieved, 2), "peak": peak, "unit": roof_unit,
                "frac": round(achieved / peak, 4) if peak else None,
                "traffic": TRAFFIC.get(wl.name) if world == 1 else None,
                "kernel": dom_op, "kernel_ms": round(dom_ms, 4),
                "kernel_share_of_step": round(dom_ms / step_total, 3) if step_total else None,
                "peak_source": peak_note,
                "steps_ms": {f"{i}:{op}": round(ms, 4) for i, (op, ms) in enumerate(prof) if ms > 0}
                if sum(1 for _, ms in prof if ms > 0) <= 40 else None}

    # ---- sustained: two seconds of back-to-back steps (the power cap sets the clock) ----------------------
    if tensor_bound and wl.is_gemm and not args.no_sustained:
        n_sus = int(max(50, min(20000, 2000.0 / max(ms_per_step, 1e-3))))
        barrier()
        ts0 = time.time()
        sus_ms = max_over_ranks(dist, local_rank, pb.timed_steps(n_sus))
        ts1 = time.time()
        sus_val = wl.units_total * n_sus / (sus_ms / 1e3)
        sus_peak = peaks.get("bf16_tflops_sustained")
        if wl.arith == "tf32" and sus_peak:
            sus_peak = sus_peak / 2.0
        sus_clock = sampler.window(ts0, ts1) if rank == 0 and sampler.nvml is not None else None
        # whole-job figure over `world` GPUs against `world` times the one-GPU peak
        roofline["sustained"] = {"tflops": round(sus_val, 1), "steps": n_sus, "seconds": round(sus_ms / 1e3, 2),
                                 "peak": sus_peak, "frac": round(sus_val / (world * sus_peak), 4) if sus_peak else None,
                                 "sm_mhz": sus_clock["sm_mhz"] if sus_clock else None,
                                 "reasons": sus_clock["reasons"] if sus_clock else None}
    if rank == 0 and clocks is None:
        clocks = sampler.stop(t_wall0, t_wall1)
    sampler._stop = True

    # ---- reference CPU backend on a slab (rank 0, N=1 only), and parity of the GPU result with it --------
    cpu_baseline = parity = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        pb.run()
        pb.sync()
        cpu_baseline, parity = cpu_slab_baseline(wl, pb.output_host(0))

    # ---- the same graph through the reference framework's own API with this backend plugged in ----------
    via_frame = None
    if rank == 0 and world == 1 and not wl.is_gemm and not args.no_cpu_baseline:
        via_frame = via_frame_leg(wl)

    extras = {}
    if args.workload == DEFAULT_WORKLOAD and not args.no_extras:
        extras = default_workload_extras(args, rank, local_rank, world, device, stream, dist, wl, pb)

    if rank == 0:
        ok = parity is None or parity.get("ok", False)
        line = {
            "metric": wl.metric, "value": round(value, 3) if ok else None, "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": wl.arith,
            "data": "synthetic", "impl": "frame_b200",
            "config": bench_config(wl, world),
            "run": {"plan": pb.plan_name, "l2": pb.l2_note, "accumulate": "fp32",
                    "launches_per_step": pb.plan.launches_per_run, "arena_bytes": pb.plan.arena_bytes,
                    "partition": f"{wl.batch // world} of {wl.batch} {'rows of A' if wl.is_gemm else 'samples'} per rank, no collective",
                    "via_frame": via_frame},
            "e2e": {"value": round(e2e_value, 3) if ok else None, "unit": wl.unit, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 3),
                    "resident": "parameters (weights, full-shape biases) stay on the device; activations and results travel"},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
            "cpu_baseline": cpu_baseline, "parity": parity,
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


DEFAULT_WORKLOAD = "gemm_bias_gelu_bf16_8192"


def bench_config(wl, world):
    """The workload description both arms print (same keys, same values)."""
    return {"workload": wl.name, "batch": wl.batch, "partition": "contiguous batch ranges, one graph per GPU",
            "n_shards": world}


def via_frame_leg(wl):
    """ms per Executable::run of the SAME graph compiled by the reference framework's runtime::compile
    for backend "cuda" with this repository's plugin loaded (cache, nine-pass pipeline,
    B200Backend::compile, then B200Executable::run on resident tensors): what a Frame user's call costs,
    adapter validation and locking included.  Host wall clock over back-to-back runs and one stream
    synchronise.  The framework is the reference build of oracle/_ref used as the HOST of the plugin."""
    from oracle import ref_runtime
    if not ref_runtime.available():
        return None
    try:
        ref_runtime.load_b200_backend()
        full = wl.full()
        comp = ref_runtime.Compiled(full.with_backend("cuda"), "cuda", allow_tf32=wl.allow_tf32)
        comp.run(full.inputs)
        comp.time_run(20)
        iters = 200 if wl.key == "mlp" else 50
        ms = comp.time_run(iters) * 1e3
        comp.close()
        return {"ms_per_step": round(ms, 4), "runs": iters,
                "path": "runtime::compile(graph, \"cuda\") -> Executable::run through the C++ adapter, resident tensors"}
    except Exception as e:   # the leg is informational: the plan path above is what the line reports
        return {"error": str(e)[:200]}


# ---- the reference CPU backend on a slab of the workload ---------------------------------------------
def slab_case(wl):
    """(IR text for backend cpu, inputs, units of the metric the slab stands for, description)."""
    from frame_public_b200 import configs, irtext
    full = wl.full()
    if wl.is_gemm:
        rows, n = configs.GEMM_SLAB_ROWS, wl.n
        dt = "bfloat16" if wl.gemm_dtype == "bf16" else "float32"
        g = irtext.IrGraph("cpu")
        va, vb, vbias = g.input(dt, (rows, n)), g.input(dt, (n, n)), g.input(dt, (rows, n))
        g.output(g.unary("gelu", g.add(g.matmul(va, vb), vbias)))
        ins = [full.inputs[0][:rows], full.inputs[1], full.inputs[2][:rows]]
        return g.text(), ins, 2.0 * rows * n * n / 1e12, f"the first {rows} rows of A (matmul, add, gelu)"
    ins = configs.slab_inputs(wl.key, full.inputs)
    units = float(wl.batch) if wl.key == "mlp" else 1.0
    what = "the whole batch" if wl.key == "mlp" else "sample 0 of the full-size batch"
    return configs.slab_graph(wl.key), ins, units, what


def slab_rows(wl, full_output):
    from frame_public_b200 import configs
    if wl.is_gemm:
        return full_output[:configs.GEMM_SLAB_ROWS]
    return configs.slab_of_output(wl.key, full_output)


def cpu_slab_baseline(wl, gpu_output):
    from oracle import ref_runtime
    from oracle import frame_oracle as fo
    from frame_public_b200 import configs
    if not ref_runtime.available():
        return ({"value": None, "unit": wl.unit, "cores": 0, "kind": "reference",
                 "sample": "oracle/_ref (the reference build) is not present on this box"}, None)
    ref_runtime.load_b200_backend()   # CPU kernels of the ops the reference lacks (gelu, silu, ...)
    text, ins, units, what = slab_case(wl)
    comp = ref_runtime.Compiled(text, "cpu")
    t0 = time.time()
    (expected,) = comp.run(ins)
    dt = time.time() - t0
    runs = 1
    if dt < 2.0:   # a short slab: repeat it for about three seconds
        runs = int(max(2, min(2000, 3.0 / max(dt, 1e-4))))
        dt = comp.time_run(runs)
    comp.close()
    cpu = {"value": units / dt, "unit": wl.unit, "cores": 1, "kind": "reference",
           "sample": f"{what} through the reference CPU backend's compiled graph, {dt:.2f} s per run"
                     f"{'' if runs == 1 else f' (mean of {runs})'} on one core (the backend is single-threaded)"}
    dtype = wl.full().dtype
    got = slab_rows(wl, gpu_output)
    tol = configs.parity_tolerance(wl.key, dtype, wl.allow_tf32, fo.to_accum(expected, dtype), wl.full().inputs)
    max_abs, _ = fo.max_err(got, expected, dtype)
    # relative error only where the expected value is above the absolute bound (at an expected value of
    # zero a ratio says nothing); worst_over_bound is |difference| / (atol + rtol |expected|), at most 1
    a64 = fo.to_accum(got, dtype).astype(np.float64)
    e64 = fo.to_accum(expected, dtype).astype(np.float64)
    diff = np.abs(a64 - e64)
    big = np.abs(e64) > float(tol["atol"])
    max_rel = float((diff[big] / np.abs(e64[big])).max(initial=0.0))
    worst = float((diff / (float(tol["atol"]) + float(tol["rtol"]) * np.abs(e64))).max(initial=0.0))
    parity = {"rows": int(np.prod(expected.shape[:-1])), "elements": int(expected.size), "max_abs": max_abs,
              "max_rel": max_rel, "worst_over_bound": worst, "rtol": tol["rtol"], "atol": tol["atol"],
              "ok": bool(fo.all_close(got, expected, dtype, **tol)),
              "against": "the reference CPU backend on the same seeded inputs, " + what}
    return cpu, parity


# ---- extra legs of the default workload: batch-sharded Mamba block, column-split GEMM ------------------
def default_workload_extras(args, rank, local_rank, world, device, stream, dist, wl, pb):
    from frame_public_b200 import capi, sharding
    lib = capi.load()
    out = {}

    def barrier():
        pb.sync()
        if dist is not None:
            dist.barrier()

    # (1) the Mamba block (batch 16, sequence 2048) batch-sharded over the ranks: samples/s of the job
    mw = Workload("mamba")
    mpb = PlanBench(mw, rank, world, device, stream)
    for _ in range(3):
        mpb.run()
    barrier()
    ms = max_over_ranks(dist, local_rank, mpb.timed_steps(args.steps)) / args.steps
    if capi.kernel_status(device) != 0:
        raise SystemExit("bench.py: a bounded wait gave up inside a kernel of the Mamba plan")
    out["batch_sharded"] = {"workload": mw.name, "plan_per_rank": mpb.plan_name, "samples_per_s": round(mw.units_total / (ms / 1e3), 1),
                            "ms_per_step": round(ms, 4), "unit": "samples/s", "scaling": "strong",
                            "partition": f"{mw.batch // world} of {mw.batch} samples per rank, no collective",
                            "launches_per_step": mpb.plan.launches_per_run}
    del mpb

    # (2) column-split GEMM: rank j multiplies A by its column block of B; the epilogue stores the block
    # into every rank's C through peer pointers (plain stores over NVLink), so each GPU ends with all of C
    if world > 1 and wl.is_gemm:
        from frame_public_b200 import colsplit
        n = wl.n
        es = 2 if wl.gemm_dtype == "bf16" else 4
        dt = capi.BF16 if wl.gemm_dtype == "bf16" else capi.F32
        a, b, bias = wl.full().inputs
        nl = n // world
        cols = slice(rank * nl, (rank + 1) * nl)
        da = capi.DeviceBuffer.from_numpy(a, device)
        db = capi.DeviceBuffer.from_numpy(np.ascontiguousarray(b[:, cols]), device)
        dbias = capi.DeviceBuffer.from_numpy(np.ascontiguousarray(bias[:, cols]), device)
        c = colsplit.PeerMatrix(n * n * es, rank, world, device, dist)
        epi = capi.make_epilogue([("add", dbias.ptr, capi.OPERAND_FULL), ("gelu", None, 0)])

        def step():
            colsplit.matmul_colsplit(da.ptr, db.ptr, c, n, n, n, dt, wl.allow_tf32, epi, stream)

        for _ in range(3):
            step()
        barrier()
        ev = pb.events
        capi.check(lib.fb200_event_record(device, ev[0], stream))
        for _ in range(args.steps):
            step()
        capi.check(lib.fb200_event_record(device, ev[1], stream))
        barrier()
        cms = max_over_ranks(dist, local_rank, pb.elapsed(ev[0], ev[1])) / args.steps
        status = capi.kernel_status(device)
        bytes_in = n * n * es * (world - 1) / world
        same = None
        if rank == 0:
            from oracle import frame_oracle as fo
            rows = 16
            got = c.local.download(capi.NP_STORAGE[dt], (n, n))[:rows]
            exp = pb.output_host(0)[:rows]
            dcode = wl.full().dtype
            same = bool(status == 0 and fo.all_close(got, exp, dcode, rtol=2e-2 if es == 2 else 1e-3, atol=2e-3))
        out["colsplit"] = {"ms": round(cms, 4), "tflops": round(2.0 * n ** 3 / 1e12 / (cms / 1e3), 1),
                           "nvlink_bytes_in_per_gpu": int(bytes_in),
                           "nvlink_gbs_in_per_gpu": round(bytes_in / 1e9 / (cms / 1e3), 1),
                           "nvlink_peak_gbs": 770.0, "peak_source": "measured peer copy per direction on this pool (900 nominal)",
                           "how": "tcgen05 GEMM on this rank's column block, epilogue stores to every rank's C over NVLink (peer pointers, no multicast)",
                           "first_rows_match_row_sharded_result": same, "kernel_status": status}
        barrier()
        c.close()
    return out


# ---- reference arm ------------------------------------------------------------------------------------
REF_GEMM_ROWS = 8   # rows of A per process per step


def gelu_composition_graph(rows, n, dt):
    """matmul -> add -> tanh-GELU written with reference-native ops only (mul, add, square, tanh); the
    four constants are full-shape inputs because the reference's add/mul do not broadcast."""
    from frame_public_b200 import irtext
    g = irtext.IrGraph("cpu")
    va, vb, vbias = g.input(dt, (rows, n)), g.input(dt, (n, n)), g.input(dt, (rows, n))
    c_half, c_one, c_k, c_c = (g.input(dt, (rows, n)) for _ in range(4))
    x = g.add(g.matmul(va, vb), vbias)
    x3 = g.mul(g.unary("square", x), x)
    inner = g.mul(c_k, g.add(x, g.mul(c_c, x3)))
    g.output(g.mul(g.mul(c_half, x), g.add(c_one, g.unary("tanh", inner))))
    return g.text()


def _ref_worker(args_tuple):
    name, steps, warmup, seed = args_tuple
    sys.path.insert(0, ROOT)
    from oracle import ref_runtime
    from frame_public_b200 import configs
    wl = Workload(name)
    if wl.is_gemm:
        # the unmodified reference only: GELU as a composition of its own ops
        rows, n = REF_GEMM_ROWS, wl.n
        bf = wl.gemm_dtype == "bf16"
        conv = configs._bf16 if bf else (lambda x: x)
        rng = np.random.default_rng(seed)
        ins = [conv(rng.uniform(-1, 1, (rows, n)).astype(np.float32)), conv(rng.uniform(-1, 1, (n, n)).astype(np.float32)),
               conv(rng.normal(0, 0.1, (rows, n)).astype(np.float32))]
        ins += [conv(np.full((rows, n), v, np.float32)) for v in (0.5, 1.0, 0.7978845608028654, 0.044715)]
        text, units = gelu_composition_graph(rows, n, "bfloat16" if bf else "float32"), 2.0 * rows * n * n / 1e12
    else:
        if wl.key in ("transformer", "mamba"):
            ref_runtime.load_b200_backend()   # gelu / silu / softplus / mamba_scan are not reference ops
        text, ins, units, _ = slab_case(wl)
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
    wl = Workload(args.workload)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not ref_runtime.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref (the reference CPU backend built from its sources) is not present"}))
        return
    import multiprocessing as mp
    cores = os.cpu_count() or 1
    procs = max(1, min(cores, 64))
    warm = max(0, args.warmup)
    steps = max(1, args.steps)
    ctx = mp.get_context("spawn")
    with ctx.Pool(procs) as pool:
        res = pool.map(_ref_worker, [(args.workload, steps, warm, 100 + i) for i in range(procs)])
    t_step = max(r[0] for r in res)
    units = sum(r[1] for r in res)
    value = units / t_step
    if wl.is_gemm:
        sample = (f"{procs} processes x {REF_GEMM_ROWS} rows of A per step through the unmodified reference CPU backend's "
                  f"compiled graph (matmul, add, tanh-GELU composed of mul/add/square/tanh); the backend is single-threaded")
    else:
        sample = (f"{procs} processes x sample 0 of the full-size batch per step through the reference CPU backend's compiled graph"
                  + ("; gelu/silu/softplus/mamba_scan are not reference ops: their CPU kernels come from this repository's plugin"
                     if wl.key in ("transformer", "mamba") else ""))
    line = {
        "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world,
        "steps": steps, "warmup": warm, "ms_per_step": t_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": wl.arith, "data": "synthetic", "impl": "reference",
        "config": bench_config(wl, world),
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": procs, "kind": "reference", "sample": sample},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the batch-sharded Mamba and column-split legs")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second back-to-back leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
