"""Times one kernel of libframe_b200.so through the C ABI with CUDA events, and prints one JSON
line: launch time, algorithmic bytes or FLOPs per launch, achieved rate and the fraction of the
measured peak (the peaks file at the repository root, when present).

    python -m frame_public_b200.microbench --op scan_rows --rows 32768 --cols 2048 --dtype f32
    python -m frame_public_b200.microbench --op fused_add_relu --numel 67108864
    python -m frame_public_b200.microbench --op gemm --m 4096 --n 4096 --k 4096 --dtype bf16

Ops: fused_add_relu, gelu, silu, softmax, layer_norm, scan_rows, mamba_scan, transpose, slice,
max_pool, conv1d_depthwise, dwconv_time_major, conv2d_tf32, conv2d_stem, conv2d_stem_pool, attention (--batch, --cols = sequence length, --m = model
width), gemm.  Inputs are seeded random data; between timed
launches nothing is flushed, so choose sizes larger than the 126 MB L2 for HBM figures.  This is
also the command the ncu captures summarised under profiles/ were taken with.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"f32": capi.F32, "bf16": capi.BF16}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def _rand(shape, dtype, rng, lo=-1.0, hi=1.0):
    x = rng.uniform(lo, hi, shape).astype(np.float32)
    if dtype == capi.BF16:
        bits = x.view(np.uint32)
        x = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    return capi.DeviceBuffer.from_numpy(x)


def _time(fn, iters, warm):
    lib = capi.load()
    e0, e1 = capi.c_void_p(), capi.c_void_p()
    capi.check(lib.fb200_event_create(0, 1, capi.byref(e0)))
    capi.check(lib.fb200_event_create(0, 1, capi.byref(e1)))
    for _ in range(warm):
        fn()
    capi.synchronize()
    capi.check(lib.fb200_event_record(0, e0, None))
    for _ in range(iters):
        fn()
    capi.check(lib.fb200_event_record(0, e1, None))
    capi.check(lib.fb200_event_synchronize(0, e1))
    ms = capi.c_float(0)
    capi.check(lib.fb200_event_elapsed_ms(e0, e1, capi.byref(ms)))
    return ms.value / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True)
    ap.add_argument("--dtype", default="f32", choices=list(DT))
    ap.add_argument("--numel", type=int, default=64 * 1024 * 1024)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--cols", type=int, default=2048)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    if capi.device_count() < 1:
        raise SystemExit("microbench needs a B200: the library has no CPU fallback")
    dt = DT[a.dtype]
    es = capi.ITEMSIZE[dt]
    rng = np.random.default_rng(0)
    flops = 0.0
    if a.op in ("fused_add_relu", "gelu", "silu"):
        n = a.numel
        x, y, o = _rand((n,), dt, rng), _rand((n,), dt, rng), capi.DeviceBuffer(n * es)
        if a.op == "fused_add_relu":
            fn, nbytes = (lambda: capi.fused_elementwise([x.ptr, y.ptr], o.ptr, n, dt, ["add", "relu"])), 3 * n * es
        else:
            fn, nbytes = (lambda: capi.fused_elementwise([x.ptr], o.ptr, n, dt, [a.op])), 2 * n * es
    elif a.op in ("softmax", "layer_norm"):
        r, c = a.rows, a.cols
        x, o = _rand((r, c), dt, rng), capi.DeviceBuffer(r * c * es)
        g, b = _rand((c,), dt, rng), _rand((c,), dt, rng)
        fn = (lambda: capi.softmax(x.ptr, o.ptr, r, c, dt)) if a.op == "softmax" else \
             (lambda: capi.layer_norm(x.ptr, g.ptr, b.ptr, o.ptr, r, c, 1e-5, dt))
        nbytes = 2 * r * c * es
    elif a.op == "scan_rows":
        r, c = a.rows, a.cols
        ins = [_rand((r, c), dt, rng, 0.5, 0.99) for _ in range(5)]
        o = capi.DeviceBuffer(r * c * es)
        fn = lambda: capi.selective_scan(*[t.ptr for t in ins], o.ptr, r, c, dt)
        nbytes = 6 * r * c * es
    elif a.op == "mamba_scan":
        bt, L, dm, ns = a.batch, a.cols, a.m, 16
        u, d, z = _rand((bt, L, dm), capi.F32, rng), _rand((bt, L, dm), capi.F32, rng, 1e-3, 1e-1), _rand((bt, L, dm), capi.F32, rng)
        A = capi.DeviceBuffer.from_numpy(-np.tile(np.arange(1, ns + 1, dtype=np.float32), (dm, 1)))
        B, C, D = _rand((bt, L, ns), capi.F32, rng), _rand((bt, L, ns), capi.F32, rng), _rand((dm,), capi.F32, rng)
        y = capi.DeviceBuffer(bt * L * dm * 4)
        fn = lambda: capi.mamba_scan(u.ptr, d.ptr, A.ptr, B.ptr, C.ptr, D.ptr, z.ptr, y.ptr, bt, L, dm, ns)
        nbytes = (4 * bt * L * dm + 2 * bt * L * ns) * 4
    elif a.op == "transpose":
        bt, r, c = a.batch, a.rows, a.cols
        x, o = _rand((bt, r, c), dt, rng), capi.DeviceBuffer(bt * r * c * es)
        fn = lambda: capi.transpose(x.ptr, o.ptr, (bt, r, c), (0, 2, 1), es)
        nbytes = 2 * bt * r * c * es
    elif a.op == "slice":
        r, c = a.rows, a.cols
        x, o = _rand((r, c), dt, rng), capi.DeviceBuffer(r * (c // 2) * es)
        fn = lambda: capi.slice_(x.ptr, o.ptr, (r, c), 1, c // 2, c, es)
        nbytes = 2 * r * (c // 2) * es
    elif a.op == "max_pool":
        n, c, h = a.batch, 64, 112
        x, o = _rand((n, c, h, h), dt, rng), capi.DeviceBuffer(n * c * 56 * 56 * es)
        fn = lambda: capi.max_pool2d(x.ptr, o.ptr, n, c, h, h, 3, 3, 2, 2, 1, 1, dt)
        nbytes = (n * c * h * h + n * c * 56 * 56) * es
    elif a.op == "conv1d_depthwise":
        bt, ch, L = a.batch, a.m, a.cols
        x, w, b = _rand((bt, ch, L), dt, rng), _rand((ch, 1, 4), dt, rng), _rand((ch,), dt, rng)
        o = capi.DeviceBuffer(bt * ch * (L + 3) * es)
        fn = lambda: capi.conv1d(x.ptr, w.ptr, b.ptr, o.ptr, bt, ch, L, ch, 4, 1, 3, ch, dt)
        nbytes = (bt * ch * L + bt * ch * (L + 3)) * es
    elif a.op == "dwconv_time_major":
        # the Mamba block's causal conv: a 1536-wide window of the [batch*len, 3072] in_proj output
        bt, L, ch = a.batch, a.cols, a.m
        x, w, b = _rand((bt * L, 2 * ch), dt, rng), _rand((ch, 1, 4), dt, rng), _rand((ch,), dt, rng)
        o = capi.DeviceBuffer(bt * L * ch * es)
        fn = lambda: capi.dwconv1d_time_major(x.ptr, 2 * ch, w.ptr, b.ptr, o.ptr, ch, bt, L, L, ch, 4, -3, ["silu"], dt)
        nbytes = 2 * bt * L * ch * es
    elif a.op == "conv2d_tf32":
        n, cin, h, cout, k = a.batch, 64, 56, 64, 3
        x, w, b = _rand((n, cin, h, h), capi.F32, rng), _rand((cout, cin, k, k), capi.F32, rng), _rand((cout,), capi.F32, rng)
        o = capi.DeviceBuffer(n * cout * h * h * 4)
        p = capi.Conv2dParams(n, cin, h, h, cout, k, k, 1, 1, 1, 1, 1)
        fn = lambda: capi.conv2d(x.ptr, w.ptr, b.ptr, o.ptr, p, capi.F32, True)
        nbytes = (n * cin * h * h + n * cout * h * h) * 4
        flops = 2.0 * n * cout * h * h * cin * k * k
    elif a.op in ("conv2d_stem", "conv2d_stem_pool"):
        # the conv-stack workload's stem: 3 -> 64 channels, 7x7, stride 2, pad 3, + ReLU; _pool adds the
        # 3x3 / stride-2 max-pool through fb200_conv2d_max_pool (one kernel)
        n, cin, h, cout, k = a.batch, 3, 224, 64, 7
        oh, ph = 112, 56
        x, w, b = _rand((n, cin, h, h), capi.F32, rng), _rand((cout, cin, k, k), capi.F32, rng), _rand((cout,), capi.F32, rng)
        p = capi.Conv2dParams(n, cin, h, h, cout, k, k, 2, 2, 3, 3, 1)
        epi = capi.make_epilogue([("relu", None, 0)])
        if a.op == "conv2d_stem":
            o = capi.DeviceBuffer(n * cout * oh * oh * 4)
            fn = lambda: capi.conv2d(x.ptr, w.ptr, b.ptr, o.ptr, p, capi.F32, True, epi)
            nbytes = (n * cin * h * h + n * cout * oh * oh) * 4
        else:
            o = capi.DeviceBuffer(n * cout * ph * ph * 4)
            fn = lambda: capi.conv2d_max_pool(x.ptr, w.ptr, b.ptr, None, o.ptr, p, (3, 3, 2, 2, 1, 1), capi.F32, True, epi)
            nbytes = (n * cin * h * h + n * cout * ph * ph) * 4
        flops = 2.0 * n * cout * oh * oh * cin * k * k
    elif a.op == "attention":
        # the transformer workload's layout: [batch*seq, 3*heads*64] projection, 64-wide heads
        bt, seq, heads = a.batch, a.cols, a.m // 64
        width = heads * 64
        qkv = _rand((bt * seq, 3 * width), capi.BF16, rng)
        o = capi.DeviceBuffer(bt * seq * width * 2)
        table = np.zeros(bt * heads, dtype=capi.HEAD_DTYPE)
        for b in range(bt):
            for h in range(heads):
                table[b * heads + h] = (b * seq, h * 64, b * seq, width + h * 64, b * seq,
                                        2 * width + h * 64, b * seq * width + h * 64)
        tab = capi.DeviceBuffer.from_numpy(table.view(np.uint8))
        rows, ld = bt * seq, 3 * width
        fn = lambda: capi.attention_fan(qkv.ptr, rows, ld, qkv.ptr, rows, ld, qkv.ptr, rows, ld, o.ptr, width,
                                        tab.ptr, len(table), seq, seq, 64, capi.BF16)
        nbytes = 4 * bt * seq * width * 2
        flops = 4.0 * bt * heads * seq * seq * 64
    elif a.op == "gemm":
        m, n, k = a.m, a.n, a.k
        x, w, o = _rand((m, k), dt, rng), _rand((k, n), dt, rng), capi.DeviceBuffer(m * n * es)
        fn = lambda: capi.matmul(x.ptr, w.ptr, o.ptr, m, n, k, dt, True)
        nbytes = (m * k + k * n + m * n) * es
        flops = 2.0 * m * n * k
    else:
        raise SystemExit(f"unknown op {a.op}")
    ms = _time(fn, a.iters, a.warmup)
    assert capi.kernel_status(0) == 0
    peaks, src = _peaks()
    line = {"op": a.op, "dtype": a.dtype, "ms_per_launch": round(ms, 5), "bytes_per_launch": int(nbytes),
            "gbs": round(nbytes / ms / 1e6, 1), "hbm_frac": round(nbytes / ms / 1e6 / peaks["hbm_gbs"], 4),
            "peaks": src}
    if flops:
        line["flops_per_launch"] = flops
        line["tflops"] = round(flops / ms / 1e9, 1)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
