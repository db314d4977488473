"""Seeded single-op parity cases shared by the golden-vector generator, the oracle pin tests
(CPU) and the C-ABI parity tests (GPU).  Shapes follow the reference's own CUDA-vs-CPU
differential tests (tests/cpp/backends/test_cuda_backend.cpp:1174-2345 of the reference: the
1023/1024 vectorisation boundary, odd shapes, zero-size tensors) and the five benchmark workloads
in miniature.  Every case names the reference op, its attributes and its inputs in storage form
(uint16 bit patterns for bf16)."""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field
from typing import Callable, Dict, List

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import frame_oracle as fo  # noqa: E402
from frame_public_b200 import irtext  # noqa: E402

F32, BF16, I32, I64 = fo.DT_F32, fo.DT_BF16, fo.DT_I32, fo.DT_I64


@dataclass
class Case:
    name: str
    op: str
    dtype: int
    inputs: List[np.ndarray]
    attrs: Dict[str, object] = field(default_factory=dict)
    oracle: Callable[..., np.ndarray] = None
    exact: bool = False       # integer/indexing work or fp32 without libm: bit-exact expected
    new_op: bool = False      # no golden from the reference CPU backend: an op that is not in the reference, or
                              # one whose CPU kernel needs a library that is absent here (rfft / irfft: pocketfft)
    in_dtypes: List[int] = None   # dtype code per input when they differ from `dtype` (indices)

    def expected(self) -> np.ndarray:
        return self.oracle(*self.inputs)

    def ir_text(self, backend: str = "cpu") -> str:
        g = irtext.IrGraph(backend)
        dt = irtext.DTYPE_NAMES[self.dtype]
        in_dts = self.in_dtypes or [self.dtype] * len(self.inputs)
        vals = [g.input(irtext.DTYPE_NAMES[d], a.shape) for d, a in zip(in_dts, self.inputs)]
        out_shape = self.expected().shape
        attrs = dict(self.attrs)
        for key in ("target_shape", "output_shape", "input_shape", "filter_shape"):
            if key in attrs:
                attrs[key] = irtext.Shape(tuple(attrs[key]))
        out = g.node(self.op, vals, attrs, dt, out_shape)
        g.output(out)
        return g.text()


def _store(x, dtype):
    return fo.from_accum(np.asarray(x, dtype=np.float32), dtype) if dtype in (F32, BF16) else x


def _rng(seed):
    return np.random.default_rng(seed)


def build_cases() -> List[Case]:
    cases: List[Case] = []
    seed = [1000]

    def rnd(shape, dtype=F32, lo=None, scale=1.0):
        seed[0] += 1
        r = _rng(seed[0])
        if lo is not None:
            v = r.uniform(lo[0], lo[1], size=shape).astype(np.float32)
        else:
            v = (r.standard_normal(size=shape) * scale).astype(np.float32)
        return _store(v, dtype)

    # ---- matmul ----------------------------------------------------------------------------
    for name, (m, k, n), dt in [("matmul_f32_5x7x3", (5, 7, 3), F32),
                                ("matmul_f32_64x784x256", (64, 784, 256), F32),
                                ("matmul_f32_33x17x9", (33, 17, 9), F32),
                                ("matmul_f32_64x256x10", (64, 256, 10), F32),
                                ("matmul_f32_130x70x200", (130, 70, 200), F32),
                                ("matmul_bf16_64x64x64", (64, 64, 64), BF16),
                                ("matmul_bf16_37x50x21", (37, 50, 21), BF16)]:
        a, b = rnd((m, k), dt, lo=(-1, 1)), rnd((k, n), dt, lo=(-1, 1))
        cases.append(Case(name, "matmul", dt, [a, b], {}, lambda a, b, dt=dt: fo.matmul(a, b, dt),
                          exact=True))

    # ---- elementwise and fused groups --------------------------------------------------------
    for dt, tag in [(F32, "f32"), (BF16, "bf16")]:
        for n in (1023, 1024, 5):
            for op in ("add", "mul"):
                cases.append(Case(f"{op}_{tag}_{n}", op, dt, [rnd((n,), dt), rnd((n,), dt)], {},
                                  lambda a, b, op=op, dt=dt: fo.BINARY[op](a, b, dt), exact=True))
            for op in ("relu", "square"):
                cases.append(Case(f"{op}_{tag}_{n}", op, dt, [rnd((n,), dt)], {},
                                  lambda a, op=op, dt=dt: fo.UNARY[op](a, dt), exact=True))
            for op in ("sigmoid", "tanh"):
                cases.append(Case(f"{op}_{tag}_{n}", op, dt, [rnd((n,), dt, scale=3.0)], {},
                                  lambda a, op=op, dt=dt: fo.UNARY[op](a, dt)))
            cases.append(Case(f"rsqrt_{tag}_{n}", "rsqrt", dt, [rnd((n,), dt, lo=(0.01, 9.0))], {},
                              lambda a, dt=dt: fo.rsqrt(a, dt), exact=True))
        for chain, ar in [("add;relu", [2, 1]), ("add;mul;relu", [2, 2, 1]),
                          ("relu;add", [1, 2]), ("square;add;mul;relu", [1, 2, 2, 1])]:
            n_in = sum(ar) - (len(ar) - 1)
            ins = [rnd((6, 171), dt) for _ in range(n_in)]
            cases.append(Case(f"fused_{chain.replace(';', '_')}_{tag}", "fused_elementwise_internal",
                              dt, ins, {"ops": chain, "arities": ar},
                              lambda *xs, chain=chain, ar=ar, dt=dt: fo.fused_elementwise(list(xs), chain, ar, dt),
                              exact=True))
    for dt, tag, npdt in [(I32, "i32", np.int32), (I64, "i64", np.int64)]:
        r = _rng(77)
        a = r.integers(-1000, 1000, size=(1023,)).astype(npdt)
        b = r.integers(-1000, 1000, size=(1023,)).astype(npdt)
        cases.append(Case(f"add_{tag}_1023", "add", dt, [a, b], {}, lambda a, b, dt=dt: fo.add(a, b, dt),
                          exact=True))

    # ---- row kernels -------------------------------------------------------------------------
    for name, shape, dt in [("softmax_f32_64x10", (64, 10), F32), ("softmax_f32_5x33", (5, 33), F32),
                            ("softmax_f32_9x512", (9, 512), F32), ("softmax_bf16_8x512", (8, 512), BF16),
                            ("softmax_bf16_3x40", (3, 40), BF16), ("softmax_f32_2x4100", (2, 4100), F32)]:
        cases.append(Case(name, "softmax", dt, [rnd(shape, dt, scale=2.0)], {},
                          lambda x, dt=dt: fo.softmax(x, dt)))
    for name, shape, dt in [("layer_norm_f32_4x100", (4, 100), F32), ("layer_norm_f32_7x1024", (7, 1024), F32),
                            ("layer_norm_bf16_7x1024", (7, 1024), BF16), ("layer_norm_bf16_5x24", (5, 24), BF16)]:
        g = _store(1.0 + 0.1 * _rng(5).standard_normal(shape[1]).astype(np.float32), dt)
        b = _store(0.1 * _rng(6).standard_normal(shape[1]).astype(np.float32), dt)
        cases.append(Case(name, "layer_norm", dt, [rnd(shape, dt), g, b], {"eps": 1e-5},
                          lambda x, g, b, dt=dt: fo.layer_norm(x, g, b, 1e-5, dt)))

    # ---- selective scan ----------------------------------------------------------------------
    for name, shape, dt in [("scan_f32_3x5x37", (3, 5, 37), F32), ("scan_f32_70x64", (70, 64), F32),
                            ("scan_f32_2x2048", (2, 2048), F32), ("scan_bf16_40x96", (40, 96), BF16),
                            ("scan_f32_1", (1,), F32), ("scan_f32_0x3", (0, 3), F32)]:
        x = rnd(shape, dt)
        a = rnd(shape, dt, lo=(0.5, 0.99))
        b, c, d = rnd(shape, dt), rnd(shape, dt), rnd(shape, dt)
        exact = name != "scan_f32_2x2048"  # few long rows take the time-parallel kernel
        cases.append(Case(name, "selective_scan", dt, [x, a, b, c, d], {},
                          lambda x, a, b, c, d, dt=dt: fo.selective_scan(x, a, b, c, d, dt), exact=exact))

    # ---- conv / pool ---------------------------------------------------------------------------
    def conv_case(name, xs, ws, stride, padding, groups, bias, dt=F32):
        x, w = rnd(xs, dt), rnd(ws, dt, scale=0.3)
        ins = [x, w] + ([rnd((ws[0],), dt)] if bias else [])
        cases.append(Case(name, "conv2d", dt, ins,
                          {"stride": list(stride), "padding": list(padding), "groups": groups},
                          lambda x, w, b=None, dt=dt: fo.conv2d(x, w, b, stride, padding, groups, dt),
                          exact=True))

    conv_case("conv2d_f32_3x3_s1_p1", (2, 3, 9, 9), (4, 3, 3, 3), (1, 1), (1, 1), 1, True)
    conv_case("conv2d_f32_7x7_s2_p3", (1, 3, 20, 20), (8, 3, 7, 7), (2, 2), (3, 3), 1, True)
    conv_case("conv2d_f32_groups2", (2, 4, 6, 7), (6, 2, 3, 2), (1, 2), (0, 1), 2, False)
    conv_case("conv2d_f32_64ch_3x3", (2, 64, 10, 10), (64, 64, 3, 3), (1, 1), (1, 1), 1, True)
    conv_case("conv2d_bf16_3x3", (1, 4, 8, 8), (5, 4, 3, 3), (1, 1), (1, 1), 1, True, BF16)
    xs, ws = (2, 6, 20), (6, 1, 4)
    cases.append(Case("conv1d_f32_depthwise_causal", "conv1d", F32,
                      [rnd(xs), rnd(ws, scale=0.5), rnd((6,))], {"stride": 1, "padding": 3, "groups": 6},
                      lambda x, w, b: fo.conv1d(x, w, b, 1, 3, 6, F32), exact=True))
    cases.append(Case("conv1d_f32_dense_s2", "conv1d", F32, [rnd((2, 4, 15)), rnd((3, 4, 3), scale=0.5)],
                      {"stride": 2, "padding": 1, "groups": 1},
                      lambda x, w: fo.conv1d(x, w, None, 2, 1, 1, F32), exact=True))
    tie = np.array([[[[5, 5, 1, 2], [5, 5, 2, 2], [1, 1, 3, 3], [0, 1, 3, 3]]]], dtype=np.float32)
    cases.append(Case("max_pool2d_f32_ties", "max_pool2d", F32, [tie],
                      {"kernel": [2, 2], "stride": [2, 2], "padding": [0, 0]},
                      lambda x: fo.max_pool2d(x, (2, 2), (2, 2), (0, 0), F32), exact=True))
    cases.append(Case("max_pool2d_f32_k3_s2_p1", "max_pool2d", F32, [rnd((2, 3, 9, 11))],
                      {"kernel": [3, 3], "stride": [2, 2], "padding": [1, 1]},
                      lambda x: fo.max_pool2d(x, (3, 3), (2, 2), (1, 1), F32), exact=True))
    cases.append(Case("max_pool2d_bf16_k3_s2_p1", "max_pool2d", BF16, [rnd((1, 2, 8, 8), BF16)],
                      {"kernel": [3, 3], "stride": [2, 2], "padding": [1, 1]},
                      lambda x: fo.max_pool2d(x, (3, 3), (2, 2), (1, 1), BF16), exact=True))

    # ---- data movement ---------------------------------------------------------------------------
    for name, shape, perm, dt in [("transpose_f32_5x7", (5, 7), (1, 0), F32),
                                  ("transpose_f32_2x33x65_021", (2, 33, 65), (0, 2, 1), F32),
                                  ("transpose_bf16_3x40x24_021", (3, 40, 24), (0, 2, 1), BF16),
                                  ("transpose_f32_2x3x4_201", (2, 3, 4), (2, 0, 1), F32),
                                  ("transpose_f32_2x3x4x5_0213", (2, 3, 4, 5), (0, 2, 1, 3), F32)]:
        cases.append(Case(name, "transpose", dt, [rnd(shape, dt)], {"perm": list(perm)},
                          lambda x, perm=perm: fo.transpose(x, perm), exact=True))
    cases.append(Case("slice_f32_cols", "slice", F32, [rnd((6, 30))], {"axis": 1, "start": 10, "stop": 20},
                      lambda x: fo.slice_(x, 1, 10, 20), exact=True))
    cases.append(Case("slice_bf16_odd", "slice", BF16, [rnd((3, 7, 5), BF16)], {"axis": 1, "start": 1, "stop": 4},
                      lambda x: fo.slice_(x, 1, 1, 4), exact=True))
    cases.append(Case("concat_f32_axis1", "concat", F32, [rnd((4, 3)), rnd((4, 5)), rnd((4, 8))], {"axis": 1},
                      lambda *xs: fo.concat(xs, 1), exact=True))
    cases.append(Case("concat_bf16_axis0", "concat", BF16, [rnd((2, 6), BF16), rnd((3, 6), BF16)], {"axis": 0},
                      lambda *xs: fo.concat(xs, 0), exact=True))
    cases.append(Case("reshape_f32", "reshape", F32, [rnd((4, 6))], {"target_shape": (2, 12)},
                      lambda x: fo.reshape(x, (2, 12)), exact=True))
    cases.append(Case("sum_f32_axis2of4", "sum", F32, [rnd((2, 5, 16, 24))], {"axes": [2]},
                      lambda x: fo.sum_axes(x, [2], False, F32), exact=True))
    cases.append(Case("sum_f32_last", "sum", F32, [rnd((7, 33))], {"axes": [1]},
                      lambda x: fo.sum_axes(x, [1], False, F32), exact=True))

    # ---- new ops (not in the reference) ------------------------------------------------------------
    for dt, tag in [(F32, "f32"), (BF16, "bf16")]:
        for op in ("gelu", "silu", "softplus", "exp"):
            cases.append(Case(f"{op}_{tag}_1023", op, dt, [rnd((1023,), dt, scale=2.0)], {},
                              lambda a, op=op, dt=dt: fo.UNARY[op](a, dt), new_op=True))
        cases.append(Case(f"bias_add_{tag}", "bias_add", dt, [rnd((9, 40), dt), rnd((40,), dt)], {},
                          lambda x, b, dt=dt: fo.bias_add(x, b, dt), exact=True, new_op=True))
    # ---- ops added after the first golden set (kept last so that earlier seeded draws do not move) --
    cases.append(Case("avg_pool2d_f32_k3_s2_p1", "avg_pool2d", F32, [rnd((2, 3, 9, 11))],
                      {"kernel": [3, 3], "stride": [2, 2], "padding": [1, 1]},
                      lambda x: fo.avg_pool2d(x, (3, 3), (2, 2), (1, 1), F32), exact=True))
    cases.append(Case("avg_pool2d_f32_k2_s2", "avg_pool2d", F32, [rnd((1, 4, 8, 6))],
                      {"kernel": [2, 2], "stride": [2, 2], "padding": [0, 0]},
                      lambda x: fo.avg_pool2d(x, (2, 2), (2, 2), (0, 0), F32), exact=True))
    cases.append(Case("avg_pool2d_bf16_k3_s1_p1", "avg_pool2d", BF16, [rnd((1, 2, 7, 7), BF16)],
                      {"kernel": [3, 3], "stride": [1, 1], "padding": [1, 1]},
                      lambda x: fo.avg_pool2d(x, (3, 3), (1, 1), (1, 1), BF16), exact=True))
    cases.append(Case("heaviside_f32_1023", "heaviside_surrogate", F32,
                      [np.concatenate([rnd((1021,)), np.array([0.0, -0.0], np.float32)])], {"alpha": 2.0},
                      lambda x: fo.heaviside_surrogate(x, F32), exact=True))
    cases.append(Case("heaviside_bf16_40x9", "heaviside_surrogate", BF16, [rnd((40, 9), BF16)], {"alpha": 1.0},
                      lambda x: fo.heaviside_surrogate(x, BF16), exact=True))

    # ---- gather / scatter_add (indices int32 or int64, repeated indices accumulate) -----------------
    idx_a = _rng(41).integers(0, 13, size=(29,))
    for tag, idt, npdt in (("i32", I32, np.int32), ("i64", I64, np.int64)):
        cases.append(Case(f"gather_f32_13x20_{tag}", "gather", F32, [rnd((13, 20)), idx_a.astype(npdt)], {},
                          lambda x, i: fo.gather(x, i), exact=True, in_dtypes=[F32, idt]))
        cases.append(Case(f"scatter_add_f32_29x20_{tag}", "scatter_add", F32, [rnd((29, 20)), idx_a.astype(npdt)],
                          {"output_shape": [13, 20]},
                          lambda u, i: fo.scatter_add(u, i, (13, 20), F32), in_dtypes=[F32, idt]))
    cases.append(Case("gather_bf16_13x7_i64", "gather", BF16, [rnd((13, 7), BF16), idx_a.astype(np.int64)], {},
                      lambda x, i: fo.gather(x, i), exact=True, in_dtypes=[BF16, I64]))
    cases.append(Case("scatter_add_bf16_29x8_i32", "scatter_add", BF16, [rnd((29, 8), BF16), idx_a.astype(np.int32)],
                      {"output_shape": [13, 8]},
                      lambda u, i: fo.scatter_add(u, i, (13, 8), BF16), in_dtypes=[BF16, I32]))
    cases.append(Case("gather_grad_f32_29x5_i64", "gather_grad_internal", F32, [rnd((29, 5)), idx_a.astype(np.int64)],
                      {"input_shape": [13, 5]},
                      lambda u, i: fo.scatter_add(u, i, (13, 5), F32), in_dtypes=[F32, I64]))

    cases.append(Case("max_pool2d_f32_k3_s2_p1_w16", "max_pool2d", F32, [rnd((2, 3, 10, 16))],
                      {"kernel": [3, 3], "stride": [2, 2], "padding": [1, 1]},
                      lambda x: fo.max_pool2d(x, (3, 3), (2, 2), (1, 1), F32), exact=True))

    # ---- gradient-side internals of pooling and convolution (bit-exact: gathers in the CPU's order) --
    pool_geoms = [("k3_s2_p1", (2, 3, 9, 11), (3, 3), (2, 2), (1, 1)), ("k2_s2", (1, 4, 8, 6), (2, 2), (2, 2), (0, 0)),
                  ("k3_s1_p1", (1, 2, 7, 7), (3, 3), (1, 1), (1, 1)), ("k3x2_s2x1_p1x0", (2, 2, 10, 5), (3, 2), (2, 1), (1, 0))]
    for tag, xs, k, st, pd in pool_geoms:
        oshape = (xs[0], xs[1], fo.conv_out_size(xs[2], k[0], st[0], pd[0]), fo.conv_out_size(xs[3], k[1], st[1], pd[1]))
        pat = {"kernel": list(k), "stride": list(st), "padding": list(pd)}
        for dt, dtag in ((F32, "f32"), (BF16, "bf16")):
            if dt == BF16 and tag != "k3_s2_p1":
                continue
            cases.append(Case(f"max_pool2d_select_{dtag}_{tag}", "max_pool2d_select_internal", dt,
                              [rnd(xs, dt), rnd(xs, dt)], dict(pat),
                              lambda g, x, k=k, st=st, pd=pd, dt=dt: fo.max_pool2d_select(g, x, k, st, pd, dt), exact=True))
            cases.append(Case(f"max_pool2d_grad_{dtag}_{tag}", "max_pool2d_grad_internal", dt,
                              [rnd(oshape, dt), rnd(xs, dt)], dict(pat, input_shape=list(xs)),
                              lambda dy, x, k=k, st=st, pd=pd, dt=dt: fo.max_pool2d_grad(dy, x, k, st, pd, dt), exact=True))
            cases.append(Case(f"avg_pool2d_grad_{dtag}_{tag}", "avg_pool2d_grad_internal", dt,
                              [rnd(oshape, dt)], dict(pat, input_shape=list(xs)),
                              lambda dy, xs=xs, k=k, st=st, pd=pd, dt=dt: fo.avg_pool2d_grad(dy, xs, k, st, pd, dt), exact=True))
    tie_x = np.array([[[[5, 5, 1, 2], [5, 5, 2, 2], [1, 1, 3, 3], [0, 1, 3, 3]]]], dtype=np.float32)
    cases.append(Case("max_pool2d_grad_f32_ties_overlap", "max_pool2d_grad_internal", F32,
                      [rnd((1, 1, 3, 3)), tie_x], {"kernel": [2, 2], "stride": [1, 1], "padding": [0, 0], "input_shape": [1, 1, 4, 4]},
                      lambda dy, x: fo.max_pool2d_grad(dy, x, (2, 2), (1, 1), (0, 0), F32), exact=True))
    conv_geoms = [("3x3_s1_p1", (2, 3, 9, 9), (4, 3, 3, 3), (1, 1), (1, 1), 1, F32),
                  ("7x7_s2_p3", (1, 3, 20, 20), (8, 3, 7, 7), (2, 2), (3, 3), 1, F32),
                  ("groups2", (2, 4, 6, 7), (6, 2, 3, 2), (1, 2), (0, 1), 2, F32),
                  ("bf16_3x3", (1, 4, 8, 8), (5, 4, 3, 3), (1, 1), (1, 1), 1, BF16)]
    for tag, xs, ws, st, pd, groups, dt in conv_geoms:
        oshape = (xs[0], ws[0], fo.conv_out_size(xs[2], ws[2], st[0], pd[0]), fo.conv_out_size(xs[3], ws[3], st[1], pd[1]))
        cat = {"stride": list(st), "padding": list(pd), "groups": groups}
        cases.append(Case(f"conv2d_grad_input_{tag}", "conv2d_grad_input_internal", dt,
                          [rnd(oshape, dt), rnd(ws, dt, scale=0.3)], dict(cat, input_shape=list(xs)),
                          lambda dy, w, xs=xs, st=st, pd=pd, groups=groups, dt=dt: fo.conv2d_grad_input(dy, w, xs, st, pd, groups, dt),
                          exact=True))
        cases.append(Case(f"conv2d_grad_filter_{tag}", "conv2d_grad_filter_internal", dt,
                          [rnd(xs, dt), rnd(oshape, dt, scale=0.3)], dict(cat, filter_shape=list(ws)),
                          lambda x, dy, ws=ws, st=st, pd=pd, groups=groups, dt=dt: fo.conv2d_grad_filter(x, dy, ws, st, pd, groups, dt),
                          exact=True))

    # ---- training-side ops: gradients of matmul and relu, the MSE loss pair, a full reduction ---------
    for tag, (m, k, n), dt in [("f32_5x7x3", (5, 7, 3), F32), ("f32_64x96x40", (64, 96, 40), F32),
                               ("bf16_33x17x9", (33, 17, 9), BF16)]:
        cases.append(Case(f"matmul_grad_lhs_{tag}", "matmul_grad_lhs_internal", dt, [rnd((m, n), dt), rnd((k, n), dt)], {},
                          lambda gy, b, dt=dt: fo.matmul_grad_lhs(gy, b, dt), exact=True))
        cases.append(Case(f"matmul_grad_rhs_{tag}", "matmul_grad_rhs_internal", dt, [rnd((m, k), dt), rnd((m, n), dt)], {},
                          lambda a, gy, dt=dt: fo.matmul_grad_rhs(a, gy, dt), exact=True))
    for dt, tag in ((F32, "f32"), (BF16, "bf16")):
        xz = rnd((1023,), dt)
        xz[:3] = _store(np.array([0.0, -0.0, 1e-30], np.float32), dt)
        cases.append(Case(f"relu_grad_{tag}_1023", "relu_grad_internal", dt, [xz, rnd((1023,), dt)], {},
                          lambda x, gy, dt=dt: fo.relu_grad(x, gy, dt), exact=True))
        cases.append(Case(f"mse_loss_{tag}_37x29", "mse_loss", dt, [rnd((37, 29), dt), rnd((37, 29), dt)], {},
                          lambda p, t, dt=dt: fo.mse_loss(p, t, dt), exact=True))
        cases.append(Case(f"mse_loss_grad_{tag}_37x29", "mse_loss_grad_internal", dt,
                          [rnd((37, 29), dt), rnd((37, 29), dt), np.asarray(rnd((), dt)).reshape(())], {},
                          lambda p, t, g, dt=dt: fo.mse_loss_grad(p, t, g, dt), exact=True))
    cases.append(Case("sum_f32_all_axes", "sum", F32, [rnd((7, 33))], {"axes": [0, 1]},
                      lambda x: fo.sum_axes(x, [0, 1], False, F32), exact=True))

    # ---- rfft / irfft (float32; the reference CPU kernel needs pocketfft, which is not in its tree:
    #      pinned by the reference's known-answer tests instead, tests/test_fft_cpu.py) ----------------
    for tag, shape in (("n4", (4,)), ("n5", (5,)), ("2x6", (2, 6)), ("3x64", (3, 64)), ("2x5x243", (2, 5, 243)),
                       ("7x1000", (7, 1000))):
        n = shape[-1]
        cases.append(Case(f"rfft_f32_{tag}", "rfft", F32, [rnd(shape)], {}, lambda x: fo.rfft(x), new_op=True))
        zshape = shape[:-1] + (n // 2 + 1, 2)
        cases.append(Case(f"irfft_f32_{tag}", "irfft", F32, [rnd(zshape)], {"n": n},
                          lambda z, n=n: fo.irfft(z, n), new_op=True))
    # a fused group longer than one launch holds (the reference's fusion pass builds chains of any
    # length, src/compiler/passes/operator_fusion.cpp:140-157): 12 steps, 8 external inputs
    long_chain = "add;relu;mul;square;add;relu;mul;add;relu;add;mul;relu"
    long_ar = [2, 1, 2, 1, 2, 1, 2, 2, 1, 2, 2, 1]
    for dt, tag in [(F32, "f32"), (BF16, "bf16")]:
        ins = [rnd((9, 1023), dt, scale=0.8) for _ in range(sum(long_ar) - (len(long_ar) - 1))]
        cases.append(Case(f"fused_long_chain_12_{tag}", "fused_elementwise_internal", dt, ins,
                          {"ops": long_chain, "arities": long_ar},
                          lambda *xs, dt=dt: fo.fused_elementwise(list(xs), long_chain, long_ar, dt), exact=True))
    return cases


CASES = build_cases()
CASES_BY_NAME = {c.name: c for c in CASES}
# Cases whose executable plan (as the reference derives it for backend "cuda") is committed under
# tests/golden/plans/case_<name>.plan and run through the plan executor.
PLAN_CASES = ["max_pool2d_select_f32_k3_s2_p1", "max_pool2d_grad_f32_k3_s2_p1", "max_pool2d_grad_bf16_k3_s2_p1",
              "avg_pool2d_grad_f32_k3x2_s2x1_p1x0", "conv2d_grad_input_groups2", "conv2d_grad_input_3x3_s1_p1",
              "conv2d_grad_filter_7x7_s2_p3", "conv2d_grad_filter_bf16_3x3"]
