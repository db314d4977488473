"""The five compiled-graph workloads (MLP, GEMM+epilogue, conv stack, transformer encoder block,
Mamba block) as Frame IR graphs with seeded synthetic inputs.

Each builder returns a `Workload`: the IR text (reference-native ops plus the new ops this
repository registers: gelu, silu, softplus, bias_add, mamba_scan), the input arrays in storage
form (uint16 bit patterns for bf16) in graph-input order, and the algorithmic FLOPs / bytes of one
run.  Inputs come from numpy's default_rng(seed) in the order listed; bf16 tensors are the fp32
draw rounded to nearest even.  Sizes are parameters so that tests run miniatures of the same
graphs.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

import numpy as np

from . import irtext

F32, BF16 = 0, 3


def _bf16(x: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (bits.astype(np.uint64) + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFFFFFF
    return (rounded >> 16).astype(np.uint16)


def _store(x, dtype):
    x = np.ascontiguousarray(x, dtype=np.float32)
    return _bf16(x) if dtype == BF16 else x


@dataclass
class Workload:
    name: str
    ir_text: str
    inputs: List[np.ndarray]
    dtype: int
    samples: int                 # samples one run processes
    flops: float                 # algorithmic FLOPs of one run
    bytes: float                 # algorithmic bytes of one run (inputs + weights + outputs once)
    allow_tf32: bool = False
    meta: Dict[str, object] = field(default_factory=dict)

    def with_backend(self, backend: str, device: int = 0) -> str:
        """The same graph addressed to another backend/device (`@cpu:0` <-> `@cuda:i`)."""
        import re
        return re.sub(r"@(cpu|cuda):\d+", f"@{backend}:{device}", self.ir_text)


def mlp(batch: int = 64, d_in: int = 784, hidden: int = 256, d_out: int = 10, seed: int = 0,
        backend: str = "cpu") -> Workload:
    """Config 1: Linear+ReLU, Linear+ReLU, Linear, softmax; fp32; full-shape zero biases (the
    reference's Linear convention)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, d_in)).astype(np.float32)

    def kaiming_uniform(fan_in, fan_out):
        bound = np.sqrt(6.0 / fan_in)
        return rng.uniform(-bound, bound, (fan_in, fan_out)).astype(np.float32)

    w1, w2, w3 = kaiming_uniform(d_in, hidden), kaiming_uniform(hidden, hidden), kaiming_uniform(hidden, d_out)
    b1 = np.zeros((batch, hidden), np.float32)
    b2 = np.zeros((batch, hidden), np.float32)
    b3 = np.zeros((batch, d_out), np.float32)
    g = irtext.IrGraph(backend)
    vx = g.input("float32", x.shape)
    vw1, vb1 = g.input("float32", w1.shape), g.input("float32", b1.shape)
    vw2, vb2 = g.input("float32", w2.shape), g.input("float32", b2.shape)
    vw3, vb3 = g.input("float32", w3.shape), g.input("float32", b3.shape)
    h = g.unary("relu", g.add(g.matmul(vx, vw1), vb1))
    h = g.unary("relu", g.add(g.matmul(h, vw2), vb2))
    out = g.softmax(g.add(g.matmul(h, vw3), vb3))
    g.output(out)
    ins = [x, w1, b1, w2, b2, w3, b3]
    flops = 2.0 * batch * (d_in * hidden + hidden * hidden + hidden * d_out)
    nbytes = sum(a.nbytes for a in ins) + batch * d_out * 4
    return Workload(f"mlp_f32_b{batch}", g.text(), ins, F32, batch, flops, nbytes)


def gemm_epilogue(n: int = 8192, dtype: int = BF16, seed: int = 1, m: int = None,
                  broadcast_bias: bool = False, backend: str = "cpu") -> Workload:
    """Config 2: C = GELU(A.B + bias), row-major, square by default.  The bias vector is
    replicated to a full [M,N] tensor for the reference-native `add` unless broadcast_bias."""
    m = n if m is None else m
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    b = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    bias = rng.normal(0, 0.1, (n,)).astype(np.float32)
    dt = irtext.DTYPE_NAMES[dtype]
    g = irtext.IrGraph(backend)
    va, vb = g.input(dt, a.shape), g.input(dt, b.shape)
    if broadcast_bias:
        vbias = g.input(dt, (n,))
        out = g.unary("gelu", g.bias_add(g.matmul(va, vb), vbias))
        bias_in = bias
    else:
        vbias = g.input(dt, (m, n))
        out = g.unary("gelu", g.add(g.matmul(va, vb), vbias))
        bias_in = np.tile(bias[None, :], (m, 1))
    g.output(out)
    ins = [_store(a, dtype), _store(b, dtype), _store(bias_in, dtype)]
    es = 2 if dtype == BF16 else 4
    flops = 2.0 * m * n * n
    nbytes = (m * n + n * n + bias_in.size + m * n) * es
    tag = "bf16" if dtype == BF16 else "f32"
    tag += "_bcast" if broadcast_bias else ""
    return Workload(f"gemm_bias_gelu_{tag}_{m}x{n}x{n}", g.text(), ins, dtype, 1, flops, nbytes,
                    allow_tf32=(dtype == F32))


def conv_stack(batch: int = 32, hw: int = 224, seed: int = 2, backend: str = "cpu") -> Workload:
    """Config 3: 7x7 s2 p3 conv 3->64 + folded BN + ReLU + 3x3 s2 p1 maxpool, then two 3x3 convs
    64->64 with folded BN + ReLU and a residual add; fp32 NCHW.  BN (running mean 0, var 1) is
    folded on the host: w' = gamma*w, bias = beta."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, 3, hw, hw)).astype(np.float32)

    def kaiming_normal(shape):
        fan_in = shape[1] * shape[2] * shape[3]
        return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)

    w1, w2a, w2b = kaiming_normal((64, 3, 7, 7)), kaiming_normal((64, 64, 3, 3)), kaiming_normal((64, 64, 3, 3))
    folded = []
    for w in (w1, w2a, w2b):
        gamma = rng.normal(1.0, 0.1, (w.shape[0],)).astype(np.float32)
        beta = rng.normal(0.0, 0.1, (w.shape[0],)).astype(np.float32)
        folded.append(((gamma[:, None, None, None] * w).astype(np.float32), beta))
    g = irtext.IrGraph(backend)
    vx = g.input("float32", x.shape)
    vs = []
    for w, beta in folded:
        vs.append((g.input("float32", w.shape), g.input("float32", beta.shape)))
    h = g.unary("relu", g.conv2d(vx, vs[0][0], vs[0][1], (2, 2), (3, 3), 1))
    pooled = g.max_pool2d(h, (3, 3), (2, 2), (1, 1))
    h = g.unary("relu", g.conv2d(pooled, vs[1][0], vs[1][1], (1, 1), (1, 1), 1))
    h = g.unary("relu", g.conv2d(h, vs[2][0], vs[2][1], (1, 1), (1, 1), 1))
    out = g.add(h, pooled)
    g.output(out)
    ins = [x]
    for w, beta in folded:
        ins += [w, beta]
    oh1 = irtext.conv_out(hw, 7, 2, 3)
    oh2 = irtext.conv_out(oh1, 3, 2, 1)
    flops = 2.0 * batch * 64 * (oh1 * oh1 * 147 + 2 * oh2 * oh2 * 576)
    nbytes = sum(a.nbytes for a in ins) + batch * 64 * oh2 * oh2 * 4
    return Workload(f"conv_stack_f32_b{batch}_{hw}", g.text(), ins, F32, batch, flops, nbytes,
                    allow_tf32=True)


def transformer_block(batch: int = 8, seq: int = 512, d_model: int = 1024, heads: int = 16,
                      ffn: int = 4096, seed: int = 3, backend: str = "cpu") -> Workload:
    """Config 4: pre-LayerNorm encoder block in bf16, built the reference's way: one fused QKV
    projection, per-(batch, head) rank-2 attention (slice, slice, transpose, matmul, softmax,
    matmul), concat, output projection, residual; LayerNorm, FFN with GELU, residual.
    1/sqrt(head_dim) is folded into the Q columns of Wqkv (a power of two for head_dim 64)."""
    rng = np.random.default_rng(seed)
    hd = d_model // heads
    rows = batch * seq
    x = rng.standard_normal((rows, d_model)).astype(np.float32)
    wqkv = rng.normal(0, 0.02, (d_model, 3 * d_model)).astype(np.float32)
    wo = rng.normal(0, 0.02, (d_model, d_model)).astype(np.float32)
    w1 = rng.normal(0, 0.02, (d_model, ffn)).astype(np.float32)
    w2 = rng.normal(0, 0.02, (ffn, d_model)).astype(np.float32)
    wqkv[:, :d_model] *= np.float32(1.0 / np.sqrt(hd))
    ones, zeros = np.ones(d_model, np.float32), np.zeros(d_model, np.float32)
    dt = "bfloat16"
    g = irtext.IrGraph(backend)
    vx = g.input(dt, x.shape)
    vg1, vb1 = g.input(dt, (d_model,)), g.input(dt, (d_model,))
    vwqkv, vwo = g.input(dt, wqkv.shape), g.input(dt, wo.shape)
    vg2, vb2 = g.input(dt, (d_model,)), g.input(dt, (d_model,))
    vw1, vw2 = g.input(dt, w1.shape), g.input(dt, w2.shape)
    h = g.layer_norm(vx, vg1, vb1, 1e-5)
    qkv = g.matmul(h, vwqkv)
    per_batch = []
    for b in range(batch):
        rows_b = g.slice(qkv, 0, b * seq, (b + 1) * seq)
        per_head = []
        for hh in range(heads):
            q = g.slice(rows_b, 1, hh * hd, (hh + 1) * hd)
            k = g.slice(rows_b, 1, d_model + hh * hd, d_model + (hh + 1) * hd)
            v = g.slice(rows_b, 1, 2 * d_model + hh * hd, 2 * d_model + (hh + 1) * hd)
            p = g.softmax(g.matmul(q, g.transpose(k, (1, 0))))
            per_head.append(g.matmul(p, v))
        per_batch.append(g.concat(per_head, 1) if heads > 1 else per_head[0])
    attn = g.concat(per_batch, 0) if batch > 1 else per_batch[0]
    y = g.add(g.matmul(attn, vwo), vx)
    h2 = g.layer_norm(y, vg2, vb2, 1e-5)
    f = g.matmul(g.unary("gelu", g.matmul(h2, vw1)), vw2)
    out = g.add(f, y)
    g.output(out)
    ins = [_bf16(a) for a in (x, ones, zeros, wqkv, wo, ones, zeros, w1, w2)]
    flops = 2.0 * rows * d_model * 3 * d_model + batch * heads * 2 * (2.0 * seq * seq * hd) \
        + 2.0 * rows * d_model * d_model + 2 * 2.0 * rows * d_model * ffn
    nbytes = sum(a.nbytes for a in ins) + rows * d_model * 2
    return Workload(f"transformer_bf16_b{batch}_s{seq}_d{d_model}", g.text(), ins, BF16, batch, flops, nbytes)


def mamba_block(batch: int = 16, seq: int = 2048, d_model: int = 768, expand: int = 2,
                d_state: int = 16, dt_rank: int = 48, d_conv: int = 4, seed: int = 4,
                backend: str = "cpu") -> Workload:
    """Config 5: Mamba block in fp32: in_proj, causal depthwise conv1d (the reference's idiom:
    padding d_conv-1 then slice), SiLU, x_proj, dt_proj + bias + softplus, the fused selective scan
    (new op) with A = -(1..d_state) per channel and a D skip, SiLU(z) gate, out_proj."""
    rng = np.random.default_rng(seed)
    di = expand * d_model
    rows = batch * seq
    x = rng.standard_normal((rows, d_model)).astype(np.float32)
    w_in = rng.normal(0, 0.02, (d_model, 2 * di)).astype(np.float32)
    conv_w = rng.normal(0, 0.02, (di, 1, d_conv)).astype(np.float32)
    conv_b = rng.normal(0, 0.02, (di,)).astype(np.float32)
    w_x = rng.normal(0, 0.02, (di, dt_rank + 2 * d_state)).astype(np.float32)
    w_dt = rng.normal(0, 0.02, (dt_rank, di)).astype(np.float32)
    w_out = rng.normal(0, 0.02, (di, d_model)).astype(np.float32)
    dt_target = rng.uniform(1e-3, 1e-1, (di,))
    dt_bias = np.log(np.expm1(dt_target)).astype(np.float32)       # softplus^-1
    A = -np.tile(np.arange(1, d_state + 1, dtype=np.float32), (di, 1))
    D = np.ones(di, np.float32)
    g = irtext.IrGraph(backend)
    f = "float32"
    vx, vwin = g.input(f, x.shape), g.input(f, w_in.shape)
    vcw, vcb = g.input(f, conv_w.shape), g.input(f, conv_b.shape)
    vwx, vwdt, vdtb = g.input(f, w_x.shape), g.input(f, w_dt.shape), g.input(f, dt_bias.shape)
    vA, vD, vwout = g.input(f, A.shape), g.input(f, D.shape), g.input(f, w_out.shape)
    xz = g.matmul(vx, vwin)
    u = g.slice(xz, 1, 0, di)
    z = g.slice(xz, 1, di, 2 * di)
    u3 = g.transpose(g.reshape(u, (batch, seq, di)), (0, 2, 1))
    c = g.conv1d(u3, vcw, vcb, 1, d_conv - 1, di)
    c = g.unary("silu", g.slice(c, 2, 0, seq))
    uc = g.reshape(g.transpose(c, (0, 2, 1)), (rows, di))
    xdbc = g.matmul(uc, vwx)
    dr = g.slice(xdbc, 1, 0, dt_rank)
    Bm = g.slice(xdbc, 1, dt_rank, dt_rank + d_state)
    Cm = g.slice(xdbc, 1, dt_rank + d_state, dt_rank + 2 * d_state)
    delta = g.unary("softplus", g.bias_add(g.matmul(dr, vwdt), vdtb))
    y = g.mamba_scan(g.reshape(uc, (batch, seq, di)), g.reshape(delta, (batch, seq, di)), vA,
                     g.reshape(Bm, (batch, seq, d_state)), g.reshape(Cm, (batch, seq, d_state)), vD,
                     g.reshape(z, (batch, seq, di)))
    out = g.matmul(g.reshape(y, (rows, di)), vwout)
    g.output(out)
    ins = [x, w_in, conv_w, conv_b, w_x, w_dt, dt_bias, A, D, w_out]
    flops = 2.0 * rows * (d_model * 2 * di + di * (dt_rank + 2 * d_state) + dt_rank * di + di * d_model)
    nbytes = sum(a.nbytes for a in ins) + rows * d_model * 4
    return Workload(f"mamba_f32_b{batch}_s{seq}_d{d_model}", g.text(), ins, F32, batch, flops, nbytes,
                    allow_tf32=True, meta={"scan_bytes": 4.0 * rows * di * 4 + 2.0 * rows * d_state * 4})


# Miniatures of the five graphs for the parity tests (same structure, seconds on the CPU oracle).
# The reference's OWN nn:: modules (include/frame/nn/layers.h:157-234), graphs emitted by its builder
# where the reference is present (tests/golden/make_workload_golden.py): (golden name, module kind,
# builder arguments, DTypeCode).  transformer: batch, seq, embed, heads, ffn, with_bias; mamba: batch,
# steps, channels, kernel; cnn: batch, input channels, image size, conv channels, classes.
def train_mlp_forward(batch: int = 16, d_in: int = 32, hidden: int = 24, d_out: int = 8, dtype: int = F32,
                      backend: str = "cpu"):
    """Forward graph of a two-layer MLP with an MSE loss, as IR text, and its seeded inputs
    (x, w1, b1 as a full-shape tensor, w2, target).  The reference's compiler::build_backward_graph
    turns it into the training graph [loss, grad w1, grad b1, grad w2]: mse_loss_grad_internal,
    matmul_grad_lhs/rhs_internal and relu_grad_internal beside the forward ops."""
    name = irtext.DTYPE_NAMES[dtype]
    g = irtext.IrGraph(backend)
    x = g.input(name, (batch, d_in))
    w1 = g.input(name, (d_in, hidden))
    b1 = g.input(name, (batch, hidden))
    w2 = g.input(name, (hidden, d_out))
    t = g.input(name, (batch, d_out))
    h = g.node("matmul", [x, w1], {}, name, (batch, hidden))
    h = g.node("add", [h, b1], {}, name, (batch, hidden))
    h = g.node("relu", [h], {}, name, (batch, hidden))
    y = g.node("matmul", [h, w2], {}, name, (batch, d_out))
    g.output(g.node("mse_loss", [y, t], {}, name, ()))
    rng = np.random.default_rng(23)
    ins = [_store(rng.standard_normal(s).astype(np.float32) * sc, dtype)
           for s, sc in (((batch, d_in), 1.0), ((d_in, hidden), 0.3), ((batch, hidden), 0.1), ((hidden, d_out), 0.3),
                         ((batch, d_out), 1.0))]
    return g.text(), ins


TRAIN_WRT = [1, 2, 3]   # gradients w.r.t. w1, b1, w2


NN_GRAPHS = [
    ("nn_transformer_bf16_b2_s128_e128_h2", "transformer", (2, 128, 128, 2, 256, True), BF16),
    ("nn_transformer_f32_b2_s16_e32_h2", "transformer", (2, 16, 32, 2, 64, True), F32),
    ("nn_mamba_f32_b2_c16_s24_k4", "mamba", (2, 24, 16, 4, 0, True), F32),
    # nn::Sequential CNN (conv2d + bias, relu, max_pool2d, flatten = reshape, linear): the reference's
    # own golden shape, and a wider one that the tensor-core conv takes under allow_tf32
    ("nn_cnn_f32_b8_c1_hw8_o4", "cnn", (8, 1, 8, 4, 1, True), F32),
    ("nn_cnn_f32_b4_c16_hw32_o32", "cnn", (4, 16, 32, 32, 10, True), F32),
]


def nn_inputs(shapes, dtype: int, seed: int = 11) -> List[np.ndarray]:
    """Seeded inputs for a graph given the shapes of its inputs: the activation first, then the
    parameters; N(0, 1) for the activation, N(0, 0.1) for everything else, in storage form."""
    rng = np.random.default_rng(seed)
    out = []
    for i, shape in enumerate(shapes):
        x = rng.standard_normal(shape).astype(np.float32) * np.float32(1.0 if i == 0 else 0.1)
        out.append(_bf16(x) if dtype == BF16 else x)
    return out


def small_workloads(backend: str = "cpu") -> List[Workload]:
    return [
        mlp(batch=8, d_in=40, hidden=32, d_out=10, backend=backend),
        gemm_epilogue(n=64, m=48, dtype=F32, backend=backend),
        gemm_epilogue(n=128, m=64, dtype=BF16, backend=backend),
        gemm_epilogue(n=64, m=48, dtype=F32, broadcast_bias=True, backend=backend),
        conv_stack(batch=2, hw=32, backend=backend),
        transformer_block(batch=2, seq=32, d_model=64, heads=2, ffn=128, backend=backend),
        # head_dim 64 and 128 keys: the shape the fused attention launch accepts
        transformer_block(batch=2, seq=128, d_model=128, heads=2, ffn=256, backend=backend),
        mamba_block(batch=2, seq=24, d_model=16, d_state=16, dt_rank=4, backend=backend),
    ]


# ---- slabs of the full-size workloads -------------------------------------------------------------
# Every op on the path is row / sample independent, so the first sample (or the first rows of A)
# of a full-size run depends only on its own inputs: the CPU backend can compute that slab in
# seconds to a minute, and the full-size GPU result must agree with it on those rows.
FULL_BUILDERS = {
    "mlp": (mlp, dict()),
    "gemm_bf16": (gemm_epilogue, dict(n=8192, dtype=BF16)),
    "gemm_f32": (gemm_epilogue, dict(n=8192, dtype=F32)),
    "conv_stack": (conv_stack, dict()),
    "transformer": (transformer_block, dict()),
    "mamba": (mamba_block, dict()),
}
GEMM_SLAB_ROWS = 16


def slab_graph(key: str, backend: str = "cpu") -> str:
    """IR text of the slab graph of a full-size workload: the same graph at batch 1 (GEMM: the first
    GEMM_SLAB_ROWS rows of A; MLP: the whole batch)."""
    builder, kw = FULL_BUILDERS[key]
    if key == "mlp":
        return builder(backend=backend, **kw).ir_text
    if key.startswith("gemm"):
        dt = irtext.DTYPE_NAMES[kw["dtype"]]
        n = kw["n"]
        g = irtext.IrGraph(backend)
        va, vb, vbias = g.input(dt, (GEMM_SLAB_ROWS, n)), g.input(dt, (n, n)), g.input(dt, (GEMM_SLAB_ROWS, n))
        g.output(g.unary("gelu", g.add(g.matmul(va, vb), vbias)))
        return g.text()
    small = dict(kw)
    small["batch"] = 1
    return _graph_text_only(builder, backend=backend, **small)


def _graph_text_only(builder, **kw) -> str:
    """The graph text of a builder without paying for its random inputs."""
    class Zero:
        def standard_normal(self, shape):
            return np.zeros(shape, np.float32)

        def normal(self, a, b, shape):
            return np.zeros(shape, np.float32)

        def uniform(self, a, b, shape):
            return np.full(shape, 0.5 * (a + b), np.float64)

    real = np.random.default_rng
    np.random.default_rng = lambda seed=None: Zero()
    try:
        return builder(**kw).ir_text
    finally:
        np.random.default_rng = real


def slab_inputs(key: str, full_inputs: List[np.ndarray]) -> List[np.ndarray]:
    """The slab's inputs cut out of the full-size inputs (graph-input order is unchanged)."""
    ins = list(full_inputs)
    if key == "mlp":
        return ins
    if key.startswith("gemm"):
        return [ins[0][:GEMM_SLAB_ROWS], ins[1], ins[2][:GEMM_SLAB_ROWS]]
    builder, kw = FULL_BUILDERS[key]
    if key == "conv_stack":
        ins[0] = ins[0][:1]
    else:   # transformer, mamba: activations are [batch * seq, d_model]
        import inspect
        seq = inspect.signature(builder).parameters["seq"].default
        ins[0] = ins[0][:seq]
    return [np.ascontiguousarray(a) for a in ins]


def slab_of_output(key: str, full_output: np.ndarray) -> np.ndarray:
    """The rows of a full-size result that the slab graph computes."""
    if key == "mlp":
        return full_output
    if key.startswith("gemm"):
        return full_output[:GEMM_SLAB_ROWS]
    builder, _ = FULL_BUILDERS[key]
    if key == "conv_stack":
        return full_output[:1]
    import inspect
    seq = inspect.signature(builder).parameters["seq"].default
    return full_output[:seq]


def parity_tolerance(key: str, dtype: int, allow_tf32: bool, gold_f32: np.ndarray, inputs=None) -> Dict[str, float]:
    """rtol/atol of |got - expected| <= atol + rtol*|expected| for a slab comparison, by the
    reference's tiers (tests/cpp/common/tolerance.h:41-98 of the reference): bf16 2e-2 / 2e-3; strict
    fp32 1e-5 / 1e-6; fp32 on the tensor cores rtol 1e-3 plus an absolute term for outputs that cancel
    to near zero: 2e-3 * sqrt(K) * rms(a) * rms(b) for one GEMM, 5e-3 of the expected rms for graphs
    that chain several TF32 contractions."""
    if dtype == BF16:
        if key == "transformer":
            # A chain of bf16 nodes ending in residual adds: the reference's table has no tier beyond
            # bf16 ("handled case by case by the caller", tolerance.h:63-80).  Every node stores bf16, so
            # a different fp32 accumulation order inside a matmul can flip one rounding of an addend,
            # and the sum then differs by one bf16 ulp OF THE ADDEND however small the sum is.  The
            # absolute term is therefore one bf16 ulp at the largest magnitude of the residual stream.
            top = float(np.max(np.abs(np.asarray(gold_f32, np.float64))))
            return dict(rtol=2e-2, atol=float(2.0 ** (np.floor(np.log2(max(top, 1e-30))) - 7)))
        return dict(rtol=2e-2, atol=2e-3)
    if not allow_tf32:
        if key.startswith("gemm") and inputs is not None and inputs[1].shape[0] >= 1024:
            # strict fp32 above 2^30 multiply-adds runs error-compensated on the tensor cores (three TF32
            # products with the operands' low parts): no operand error, but the tensor core truncates
            # its fp32 accumulator at each of the K/8 additions; measured worst element about
            # 2^-23 * (K/8) of the output's rms, bounded here at 3 times that
            k = inputs[1].shape[0]
            rms = float(np.sqrt(np.mean(np.square(np.asarray(gold_f32, np.float64)))))
            return dict(rtol=1e-5, atol=float(3 * 2.0 ** -23 * (k / 8) * max(rms, 1.0)))
        return dict(rtol=1e-5, atol=1e-6)
    if key.startswith("gemm") and inputs is not None:
        a, b = np.asarray(inputs[0][:64], np.float64), np.asarray(inputs[1][:, :64], np.float64)
        k = inputs[1].shape[0]
        return dict(rtol=1e-3, atol=float(2e-3 * np.sqrt(k) * np.sqrt((a ** 2).mean()) * np.sqrt((b ** 2).mean())))
    rms = float(np.sqrt(np.mean(np.square(np.asarray(gold_f32, np.float64)))))
    return dict(rtol=1e-3, atol=max(1e-4, 5e-3 * rms))
