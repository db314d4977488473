"""Tensor-core implicit-GEMM conv2d (fp32 tensors, TF32 math, allow_tf32) against the CPU oracle.
Tolerance: tcgen05 reads fp32 operands as TF32 (10 explicit mantissa bits, the low 13 bits are
dropped), so each product errs by at most 2^-9 relative and an output by at most
2^-9 * sum |x||w| over its window; the test bound is that elementwise figure plus the strict-fp32
tier (rtol 1e-5, atol 1e-6) for the fp32 accumulation.  On these inputs that is tighter than the
reference's TF32 tier (rtol 1e-3 / atol 1e-4 at K=512, tests/cpp/common/tolerance.h:90-98) scaled
to the output magnitudes."""
import numpy as np
import pytest

from frame_public_b200 import capi
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu

CASES = [
    # (x shape, w shape, stride, padding, bias)
    ((2, 3, 9, 9), (4, 3, 3, 3), (1, 1), (1, 1), True),
    ((1, 3, 20, 20), (8, 3, 7, 7), (2, 2), (3, 3), True),
    ((2, 64, 10, 10), (64, 64, 3, 3), (1, 1), (1, 1), True),
    ((3, 16, 13, 17), (40, 16, 3, 3), (2, 1), (0, 1), False),
    ((2, 3, 64, 64), (64, 3, 7, 7), (2, 2), (3, 3), True),
    ((4, 64, 56, 56), (64, 64, 3, 3), (1, 1), (1, 1), True),
    ((1, 8, 9, 9), (130, 8, 1, 1), (1, 1), (0, 0), True),
    # halo-tile kernel (image width a multiple of 4): two channel blocks and more tiles per CTA than
    # TMEM accumulators (two rounds); a stride-2 7x7 stem with two rounds; ragged Cout with strides
    # that differ; three channel blocks with one tile per image
    ((44, 64, 56, 56), (64, 64, 3, 3), (1, 1), (1, 1), True),
    ((12, 3, 224, 224), (64, 3, 7, 7), (2, 2), (3, 3), True),
    ((3, 16, 12, 16), (40, 16, 3, 3), (2, 1), (0, 1), False),
    ((2, 96, 8, 8), (32, 96, 3, 3), (1, 1), (1, 1), True),
    # results through the TMA-store tile, last tile of each image only partly inside it (22 rows, 10 per tile)
    ((2, 8, 22, 12), (24, 8, 3, 3), (1, 1), (1, 1), True),
    # column-shifted planes kernel (stride 1, channels a multiple of 8): 1x1; 3x3 without padding;
    # 5x5 and 7x7 with "same" padding; rows of 28 (four per tile), 64 and 96 pixels; 256 -> 256 channels
    # (eight-channel blocks, two accumulators per round); an image shorter than a tile
    ((2, 16, 16, 16), (24, 16, 1, 1), (1, 1), (0, 0), True),
    ((1, 8, 14, 14), (16, 8, 3, 3), (1, 1), (0, 0), False),
    ((1, 8, 12, 12), (8, 8, 5, 5), (1, 1), (2, 2), True),
    ((1, 8, 16, 16), (40, 8, 7, 7), (1, 1), (3, 3), True),
    ((3, 32, 28, 28), (64, 32, 3, 3), (1, 1), (1, 1), True),
    ((1, 16, 20, 64), (32, 16, 3, 3), (1, 1), (1, 1), True),
    ((1, 8, 9, 96), (16, 8, 3, 3), (1, 1), (1, 1), False),
    ((2, 256, 28, 28), (256, 256, 3, 3), (1, 1), (1, 1), True),
    ((5, 24, 3, 8), (8, 24, 3, 3), (1, 1), (1, 1), True),
    # row-matrix kernel (stride 2, KW * Cin <= 32, output rows a multiple of 4 pixels): runs of rows
    # that cross images; 3x3 with four channels (K 12 -> 16); one channel, 5x5, odd height; no
    # padding; an even 4x4 window; Cout too large for resident weights (falls back to the halo kernel)
    ((5, 3, 90, 64), (32, 3, 7, 7), (2, 2), (3, 3), True),
    ((2, 4, 40, 48), (40, 4, 3, 3), (2, 2), (1, 1), False),
    ((2, 1, 33, 72), (16, 1, 5, 5), (2, 2), (2, 2), True),
    ((1, 2, 21, 34), (8, 2, 3, 3), (2, 2), (0, 0), True),
    ((1, 3, 16, 32), (8, 3, 4, 4), (2, 2), (1, 1), True),
    ((1, 3, 32, 64), (200, 3, 7, 7), (2, 2), (3, 3), True),
]


def _run(x, w, b, stride, padding, steps=None, extra=None):
    n, cin, h, wd = x.shape
    cout, _, kh, kw = w.shape
    oh = (h + 2 * padding[0] - kh) // stride[0] + 1
    ow = (wd + 2 * padding[1] - kw) // stride[1] + 1
    dx, dw = capi.DeviceBuffer.from_numpy(x), capi.DeviceBuffer.from_numpy(w)
    db = capi.DeviceBuffer.from_numpy(b) if b is not None else None
    dout = capi.DeviceBuffer(n * cout * oh * ow * 4)
    keep, epi = [], None
    if steps:
        lst = []
        for name, opnd, mode in steps:
            if opnd is not None:
                buf = capi.DeviceBuffer.from_numpy(opnd)
                keep.append(buf)
                lst.append((name, buf.ptr, mode))
            else:
                lst.append((name, None, 0))
        epi = capi.make_epilogue(lst)
    p = capi.Conv2dParams(n, cin, h, wd, cout, kh, kw, stride[0], stride[1], padding[0], padding[1], 1)
    capi.conv2d(dx.ptr, dw.ptr, db.ptr if db else None, dout.ptr, p, capi.F32, True, epi)
    capi.synchronize()
    assert capi.kernel_status(0) == 0
    return dout.download(np.float32, (n, cout, oh, ow))


def _within_tf32_bound(got, exp, x, w, stride, padding):
    mag = fo.conv2d(np.abs(x), np.abs(w), None, stride, padding, 1, fo.DT_F32).astype(np.float64)
    bound = mag * 2.0 ** -9 + 1e-5 * np.abs(exp) + 1e-6
    err = np.abs(got.astype(np.float64) - exp.astype(np.float64))
    return bool(np.all(err <= bound)), float((err / bound).max())


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c[0])) + "_w" + "x".join(map(str, c[1])))
def test_conv2d_tensor_cores(case):
    xs, ws, stride, padding, use_bias = case
    rng = np.random.default_rng(21)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * 0.3).astype(np.float32)
    b = rng.standard_normal(ws[0]).astype(np.float32) if use_bias else None
    got = _run(x, w, b, stride, padding)
    exp = fo.conv2d(x, w, b, stride, padding, 1, fo.DT_F32)
    ok, worst = _within_tf32_bound(got, exp, x, w, stride, padding)
    assert ok, (worst, fo.max_err(got, exp))


def test_conv2d_tensor_cores_fused_relu_and_residual():
    rng = np.random.default_rng(22)
    x = rng.standard_normal((2, 64, 28, 28)).astype(np.float32)
    w = (rng.standard_normal((64, 64, 3, 3)) * 0.05).astype(np.float32)
    b = rng.standard_normal(64).astype(np.float32)
    res = rng.standard_normal((2, 64, 28, 28)).astype(np.float32)
    got = _run(x, w, b, (1, 1), (1, 1), steps=[("relu", None, 0), ("add", res, capi.OPERAND_FULL)])
    exp = fo.add(fo.relu(fo.conv2d(x, w, b, (1, 1), (1, 1), 1)), res)
    ok, worst = _within_tf32_bound(got, exp, x, w, (1, 1), (1, 1))
    assert ok, (worst, fo.max_err(got, exp))


def test_stride2_stem_fused_relu_and_residual():
    """The stride-2 row-matrix kernel with a chain: ReLU, then a full-shape residual; 448 output rows
    over 148 CTAs (runs of three rows, image boundaries inside runs)."""
    rng = np.random.default_rng(24)
    x = rng.standard_normal((4, 3, 224, 224)).astype(np.float32)
    w = (rng.standard_normal((64, 3, 7, 7)) * 0.1).astype(np.float32)
    b = rng.standard_normal(64).astype(np.float32)
    res = rng.standard_normal((4, 64, 112, 112)).astype(np.float32)
    got = _run(x, w, b, (2, 2), (3, 3), steps=[("relu", None, 0), ("add", res, capi.OPERAND_FULL)])
    exp = fo.add(fo.relu(fo.conv2d(x, w, b, (2, 2), (3, 3), 1)), res)
    ok, worst = _within_tf32_bound(got, exp, x, w, (2, 2), (3, 3))
    assert ok, (worst, fo.max_err(got, exp))


POOL_CASES = [
    # (x shape, w shape, padding, relu): stride-2 conv followed by max_pool2d(3, 3, stride 2, pad 1)
    ((4, 3, 224, 224), (64, 3, 7, 7), (3, 3), True),    # 224 pooled rows over 148 CTAs: runs of 1-2 pooled rows
    ((20, 3, 224, 224), (64, 3, 7, 7), (3, 3), True),   # runs of 7-8 pooled rows that cross image boundaries
    ((3, 3, 64, 96), (48, 3, 7, 7), (3, 3), False),     # ragged Cout (48 of 64), negative values reach the pool
    ((2, 4, 40, 48), (40, 4, 3, 3), (1, 1), True),      # 3x3 stem over four channels
    ((2, 3, 36, 64), (64, 3, 5, 5), (2, 2), True),      # 5x5: not instantiated for the fused form -> two kernels
]


@pytest.mark.parametrize("case", POOL_CASES, ids=lambda c: "x".join(map(str, c[0])) + "_w" + "x".join(map(str, c[1])))
def test_conv2d_max_pool_fused(case):
    """conv2d -> [ReLU] -> max_pool2d(3x3, stride 2, pad 1) through fb200_conv2d_max_pool.  Where the
    shape allows, one kernel pools the rows in its epilogue and the intermediate is never written
    (checked: the buffer keeps its fill pattern).  |max a_i - max b_i| <= max |a_i - b_i|, so the
    pooled result must lie within the max-pool of the elementwise TF32 bound."""
    xs, ws, padding, relu = case
    rng = np.random.default_rng(31)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * 0.2).astype(np.float32)
    b = rng.standard_normal(ws[0]).astype(np.float32)
    n, cin, h, wd = xs
    cout, _, kh, kw = ws
    oh = (h + 2 * padding[0] - kh) // 2 + 1
    ow = (wd + 2 * padding[1] - kw) // 2 + 1
    poh, pow_ = (oh + 2 - 3) // 2 + 1, (ow + 2 - 3) // 2 + 1
    dx, dw, db = (capi.DeviceBuffer.from_numpy(t) for t in (x, w, b))
    fill = np.full((n, cout, oh, ow), 12345.0, np.float32)
    dmid = capi.DeviceBuffer.from_numpy(fill)
    dout = capi.DeviceBuffer(n * cout * poh * pow_ * 4)
    epi = capi.make_epilogue([("relu", None, 0)]) if relu else None
    p = capi.Conv2dParams(n, cin, h, wd, cout, kh, kw, 2, 2, padding[0], padding[1], 1)
    before = capi.load().fb200_launch_count()
    capi.conv2d_max_pool(dx.ptr, dw.ptr, db.ptr, dmid.ptr, dout.ptr, p, (3, 3, 2, 2, 1, 1), capi.F32, True, epi)
    launches = capi.load().fb200_launch_count() - before
    capi.synchronize()
    assert capi.kernel_status(0) == 0
    got = dout.download(np.float32, (n, cout, poh, pow_))
    fused = launches == 1
    assert fused == (kh != 5), launches
    if fused:
        assert np.array_equal(dmid.download(np.float32, fill.shape), fill)
    conv = fo.conv2d(x, w, b, (2, 2), padding, 1, fo.DT_F32)
    if relu:
        conv = fo.relu(conv)
    exp = fo.max_pool2d(conv, (3, 3), (2, 2), (1, 1))
    mag = fo.conv2d(np.abs(x), np.abs(w), None, (2, 2), padding, 1, fo.DT_F32).astype(np.float64)
    bound = fo.max_pool2d((mag * 2.0 ** -9 + 1e-5 * np.abs(conv) + 1e-6).astype(np.float32), (3, 3), (2, 2), (1, 1))
    err = np.abs(got.astype(np.float64) - exp.astype(np.float64))
    assert np.all(err <= bound), float((err / bound).max())


def test_strict_conv2d_stays_bit_identical():
    rng = np.random.default_rng(23)
    x = rng.standard_normal((2, 8, 12, 12)).astype(np.float32)
    w = rng.standard_normal((16, 8, 3, 3)).astype(np.float32)
    n, cin, h, wd = x.shape
    dx, dw = capi.DeviceBuffer.from_numpy(x), capi.DeviceBuffer.from_numpy(w)
    dout = capi.DeviceBuffer(2 * 16 * 12 * 12 * 4)
    p = capi.Conv2dParams(n, cin, h, wd, 16, 3, 3, 1, 1, 1, 1, 1)
    capi.conv2d(dx.ptr, dw.ptr, None, dout.ptr, p, capi.F32, False)
    capi.synchronize()
    got = dout.download(np.float32, (2, 16, 12, 12))
    assert np.array_equal(got, fo.conv2d(x, w, None, (1, 1), (1, 1), 1))
