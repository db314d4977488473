"""Tensor-core (tcgen05/TMEM/TMA) matmul parity against the CPU oracle.

bf16: products of bf16 values are exact in fp32, so the only difference from the CPU reference
is the order of the fp32 accumulation; tolerance = the reference's bf16 tier (rtol 2e-2,
atol 2e-3).  fp32 with allow_tf32: operands are read as TF32 (10 explicit mantissa bits), so the
error of a K-term dot product is about 2^-10 * sqrt(K) * rms(a) * rms(b); tolerance =
rtol 1e-3 (the reference's TF32 tier, tests/cpp/common/tolerance.h:90-98) plus
atol = 2e-3 * sqrt(K) * rms(a) * rms(b) for outputs that cancel to near zero."""
import json
import os

import numpy as np
import pytest

from frame_public_b200 import capi
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu


def _gen(m, k, n, dt, seed):
    rng = np.random.default_rng(seed)
    a = fo.from_accum(rng.uniform(-1, 1, (m, k)).astype(np.float32), dt)
    b = fo.from_accum(rng.uniform(-1, 1, (k, n)).astype(np.float32), dt)
    return a, b


def _run(a, b, dt, allow_tf32, steps=None, operands=None):
    m, k = a.shape
    n = b.shape[1]
    da, db = capi.DeviceBuffer.from_numpy(a), capi.DeviceBuffer.from_numpy(b)
    dc = capi.DeviceBuffer(m * n * capi.ITEMSIZE[dt])
    keep = []
    epi = None
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
    capi.matmul(da.ptr, db.ptr, dc.ptr, m, n, k, dt, allow_tf32, epi)
    capi.synchronize()
    assert capi.kernel_status(0) == 0
    return dc.download(capi.NP_STORAGE[dt], (m, n))


SHAPES = [(128, 64, 256), (256, 256, 256), (128, 512, 64), (300, 136, 520), (64, 784, 256),
          (1024, 1024, 1024), (4096, 64, 512), (512, 512, 64), (130, 72, 80)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_bf16_matmul_tensor_cores(shape):
    m, k, n = shape
    assert capi.load().fb200_matmul_uses_tensor_cores(m, n, k, capi.BF16, 0) == 1
    a, b = _gen(m, k, n, fo.DT_BF16, 11)
    got = _run(a, b, fo.DT_BF16, False)
    exp = fo.matmul(a, b, fo.DT_BF16)
    assert fo.all_close(got, exp, fo.DT_BF16), fo.max_err(got, exp, fo.DT_BF16)


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_tf32_matmul_tensor_cores(shape):
    m, k, n = shape
    assert capi.load().fb200_matmul_uses_tensor_cores(m, n, k, capi.F32, 1) == 1
    a, b = _gen(m, k, n, fo.DT_F32, 12)
    got = _run(a, b, fo.DT_F32, True)
    exp = fo.matmul(a, b, fo.DT_F32)
    atol = 2e-3 * np.sqrt(k) * float(np.sqrt((a ** 2).mean()) * np.sqrt((b ** 2).mean()))
    assert fo.all_close(got, exp, fo.DT_F32, rtol=1e-3, atol=atol), fo.max_err(got, exp)


def test_strict_fp32_is_bit_identical_to_the_cpu_reference():
    a, b = _gen(200, 300, 136, fo.DT_F32, 13)
    got = _run(a, b, fo.DT_F32, False)
    assert np.array_equal(got, fo.matmul(a, b, fo.DT_F32))


@pytest.mark.parametrize("dt,tf32", [(fo.DT_BF16, False), (fo.DT_F32, True), (fo.DT_F32, False)],
                         ids=["bf16", "tf32", "fp32_strict"])
def test_fused_epilogue_bias_full_then_gelu_then_residual(dt, tf32):
    m, k, n = 384, 256, 520
    a, b = _gen(m, k, n, dt, 14)
    rng = np.random.default_rng(15)
    bias_full = fo.from_accum(np.tile(rng.normal(0, 0.1, (1, n)).astype(np.float32), (m, 1)), dt)
    resid = fo.from_accum(rng.standard_normal((m, n)).astype(np.float32), dt)
    got = _run(a, b, dt, tf32, steps=[("add", bias_full, capi.OPERAND_FULL), ("gelu", None, 0),
                                      ("add", resid, capi.OPERAND_FULL)])
    mm = fo.matmul(a, b, dt)
    exp = fo.add(fo.gelu(fo.add(mm, bias_full, dt), dt), resid, dt)
    if dt == fo.DT_F32 and not tf32:
        assert fo.all_close(got, exp, dt), fo.max_err(got, exp, dt)
    elif dt == fo.DT_F32:
        atol = 2e-3 * np.sqrt(k) * float(np.sqrt((a ** 2).mean()) * np.sqrt((b ** 2).mean()))
        assert fo.all_close(got, exp, dt, rtol=1e-3, atol=atol), fo.max_err(got, exp, dt)
    else:
        assert fo.all_close(got, exp, dt, rtol=2e-2, atol=2e-2), fo.max_err(got, exp, dt)


def test_epilogue_column_and_row_operands():
    m, k, n = 256, 128, 264
    dt = fo.DT_BF16
    a, b = _gen(m, k, n, dt, 16)
    rng = np.random.default_rng(17)
    col = fo.from_accum(rng.standard_normal(n).astype(np.float32), dt)
    row = fo.from_accum(rng.uniform(0.5, 1.5, m).astype(np.float32), dt)
    got = _run(a, b, dt, False, steps=[("add", col, capi.OPERAND_COL), ("relu", None, 0),
                                       ("mul", row, capi.OPERAND_ROW)])
    mm = fo.to_accum(fo.matmul(a, b, dt), dt)
    e1 = fo.round_through(mm + fo.to_accum(col, dt)[None, :], dt)
    e2 = np.where(e1 < 0, 0, e1).astype(np.float32)
    exp = fo.from_accum(e2 * fo.to_accum(row, dt)[:, None], dt)
    assert fo.all_close(got, exp, dt, rtol=2e-2, atol=2e-2), fo.max_err(got, exp, dt)


@pytest.mark.parametrize("dt,tf32,k", [(fo.DT_BF16, False, 8200), (fo.DT_F32, True, 4104)], ids=["bf16", "tf32"])
def test_large_gemm_on_256x256_tiles_with_a_light_epilogue(dt, tf32, k):
    """17 x 17 tiles of 256 x 256 (two waves of 148) against 33 x 17 of 128 x 256 (four waves), at
    least 128 k-blocks and a light epilogue: the kernel takes the 256-row form (two M = 128
    instructions per B stage, both accumulators of TMEM in one tile).  Ragged in M (4200 = 16 * 256 +
    104), N (4168 = 16 * 256 + 72) and K; column bias + ReLU epilogue.  At this size the checker is
    the float64 product of the stored operands (the ordered fp32 sum of the oracle would take
    minutes), compared within the tensor-core tolerance tiers."""
    m, n = 4200, 4168
    a, b = _gen(m, k, n, dt, 21)
    rng = np.random.default_rng(22)
    col = fo.from_accum(rng.standard_normal(n).astype(np.float32), dt)
    got = _run(a, b, dt, tf32, steps=[("add", col, capi.OPERAND_COL), ("relu", None, 0)])
    mm = (fo.to_accum(a, dt).astype(np.float64) @ fo.to_accum(b, dt).astype(np.float64)).astype(np.float32)
    e1 = fo.round_through(fo.round_through(mm, dt) + fo.to_accum(col, dt)[None, :], dt)
    exp = fo.from_accum(np.where(e1 < 0, 0, e1).astype(np.float32), dt)
    if dt == fo.DT_F32:
        atol = 2e-3 * np.sqrt(k) * float(np.sqrt((a ** 2).mean()) * np.sqrt((b ** 2).mean()))
        assert fo.all_close(got, exp, dt, rtol=1e-3, atol=atol), fo.max_err(got, exp, dt)
    else:
        assert fo.all_close(got, exp, dt, rtol=2e-2, atol=2e-2 * np.sqrt(k / 136.0)), fo.max_err(got, exp, dt)


@pytest.mark.parametrize("dt,tf32", [(fo.DT_BF16, False), (fo.DT_F32, True), (fo.DT_F32, False)],
                         ids=["bf16", "tf32", "fp32_strict"])
def test_matmul_gradients_on_the_tensor_cores_and_strict(dt, tf32):
    """ga = gy * b^T and gb = a^T * gy (src/backends/cpu/kernels/matmul.cpp:187-232, :289-330): the
    transposed operand goes through a scratch transpose and the tcgen05 GEMM when reduced-precision
    math is allowed, and is read in place by the strict kernel otherwise (bit-identical)."""
    m, n, k = 520, 392, 264
    rng = np.random.default_rng(31)
    gy = fo.from_accum(rng.uniform(-1, 1, (m, n)).astype(np.float32), dt)
    a = fo.from_accum(rng.uniform(-1, 1, (m, k)).astype(np.float32), dt)
    b = fo.from_accum(rng.uniform(-1, 1, (k, n)).astype(np.float32), dt)
    d_gy, d_a, d_b = (capi.DeviceBuffer.from_numpy(t) for t in (gy, a, b))
    d_ga = capi.DeviceBuffer(m * k * capi.ITEMSIZE[dt])
    d_gb = capi.DeviceBuffer(k * n * capi.ITEMSIZE[dt])
    capi.matmul_grad_lhs(d_gy.ptr, d_b.ptr, d_ga.ptr, m, n, k, dt, tf32)
    capi.matmul_grad_rhs(d_a.ptr, d_gy.ptr, d_gb.ptr, m, n, k, dt, tf32)
    capi.synchronize()
    assert capi.kernel_status(0) == 0
    ga = d_ga.download(capi.NP_STORAGE[dt], (m, k))
    gb = d_gb.download(capi.NP_STORAGE[dt], (k, n))
    exp_a, exp_b = fo.matmul_grad_lhs(gy, b, dt), fo.matmul_grad_rhs(a, gy, dt)
    if dt == fo.DT_F32 and not tf32:
        assert np.array_equal(ga, exp_a) and np.array_equal(gb, exp_b)
    elif dt == fo.DT_F32:
        for got, exp, red in ((ga, exp_a, n), (gb, exp_b, m)):
            assert fo.all_close(got, exp, dt, rtol=1e-3, atol=2e-3 * np.sqrt(red) / 3), fo.max_err(got, exp, dt)
    else:
        assert fo.all_close(ga, exp_a, dt, rtol=2e-2, atol=2e-2) and fo.all_close(gb, exp_b, dt, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dt,tf32,tail_col", [(fo.DT_F32, True, 160), (fo.DT_BF16, False, 256), (fo.DT_F32, True, 64)],
                         ids=["tf32_160", "bf16_256", "tf32_ragged_tail"])
def test_matmul_split_stores_the_trailing_columns_separately(dt, tf32, tail_col):
    """fb200_matmul_split: columns [0, tail_col) where fb200_matmul puts them (the rest of `c` keeps
    its old bytes), columns [tail_col, n) in a dense matrix of their own; with an epilogue on both."""
    m, k, n = 300, 96, 80 if tail_col == 64 else 416
    a, b = _gen(m, k, n, dt, 17)
    rng = np.random.default_rng(18)
    bias = fo.from_accum(rng.normal(0, 0.5, (n,)).astype(np.float32), dt)
    es = capi.ITEMSIZE[dt]
    da, db, dbias = (capi.DeviceBuffer.from_numpy(t) for t in (a, b, bias))
    fill = np.full((m, n), 0x3C3C if es == 2 else 0, capi.NP_STORAGE[dt])
    dc = capi.DeviceBuffer.from_numpy(fill)
    dtail = capi.DeviceBuffer(m * (n - tail_col) * es)
    epi = capi.make_epilogue([("add", dbias.ptr, capi.OPERAND_COL), ("relu", None, 0)])
    capi.matmul_split(da.ptr, db.ptr, dc.ptr, dtail.ptr, tail_col, m, n, k, dt, tf32, epi)
    capi.synchronize()
    assert capi.kernel_status(0) == 0
    head = dc.download(capi.NP_STORAGE[dt], (m, n))
    tail = dtail.download(capi.NP_STORAGE[dt], (m, n - tail_col))
    exp = fo.relu(fo.bias_add(fo.matmul(a, b, dt), bias, dt), dt)
    if tf32:
        atol = 2e-3 * np.sqrt(k) * float(np.sqrt((a ** 2).mean()) * np.sqrt((b ** 2).mean()))
        tol = dict(rtol=1e-3, atol=atol)
    else:
        tol = dict(rtol=2e-2, atol=2e-3)
    assert fo.all_close(head[:, :tail_col], exp[:, :tail_col], dt, **tol)
    assert fo.all_close(tail, exp[:, tail_col:], dt, **tol)
    assert np.array_equal(head[:, tail_col:], fill[:, tail_col:])      # untouched


@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (2048, 512, 1536), (1152, 4096, 256)], ids=lambda s: "x".join(map(str, s)))
def test_large_strict_fp32_matmul_is_error_compensated_on_the_tensor_cores(shape):
    """allow_tf32 = 0 from 2^30 multiply-adds on: three TF32 products with the operands' low parts.  The
    operand error of TF32 is gone; what remains is the tensor core's own accumulation, which truncates
    the fp32 accumulator at each of its K/8 additions: measured mean error 0.13 * 2^-23 * (K/8) * rms(out)
    (K = 512..8192), i.e. 5-30 times a round-to-nearest fp32 summation and 50-100 times below plain
    TF32.  Bounds: mean <= 0.3 and max <= 3 of that unit, against a float64 product."""
    m, k, n = shape
    a, b = _gen(m, k, n, fo.DT_F32, 19)
    got = _run(a, b, fo.DT_F32, False)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    err = np.abs(got.astype(np.float64) - exact)
    unit = 2.0 ** -23 * (k / 8) * float(np.sqrt(np.mean(exact ** 2)))
    tf32_level = 2.0 ** -11 * np.sqrt(k) * float(np.sqrt((a ** 2).mean()) * np.sqrt((b ** 2).mean()))
    err_fp32_sum = np.abs((a @ b).astype(np.float64) - exact)
    path = os.environ.get("FRAME_B200_ERROR_TABLE")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"case": "compensated_fp32_matmul", "shape": list(shape), "max_abs": float(err.max()),
                                "mean_abs": float(err.mean()), "fp32_sum_mean_abs": float(err_fp32_sum.mean()),
                                "fp32_sum_max_abs": float(err_fp32_sum.max()), "unit": unit, "tf32_level": tf32_level}) + "\n")
    assert err.mean() <= 0.3 * unit and err.max() <= 3.0 * unit, (float(err.mean() / unit), float(err.max() / unit))
    assert err.mean() <= tf32_level / 20, (float(err.mean()), tf32_level)


def test_exact_order_can_be_forced_at_any_size():
    """allow_tf32 < 0: the CPU reference's order of additions (bit-identical) even above the size from
    which strict fp32 moves to the tensor cores."""
    m, k, n = 1024, 1024, 1024
    a, b = _gen(m, k, n, fo.DT_F32, 20)
    da, db = capi.DeviceBuffer.from_numpy(a), capi.DeviceBuffer.from_numpy(b)
    dc = capi.DeviceBuffer(m * n * 4)
    capi.check(capi.load().fb200_matmul(da.ptr, db.ptr, dc.ptr, m, n, k, capi.F32, -1, None, None))
    capi.synchronize()
    got = dc.download(np.float32, (m, n))
    rows = slice(0, 8)
    assert np.array_equal(got[rows], fo.matmul(a[rows], b, fo.DT_F32))


SPLIT_CASES = [
    # m, k, n, dtype, allow_tf32, chain: a few tiles with a long K, split over the SMs
    (512, 8192, 1024, fo.DT_BF16, False, "residual"),    # 16 tiles of 128 x 256, 128 k-blocks each
    (640, 8192, 1280, fo.DT_BF16, False, None),          # 25 tiles, 128 k-blocks: ranges of 16
    (500, 4104, 520, fo.DT_F32, True, "col_gelu"),       # TF32, ragged in M, N and K, interpreter chain
    (256, 8192, 512, fo.DT_BF16, False, None),           # four tiles, each shared by eight CTAs
    (1024, 2048, 1024, fo.DT_F32, False, None),          # strict fp32: three passes over K in one range list
]


@pytest.mark.parametrize("m,k,n,dt,tf32,chain", SPLIT_CASES, ids=lambda v: str(v))
def test_long_k_split_over_the_sms(m, k, n, dt, tf32, chain):
    """Products of a few tiles with a long K: the tiles' k-blocks are dealt out in ranges to more
    CTAs than there are tiles, partial accumulators travel through scratch memory and are added in
    range order.  Checked
    against the float64 product of the stored operands within the tensor-core tiers, and for
    run-to-run identity (the order of the additions is fixed)."""
    sched = capi.matmul_schedule(m, n, k, capi.BF16 if dt == fo.DT_BF16 else capi.F32,
                                 light_epilogue=chain in (None, "residual"),
                                 compensated=(dt == fo.DT_F32 and not tf32))
    assert sched["sk_units"] > 0, sched
    a, b = _gen(m, k, n, dt, 31)
    rng = np.random.default_rng(32)
    steps, ref = None, None
    mm = (fo.to_accum(a, dt).astype(np.float64) @ fo.to_accum(b, dt).astype(np.float64)).astype(np.float32)
    exp = fo.round_through(mm, dt)
    if chain == "residual":
        resid = fo.from_accum(rng.standard_normal((m, n)).astype(np.float32), dt)
        steps = [("add", resid, capi.OPERAND_FULL)]
        exp = fo.round_through(exp + fo.to_accum(resid, dt), dt)
    elif chain == "col_gelu":
        col = fo.from_accum(rng.standard_normal(n).astype(np.float32), dt)
        steps = [("add", col, capi.OPERAND_COL), ("gelu", None, 0)]
        exp = fo.to_accum(fo.gelu(fo.from_accum(fo.round_through(exp + fo.to_accum(col, dt)[None, :], dt), dt), dt), dt)
    got = _run(a, b, dt, tf32, steps=steps)
    again = _run(a, b, dt, tf32, steps=steps)
    assert np.array_equal(got, again)
    got32 = fo.to_accum(got, dt)
    scale = np.sqrt(k) * float(np.sqrt((fo.to_accum(a, dt) ** 2).mean()) * np.sqrt((fo.to_accum(b, dt) ** 2).mean()))
    if dt == fo.DT_BF16:
        rtol, atol = 2e-2, 2e-3 * max(scale, 1.0)
    elif tf32:
        rtol, atol = 1e-3, 2e-3 * scale
    else:
        rtol, atol = 1e-5, 3 * 2.0 ** -23 * (k / 8) * max(scale, 1.0)
    err = np.abs(got32 - exp)
    assert np.all(err <= atol + rtol * np.abs(exp)), (float(err.max()), atol)


def test_split_products_on_two_streams_from_two_threads():
    """Two host threads, each with its own stream, run split products (CTAs of one launch wait for
    partial tiles of CTAs of the same launch) back to back.  The launches may be resident on the GPU
    at the same time; ranges are handed out against the order in which CTAs start, so a waiting CTA
    only ever depends on CTAs that are already running, and each stream has its own partial-tile
    workspace: every run must give bit for bit what a lone run gives, and no wait may time out."""
    import threading
    lib = capi.load()
    dt = fo.DT_BF16
    shapes = [(256, 8192, 512), (512, 8192, 1024)]
    jobs = []
    for i, (m, k, n) in enumerate(shapes):
        assert capi.matmul_schedule(m, n, k, capi.BF16)["sk_units"] > 0
        a, b = _gen(m, k, n, dt, 40 + i)
        jobs.append((a, b, _run(a, b, dt, False)))
    errors = []

    def worker(idx):
        try:
            a, b, expected = jobs[idx]
            m, k = a.shape
            n = b.shape[1]
            stream = capi.c_void_p()
            capi.check(lib.fb200_stream_create(0, capi.byref(stream)))
            da, db = capi.DeviceBuffer.from_numpy(a), capi.DeviceBuffer.from_numpy(b)
            dc = capi.DeviceBuffer(m * n * 2)
            for it in range(50):
                capi.matmul(da.ptr, db.ptr, dc.ptr, m, n, k, dt, False, None, stream)
                if it % 10 == 9:
                    capi.synchronize(0, stream)
                    got = dc.download(capi.NP_STORAGE[dt], (m, n))
                    if not np.array_equal(got, expected):
                        errors.append((idx, it))
                        return
            capi.synchronize(0, stream)
        except Exception as e:   # surfaced in the main thread
            errors.append((idx, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert capi.kernel_status(0) == 0
    assert errors == [], errors


@pytest.mark.parametrize("dt,tf32,k,chain", [(fo.DT_F32, True, 48, "col_softplus"), (fo.DT_BF16, False, 64, None),
                                               (fo.DT_BF16, False, 200, "residual")],
                         ids=["tf32_k48_softplus", "bf16_k64", "bf16_k200_residual"])
def test_short_k_products_with_two_epilogue_groups(dt, tf32, k, chain):
    """A K of one to four k-blocks under 296+ tiles: the launch is all epilogue and runs with two
    epilogue groups, one per TMEM accumulator (Mamba's dt_proj: K = 48, bias + softplus).  Ragged M and
    N; float64 product of the stored operands as the checker."""
    m, n = 4700, 2056
    a, b = _gen(m, k, n, dt, 61)
    rng = np.random.default_rng(62)
    mm = (fo.to_accum(a, dt).astype(np.float64) @ fo.to_accum(b, dt).astype(np.float64)).astype(np.float32)
    exp = fo.round_through(mm, dt)
    steps = None
    if chain == "col_softplus":
        col = fo.from_accum(rng.standard_normal(n).astype(np.float32), dt)
        steps = [("add", col, capi.OPERAND_COL), ("softplus", None, 0)]
        z = (exp + fo.to_accum(col, dt)[None, :]).astype(np.float64)
        exp = np.where(z > 20, z, np.log1p(np.exp(np.minimum(z, 20)))).astype(np.float32)
    elif chain == "residual":
        resid = fo.from_accum(rng.standard_normal((m, n)).astype(np.float32), dt)
        steps = [("add", resid, capi.OPERAND_FULL)]
        exp = fo.round_through(exp + fo.to_accum(resid, dt), dt)
    got = fo.to_accum(_run(a, b, dt, tf32, steps=steps), dt)
    scale = np.sqrt(k) * float(np.sqrt((fo.to_accum(a, dt) ** 2).mean()) * np.sqrt((fo.to_accum(b, dt) ** 2).mean()))
    rtol, atol = (2e-2, 2e-3 * max(scale, 1.0)) if dt == fo.DT_BF16 else (1e-3, 2e-3 * scale)
    err = np.abs(got - exp)
    assert np.all(err <= atol + rtol * np.abs(exp)), (float(err.max()), atol)
