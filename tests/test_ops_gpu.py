"""GPU parity tests proper: every case of tests/cases.py through the C ABI of libframe_b200.so
against the CPU oracle.  Bit-exact for integer / indexing work and for fp32 ops whose kernel
keeps the CPU's order of operations; |a-e| <= atol + rtol*|e| with the reference's tolerances
(fp32 1e-5/1e-6, bf16 2e-2/2e-3; tests/cpp/common/tolerance.h:41-98 of the reference) for the
rest."""
import numpy as np
import pytest

import cases
import gpu_dispatch
from frame_public_b200 import capi
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _require_gpu():
    assert capi.device_count() >= 1, "no CUDA device: the GPU tests need a B200"
    yield
    assert capi.kernel_status(0) == 0, "a bounded wait gave up inside a tensor-core kernel"


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.name)
def test_case_matches_oracle(case):
    exact = case.exact
    if case.op == "matmul":
        m, k = case.inputs[0].shape
        n = case.inputs[1].shape[1]
        if capi.load().fb200_matmul_uses_tensor_cores(m, n, k, case.dtype, 0):
            exact = False  # tensor-core accumulation order differs from the CPU's
    got = gpu_dispatch.run_case(case)
    gpu_dispatch.assert_parity(case, got, exact)


def test_launches_are_counted():
    before = capi.launch_count()
    gpu_dispatch.run_case(cases.CASES_BY_NAME["add_f32_1024"])
    assert capi.launch_count() == before + 1


def test_invalid_arguments_are_rejected_with_messages():
    lib = capi.load()
    rc = lib.fb200_softmax(None, None, 4, 4, capi.F32, None)
    assert rc == 1 and b"null" in lib.fb200_last_error()
    rc = lib.fb200_softmax(None, None, 4, 4, capi.I32, None)
    assert rc == 1
    buf = capi.DeviceBuffer(64)
    rc = lib.fb200_selective_scan(buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, 4, 0, capi.F32, None)
    assert rc == 1 and b"steps" in lib.fb200_last_error()
    ops = (capi.c_int * 1)(99)
    ar = (capi.c_int * 1)(1)
    ptrs = (capi.c_void_p * 1)(buf.ptr.value)
    rc = lib.fb200_fused_elementwise(ptrs, 1, buf.ptr, 4, capi.F32, ops, ar, 1, None)
    assert rc == 4  # UNIMPLEMENTED names the unknown sub-op
    # zero-size tensors are legal and launch nothing
    before = capi.launch_count()
    assert lib.fb200_softmax(None, None, 0, 4, capi.F32, None) == 0
    assert capi.launch_count() == before


def test_hal_allocator_and_copies_round_trip():
    lib = capi.load()
    p = capi.c_void_p()
    assert lib.fb200_malloc(0, 0, 64, capi.byref(p)) == 1          # zero bytes rejected
    assert lib.fb200_malloc(0, 64, 512, capi.byref(p)) == 1        # alignment > 256 rejected
    assert lib.fb200_malloc(0, 1000, 64, capi.byref(p)) == 0
    assert p.value % 256 == 0
    src = np.arange(250, dtype=np.int32)
    dst = np.zeros_like(src)
    q = capi.DeviceBuffer(1000)
    capi.check(lib.fb200_memcpy(0, p, src.ctypes.data, 1000, capi.H2D, None, 1))
    capi.check(lib.fb200_memcpy(0, q.ptr, p, 1000, capi.D2D, None, 1))
    capi.check(lib.fb200_memcpy(0, dst.ctypes.data, q.ptr, 1000, capi.D2H, None, 1))
    assert np.array_equal(src, dst)
    assert lib.fb200_memcpy(0, None, None, 0, capi.H2D, None, 1) == 0
    assert lib.fb200_memcpy(0, None, src.ctypes.data, 8, capi.H2D, None, 1) == 1
    capi.check(lib.fb200_free(0, p))
    # un-recorded event reports complete; record -> wait -> sync
    ev, st = capi.c_void_p(), capi.c_void_p()
    capi.check(lib.fb200_event_create(0, 0, capi.byref(ev)))
    capi.check(lib.fb200_stream_create(0, capi.byref(st)))
    done = capi.c_int(0)
    capi.check(lib.fb200_event_query(0, ev, capi.byref(done)))
    assert done.value == 1
    capi.check(lib.fb200_event_record(0, ev, st))
    capi.check(lib.fb200_stream_wait_event(0, st, ev))
    capi.check(lib.fb200_event_synchronize(0, ev))
    capi.check(lib.fb200_stream_synchronize(0, st))
    capi.check(lib.fb200_event_destroy(0, ev))
    capi.check(lib.fb200_stream_destroy(0, st))


def test_gather_names_an_out_of_range_index():
    lib = capi.load()
    x = capi.DeviceBuffer.from_numpy(np.zeros((5, 4), np.float32))
    out = capi.DeviceBuffer(3 * 4 * 4)
    for bad, npdt, code in ((7, np.int32, capi.I32), (-2, np.int64, capi.I64)):
        idx = capi.DeviceBuffer.from_numpy(np.array([0, bad, 4], dtype=npdt))
        rc = lib.fb200_gather(x.ptr, idx.ptr, out.ptr, 5, 4, 3, capi.F32, code, None)
        assert rc == 1 and f"index {bad} is out of range [0, 5)".encode() in lib.fb200_last_error()
        rc = lib.fb200_scatter_add(out.ptr, idx.ptr, x.ptr, 3, 4, 5, capi.F32, code, None)
        assert rc == 1 and f"index {bad} is out of range".encode() in lib.fb200_last_error()


@pytest.mark.parametrize("dt", [fo.DT_F32, fo.DT_BF16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", [(37, 1024), (5, 24), (300, 4096)], ids=lambda s: "x".join(map(str, s)))
def test_add_layer_norm_equals_add_then_layer_norm(dt, shape):
    """layer_norm(x + res) in one pass: the stored sum is bit for bit what `add` stores, the
    normalised rows bit for bit what layer_norm makes of that sum ([5, 24] in fp32 is outside the
    vector path for bf16 only by alignment of 24 % 8: both routes must agree all the same).  Also
    with the result written exactly over x, as the memory planner lays a transformer block out."""
    rows, cols = shape
    rng = np.random.default_rng(51)
    x = fo.from_accum(rng.standard_normal(shape).astype(np.float32), dt)
    res = fo.from_accum(rng.standard_normal(shape).astype(np.float32), dt)
    g = fo.from_accum(rng.uniform(0.5, 1.5, cols).astype(np.float32), dt)
    b = fo.from_accum(rng.standard_normal(cols).astype(np.float32), dt)
    cdt = capi.F32 if dt == fo.DT_F32 else capi.BF16
    es = capi.ITEMSIZE[cdt]
    dx, dr, dg, db = (capi.DeviceBuffer.from_numpy(t) for t in (x, res, g, b))
    ds, do = capi.DeviceBuffer(rows * cols * es), capi.DeviceBuffer(rows * cols * es)
    # reference: the two operators of this library (each pinned against the oracle elsewhere)
    capi.fused_elementwise([dx.ptr, dr.ptr], ds.ptr, rows * cols, cdt, ["add"])
    capi.layer_norm(ds.ptr, dg.ptr, db.ptr, do.ptr, rows, cols, 1e-5, cdt)
    capi.synchronize()
    sum_ref = ds.download(capi.NP_STORAGE[cdt], shape)
    out_ref = do.download(capi.NP_STORAGE[cdt], shape)
    ds2, do2 = capi.DeviceBuffer(rows * cols * es), capi.DeviceBuffer(rows * cols * es)
    capi.add_layer_norm(dx.ptr, dr.ptr, dg.ptr, db.ptr, ds2.ptr, do2.ptr, rows, cols, 1e-5, cdt)
    capi.synchronize()
    assert np.array_equal(ds2.download(capi.NP_STORAGE[cdt], shape), sum_ref)
    assert np.array_equal(do2.download(capi.NP_STORAGE[cdt], shape), out_ref)
    # result over x itself
    capi.add_layer_norm(dx.ptr, dr.ptr, dg.ptr, db.ptr, ds2.ptr, dx.ptr, rows, cols, 1e-5, cdt)
    capi.synchronize()
    assert np.array_equal(dx.download(capi.NP_STORAGE[cdt], shape), out_ref)
    assert fo.all_close(out_ref, fo.layer_norm(fo.add(x, res, dt), g, b, 1e-5, dt), dt, rtol=2e-2 if dt == fo.DT_BF16 else 1e-5, atol=2e-2 if dt == fo.DT_BF16 else 1e-5)
