"""fb200_selective_scan_noalloc — the scan for hosts that may not allocate device memory while it
runs (graph capture in progress, or all device memory planned ahead): its scratch is a fixed array
inside the library instead of a stream-ordered allocation.  Called through the C ABI and compared
with fb200_selective_scan on the same inputs, twice in a row with different data (the array keeps
the previous call's contents, which must not leak into the next result).  Collected last on
purpose: a failure here must not hide any other test from a run that stops at the first failure."""
import numpy as np
import pytest

from frame_public_b200 import capi
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu


def _inputs(rows, steps, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, steps)).astype(np.float32)
    a = rng.uniform(0.5, 0.99, (rows, steps)).astype(np.float32)
    b, c, d = (rng.standard_normal((rows, steps)).astype(np.float32) for _ in range(3))
    return [x, a, b, c, d]


def _run(entry, arrays):
    rows, steps = arrays[0].shape
    bufs = [capi.DeviceBuffer.from_numpy(t) for t in arrays]
    out = capi.DeviceBuffer(arrays[0].nbytes)
    capi.check(entry(*[t.ptr for t in bufs], out.ptr, rows, steps, capi.F32, None))
    capi.synchronize()
    return out.download(np.float32, (rows, steps))


def test_noalloc_scan_matches_the_allocating_entry_point_twice():
    lib = capi.load()
    for seed, (rows, steps) in ((41, (8, 16384)), (42, (3, 40960))):
        arrays = _inputs(rows, steps, seed)
        ref = _run(lib.fb200_selective_scan, arrays)
        got = _run(lib.fb200_selective_scan_noalloc, arrays)
        # same tolerance tier as the other fp32 scan tests (1e-5 relative, 1e-6 absolute)
        assert fo.all_close(got, ref, fo.DT_F32), fo.max_err(got, ref)
    # and against the CPU oracle for the last case (the chunked association differs from the CPU's
    # sequential one and outputs near zero come from cancellation, hence the absolute term)
    exp = fo.selective_scan(*arrays)
    assert fo.all_close(got, exp, fo.DT_F32, rtol=1e-4, atol=1e-4), fo.max_err(got, exp)


def test_noalloc_scan_rejects_what_its_fixed_scratch_cannot_hold():
    lib = capi.load()
    buf = capi.DeviceBuffer(1024)
    rc = lib.fb200_selective_scan_noalloc(buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr,
                                          65537, 4, capi.F32, None)
    assert rc == 1 and b"exceed the fixed scratch" in lib.fb200_last_error()
    rc = lib.fb200_selective_scan_noalloc(buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr,
                                          4, 6, capi.F32, None)
    assert rc == 1 and b"multiple of 4" in lib.fb200_last_error()
