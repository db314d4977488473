"""fb200_dwconv1d_time_major against the oracle's five-step form (transpose, conv1d with
groups = C, slice, unary op, transpose back).  The kernel performs the same fp32 operations in
the same order with the same roundings, so the comparison is bit-exact whenever the unary op is
(relu, or none); SiLU goes through the GPU's exp approximation and is compared in the fp32 /
bf16 tolerance tier."""
import numpy as np
import pytest

from frame_public_b200 import capi
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu


def _five_step(x, w, bias, k, padding, start, stop, op, dt):
    """x: [B, L, C] storage; returns [B, stop-start, C] storage."""
    xt = fo.transpose(x, (0, 2, 1))
    y = fo.conv1d(xt, w, bias, 1, padding, x.shape[2], dt)
    y = fo.slice_(y, 2, start, stop)
    if op is not None:
        y = getattr(fo, op)(y, dt)
    return fo.transpose(y, (0, 2, 1))


@pytest.mark.parametrize("dt,batch,length,chan,k,padding,start,op,exact", [
    (fo.DT_F32, 2, 70, 16, 4, 3, 0, "relu", True),       # the causal form of the Mamba block
    (fo.DT_F32, 1, 33, 8, 3, 1, 0, None, True),          # 'same' convolution, no slice offset
    (fo.DT_F32, 2, 40, 12, 4, 3, 2, "relu", True),       # slice starting inside the padded output
    (fo.DT_BF16, 2, 65, 24, 4, 3, 0, "relu", True),
    (fo.DT_F32, 2, 70, 16, 4, 3, 0, "silu", False),
    (fo.DT_BF16, 1, 50, 16, 2, 1, 0, "silu", False),
])
def test_matches_the_five_step_form(dt, batch, length, chan, k, padding, start, op, exact):
    rng = np.random.default_rng(batch * 1000 + length)
    wide = chan * 2 + (8 if dt != fo.DT_F32 else 4)       # the input is a column window of a wider matrix
    col0 = chan
    xw = fo.from_accum(rng.standard_normal((batch, length, wide)).astype(np.float32), dt)
    x = np.ascontiguousarray(xw[:, :, col0:col0 + chan])
    w = fo.from_accum(rng.normal(0, 0.5, (chan, 1, k)).astype(np.float32), dt)
    bias = fo.from_accum(rng.normal(0, 0.5, (chan,)).astype(np.float32), dt)
    full = length + 2 * padding - k + 1
    stop = min(full, start + length)
    exp = _five_step(x, w, bias, k, padding, start, stop, op, dt)
    out_len = stop - start
    es = capi.ITEMSIZE[dt]
    d_x, d_w, d_b = (capi.DeviceBuffer.from_numpy(t) for t in (xw, w, bias))
    d_o = capi.DeviceBuffer(batch * out_len * chan * es)
    capi.dwconv1d_time_major(capi.c_void_p(d_x.ptr.value + col0 * es), wide, d_w.ptr, d_b.ptr, d_o.ptr, chan, batch, length,
                             out_len, chan, k, start - padding, [op] if op else [], dt)
    capi.synchronize()
    got = d_o.download(capi.NP_STORAGE[dt], (batch, out_len, chan))
    if exact:
        assert np.array_equal(got.view(np.uint8), np.ascontiguousarray(exp).view(np.uint8)), fo.max_err(got, exp, dt)
    else:
        assert fo.all_close(got, exp, dt), fo.max_err(got, exp, dt)


def test_rejects_what_the_vector_layout_cannot_address():
    lib = capi.load()
    buf = capi.DeviceBuffer(4096)
    ops = (capi.c_int * 1)(capi.EW["relu"])
    rc = lib.fb200_dwconv1d_time_major(buf.ptr, 6, buf.ptr, None, buf.ptr, 6, 1, 8, 8, 6, 4, -3, ops, 1, capi.F32, None)
    assert rc == 1 and b"multiples of 4" in lib.fb200_last_error()
    rc = lib.fb200_dwconv1d_time_major(buf.ptr, 8, buf.ptr, None, buf.ptr, 8, 1, 8, 8, 8, 9, -3, ops, 1, capi.F32, None)
    assert rc == 1 and b"k <= 8" in lib.fb200_last_error()
