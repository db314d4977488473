"""The sm_100a kernels of gelu, silu, softplus and exp against float64 libm on dense and edge inputs
(the reference has no such ops, so nothing of the reference pins them).  The kernels use the
hardware's ex2 / lg2 approximations: exp(x) as ex2(x * log2 e) loses about |x| * 2^-24 relative in
the argument scaling, so the bound grows with |x|:

    |got - ref| <= (ulps + slope * |x|) * ulp32(ref) + cancel * 2^-24 * |x|

softplus adds lg2.approx, whose absolute error of about 2^-22 is up to 20 ulps where the result is
near 0.1.  fp32 `exp` itself goes through the accurate expf.  Every bound stays inside the fp32 tolerance tier
(rtol 1e-5, atol 1e-6) the parity tests use; that tier is asserted as well."""
import json
import os

import numpy as np
import pytest

import new_op_pins as pins
from frame_public_b200 import capi

pytestmark = pytest.mark.gpu

# (ulps, cancellation factor, ulps per unit of |x|)
BOUNDS = {"gelu": (8, 6, 2.0), "silu": (8, 4, 2.0), "softplus": (32, 0, 2.0), "exp": (3, 0, 0.0)}


def _run(op, x):
    dx = capi.DeviceBuffer.from_numpy(x)
    out = capi.DeviceBuffer(x.nbytes)
    capi.fused_elementwise([dx.ptr], out.ptr, x.size, capi.F32, [op])
    capi.synchronize()
    return out.download(np.float32, x.shape)


@pytest.mark.parametrize("op", pins.OPS)
def test_gpu_kernel_against_float64(op):
    x = pins.inputs()
    got = _run(op, x)
    ulps, cancel, slope = BOUNDS[op]
    ref = pins.reference(op, x)
    finite = np.isfinite(ref) & np.isfinite(x) & (np.abs(ref) < 3e38)
    err = np.abs(got.astype(np.float64) - ref)
    x_abs = np.where(np.isfinite(x), np.abs(x.astype(np.float64)), 0.0)
    in_ulps = np.where(finite, np.maximum(err - cancel * 2.0 ** -24 * x_abs, 0.0) / pins.ulp32(ref), 0.0)
    worst = int(np.argmax(in_ulps - slope * x_abs))
    path = os.environ.get("FRAME_B200_ERROR_TABLE")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"case": "new_op_pin_" + op, "max_ulps": float(in_ulps.max()), "at_x": float(x[int(np.argmax(in_ulps))]),
                                "max_ulps_small_x": float(in_ulps[x_abs <= 2.0].max())}) + "\n")
    assert np.all(in_ulps[finite] <= ulps + slope * x_abs[finite]), (op, float(in_ulps[worst]), float(x[worst]), float(got[worst]))
    # non-finite inputs and overflow: NaN stays NaN, infinities agree
    rest = ~finite
    r, g = ref[rest], got[rest].astype(np.float64)
    r = np.where(np.abs(r) > 3.4028234663852886e38, np.sign(r) * np.inf, r)
    assert np.all((np.isnan(r) & np.isnan(g)) | (r == g)), (op, r, g)
    # and the tier the parity tests use
    assert np.all(err[finite] <= 1e-6 + 1e-5 * np.abs(ref[finite]))
