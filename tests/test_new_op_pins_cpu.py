"""gelu, silu, softplus and exp exist in this repository only (the reference has no such ops), so
nothing of the reference pins them.  Here their two CPU statements, the numpy restatement used as the
GPU tests' oracle and the C++ CPU kernels registered with the reference's OpRegistry, are pinned
against float64 libm on dense and edge inputs, with a stated bound in units in the last place."""
import numpy as np
import pytest

import new_op_pins as pins
from oracle import frame_oracle as fo
from oracle import ref_runtime

# fp32 libm evaluation of the defining formula: a few rounded operations each
BOUNDS = {"gelu": (6, 4), "silu": (4, 2), "softplus": (3, 0), "exp": (3, 0)}   # (ulps, cancellation factor); numpy's vectorised float32 exp is good to about 2.5


@pytest.mark.parametrize("op", pins.OPS)
def test_numpy_restatement_against_float64(op):
    x = pins.inputs()
    with np.errstate(all="ignore"):
        got = fo.UNARY[op](x, fo.DT_F32)
    ok, worst, at = pins.check(op, x, got, *BOUNDS[op])
    assert ok, (op, worst, float(x[at]), float(got[at]))


@pytest.mark.skipif(not ref_runtime.available(), reason="the reference build (oracle/_ref) is not present")
@pytest.mark.parametrize("op", pins.OPS)
def test_registered_cpu_kernel_against_float64(op):
    from frame_public_b200 import irtext
    ref_runtime.load_b200_backend()
    x = pins.inputs()
    g = irtext.IrGraph("cpu")
    g.output(g.unary(op, g.input("float32", x.shape)))
    comp = ref_runtime.Compiled(g.text(), "cpu")
    (got,) = comp.run([x])
    comp.close()
    ok, worst, at = pins.check(op, x, got, *BOUNDS[op])
    assert ok, (op, worst, float(x[at]), float(got[at]))
