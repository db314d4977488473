"""Independent pins for the ops the reference does not have (gelu, silu, softplus, exp): float64
libm evaluations of the defining formulas on dense and edge inputs, and the error bound each
implementation must meet.

Bound: |got - ref| <= ulps * ulp32(ref) + cancel * 2^-24 * |x|, where ulp32(ref) is the spacing of
float32 at the float64 reference value.  The second term is only non-zero for gelu and silu, whose
defining formulas cancel in fp32 for negative x (0.5*x*(1 + tanh(t)) with tanh(t) -> -1): the
absolute error there is a few rounding errors of the factor that multiplies x.  NaN must map to
NaN, +-inf to the formula's own limit, and the sign of a zero result is not compared."""
import numpy as np

OPS = ("gelu", "silu", "softplus", "exp")


def inputs() -> np.ndarray:
    dense = np.linspace(-30.0, 30.0, 120001, dtype=np.float64).astype(np.float32)
    fine = np.linspace(-2.0, 2.0, 40001, dtype=np.float64).astype(np.float32)
    t = np.float32(20.0)
    edge = np.array([0.0, -0.0, 1e-40, -1e-40, 1.1754944e-38, -1.1754944e-38, 1e-20, -1e-20,
                     t, np.nextafter(t, np.float32(0)), np.nextafter(t, np.float32(40)), -t,
                     15.0, -15.0, 50.0, -50.0, 80.0, -80.0, 88.0, -87.0, -100.0, -104.0,
                     np.inf, -np.inf, np.nan], dtype=np.float32)
    return np.concatenate([dense, fine, edge])


def reference(op: str, x32: np.ndarray) -> np.ndarray:
    x = x32.astype(np.float64)
    with np.errstate(all="ignore"):
        if op == "gelu":
            inner = 0.7978845608028654 * (x + 0.044715 * x * x * x)
            r = 0.5 * x * (1.0 + np.tanh(inner))
        elif op == "silu":
            r = x / (1.0 + np.exp(-x))
            r = np.where(np.isneginf(x), np.nan, r)        # -inf * 0 in the defining product x * sigmoid(x)
        elif op == "softplus":
            r = np.where(x > 20.0, x, np.log1p(np.exp(np.minimum(x, 30.0))))
        elif op == "exp":
            r = np.exp(x)
        else:
            raise KeyError(op)
    return r


def ulp32(ref64: np.ndarray) -> np.ndarray:
    a = np.abs(ref64)
    a32 = np.minimum(a, np.finfo(np.float32).max).astype(np.float32)
    with np.errstate(all="ignore"):
        up = np.nextafter(a32, np.float32(np.inf)).astype(np.float64) - a32.astype(np.float64)
    return np.where(np.isfinite(up), np.maximum(up, 2.0 ** -149), 2.0 ** 104)


def check(op: str, x32: np.ndarray, got32: np.ndarray, ulps: float, cancel: float):
    """(ok, worst error in ulps of the reference, index of the worst element)."""
    ref = reference(op, x32)
    got = got32.astype(np.float64)
    both_nan = np.isnan(ref) & np.isnan(got)
    overflow = np.abs(ref) > np.finfo(np.float32).max       # float32 has no finite value there
    ref_c = np.where(overflow, np.sign(ref) * np.inf, ref)
    same_inf = np.isinf(ref_c) & np.isinf(got) & (np.sign(ref_c) == np.sign(got))
    x_abs = np.where(np.isfinite(x32), np.abs(x32.astype(np.float64)), 0.0)
    with np.errstate(all="ignore"):
        err = np.abs(got - ref_c)
        bound = ulps * ulp32(ref) + cancel * 2.0 ** -24 * x_abs
        ok = (err <= bound) | both_nan | same_inf
        in_ulps = np.where(both_nan | same_inf, 0.0, (err - cancel * 2.0 ** -24 * x_abs) / ulp32(ref))
    in_ulps = np.where(ok, np.where(np.isfinite(in_ulps), np.maximum(in_ulps, 0.0), 0.0), np.where(np.isfinite(in_ulps), in_ulps, 1e30))
    worst = int(np.nanargmax(in_ulps))
    return bool(np.all(ok)), float(in_ulps[worst]), worst
