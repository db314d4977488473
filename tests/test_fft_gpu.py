"""rfft / irfft on the GPU through the C ABI: the reference's known-answer vectors
(tests/cpp/ops/test_op_fft.cpp:287-395, :477-500), round trips at larger sizes, and the float32-only
rule."""
import numpy as np
import pytest

from frame_public_b200 import capi
from oracle import frame_oracle as fo
from test_fft_cpu import RFFT_KNOWN

pytestmark = pytest.mark.gpu


def _rfft(x):
    x = np.ascontiguousarray(x, np.float32)
    n = x.shape[-1]
    dx = capi.DeviceBuffer.from_numpy(x)
    out = capi.DeviceBuffer(x.size // n * (n // 2 + 1) * 8)
    capi.rfft(dx.ptr, out.ptr, x.size // n, n, capi.F32)
    capi.synchronize()
    return out.download(np.float32, x.shape[:-1] + (n // 2 + 1, 2))


def _irfft(z, n):
    z = np.ascontiguousarray(z, np.float32)
    dz = capi.DeviceBuffer.from_numpy(z)
    rows = z.size // (2 * (n // 2 + 1))
    out = capi.DeviceBuffer(rows * n * 4)
    capi.irfft(dz.ptr, out.ptr, rows, n, capi.F32)
    capi.synchronize()
    return out.download(np.float32, z.shape[:-2] + (n,))


@pytest.mark.parametrize("x,expected", RFFT_KNOWN)
def test_rfft_known_answers(x, expected):
    np.testing.assert_allclose(_rfft(x).reshape(-1), np.asarray(expected, np.float32), rtol=1e-5, atol=1e-6)


def test_irfft_known_answer():
    z = np.asarray([0, 0, 2, 0, 0, 0], np.float32).reshape(3, 2)
    np.testing.assert_allclose(_irfft(z, 4), np.asarray([1, 0, -1, 0], np.float32), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("shape", [(6,), (5,), (2, 6), (16, 1024), (4, 3, 729), (3, 4099)])
def test_round_trip_and_parseval(shape):
    x = np.random.default_rng(9).standard_normal(shape).astype(np.float32)
    n = shape[-1]
    spec = _rfft(x)
    np.testing.assert_allclose(_irfft(spec, n), x, rtol=1e-5, atol=2e-6)
    # Parseval with the Hermitian weights: sum x^2 = (1/n) sum w_k |X_k|^2
    w = np.full(n // 2 + 1, 2.0)
    w[0] = 1.0
    if n % 2 == 0:
        w[-1] = 1.0
    power = (spec.astype(np.float64) ** 2).sum(-1)
    np.testing.assert_allclose((power * w).sum(-1) / n, (x.astype(np.float64) ** 2).sum(-1), rtol=1e-5)
    assert fo.all_close(spec, fo.rfft(x), fo.DT_F32, rtol=1e-5, atol=1e-5)


def test_only_float32_is_accepted():
    buf = capi.DeviceBuffer(64)
    with pytest.raises(capi.Fb200Error, match="float32"):
        capi.rfft(buf.ptr, buf.ptr, 1, 4, capi.BF16)
    with pytest.raises(capi.Fb200Error, match=">= 2"):
        capi.rfft(buf.ptr, buf.ptr, 1, 1, capi.F32)
