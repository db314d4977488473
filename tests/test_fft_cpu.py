"""rfft / irfft oracle against the reference's own known-answer tests
(tests/cpp/ops/test_op_fft.cpp:287-395 eager rfft, :454-500 compiled rfft / irfft, :525-570 round
trips).  The reference's CPU kernel calls pocketfft, which its build downloads and which is absent
here, so these literal vectors — not outputs of the reference binary — pin the restatement."""
import numpy as np
import pytest

from oracle import frame_oracle as fo

RFFT_KNOWN = [
    ([1, 0, 0, 0], [1, 0, 1, 0, 1, 0]),                      # impulse, even n
    ([2, 2, 2, 2], [8, 0, 0, 0, 0, 0]),                      # constant, even n
    ([1, 0, -1, 0], [0, 0, 2, 0, 0, 0]),                     # one cycle of a cosine, even n
    ([1, 0, 0, 0, 0], [1, 0, 1, 0, 1, 0]),                   # impulse, odd n
    ([2, 2, 2, 2, 2], [10, 0, 0, 0, 0, 0]),                  # constant, odd n
    ([1.0, 0.30901699, -0.80901699, -0.80901699, 0.30901699], [0, 0, 2.5, 0, 0, 0]),   # cos(2*pi*j/5)
]


@pytest.mark.parametrize("x,expected", RFFT_KNOWN)
def test_rfft_known_answers_of_the_reference(x, expected):
    got = fo.rfft(np.asarray(x, np.float32))
    assert got.shape == (len(x) // 2 + 1, 2)
    np.testing.assert_allclose(got.reshape(-1), np.asarray(expected, np.float32), rtol=1e-5, atol=1e-6)


def test_irfft_known_answer_of_the_reference():
    z = np.asarray([0, 0, 2, 0, 0, 0], np.float32).reshape(3, 2)
    np.testing.assert_allclose(fo.irfft(z, 4), np.asarray([1, 0, -1, 0], np.float32), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("x", [[1, 2, 3, 4, 5, 6], [1, -2, 3, 0.5, 4],
                               [[1, 2, 3, 4, 5, 6], [-1, 0.5, 2.5, -3, 4.5, 0]]])
def test_round_trips_of_the_reference(x):
    xv = np.asarray(x, np.float32)
    n = xv.shape[-1]
    np.testing.assert_allclose(fo.irfft(fo.rfft(xv), n), xv, rtol=1e-5, atol=1e-6)


def test_oracle_agrees_with_numpy_fft_and_ignores_the_imaginary_dc_and_nyquist():
    rng = np.random.default_rng(5)
    for n in (8, 9, 64, 243):
        x = rng.standard_normal((3, n)).astype(np.float32)
        ref = np.fft.rfft(x.astype(np.float64), axis=-1)
        got = fo.rfft(x)
        np.testing.assert_allclose(got[..., 0], ref.real, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(got[..., 1], ref.imag, rtol=1e-5, atol=1e-5)
        z = rng.standard_normal((3, n // 2 + 1, 2)).astype(np.float32)
        zc = z[..., 0].astype(np.float64) + 1j * z[..., 1].astype(np.float64)
        np.testing.assert_allclose(fo.irfft(z, n), np.fft.irfft(zc, n=n, axis=-1), rtol=1e-5, atol=1e-6)
