"""The fused Mamba scan (a new op: no counterpart in the reference, parity unpinned by it) through
the C ABI against the numpy oracle, which itself is pinned to the reference's selective_scan on
materialised operands (tests/test_oracle_pins.py).  fp32; the state sum is associated differently
on the GPU (four partial sums + two shuffles), hence the fp32 tolerance tier rather than bit
equality.  Sequences of a few hundred steps with few channels run as several time chunks: the state
a chunk starts from is rebuilt from the earlier chunks' end states and decays."""
import numpy as np
import pytest

from frame_public_b200 import capi
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(2, 9, 5, 4), (1, 33, 40, 16), (3, 64, 70, 16), (2, 17, 32, 8),
                                   (2, 100, 48, 16), (1, 8, 64, 16), (1, 3, 32, 4),   # cp.async pipeline
                                   # long enough for several time chunks (summary + apply passes):
                                   # chunk boundaries inside and at the end of the sequence
                                   (1, 512, 64, 16), (2, 300, 32, 16), (1, 1000, 32, 8), (3, 257, 16, 16)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("gated", [True, False], ids=["gated", "ungated"])
def test_mamba_scan_matches_oracle(shape, gated):
    bt, L, dm, n = shape
    rng = np.random.default_rng(31)
    u = rng.standard_normal((bt, L, dm)).astype(np.float32)
    delta = rng.uniform(1e-3, 1e-1, (bt, L, dm)).astype(np.float32)
    A = -np.tile(np.arange(1, n + 1, dtype=np.float32), (dm, 1))
    B = rng.standard_normal((bt, L, n)).astype(np.float32)
    C = rng.standard_normal((bt, L, n)).astype(np.float32)
    D = rng.standard_normal(dm).astype(np.float32)
    z = rng.standard_normal((bt, L, dm)).astype(np.float32) if gated else None
    bufs = [capi.DeviceBuffer.from_numpy(t) for t in (u, delta, A, B, C, D)]
    dz = capi.DeviceBuffer.from_numpy(z) if gated else None
    dy = capi.DeviceBuffer(u.nbytes)
    capi.mamba_scan(*[b.ptr for b in bufs], dz.ptr if gated else None, dy.ptr, bt, L, dm, n)
    capi.synchronize()
    got = dy.download(np.float32, u.shape)
    exp = fo.mamba_scan(u, delta, A, B, C, D, z)
    assert fo.all_close(got, exp, fo.DT_F32, rtol=1e-5, atol=2e-6), fo.max_err(got, exp)
