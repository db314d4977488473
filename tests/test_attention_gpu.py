"""fb200_attention_fan (tcgen05/TMEM/TMA) against the CPU oracle's matmul -> softmax -> matmul
per head.  Every intermediate is rounded to the storage dtype at the same three points as the
separate operators; what differs is the order of the fp32 additions, and a score that lands on
the other side of a 16-bit rounding boundary moves its probability by one storage ulp of the
score (2^-8 relative for bf16).  Tolerance: the bf16 tier, one notch looser in the absolute term
for a chain of three 16-bit operators (rtol 2e-2, atol 2e-2 of outputs that are O(1))."""
import numpy as np
import pytest

from frame_public_b200 import capi
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu

TOL = dict(rtol=2e-2, atol=2e-2)


def _store(x, dt):
    return fo.from_accum(np.asarray(x, dtype=np.float32), dt)


def _fused_qkv_case(batch, heads, seq, dt, seed):
    """The layout of the transformer workload: one [batch*seq, 3*heads*64] projection, the output
    in the concatenated [batch*seq, heads*64] layout."""
    rng = np.random.default_rng(seed)
    width = heads * 64
    qkv = _store(rng.uniform(-1, 1, (batch * seq, 3 * width)), dt)
    table = np.zeros(batch * heads, dtype=capi.HEAD_DTYPE)
    for b in range(batch):
        for h in range(heads):
            table[b * heads + h] = (b * seq, h * 64, b * seq, width + h * 64, b * seq,
                                    2 * width + h * 64, b * seq * width + h * 64)
    exp = np.zeros((batch * seq, width), dtype=np.uint16)
    for b in range(batch):
        rows = slice(b * seq, (b + 1) * seq)
        for h in range(heads):
            q = qkv[rows, h * 64:(h + 1) * 64]
            k = qkv[rows, width + h * 64:width + (h + 1) * 64]
            v = qkv[rows, 2 * width + h * 64:2 * width + (h + 1) * 64]
            exp[rows, h * 64:(h + 1) * 64] = fo.attention_fan(q, k, v, dt)
    return qkv, table, exp


@pytest.mark.parametrize("batch,heads,seq,dt", [(2, 3, 128, fo.DT_BF16), (1, 2, 512, fo.DT_BF16),
                                                (2, 1, 256, fo.DT_F16), (1, 2, 64, fo.DT_BF16)])
def test_fan_over_a_fused_qkv_projection(batch, heads, seq, dt):
    qkv, table, exp = _fused_qkv_case(batch, heads, seq, dt, seed=seq + heads)
    rows, ld = qkv.shape
    width = heads * 64
    d_qkv = capi.DeviceBuffer.from_numpy(qkv)
    d_tab = capi.DeviceBuffer.from_numpy(table.view(np.uint8))
    d_out = capi.DeviceBuffer(rows * width * 2)
    for _ in range(2):   # a second launch over the same buffers must agree
        capi.attention_fan(d_qkv.ptr, rows, ld, d_qkv.ptr, rows, ld, d_qkv.ptr, rows, ld, d_out.ptr,
                           width, d_tab.ptr, len(table), seq, seq, 64, dt)
        capi.synchronize()
        assert capi.kernel_status(0) == 0
        got = d_out.download(np.uint16, (rows, width))
        assert fo.all_close(got, exp, dt, **TOL), fo.max_err(got, exp, dt)


def test_launches_over_the_same_buffers_are_bit_identical_at_the_transformer_size():
    """8 sequences x 16 heads x 512 keys (128 CTAs walking four query blocks each): every hand-over
    inside the kernel is ordered, so repeated launches agree bit for bit."""
    batch, heads, seq, dt = 8, 16, 512, fo.DT_BF16
    rng = np.random.default_rng(11)
    width = heads * 64
    qkv = _store(rng.uniform(-1, 1, (batch * seq, 3 * width)), dt)
    table = np.zeros(batch * heads, dtype=capi.HEAD_DTYPE)
    for b in range(batch):
        for h in range(heads):
            table[b * heads + h] = (b * seq, h * 64, b * seq, width + h * 64, b * seq,
                                    2 * width + h * 64, b * seq * width + h * 64)
    rows, ld = qkv.shape
    d_qkv = capi.DeviceBuffer.from_numpy(qkv)
    d_tab = capi.DeviceBuffer.from_numpy(table.view(np.uint8))
    d_out = capi.DeviceBuffer(rows * width * 2)
    first = None
    for i in range(6):
        capi.attention_fan(d_qkv.ptr, rows, ld, d_qkv.ptr, rows, ld, d_qkv.ptr, rows, ld, d_out.ptr,
                           width, d_tab.ptr, len(table), seq, seq, 64, dt, scale=0.125)
        capi.synchronize()
        assert capi.kernel_status(0) == 0
        got = d_out.download(np.uint16, (rows, width))
        if first is None:
            first = got
            # one head against the oracle
            q, k, v = qkv[:seq, :64], qkv[:seq, width:width + 64], qkv[:seq, 2 * width:2 * width + 64]
            const = _store(np.full((seq, seq), 0.125, dtype=np.float32), dt)
            exp = fo.matmul(fo.softmax(fo.mul(fo.matmul(q, np.ascontiguousarray(k.T), dt), const, dt), dt), v, dt)
            assert fo.all_close(got[:seq, :64], exp, dt, **TOL), fo.max_err(got[:seq, :64], exp, dt)
        else:
            assert np.array_equal(first, got), (i, int((first != got).sum()))


@pytest.mark.parametrize("scale", [0.125, 0.3])
def test_scores_scaled_by_a_constant_before_the_softmax(scale):
    """The reference's own attention multiplies the scores by a constant tensor filled with
    1/sqrt(head_dim) (an elementwise mul, rounded to the storage dtype) before the softmax."""
    dt = fo.DT_BF16
    rng = np.random.default_rng(5)
    q, k, v = (_store(rng.uniform(-1, 1, (128, 64)), dt) for _ in range(3))
    const = _store(np.full((128, 128), scale, dtype=np.float32), dt)
    s = fo.mul(fo.matmul(q, np.ascontiguousarray(k.T), dt), const, dt)
    exp = fo.matmul(fo.softmax(s, dt), v, dt)
    table = np.zeros(1, dtype=capi.HEAD_DTYPE)
    bufs = [capi.DeviceBuffer.from_numpy(t) for t in (q, k, v)]
    out = capi.DeviceBuffer(128 * 64 * 2)
    d_tab = capi.DeviceBuffer.from_numpy(table.view(np.uint8))
    stored_scale = float(fo.to_accum(const, dt)[0, 0])
    capi.attention_fan(bufs[0].ptr, 128, 64, bufs[1].ptr, 128, 64, bufs[2].ptr, 128, 64, out.ptr, 64,
                       d_tab.ptr, 1, 128, 128, 64, dt, scale=stored_scale)
    capi.synchronize()
    assert capi.kernel_status(0) == 0
    got = out.download(np.uint16, (128, 64))
    assert fo.all_close(got, exp, dt, **TOL), fo.max_err(got, exp, dt)


def test_ragged_queries_separate_operands_and_untouched_neighbours():
    """sq = 200 (two query blocks, the second partly empty), sk = 192, q / k / v in separate
    matrices with different pitches, the output inside a wider matrix whose other bytes stay."""
    dt = fo.DT_BF16
    rng = np.random.default_rng(7)
    sq, sk = 200, 192
    qm = _store(rng.uniform(-1, 1, (sq + 9, 72)), dt)
    km = _store(rng.uniform(-1, 1, (sk + 3, 136)), dt)
    vm = _store(rng.uniform(-1, 1, (sk, 64)), dt)
    q, k, v = qm[9:, 8:72], km[3:, 64:128], vm
    exp = fo.attention_fan(np.ascontiguousarray(q), np.ascontiguousarray(k), v, dt)
    o_ld = 80
    out0 = np.full((sq + 2, o_ld), 0x4049, dtype=np.uint16)
    table = np.zeros(1, dtype=capi.HEAD_DTYPE)
    table[0] = (9, 8, 3, 64, 0, 0, 1 * o_ld + 8)
    bufs = [capi.DeviceBuffer.from_numpy(t) for t in (qm, km, vm, out0)]
    d_tab = capi.DeviceBuffer.from_numpy(table.view(np.uint8))
    capi.attention_fan(bufs[0].ptr, qm.shape[0], 72, bufs[1].ptr, km.shape[0], 136, bufs[2].ptr, sk, 64,
                       bufs[3].ptr, o_ld, d_tab.ptr, 1, sq, sk, 64, dt)
    capi.synchronize()
    assert capi.kernel_status(0) == 0
    got = bufs[3].download(np.uint16, out0.shape)
    assert fo.all_close(got[1:1 + sq, 8:72], exp, dt, **TOL), fo.max_err(got[1:1 + sq, 8:72], exp, dt)
    mask = np.ones(out0.shape, dtype=bool)
    mask[1:1 + sq, 8:72] = False
    assert np.all(got[mask] == 0x4049)


def test_unsupported_shapes_are_unimplemented_not_wrong():
    lib = capi.load()
    buf = capi.DeviceBuffer(4096)
    for sq, sk, d, dt in [(128, 1024, 64, capi.BF16), (128, 96, 64, capi.BF16), (128, 128, 32, capi.BF16),
                          (128, 128, 64, capi.F32)]:
        assert lib.fb200_attention_fan_supported(sq, sk, d, dt) == 0
        rc = lib.fb200_attention_fan(buf.ptr, 128, 64, buf.ptr, 128, 64, buf.ptr, 128, 64, buf.ptr, 64,
                                     buf.ptr, 1, sq, sk, d, 1.0, dt, None)
        assert rc == 4 and b"attention_fan" in lib.fb200_last_error()
    assert lib.fb200_attention_fan_supported(512, 512, 64, capi.BF16) == 1
