"""Pins the CPU oracle (oracle/frame_oracle.py): against the known-answer vectors of the
reference's own unit tests, against committed outputs of the unmodified reference CPU backend
(tests/golden/ref_cpu_cases.npz), and, where oracle/_ref is present, against the reference CPU
backend run live."""
import hashlib
import os

import numpy as np
import pytest

import cases
import known_answers
from oracle import frame_oracle as fo
from oracle import ref_runtime

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_cpu_cases.npz")


@pytest.mark.parametrize("entry", known_answers.load(), ids=lambda e: e[0].split("/")[-1] + ":" + e[1])
def test_oracle_matches_reference_known_answers(entry):
    cite, op, dt, ins, attrs, exp, bits = entry
    got = known_answers.oracle_eval(op, dt, ins, attrs)
    assert got.shape == exp.shape
    assert fo.all_close(got, exp, dt), (cite, got, exp)
    if bits is not None:
        assert list(np.asarray(got).reshape(-1)) == bits


def test_bf16_conversion_bit_patterns():
    # include/frame/core/dtype.h:117-131 of the reference: RTNE, NaN keeps payload + quiet bit
    vals = np.array([1.0, 2.0, 3.0, 19.0, 22.0, 43.0, 50.0], dtype=np.float32)
    assert list(fo.f32_to_bf16_bits(vals)) == [0x3F80, 0x4000, 0x4040, 0x4198, 0x41B0, 0x422C, 0x4248]
    tie = np.array([0x3F808000, 0x3F818000], dtype=np.uint32).view(np.float32)  # ties: to even
    assert list(fo.f32_to_bf16_bits(tie)) == [0x3F80, 0x3F82]
    nan = np.array([0x7F800001, 0xFFC12345], dtype=np.uint32).view(np.float32)
    assert list(fo.f32_to_bf16_bits(nan)) == [0x7FC0, 0xFFC1]
    assert np.array_equal(fo.bf16_bits_to_f32(fo.f32_to_bf16_bits(vals)), vals)


def _digest(case):
    h = hashlib.sha256()
    for a in case.inputs:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()[:16]


REF_CASES = [c for c in cases.CASES if not c.new_op and c.expected().size > 0]


@pytest.mark.parametrize("case", REF_CASES, ids=lambda c: c.name)
def test_oracle_matches_committed_reference_outputs(case):
    gold = np.load(GOLDEN)
    assert case.name in gold.files, "regenerate tests/golden/ref_cpu_cases.npz"
    assert bytes(gold["digest__" + case.name]).decode() == _digest(case), "seeded inputs drifted"
    ref = gold[case.name]
    got = case.expected()
    assert got.shape == ref.shape
    if case.exact:
        assert np.array_equal(np.asarray(got).reshape(-1).view(np.uint8), np.asarray(ref).reshape(-1).view(np.uint8)), case.name
    else:
        assert fo.all_close(got, ref, case.dtype), fo.max_err(got, ref, case.dtype)


@pytest.mark.skipif(not ref_runtime.available(), reason="oracle/_ref not built")
@pytest.mark.parametrize("case", REF_CASES[::4], ids=lambda c: c.name)
def test_oracle_matches_live_reference(case):
    comp = ref_runtime.Compiled(case.ir_text("cpu"), "cpu")
    (ref,) = comp.run(case.inputs)
    comp.close()
    got = case.expected()
    if case.exact:
        assert np.array_equal(np.asarray(got).reshape(-1).view(np.uint8), np.asarray(ref).reshape(-1).view(np.uint8))
    else:
        assert fo.all_close(got, ref, case.dtype)


def test_new_ops_agree_with_compositions_of_reference_ops():
    # silu = mul(x, sigmoid(x)); gelu(tanh form) = composition of mul/add/square/tanh
    x = cases.CASES_BY_NAME["silu_f32_1023"].inputs[0]
    assert np.array_equal(fo.silu(x), fo.mul(x, fo.sigmoid(x)))
    g = fo.gelu(x)
    x3 = fo.mul(fo.square(x), x)
    inner = fo.mul(np.full_like(x, 0.7978845608028654), fo.add(x, fo.mul(np.full_like(x, 0.044715), x3)))
    comp = fo.mul(fo.mul(np.full_like(x, 0.5), x), fo.add(np.ones_like(x), fo.tanh(inner)))
    assert fo.all_close(g, comp, fo.DT_F32)


def test_mamba_scan_equals_selective_scan_on_materialised_operands():
    rng = np.random.default_rng(3)
    bt, L, dm, n = 2, 9, 5, 4
    u = rng.standard_normal((bt, L, dm)).astype(np.float32)
    delta = rng.uniform(1e-3, 1e-1, (bt, L, dm)).astype(np.float32)
    A = -np.tile(np.arange(1, n + 1, dtype=np.float32), (dm, 1))
    B = rng.standard_normal((bt, L, n)).astype(np.float32)
    C = rng.standard_normal((bt, L, n)).astype(np.float32)
    D = np.ones(dm, dtype=np.float32)
    y = fo.mamba_scan(u, delta, A, B, C, D)
    # reference-op form: [bt, dm, n, L] operands
    x4 = np.broadcast_to(u.transpose(0, 2, 1)[:, :, None, :], (bt, dm, n, L))
    a4 = np.exp(delta.transpose(0, 2, 1)[:, :, None, :] * A[None, :, :, None]).astype(np.float32)
    b4 = (delta.transpose(0, 2, 1)[:, :, None, :] * B.transpose(0, 2, 1)[:, None, :, :]).astype(np.float32)
    c4 = np.broadcast_to(C.transpose(0, 2, 1)[:, None, :, :], (bt, dm, n, L))
    d4 = np.zeros((bt, dm, n, L), dtype=np.float32)
    s = fo.selective_scan(np.ascontiguousarray(x4), a4, b4, np.ascontiguousarray(c4), d4)
    ysum = fo.sum_axes(s, [2]).transpose(0, 2, 1) + D[None, None, :] * u
    assert fo.all_close(y, ysum, fo.DT_F32, rtol=1e-5, atol=1e-6)
