"""Parity at the benchmark sizes.  The full-size plans of frame_public_b200/plans (fused, replayed
from a CUDA graph: the path bench.py times) run on seeded full-size inputs; the rows of the result
that belong to the first sample (the first 16 rows of the 8192^3 GEMM) must match what the reference
CPU backend computed for that slab (tests/golden/ref_cpu_fullsize.npz, made by
tests/golden/make_fullsize_golden.py).  Rows and samples are independent on this path, so the slab
is exactly what the CPU backend would produce for those rows of the full batch.

Tolerances are the reference's tiers (tests/cpp/common/tolerance.h:41-98 of the reference): bf16
rtol 2e-2 / atol 2e-3; strict fp32 1e-5 / 1e-6; fp32 on the tensor cores (allow_tf32) rtol 1e-3 plus
an absolute term for outputs that cancel to near zero: 2e-3 * sqrt(K) * rms(a) * rms(b) for a single
GEMM (= 2e-3 of the output's rms), and 5e-3 of the golden's rms for graphs that chain three or four
TF32 contractions (operand errors of 2^-11 relative add up over the chain; the worst element of
10^5..10^6 sits 4-5 standard deviations out).  The bf16 transformer block is a chain of bf16 nodes
ending in residual adds: its absolute term is one bf16 ulp of the largest residual value (a flipped
rounding of an addend), and at most 2 % of its elements may fall outside the single-op bf16 tier.  Setting FRAME_B200_ERROR_TABLE=<file> appends the
measured errors of every case as JSON lines."""
import json
import os

import numpy as np
import pytest

from frame_public_b200 import capi, configs, runtime
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden", "ref_cpu_fullsize.npz")

# key -> (plan name, allow_tf32 variants)
CASES = {
    "mlp": ("mlp_f32_b64", (False, True)),
    "gemm_bf16": ("gemm_bias_gelu_bf16_8192", (False,)),
    "gemm_f32": ("gemm_bias_gelu_f32_8192", (True, False)),
    "conv_stack": ("conv_stack_f32_b32_224", (True, False)),
    "transformer": ("transformer_bf16_b8_s512_d1024", (False,)),
    "mamba": ("mamba_f32_b16_s2048_d768", (True,)),
}


def _record(row):
    path = os.environ.get("FRAME_B200_ERROR_TABLE")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(row) + "\n")


def _tolerance(key, wl, tf32, gold):
    return configs.parity_tolerance(key, wl.dtype, tf32, fo.to_accum(gold, wl.dtype), wl.inputs)


@pytest.mark.parametrize("key", list(CASES))
def test_full_size_plan_matches_the_reference_cpu_slab(key):
    plan_name, variants = CASES[key]
    gold_file = np.load(GOLD)
    gold = gold_file[key]
    builder, kw = configs.FULL_BUILDERS[key]
    wl = builder(**kw)
    for tf32 in variants:
        plan = runtime.CompiledPlan(runtime.load_plan_text(plan_name), 0, allow_tf32=tf32)
        (first,) = plan.run_host(wl.inputs)
        (got,) = plan.run_host(wl.inputs)      # second run: the captured CUDA graph is replayed
        assert capi.kernel_status(0) == 0
        assert np.array_equal(first.view(np.uint8), got.view(np.uint8))
        rows = configs.slab_of_output(key, got)
        if key == "mamba":
            rows = rows[gold_file["mamba_rows"]]
        tol = _tolerance(key, wl, tf32, gold)
        max_abs, max_rel = fo.max_err(rows, gold, wl.dtype)
        g64 = fo.to_accum(gold, wl.dtype).astype(np.float64)
        err = np.abs(fo.to_accum(rows, wl.dtype).astype(np.float64) - g64)
        base = dict(rtol=2e-2, atol=2e-3) if wl.dtype == configs.BF16 else tol
        outside_base = float(np.mean(err > base["atol"] + base["rtol"] * np.abs(g64)))
        rms = float(np.sqrt(np.mean(np.square(fo.to_accum(gold, wl.dtype).astype(np.float64)))))
        _record({"case": key, "plan": plan_name, "allow_tf32": bool(tf32), "rows": int(rows.shape[0]),
                 "max_abs": max_abs, "max_rel": max_rel, "gold_rms": rms, "rtol": tol["rtol"], "atol": float(tol["atol"]),
                 "fraction_outside_single_op_tier": outside_base})
        assert fo.all_close(rows, gold, wl.dtype, **tol), (key, tf32, max_abs, max_rel, rms, tol)
        # the chain tolerance of the bf16 transformer block covers single flipped roundings only: all
        # but a small share of the elements must still meet the single-op bf16 tier
        assert outside_base <= 0.02, (key, outside_base)
        plan.close()
