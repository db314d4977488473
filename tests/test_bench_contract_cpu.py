"""bench.py on a machine without a GPU: the product arm refuses to run (there is no CPU fallback),
the reference arm times the reference CPU backend and prints the contract's JSON line."""
import json
import os
import subprocess
import sys

import pytest

from oracle import ref_runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True,
                          text=True, timeout=600, cwd=ROOT)


def test_product_arm_fails_loudly_without_a_gpu():
    from frame_public_b200 import capi
    if capi.device_count() > 0:
        pytest.skip("a GPU is present")
    res = _run("--steps", "1", "--warmup", "0")
    assert res.returncode != 0
    assert "no CPU fallback" in (res.stdout + res.stderr)


@pytest.mark.skipif(not ref_runtime.available(), reason="oracle/_ref is not built")
def test_reference_arm_prints_the_contract_line():
    res = _run("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert res.returncode == 0, res.stderr[-500:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "impl", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["steps"] == 1 and line["warmup"] == 0
    assert line["cpu_baseline"]["kind"] == "reference" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["value"] > 0 and line["config"]["workload"] == "gemm_bias_gelu_bf16_8192"
