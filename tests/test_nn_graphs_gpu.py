"""The reference's OWN nn:: modules on this backend: nn::TransformerEncoderBlock, nn::Mamba and an
nn::Sequential CNN (include/frame/nn/layers.h:32-234), their graphs emitted by the reference's builder, run through
the reference's nine-pass pipeline and memory planner for backend "cuda" (committed as
tests/golden/plans/nn_*.plan), executed here by the plan executor, and compared with the output
of the reference CPU backend on the same seeded inputs (tests/golden/ref_cpu_workloads.npz; both
made by tests/golden/make_workload_golden.py).  Every op of these graphs has a kernel here: no step
falls back, and the attention of the bf16 block runs as one attention_fan launch (its scores are
scaled by the `mul` with a constant that the reference's builder emits)."""
import os

import numpy as np
import pytest

from frame_public_b200 import capi, configs, runtime
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden", "ref_cpu_workloads.npz")


def _plan(name):
    with open(os.path.join(HERE, "golden", "plans", name + ".plan")) as f:
        return f.read()


@pytest.mark.parametrize("spec", configs.NN_GRAPHS, ids=lambda s: s[0])
@pytest.mark.parametrize("opt", [1, 0], ids=["fused", "unfused"])
def test_reference_nn_module_matches_reference_cpu(spec, opt):
    name, kind, _, dtype = spec
    gold = np.load(GOLD)[name]
    plan = runtime.CompiledPlan(_plan(name), 0, allow_tf32=False, opt_level=opt)
    ins = configs.nn_inputs([shape for _, shape in plan.inputs], dtype)
    (got,) = plan.run_host(ins)
    (again,) = plan.run_host(ins)
    assert capi.kernel_status(0) == 0
    assert np.array_equal(got.view(np.uint8), again.view(np.uint8))
    if dtype == configs.BF16:
        tol = dict(rtol=2e-2, atol=2e-3)     # the reference's bf16 tier
    else:
        tol = dict(rtol=1e-5, atol=2e-6)     # strict fp32: same operations as the CPU backend
    assert fo.all_close(got, gold, dtype, **tol), (name, fo.max_err(got, gold, dtype))
    plan.close()


def test_reference_attention_becomes_one_launch():
    name = "nn_transformer_bf16_b2_s128_e128_h2"
    fused = runtime.CompiledPlan(_plan(name), 0, opt_level=1)
    plain = runtime.CompiledPlan(_plan(name), 0, opt_level=0)
    names = fused.step_names()
    assert names.count("attention_fan") == 1
    assert not any(n in ("softmax", "transpose", "concat") for n in names)
    assert fused.launches_per_run < plain.launches_per_run / 3


def test_reference_cnn_on_the_tensor_core_conv():
    """The wider nn::Sequential CNN with allow_tf32: conv2d + bias + relu run on the tcgen05 implicit
    GEMM, the Linear on the tcgen05 GEMM; TF32 tier against the reference CPU backend."""
    name, _, _, dtype = next(s for s in configs.NN_GRAPHS if s[0] == "nn_cnn_f32_b4_c16_hw32_o32")
    gold = np.load(GOLD)[name]
    plan = runtime.CompiledPlan(_plan(name), 0, allow_tf32=True)
    ins = configs.nn_inputs([shape for _, shape in plan.inputs], dtype)
    (got,) = plan.run_host(ins)
    assert capi.kernel_status(0) == 0
    tol = configs.parity_tolerance("cnn", dtype, True, gold)
    assert fo.all_close(got, gold, dtype, **tol), fo.max_err(got, gold, dtype)
    plan.close()
