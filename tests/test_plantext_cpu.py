"""Host-side bookkeeping that needs no GPU: the plan-text reader used by the benchmark, the work
figures it derives, and the seeded input generators shared by the golden script and the GPU tests."""
import os

import numpy as np

from frame_public_b200 import configs, plantext, runtime

HERE = os.path.dirname(os.path.abspath(__file__))


def test_bench_plans_parse_and_report_their_work():
    plan = plantext.parse(runtime.load_plan_text("transformer_bf16_b8_s512_d1024"))
    ops = [s.op for s in plan.steps]
    assert ops.count("softmax") == 128 and ops.count("matmul") == 260 and ops.count("concat") == 9
    flops, nbytes = plantext.attention_fan_work(plan)
    assert flops == 128 * 4.0 * 512 * 512 * 64          # QK^T and PV of 128 heads
    assert nbytes == 128 * 4 * 512 * 64 * 2              # q, k, v read and the result written, bf16
    first = next(i for i, s in enumerate(plan.steps) if s.op == "matmul")
    assert plantext.step_work(plan, first)[0] == 2.0 * 4096 * 3072 * 1024


def test_every_golden_plan_parses():
    plan_dir = os.path.join(HERE, "golden", "plans")
    names = sorted(os.listdir(plan_dir))
    assert any(n.startswith("nn_transformer") for n in names)
    for n in names:
        with open(os.path.join(plan_dir, n)) as f:
            plan = plantext.parse(f.read())
        assert plan.steps and plan.outputs, n


def test_nn_inputs_are_reproducible_and_in_storage_form():
    shapes = [(4, 8), (8, 8), (8,)]
    a = configs.nn_inputs(shapes, configs.BF16)
    b = configs.nn_inputs(shapes, configs.BF16)
    assert all(x.dtype == np.uint16 and x.shape == s for x, s in zip(a, shapes))
    assert all(np.array_equal(x, y) for x, y in zip(a, b))
    f = configs.nn_inputs(shapes, configs.F32)
    assert f[0].dtype == np.float32 and abs(float(f[1].std()) - 0.1) < 0.05
    # every graph listed has its plan and its golden output committed
    gold = np.load(os.path.join(HERE, "golden", "ref_cpu_workloads.npz"))
    for name, _, _, _ in configs.NN_GRAPHS:
        assert name in gold.files and os.path.exists(os.path.join(HERE, "golden", "plans", name + ".plan"))
