"""bench.py's partition of ONE workload over N ranks, checked without a GPU: a plan exists for every
shard size, every rank's inputs have the shapes that plan declares, and the ranks' shards put
together are the full-size inputs (every sample owned exactly once; weights whole on every rank)."""
import importlib.util
import os

import numpy as np
import pytest

from frame_public_b200 import plantext, runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def _plan_inputs(name):
    plan = plantext.parse(runtime.load_plan_text(name))
    return [(plan.slots[i].dtype, plan.slots[i].dims) for i in plan.inputs]


@pytest.mark.parametrize("name", ["mlp", "conv_stack", "transformer", "mamba"])
def test_graph_workloads_partition_over_1_2_4_8_ranks(name):
    wl = bench.Workload(name)
    full = wl.full().inputs
    for world in (1, 2, 4, 8):
        specs = _plan_inputs(wl.plan_name(world))
        shards = [wl.shard_inputs(specs, r, world)[0] for r in range(world)]
        for shard in shards:
            assert [tuple(a.shape) for a in shard] == [tuple(s) for _, s in specs]
        for i, arr in enumerate(full):
            if tuple(arr.shape) == tuple(specs[i][1]) and world > 1:
                assert all(np.array_equal(s[i], arr) for s in shards)          # a weight: whole everywhere
            else:
                assert np.array_equal(np.concatenate([s[i] for s in shards], axis=0), arr)


def test_gemm_shard_plans_exist_with_the_row_split_shapes():
    wl = bench.Workload("gemm_bias_gelu_bf16_8192")
    for world, rows in ((1, 8192), (2, 4096), (4, 2048), (8, 1024)):
        specs = _plan_inputs(wl.plan_name(world))
        assert [s for _, s in specs] == [(rows, 8192), (8192, 8192), (rows, 8192)]
    assert wl.units_total == pytest.approx(2 * 8192 ** 3 / 1e12)
