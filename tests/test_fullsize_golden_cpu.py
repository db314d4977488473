"""The full-size slab goldens (tests/golden/ref_cpu_fullsize.npz) against what can be recomputed on
the CPU in seconds: the MLP through the numpy restatement of the reference kernels, and the MLP and
conv-stack slabs through the reference CPU backend itself where it is built."""
import os

import numpy as np
import pytest

from frame_public_b200 import configs
from oracle import frame_oracle as fo
from oracle import ref_runtime

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = np.load(os.path.join(HERE, "golden", "ref_cpu_fullsize.npz"))


def test_golden_has_every_full_size_workload_with_the_slab_shape():
    expected = {"mlp": (64, 10), "gemm_bf16": (16, 8192), "gemm_f32": (16, 8192), "conv_stack": (1, 64, 56, 56),
                "transformer": (512, 1024), "mamba": (len(GOLD["mamba_rows"]), 768)}
    for key, shape in expected.items():
        assert GOLD[key].shape == shape, key
        assert key in configs.FULL_BUILDERS
    assert GOLD["gemm_bf16"].dtype == np.uint16 and GOLD["transformer"].dtype == np.uint16
    rows = GOLD["mamba_rows"]
    assert rows[0] == 0 and rows[-1] == 2047 and np.all(np.diff(rows) > 0)


def test_mlp_golden_matches_the_numpy_restatement():
    x, w1, b1, w2, b2, w3, b3 = configs.mlp().inputs
    h = fo.relu(fo.add(fo.matmul(x, w1), b1))
    h = fo.relu(fo.add(fo.matmul(h, w2), b2))
    exp = fo.softmax(fo.add(fo.matmul(h, w3), b3))
    assert fo.all_close(GOLD["mlp"], exp, fo.DT_F32)


@pytest.mark.skipif(not ref_runtime.available(), reason="the reference build (oracle/_ref) is not present")
@pytest.mark.parametrize("key", ["mlp", "conv_stack"])
def test_cheap_slabs_recomputed_by_the_reference_cpu_backend(key):
    builder, kw = configs.FULL_BUILDERS[key]
    full = builder(**kw)
    comp = ref_runtime.Compiled(configs.slab_graph(key), "cpu")
    (res,) = comp.run(configs.slab_inputs(key, full.inputs))
    comp.close()
    assert np.array_equal(res.view(np.uint8), GOLD[key].view(np.uint8))
