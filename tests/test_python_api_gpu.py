"""The reference's Python surface on this backend: the reference's own pybind11 module (`_core`,
compiled from its python/src by oracle/build_ref.sh) with this repository's plugin registered as
backend "cuda".  A user's flow — from_numpy, Tensor.to("cuda"), compile(graph, "cuda"),
Executable.run, Tensor.numpy — runs unchanged (python/src/bind_runtime.cpp:34-54,
bind_core.cpp), and gives what the reference CPU backend gives."""
import glob
import os
import sys

import numpy as np
import pytest

from oracle import frame_oracle as fo
from oracle import ref_runtime

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")
if not ref_runtime.available() or not glob.glob(os.path.join(REF_DIR, "_core*.so")):
    pytest.skip("the reference's Python module (oracle/_ref/_core*.so) is not built", allow_module_level=True)


@pytest.fixture(scope="module")
def core():
    ref_runtime.load()
    ref_runtime.load_b200_backend()
    sys.path.insert(0, REF_DIR)
    import _core
    return _core


def _run_module(core, module, x, params, backend):
    g = core.Graph(f"py_{backend}")
    vx = g.add_graph_input(list(x.shape), core.DType.float32, backend=backend)
    vps = [g.add_graph_input(list(p.shape), core.DType.float32, backend=backend) for p in params]
    (out,) = module.build(g, [vx], vps)
    g.mark_output(out)
    exe = core.compile(g, backend)
    tensors = [core.from_numpy(a) for a in [x] + params]
    if backend != "cpu":
        tensors = [t.to(backend) for t in tensors]
        assert all(t.device.backend == backend for t in tensors)
    (res,) = exe.run(tensors)
    assert res.device.backend == backend
    return res.numpy()


def test_tensor_to_cuda_compile_run_numpy(core):
    def graph(backend):
        g = core.Graph(f"add_relu_{backend}")
        a = g.add_graph_input([4, 6], core.DType.float32, backend=backend)
        b = g.add_graph_input([4, 6], core.DType.float32, backend=backend)
        g.mark_output(core.relu(g, core.add(g, a, b)))
        return g
    rng = np.random.default_rng(0)
    a, b = (rng.standard_normal((4, 6)).astype(np.float32) for _ in range(2))
    exp = core.compile(graph("cpu"), "cpu").run([core.from_numpy(a), core.from_numpy(b)])[0].numpy()
    exe = core.compile(graph("cuda"), "cuda")
    (out,) = exe.run([core.from_numpy(a).to("cuda"), core.from_numpy(b).to("cuda")])
    assert out.device.backend == "cuda"
    got = out.numpy()
    assert np.array_equal(got, exp) and np.array_equal(got, np.maximum(a + b, 0))


@pytest.mark.parametrize("kind", ["transformer", "mamba"])
def test_reference_nn_modules_through_the_python_api(core, kind):
    rng = np.random.default_rng(3)
    if kind == "transformer":
        module = core.TransformerEncoderBlock("block", 2, 16, 32, 2, 64, True, core.DType.float32)
        x = rng.standard_normal((32, 32)).astype(np.float32)
    else:
        module = core.Mamba("mamba", 2, 16, 24, 4, core.DType.float32)
        x = rng.standard_normal((2, 16, 24)).astype(np.float32)
    params = [(0.1 * rng.standard_normal(tuple(shape))).astype(np.float32) for _, shape, _ in module.parameters()]
    exp = _run_module(core, module, x, params, "cpu")
    got = _run_module(core, module, x, params, "cuda")
    assert fo.all_close(got, exp, fo.DT_F32, rtol=1e-5, atol=2e-6), fo.max_err(got, exp)
