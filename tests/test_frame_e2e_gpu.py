"""End to end through the reference's own API on the GPU: the reference framework (oracle/_ref,
built from its sources) with this repository's plugin loaded as backend "cuda"; graphs go through
runtime::compile (cache, nine-pass pipeline, Backend::compile) and Executable::run with tensors
allocated by the plugin's hal::Allocator and moved with hal::Backend::copy.  Results are compared
with the reference CPU backend run in the same process; FallbackStats must stay at zero."""
import numpy as np
import pytest

from frame_public_b200 import configs
from oracle import frame_oracle as fo
from oracle import ref_runtime

pytestmark = pytest.mark.gpu

if not ref_runtime.available():
    pytest.skip("oracle/_ref (the reference build) is not present", allow_module_level=True)

WORKLOADS = configs.small_workloads("cpu")
OPS = ["matmul", "conv2d", "conv1d", "max_pool2d", "softmax", "layer_norm", "selective_scan", "add",
       "mul", "relu", "fused_elementwise_internal", "slice", "concat", "transpose", "reshape", "gelu",
       "silu", "softplus", "bias_add", "mamba_scan"]


@pytest.fixture(scope="module", autouse=True)
def _plugin():
    ref_runtime.load_b200_backend()
    assert ref_runtime.has_backend("cuda")
    yield


@pytest.mark.parametrize("wl", WORKLOADS, ids=lambda w: w.name)
def test_graph_compiled_on_cuda_matches_cpu_backend(wl):
    cpu = ref_runtime.Compiled(wl.ir_text, "cpu")
    (exp,) = cpu.run(wl.inputs)
    gpu = ref_runtime.Compiled(wl.with_backend("cuda"), "cuda")
    (got,) = gpu.run(wl.inputs)
    tol = dict(rtol=2e-2, atol=2e-3) if wl.dtype == configs.BF16 else dict(rtol=1e-5, atol=1e-6)
    assert fo.all_close(got, exp, wl.dtype, **tol), (wl.name, fo.max_err(got, exp, wl.dtype))
    for op in OPS:
        assert ref_runtime.fallback_count(op, "cuda") == 0, f"op {op} fell back to the eager chain"


def test_every_path_op_has_a_cuda_kernel():
    for op in OPS + ["square", "sigmoid", "tanh", "rsqrt", "sum", "constant", "exp"]:
        assert ref_runtime.has_kernel(op, "cuda"), op


def test_selective_scan_through_reference_api_matches_known_answer():
    from frame_public_b200 import irtext
    g = irtext.IrGraph("cuda")
    vals = [g.input("float32", (3,)) for _ in range(5)]
    g.output(g.selective_scan(*vals))
    comp = ref_runtime.Compiled(g.text(), "cuda")
    ins = [np.array(v, np.float32) for v in ([1, 2, -1], [0.5, 0.25, -0.5], [2, 1, 3], [1, 2, 0.5], [0.1, -1, 2])]
    (out,) = comp.run(ins)
    assert fo.all_close(out, np.array([2.1, 3.0, -4.125], np.float32))


@pytest.mark.parametrize("spec", configs.NN_GRAPHS, ids=lambda s: s[0])
def test_reference_nn_module_runs_on_cuda_without_fallback(spec):
    """The reference's own nn:: builders (nn::TransformerEncoderBlock, nn::Mamba) emit the graph; the
    reference's runtime::compile sends it to backend "cuda" (this plugin) and to its CPU backend; both
    run the same seeded parameters.  Nothing may fall back to the eager chain."""
    name, kind, args, dtype = spec
    text_cpu = ref_runtime.nn_graph_text(kind, *args, dtype_code=dtype, backend="cpu")
    text_gpu = ref_runtime.nn_graph_text(kind, *args, dtype_code=dtype, backend="cuda")
    cpu = ref_runtime.Compiled(text_cpu, "cpu")
    ins = configs.nn_inputs([shape for _, shape in cpu.inputs], dtype)
    (exp,) = cpu.run(ins)
    gpu = ref_runtime.Compiled(text_gpu, "cuda")
    (got,) = gpu.run(ins)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype == configs.BF16 else dict(rtol=1e-5, atol=2e-6)
    assert fo.all_close(got, exp, dtype, **tol), (name, fo.max_err(got, exp, dtype))
    for op in OPS + ["sigmoid", "tanh", "constant"]:
        assert ref_runtime.fallback_count(op, "cuda") == 0, f"op {op} fell back to the eager chain"


NEW_OP_CASES = [c for c in __import__("cases").CASES
                if c.op in ("avg_pool2d", "heaviside_surrogate", "gather", "scatter_add", "gather_grad_internal",
                            "max_pool2d_select_internal", "max_pool2d_grad_internal", "avg_pool2d_grad_internal",
                            "conv2d_grad_input_internal", "conv2d_grad_filter_internal", "matmul_grad_lhs_internal",
                            "matmul_grad_rhs_internal", "relu_grad_internal", "mse_loss", "mse_loss_grad_internal")
                or c.name == "sum_f32_all_axes"]


@pytest.mark.parametrize("case", NEW_OP_CASES, ids=lambda c: c.name)
def test_pool_step_and_index_ops_through_the_reference_api(case):
    """avg_pool2d, heaviside_surrogate, gather, scatter_add, gather_grad_internal and the pooling /
    convolution gradient internals compiled by the
    reference's runtime::compile for backend "cuda": no fallback, same numbers as its CPU backend."""
    cpu = ref_runtime.Compiled(case.ir_text("cpu"), "cpu")
    (exp,) = cpu.run(case.inputs)
    gpu = ref_runtime.Compiled(case.ir_text("cuda"), "cuda")
    (got,) = gpu.run(case.inputs)
    if case.exact:
        assert np.array_equal(np.asarray(got).reshape(-1).view(np.uint8), np.asarray(exp).reshape(-1).view(np.uint8)), case.name
    else:
        assert fo.all_close(got, exp, case.dtype), (case.name, fo.max_err(got, exp, case.dtype))
    assert ref_runtime.fallback_count(case.op, "cuda") == 0


FFT_CASES = [c for c in __import__("cases").CASES if c.op in ("rfft", "irfft")]


@pytest.mark.parametrize("case", FFT_CASES, ids=lambda c: c.name)
def test_rfft_irfft_through_the_reference_api(case):
    """rfft / irfft compiled by the reference's runtime::compile for backend "cuda" (its shape
    inference and attribute checks, this repository's kernels): no fallback; compared with the oracle,
    because the reference's CPU kernel needs pocketfft, which its tree does not contain."""
    gpu = ref_runtime.Compiled(case.ir_text("cuda"), "cuda")
    (got,) = gpu.run(case.inputs)
    exp = case.expected()
    assert fo.all_close(got, exp, case.dtype, rtol=1e-5, atol=1e-5), (case.name, fo.max_err(got, exp, case.dtype))
    assert ref_runtime.fallback_count(case.op, "cuda") == 0


def test_training_graph_through_the_reference_api_without_fallback():
    """compiler::build_backward_graph of a two-layer MLP with an MSE loss, compiled by the reference's
    runtime::compile for backend "cuda": [loss, grad w1, grad b1, grad w2] bit-identical to its CPU
    backend (strict fp32) and no op of the training graph takes the fallback chain."""
    fwd_cpu, ins = configs.train_mlp_forward(backend="cpu")
    fwd_cuda, _ = configs.train_mlp_forward(backend="cuda")
    cpu = ref_runtime.Compiled(ref_runtime.backward_text(fwd_cpu, 0, configs.TRAIN_WRT), "cpu")
    exp = cpu.run(ins)
    gpu = ref_runtime.Compiled(ref_runtime.backward_text(fwd_cuda, 0, configs.TRAIN_WRT), "cuda")
    got = gpu.run(ins)
    assert len(got) == len(exp) == 4
    for g, e in zip(got, exp):
        assert np.array_equal(np.asarray(g).reshape(-1).view(np.uint8), np.asarray(e).reshape(-1).view(np.uint8))
    for op in ("matmul", "add", "relu", "mse_loss", "mse_loss_grad_internal", "matmul_grad_lhs_internal",
               "matmul_grad_rhs_internal", "relu_grad_internal", "constant"):
        assert ref_runtime.fallback_count(op, "cuda") == 0, f"op {op} fell back to the eager chain"


def test_twelve_elementwise_ops_fuse_into_one_group_and_run():
    """Twelve consecutive fusable ops: the reference's fusion pass makes ONE fused_elementwise_internal
    node of them (it has no length limit), longer than a single launch of the plugin's chain kernel
    holds; the plugin runs it as successive launches.  fp32 elementwise without libm: bit-identical to
    the CPU backend, which runs the same group one sub-kernel at a time."""
    from frame_public_b200 import irtext

    def build(backend):
        g = irtext.IrGraph(backend)
        xs = [g.input("float32", (9, 1023)) for _ in range(8)]
        v = g.unary("relu", g.add(xs[0], xs[1]))
        v = g.unary("square", g.mul(v, xs[2]))
        v = g.unary("relu", g.add(v, xs[3]))
        v = g.unary("relu", g.add(g.mul(v, xs[4]), xs[5]))
        v = g.unary("relu", g.mul(g.add(v, xs[6]), xs[7]))
        g.output(v)
        return g.text()

    assert ref_runtime.pipeline_text(build("cpu"), "cpu").count("fused_elementwise_internal") == 1
    rng = np.random.default_rng(77)
    ins = [(rng.standard_normal((9, 1023)) * 0.8).astype(np.float32) for _ in range(8)]
    (exp,) = ref_runtime.Compiled(build("cpu"), "cpu").run(ins)
    (got,) = ref_runtime.Compiled(build("cuda"), "cuda").run(ins)
    assert np.array_equal(got.view(np.uint8), exp.view(np.uint8))
    assert ref_runtime.fallback_count("fused_elementwise_internal", "cuda") == 0


@pytest.mark.parametrize("kind,args,dtype", [("transformer", (1, 512, 1024, 16, 4096, True), configs.BF16),
                                             ("mamba", (2, 512, 256, 4, 0, True), configs.F32),
                                             ("cnn", (8, 16, 56, 64, 10, True), configs.F32)],
                         ids=["transformer_s512_e1024_h16", "mamba_c256_s512", "cnn_16x56x56_to_64"])
def test_reference_nn_modules_at_a_non_miniature_size(kind, args, dtype):
    """nn::TransformerEncoderBlock at sequence 512 / embed 1024 / 16 heads / FFN 4096 (bf16), nn::Mamba
    with 256 channels over 512 steps and an nn::Sequential CNN on 56 x 56 images, built by the
    reference's own builder, compiled by its runtime::compile for its CPU backend and for this plugin,
    same seeded parameters: the two must agree within the dtype's tier (the bf16 block: the chain
    tolerance of the full-size parity test), with nothing falling back to the eager chain."""
    text_cpu = ref_runtime.nn_graph_text(kind, *args, dtype_code=dtype, backend="cpu")
    text_gpu = ref_runtime.nn_graph_text(kind, *args, dtype_code=dtype, backend="cuda")
    cpu = ref_runtime.Compiled(text_cpu, "cpu")
    ins = configs.nn_inputs([shape for _, shape in cpu.inputs], dtype)
    (exp,) = cpu.run(ins)
    cpu.close()
    gpu = ref_runtime.Compiled(text_gpu, "cuda")
    (got,) = gpu.run(ins)
    gpu.close()
    tol = configs.parity_tolerance("transformer" if dtype == configs.BF16 else kind, dtype, False, fo.to_accum(exp, dtype))
    assert fo.all_close(got, exp, dtype, **tol), (kind, fo.max_err(got, exp, dtype), tol)
    for op in OPS:
        assert ref_runtime.fallback_count(op, "cuda") == 0, f"op {op} fell back to the eager chain"
