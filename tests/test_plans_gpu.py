"""Compiled-graph parity on the GPU: the miniature workloads (MLP, GEMM+epilogue, conv stack,
transformer block, Mamba block) run through the plan executor of the C ABI, fed with the plans the
reference pipeline emitted (tests/golden/plans), against outputs of the unmodified reference CPU
backend for the same seeded inputs (tests/golden/ref_cpu_workloads.npz)."""
import os

import numpy as np
import pytest

from frame_public_b200 import capi, configs, runtime
from oracle import frame_oracle as fo

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden", "ref_cpu_workloads.npz")
WORKLOADS = configs.small_workloads("cpu")


def _plan_text(name):
    with open(os.path.join(HERE, "golden", "plans", name + ".plan")) as f:
        return f.read()


def _tolerance(wl, tf32, gold):
    if wl.dtype == configs.BF16:
        return dict(rtol=2e-2, atol=2e-3)   # the reference's bf16 tier
    if tf32:
        # TF32 tier (fp32 GEMM/conv on the tensor cores): operands keep 10 explicit mantissa bits,
        # so a K-term dot product errs by about 2^-10*sqrt(K)*rms(a)*rms(b), i.e. a few 1e-3 of the
        # output's rms whatever K is (6e-3 of the rms at most was measured); rtol is the
        # reference's TF32 tier, the absolute term covers outputs that cancel to near zero.
        rms = float(np.sqrt(np.mean(np.square(gold.astype(np.float64)))))
        return dict(rtol=1e-3, atol=max(2e-3, 5e-3 * rms))
    return dict(rtol=1e-5, atol=1e-6)       # strict fp32 tier


@pytest.mark.parametrize("wl", WORKLOADS, ids=lambda w: w.name)
@pytest.mark.parametrize("tf32", [False, True], ids=["strict", "allow_tf32"])
@pytest.mark.parametrize("opt", [1, 0], ids=["fused", "unfused"])
def test_workload_matches_reference_cpu(wl, tf32, opt):
    gold = np.load(GOLD)[wl.name]
    plan = runtime.CompiledPlan(_plan_text(wl.name), 0, allow_tf32=tf32, opt_level=opt)
    (got,) = plan.run_host(wl.inputs)
    (again,) = plan.run_host(wl.inputs)   # the arena is reused: a second run must agree bit for bit
    assert capi.kernel_status(0) == 0
    assert np.array_equal(got.view(np.uint8), again.view(np.uint8))
    tol = _tolerance(wl, tf32, gold)
    assert fo.all_close(got, gold, wl.dtype, **tol), (wl.name, fo.max_err(got, gold, wl.dtype))
    plan.close()


def test_epilogue_absorption_reduces_launches():
    wl = WORKLOADS[0]  # MLP: matmul, add;relu, matmul, add;relu, matmul, add, softmax
    fused = runtime.CompiledPlan(_plan_text(wl.name), 0, opt_level=1)
    plain = runtime.CompiledPlan(_plan_text(wl.name), 0, opt_level=0)
    assert plain.launches_per_run == 7
    # matmul+add;relu, matmul+add;relu, matmul+add, softmax: the planner placed the second group's
    # output on the bytes of that matmul's own input, so the fused result goes to a private buffer.
    assert fused.launches_per_run == 4
    assert fused.private_bytes > 0 and plain.private_bytes == 0
    before = capi.launch_count()
    fused.run_host(wl.inputs)
    assert capi.launch_count() - before == 4


def test_unknown_op_is_unimplemented_with_its_name():
    lib = capi.load()
    text = "plan slots=2 arena=0\nin 0 0 1 4\nstep frobnicate nin=1 0 nout=1 1 0 -1 1 4 attrs=0\nout 1\n"
    p = capi.c_void_p()
    rc = lib.fb200_plan_create(text.encode(), 0, 0, 1, capi.byref(p))
    assert rc == 4 and b"frobnicate" in lib.fb200_last_error()


def test_attention_heads_become_one_launch():
    """2 batches x 2 heads of slice/transpose/matmul/softmax/matmul + two levels of concat: one
    attention_fan launch at opt level 1, the step-by-step path at opt level 0, same numbers within
    the bf16 tier."""
    wl = next(w for w in WORKLOADS if w.name == "transformer_bf16_b2_s128_d128")
    fused = runtime.CompiledPlan(_plan_text(wl.name), 0, opt_level=1)
    plain = runtime.CompiledPlan(_plan_text(wl.name), 0, opt_level=0)
    names = fused.step_names()
    assert names.count("attention_fan") == 1
    assert not any(n in ("softmax", "transpose", "concat", "slice") for n in names)
    assert fused.launches_per_run <= 8 < plain.launches_per_run
    (a,) = fused.run_host(wl.inputs)
    (b,) = plain.run_host(wl.inputs)
    assert capi.kernel_status(0) == 0
    assert fo.all_close(a, b, wl.dtype, rtol=2e-2, atol=2e-2), fo.max_err(a, b, wl.dtype)


def test_mamba_conv_group_becomes_one_time_major_launch():
    """transpose, conv1d, slice, silu, transpose of the Mamba block run as one depthwise convolution
    over the time-major tensor, reading the in_proj output in place.  Whether the group forms depends
    on where the planner put the buffers (in the miniature plan the x_proj output overlaps the bytes
    the result would need, so it stays step by step); the 2-sample plan of the benchmark shape does
    form it, and must give the numbers of the step-by-step path (strict fp32: same operations)."""
    wl = configs.mamba_block(batch=2)
    text = runtime.load_plan_text(wl.name)
    fused = runtime.CompiledPlan(text, 0, opt_level=1)
    plain = runtime.CompiledPlan(text, 0, opt_level=0)
    names = fused.step_names()
    assert names.count("dwconv1d_time_major") == 1
    assert "conv1d" not in names and "transpose" not in names
    assert fused.launches_per_run < plain.launches_per_run
    (a,) = fused.run_host(wl.inputs)
    (b,) = plain.run_host(wl.inputs)
    assert capi.kernel_status(0) == 0
    assert fo.all_close(a, b, wl.dtype, rtol=1e-5, atol=1e-6), fo.max_err(a, b, wl.dtype)


def test_pipelined_host_runs_deliver_each_runs_own_result():
    """fb200_plan_run_host_async: three runs in flight over two staging sets, each with its own host
    buffers, must give what the synchronous entry point gives for the same inputs."""
    wl = WORKLOADS[0]
    plan = runtime.CompiledPlan(_plan_text(wl.name), 0)
    rng = np.random.default_rng(9)
    variants = []
    for _ in range(3):
        ins = [np.ascontiguousarray(a.copy()) for a in wl.inputs]
        ins[0] = rng.standard_normal(ins[0].shape).astype(ins[0].dtype)
        variants.append(ins)
    expected = [plan.run_host(ins)[0] for ins in variants]
    stream = capi.c_void_p()
    capi.check(capi.load().fb200_stream_create(0, capi.byref(stream)))
    for round_ in range(2):   # the second round replays the captured graphs of both staging sets
        outs = [np.zeros_like(expected[0]) for _ in variants]
        for ins, out in zip(variants, outs):
            plan.run_host_async_ptrs([a.ctypes.data for a in ins], [out.ctypes.data], stream)
        plan.host_sync()
        assert capi.kernel_status(0) == 0
        for got, exp in zip(outs, expected):
            assert np.array_equal(got.view(np.uint8), exp.view(np.uint8)), round_
    plan.close()


import cases as _cases  # noqa: E402


@pytest.mark.parametrize("name", _cases.PLAN_CASES)
def test_gradient_internals_through_the_plan_executor(name):
    """Pooling / convolution gradient internals as one-step plans (the plans the reference derives for
    backend "cuda"): bit-identical to the reference CPU backend's golden output."""
    case = _cases.CASES_BY_NAME[name]
    gold = np.load(os.path.join(HERE, "golden", "ref_cpu_cases.npz"))[name]
    plan = runtime.CompiledPlan(_plan_text("case_" + name), 0)
    (got,) = plan.run_host(case.inputs)
    assert capi.kernel_status(0) == 0
    assert np.array_equal(np.asarray(got).view(np.uint8), np.asarray(gold).view(np.uint8)), name
    plan.close()


def test_training_graph_of_the_reference_autograd_runs_bit_identically():
    """The training graph compiler::build_backward_graph derives from a two-layer MLP with an MSE loss
    ([loss, grad w1, grad b1, grad w2]; mse_loss_grad_internal, matmul_grad_lhs/rhs_internal,
    relu_grad_internal beside the forward ops), planned by the reference for backend "cuda".  Strict
    fp32: every output is bit-identical to the reference CPU backend, also on CUDA-graph replays."""
    _, ins = configs.train_mlp_forward()
    gold = np.load(GOLD)
    plan = runtime.CompiledPlan(_plan_text("train_mlp_f32"), 0, allow_tf32=False)
    for _ in range(3):
        outs = plan.run_host(ins)
        assert capi.kernel_status(0) == 0
        assert len(outs) == 4
        for i, got in enumerate(outs):
            exp = gold[f"train_mlp_f32__{i}"]
            assert np.array_equal(np.asarray(got).reshape(-1).view(np.uint8), np.asarray(exp).reshape(-1).view(np.uint8)), i
    plan.close()


def test_tensor_core_matmul_gradient_inside_a_replayed_plan():
    """matmul_grad_lhs_internal on the tensor-core route (bf16: scratch transpose from the
    stream-ordered allocator + tcgen05 GEMM) as a plan step: the allocation and the free are part of
    the captured CUDA graph, so the replays must keep producing the same result."""
    m, n, k = 512, 384, 256
    text = (f"plan slots=3 arena=0\nin 0 3 2 {m} {n}\nin 1 3 2 {k} {n}\n"
            f"step matmul_grad_lhs_internal nin=2 0 1 nout=1 2 3 -1 2 {m} {k} attrs=0\nout 2\n")
    rng = np.random.default_rng(41)
    gy = fo.from_accum(rng.uniform(-1, 1, (m, n)).astype(np.float32), fo.DT_BF16)
    b = fo.from_accum(rng.uniform(-1, 1, (k, n)).astype(np.float32), fo.DT_BF16)
    exp = fo.matmul_grad_lhs(gy, b, fo.DT_BF16)
    plan = runtime.CompiledPlan(text, 0)
    first = None
    for _ in range(4):
        (got,) = plan.run_host([gy, b])
        assert capi.kernel_status(0) == 0
        assert fo.all_close(got, exp, fo.DT_BF16, rtol=2e-2, atol=2e-2), fo.max_err(got, exp, fo.DT_BF16)
        if first is None:
            first = got.copy()
        assert np.array_equal(got, first)
    plan.close()


def test_two_host_threads_on_two_streams_run_one_plan_concurrently():
    """One compiled plan, two host threads, each with its own stream, inputs and outputs: every stream
    gets a workspace of its own (arena + captured graphs), so the runs do not wait for one another
    and must not disturb one another: each thread gets, run after run, exactly what a lone run
    gives for its inputs (the reference's Executable::run is re-entrant because it allocates its
    arena per call, src/backends/cuda/cuda_executable.cpp:55-61)."""
    import threading
    lib = capi.load()
    wl = next(w for w in WORKLOADS if w.name == "transformer_bf16_b2_s128_d128")
    plan = runtime.CompiledPlan(_plan_text(wl.name), 0)
    rng = np.random.default_rng(17)
    variants = []
    for _ in range(2):
        ins = [np.ascontiguousarray(a.copy()) for a in wl.inputs]
        ins[0] = fo.from_accum(rng.standard_normal(ins[0].shape).astype(np.float32), fo.DT_BF16)
        variants.append(ins)
    expected = [plan.run_host(ins)[0].copy() for ins in variants]
    dt, shape = plan.outputs[0]
    errors = []

    def worker(k):
        try:
            stream = capi.c_void_p()
            capi.check(lib.fb200_stream_create(0, capi.byref(stream)))
            dev_in = [capi.DeviceBuffer.from_numpy(a) for a in variants[k]]
            dev_out = capi.DeviceBuffer(expected[k].nbytes)
            for it in range(40):
                capi.check(lib.fb200_memset(0, dev_out.ptr, 0, dev_out.nbytes, stream))
                plan.run_device([b.ptr for b in dev_in], [dev_out.ptr], stream)
                capi.synchronize(0, stream)
                got = dev_out.download(capi.NP_STORAGE[dt], shape)
                if not np.array_equal(got.view(np.uint8), expected[k].view(np.uint8)):
                    errors.append((k, it))
                    return
        except Exception as e:   # surfaced in the main thread
            errors.append((k, repr(e)))

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert capi.kernel_status(0) == 0
    assert errors == [], errors
    plan.close()
