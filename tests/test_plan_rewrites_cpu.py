"""The plan executor's rewrite rules, checked without a GPU through fb200_plan_describe: the same
parsing, aliasing, epilogue absorption and group recognition as fb200_plan_create, minus every
device allocation.  Plans are the ones the reference pipeline and memory planner emitted for backend
"cuda" (tests/golden/plans/, frame_public_b200/plans/)."""
import os

import pytest

from frame_public_b200 import capi, runtime

HERE = os.path.dirname(os.path.abspath(__file__))


def _golden(name):
    with open(os.path.join(HERE, "golden", "plans", name + ".plan")) as f:
        return f.read()


def _live(names):
    return [n for n in names if not n.startswith("(") and n != "constant"]


def test_transformer_block_becomes_seven_launches():
    text = runtime.load_plan_text("transformer_bf16_b8_s512_d1024")
    names, launches = runtime.describe_plan(text, opt_level=1)
    assert len(names) == 922
    assert launches == 7
    # the residual add in front of the second LayerNorm runs inside it (the planner puts the
    # normalised rows exactly on the dead addend: allowed, a warp holds its row before it writes)
    assert _live(names) == ["layer_norm", "matmul", "attention_fan", "matmul", "add+layer_norm",
                            "matmul+epilogue", "matmul+epilogue"]
    plain, plain_launches = runtime.describe_plan(text, opt_level=0)
    assert plain.count("softmax") == 128 and plain.count("attention_fan") == 0
    assert plain_launches > 900


def test_attention_fan_result_leaves_the_arena_when_the_planner_put_it_over_the_qkv_matrix():
    """The planner lays the arena out for the unfused graph, where the fused QKV projection is dead
    (sliced per head) long before the concat of the heads is written; in this plan it put the
    concat's 8 MiB result 1 MiB into the 24 MiB projection.  The fused launch reads the projection
    while it writes the result, so the result must move to a private buffer."""
    text = runtime.load_plan_text("transformer_bf16_b8_s512_d1024")
    assert runtime.plan_private_bytes(text, opt_level=1) == 8 * 512 * 1024 * 2
    assert runtime.plan_private_bytes(text, opt_level=0) == 0


def test_reference_nn_attention_with_its_scale_mul_is_recognised():
    names, _ = runtime.describe_plan(_golden("nn_transformer_bf16_b2_s128_e128_h2"))
    live = _live(names)
    assert live.count("attention_fan") == 1
    assert not any(n in ("softmax", "transpose", "concat", "slice", "mul") for n in live)
    # the fp32 block is outside the fused kernel (16-bit dtypes only): it stays step by step
    f32, _ = runtime.describe_plan(_golden("nn_transformer_f32_b2_s16_e32_h2"))
    assert f32.count("attention_fan") == 0 and f32.count("softmax") == 4


def test_mamba_conv_group_and_reshape_views():
    names, launches = runtime.describe_plan(runtime.load_plan_text("mamba_f32_b16_s2048_d768"))
    live = _live(names)
    assert live.count("dwconv1d_time_major") == 1 and live.count("mamba_scan") == 1
    assert "conv1d" not in live and "transpose" not in live and "silu" not in live
    assert live.count("reshape") == 1           # the gate's reshape: its source is still being read
    assert launches == 10
    # miniature plan: the planner put the x_proj output on the bytes the fused result would need
    small, _ = runtime.describe_plan(_golden("mamba_f32_b2_s24_d16"))
    assert small.count("dwconv1d_time_major") == 0 and small.count("conv1d") == 1


def test_mlp_absorbs_every_group_the_second_through_a_private_buffer():
    """The planner puts the second hidden layer's add;relu result on the bytes of that layer's own
    matmul input (dead in the unfused order once the matmul has run); as the matmul's epilogue it
    would overwrite rows other CTAs still read, so the result moves to a private buffer."""
    text = _golden("mlp_f32_b8")
    names, launches = runtime.describe_plan(text)
    assert launches == 4
    assert _live(names) == ["matmul+epilogue", "matmul+epilogue", "matmul+epilogue", "softmax"]
    assert runtime.plan_private_bytes(text) == 8 * 32 * 4   # the miniature has 32 hidden units
    _, plain = runtime.describe_plan(text, opt_level=0)
    assert plain == 7


def test_a_described_plan_cannot_run():
    lib = capi.load()
    h = capi.c_void_p()
    capi.check(lib.fb200_plan_describe(_golden("mlp_f32_b8").encode(), 0, 1, capi.byref(h)))
    rc = lib.fb200_plan_run(h, None, None, None)
    assert rc == 1 and b"cannot run" in lib.fb200_last_error()
    lib.fb200_plan_destroy(h)


def test_unknown_op_is_unimplemented_with_its_name_without_a_gpu():
    lib = capi.load()
    text = "plan slots=2 arena=0\nin 0 0 1 4\nstep frobnicate nin=1 0 nout=1 1 0 -1 1 4 attrs=0\nout 1\n"
    h = capi.c_void_p()
    rc = lib.fb200_plan_describe(text.encode(), 0, 1, capi.byref(h))
    assert rc == 4 and b"frobnicate" in lib.fb200_last_error()


def test_pool_and_index_ops_decode_and_opt_out_of_graph_replay_checks():
    text = ("plan slots=4 arena=1024\nin 0 0 2 5 4\nin 1 6 1 3\n"
            "step gather nin=2 0 1 nout=1 2 0 0 2 3 4 attrs=0\n"
            "step heaviside_surrogate nin=1 2 nout=1 3 0 -1 2 3 4 attrs=1\nattr alpha double 2.0\nout 3\n")
    names, launches = runtime.describe_plan(text)
    assert names == ["gather", "heaviside_surrogate"] and launches == 2
    bad = text.replace("attr alpha double 2.0", "attr alpha double -1.0")
    lib = capi.load()
    h = capi.c_void_p()
    rc = lib.fb200_plan_describe(bad.encode(), 0, 1, capi.byref(h))
    assert rc == 1 and b"alpha" in lib.fb200_last_error()


def test_gradient_internals_decode_as_single_steps():
    import sys
    sys.path.insert(0, HERE)
    import cases
    for name in cases.PLAN_CASES:
        names, launches = runtime.describe_plan(_golden("case_" + name))
        assert names == [cases.CASES_BY_NAME[name].op] and launches == 1, name
    # a malformed attribute list is rejected with the op's name
    text = _golden("case_conv2d_grad_input_groups2").replace("attr stride int64_array [1, 2]", "attr stride int64_array [1]")
    lib = capi.load()
    h = capi.c_void_p()
    rc = lib.fb200_plan_describe(text.encode(), 0, 1, capi.byref(h))
    assert rc == 1 and b"conv2d_grad_input_internal" in lib.fb200_last_error()


def test_training_graph_decodes_with_the_bias_add_absorbed():
    names, launches = runtime.describe_plan(_golden("train_mlp_f32"))
    assert _live(names) == ["matmul+epilogue", "relu", "matmul", "mse_loss", "mse_loss_grad_internal",
                            "matmul_grad_lhs_internal", "matmul_grad_rhs_internal", "relu_grad_internal",
                            "matmul_grad_rhs_internal"]
    assert launches == 9


def test_a_fused_group_longer_than_one_launch_is_split_not_rejected():
    """12 elementwise steps in one fused group (the reference's fusion pass has no length limit):
    the executor keeps it as one step that runs as two successive launches."""
    ops = "add;relu;mul;square;add;relu;mul;add;relu;add;mul;relu"
    ar = [2, 1, 2, 1, 2, 1, 2, 2, 1, 2, 2, 1]
    n_in = sum(ar) - (len(ar) - 1)
    lines = [f"plan slots={n_in + 1} arena=0"]
    lines += [f"in {i} 0 2 9 1023" for i in range(n_in)]
    lines += [f"step fused_elementwise_internal nin={n_in} " + " ".join(str(i) for i in range(n_in))
              + f" nout=1 {n_in} 0 -1 2 9 1023 attrs=2",
              "attr arities int64_array [" + ", ".join(map(str, ar)) + "]", f'attr ops string "{ops}"', f"out {n_in}"]
    names, launches = runtime.describe_plan("\n".join(lines) + "\n")
    assert names == ["fused_elementwise_internal"] and launches == 2


def test_mamba_gate_slice_is_written_by_the_projection_itself():
    """With allow_tf32 the in_proj matmul takes the tensor-core kernel, which can store a trailing
    column block into a buffer of its own: the `slice` of the gate half z and the `reshape` behind it
    (a copy, because the planner reuses the slice's bytes for the scan's result) both disappear, as
    does the slice of the last block of x_proj.  Without allow_tf32 (strict fp32 on the CUDA cores)
    the plan keeps them."""
    text = runtime.load_plan_text("mamba_f32_b16_s2048_d768")
    names, launches = runtime.describe_plan(text, allow_tf32=True)
    live = _live(names)
    assert launches == 8 and "reshape" not in live and live.count("slice") == 2
    strict, strict_launches = runtime.describe_plan(text, allow_tf32=False)
    assert strict_launches == 10 and _live(strict).count("slice") == 4


def test_stem_conv_and_its_max_pool_become_one_step_when_tf32_is_allowed():
    """conv2d + bias/ReLU epilogue followed by max_pool2d whose only reader it is: one step
    (fb200_conv2d_max_pool; on the GPU an image stem then runs as one kernel that never writes the
    convolution's result).  Strict fp32 keeps the operators apart."""
    text = runtime.load_plan_text("conv_stack_f32_b32_224")
    names, launches = runtime.describe_plan(text, allow_tf32=True)
    running = [n for n in names if not n.startswith("(")]
    assert running[0] == "conv2d+epilogue+max_pool2d", running
    assert "max_pool2d" not in running
    assert launches == 3
    strict, strict_launches = runtime.describe_plan(text, allow_tf32=False)
    assert [n for n in strict if not n.startswith("(")][:2] == ["conv2d+epilogue", "max_pool2d"]
    assert strict_launches == 4
    # the nn CNN of the reference's own layers (conv -> relu -> 2x2 pool): folded as well; the call
    # then runs the two kernels, since only the 3x3 / stride-2 pool has a fused kernel
    cnn, _ = runtime.describe_plan(_golden("nn_cnn_f32_b4_c16_hw32_o32"), allow_tf32=True)
    assert any(n.startswith("conv2d") and n.endswith("+max_pool2d") for n in cnn), cnn
