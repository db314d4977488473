"""Runs one parity case of tests/cases.py on the GPU through the C ABI (ctypes), returning the
host result in storage form.  No computation happens in Python."""
import numpy as np

from frame_public_b200 import capi
from oracle import frame_oracle as fo


def run_case(case, allow_tf32=False):
    dt = case.dtype
    exp_shape = case.expected().shape
    npdt = capi.NP_STORAGE[dt]
    bufs = [capi.DeviceBuffer.from_numpy(a) for a in case.inputs]
    ptr = [b.ptr for b in bufs]
    numel = int(np.prod(exp_shape, dtype=np.int64))
    out = capi.DeviceBuffer(max(numel, 1) * capi.ITEMSIZE[dt])
    ins = case.inputs
    op, at = case.op, case.attrs
    if op == "matmul":
        m, k = ins[0].shape
        n = ins[1].shape[1]
        capi.matmul(ptr[0], ptr[1], out.ptr, m, n, k, dt, allow_tf32)
    elif op == "fused_elementwise_internal":
        capi.fused_elementwise(ptr, out.ptr, numel, dt, at["ops"].split(";"))
    elif op in capi.EW:
        capi.fused_elementwise(ptr, out.ptr, numel, dt, [op])
    elif op == "bias_add":
        capi.bias_add(ptr[0], ptr[1], out.ptr, ins[0].shape[0], ins[0].shape[1], dt)
    elif op == "softmax":
        capi.softmax(ptr[0], out.ptr, ins[0].shape[0], ins[0].shape[1], dt)
    elif op == "layer_norm":
        capi.layer_norm(ptr[0], ptr[1], ptr[2], out.ptr, ins[0].shape[0], ins[0].shape[1], at["eps"], dt)
    elif op == "selective_scan":
        steps = ins[0].shape[-1]
        capi.selective_scan(*ptr, out.ptr, ins[0].size // steps if steps else 0, steps, dt)
    elif op == "conv2d":
        x, w = ins[0], ins[1]
        p = capi.Conv2dParams(x.shape[0], x.shape[1], x.shape[2], x.shape[3], w.shape[0], w.shape[2],
                              w.shape[3], at["stride"][0], at["stride"][1], at["padding"][0],
                              at["padding"][1], at["groups"])
        capi.conv2d(ptr[0], ptr[1], ptr[2] if len(ptr) > 2 else None, out.ptr, p, dt, allow_tf32)
    elif op == "conv1d":
        x, w = ins[0], ins[1]
        capi.conv1d(ptr[0], ptr[1], ptr[2] if len(ptr) > 2 else None, out.ptr, x.shape[0], x.shape[1],
                    x.shape[2], w.shape[0], w.shape[2], at["stride"], at["padding"], at["groups"], dt)
    elif op == "max_pool2d":
        x = ins[0]
        capi.max_pool2d(ptr[0], out.ptr, *x.shape, at["kernel"][0], at["kernel"][1], at["stride"][0],
                        at["stride"][1], at["padding"][0], at["padding"][1], dt)
    elif op == "avg_pool2d":
        x = ins[0]
        capi.avg_pool2d(ptr[0], out.ptr, *x.shape, at["kernel"][0], at["kernel"][1], at["stride"][0],
                        at["stride"][1], at["padding"][0], at["padding"][1], dt)
    elif op in ("max_pool2d_select_internal", "max_pool2d_grad_internal"):
        xs = ins[1].shape
        fn = capi.max_pool2d_select if op == "max_pool2d_select_internal" else capi.max_pool2d_grad
        fn(ptr[0], ptr[1], out.ptr, *xs, at["kernel"][0], at["kernel"][1], at["stride"][0], at["stride"][1],
           at["padding"][0], at["padding"][1], dt)
    elif op == "avg_pool2d_grad_internal":
        capi.avg_pool2d_grad(ptr[0], out.ptr, *at["input_shape"], at["kernel"][0], at["kernel"][1], at["stride"][0],
                             at["stride"][1], at["padding"][0], at["padding"][1], dt)
    elif op in ("conv2d_grad_input_internal", "conv2d_grad_filter_internal"):
        xs = at["input_shape"] if op == "conv2d_grad_input_internal" else ins[0].shape
        ws = ins[1].shape if op == "conv2d_grad_input_internal" else at["filter_shape"]
        p = capi.Conv2dParams(xs[0], xs[1], xs[2], xs[3], ws[0], ws[2], ws[3], at["stride"][0], at["stride"][1],
                              at["padding"][0], at["padding"][1], at["groups"])
        fn = capi.conv2d_grad_input if op == "conv2d_grad_input_internal" else capi.conv2d_grad_filter
        fn(ptr[0], ptr[1], out.ptr, p, dt)
    elif op == "matmul_grad_lhs_internal":
        (m, n), k = ins[0].shape, ins[1].shape[0]
        capi.matmul_grad_lhs(ptr[0], ptr[1], out.ptr, m, n, k, dt, allow_tf32)
    elif op == "matmul_grad_rhs_internal":
        (m, k), n = ins[0].shape, ins[1].shape[1]
        capi.matmul_grad_rhs(ptr[0], ptr[1], out.ptr, m, n, k, dt, allow_tf32)
    elif op == "mse_loss":
        capi.mse_loss(ptr[0], ptr[1], out.ptr, ins[0].size, dt)
    elif op == "mse_loss_grad_internal":
        capi.mse_loss_grad(ptr[0], ptr[1], ptr[2], out.ptr, ins[0].size, dt)
    elif op == "rfft":
        n = ins[0].shape[-1]
        capi.rfft(ptr[0], out.ptr, ins[0].size // n, n, dt)
    elif op == "irfft":
        n = at["n"]
        capi.irfft(ptr[0], out.ptr, ins[0].size // (2 * (n // 2 + 1)), n, dt)
    elif op == "heaviside_surrogate":
        capi.fused_elementwise(ptr, out.ptr, numel, dt, [op])
    elif op == "gather":
        capi.gather(ptr[0], ptr[1], out.ptr, ins[0].shape[0], ins[0].shape[1], ins[1].shape[0], dt,
                    capi.I32 if ins[1].dtype == np.int32 else capi.I64)
    elif op in ("scatter_add", "gather_grad_internal"):
        capi.scatter_add(ptr[0], ptr[1], out.ptr, ins[0].shape[0], ins[0].shape[1], exp_shape[0], dt,
                         capi.I32 if ins[1].dtype == np.int32 else capi.I64)
    elif op == "transpose":
        capi.transpose(ptr[0], out.ptr, ins[0].shape, at["perm"], capi.ITEMSIZE[dt])
    elif op == "slice":
        capi.slice_(ptr[0], out.ptr, ins[0].shape, at["axis"], at["start"], at["stop"], capi.ITEMSIZE[dt])
    elif op == "concat":
        capi.concat(ptr, [a.shape[at["axis"]] for a in ins], out.ptr, exp_shape, at["axis"], capi.ITEMSIZE[dt])
    elif op == "reshape":
        capi.check(capi.load().fb200_memcpy(0, out.ptr, ptr[0], ins[0].nbytes, capi.D2D, None, 1))
    elif op == "sum":
        capi.sum_axes(ptr[0], out.ptr, ins[0].shape, at["axes"], dt)
    else:
        raise KeyError(op)
    capi.synchronize()
    res = out.download(npdt, exp_shape)
    for b in bufs:
        b.free()
    out.free()
    return res


def assert_parity(case, got, exact):
    exp = case.expected()
    assert got.shape == exp.shape
    if exact:
        same = np.array_equal(np.asarray(got).reshape(-1).view(np.uint8), np.asarray(exp).reshape(-1).view(np.uint8))
        assert same, (case.name, fo.max_err(got, exp, case.dtype))
    else:
        assert fo.all_close(got, exp, case.dtype), (case.name, fo.max_err(got, exp, case.dtype))
