"""ctypes binding of libframe_b200.so (the C ABI declared in include/frame_b200.h).

This is the Python-side mirror of the reference-facing boundary: every function here is a thin
call into the shared library; nothing is computed in Python and there is no CPU fallback — if
the library is missing, or a compute entry point is called without a usable B200, an exception
is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, byref, c_char_p, c_double, c_float, c_int, c_int64,
                    c_size_t, c_void_p)

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libframe_b200.so")

# fb200_dtype == frame::DTypeCode
F32, F64, F16, BF16, I8, I16, I32, I64, U8, BOOL = range(10)
ITEMSIZE = {F32: 4, F64: 8, F16: 2, BF16: 2, I8: 1, I16: 2, I32: 4, I64: 8, U8: 1, BOOL: 1}
NP_STORAGE = {F32: np.float32, F64: np.float64, F16: np.uint16, BF16: np.uint16, I8: np.int8,
              I16: np.int16, I32: np.int32, I64: np.int64, U8: np.uint8, BOOL: np.uint8}

EW = {"add": 1, "mul": 2, "relu": 3, "square": 4, "sigmoid": 5, "tanh": 6, "rsqrt": 7,
      "gelu": 8, "silu": 9, "softplus": 10, "exp": 11, "heaviside_surrogate": 12,
      "relu_grad_internal": 13}
EW_ARITY = {"add": 2, "mul": 2, "relu_grad_internal": 2}
OPERAND_FULL, OPERAND_COL, OPERAND_ROW = 0, 1, 2
H2D, D2H, D2D = 1, 2, 3
MAX_CHAIN = 8

STATUS_NAMES = {0: "OK", 1: "INVALID_ARGUMENT", 2: "NOT_FOUND", 3: "ALREADY_EXISTS",
                4: "UNIMPLEMENTED", 5: "OUT_OF_MEMORY", 6: "INTERNAL", 7: "DEVICE_ERROR"}


class Fb200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"fb200 status {code} ({STATUS_NAMES.get(code, '?')}): {message}")
        self.code = code


class Epilogue(Structure):
    _fields_ = [("n_ops", c_int), ("ops", c_int * MAX_CHAIN), ("operands", c_void_p * MAX_CHAIN),
                ("modes", c_int * MAX_CHAIN)]


class Conv2dParams(Structure):
    _fields_ = [(n, c_int64) for n in ("n", "cin", "h", "w", "cout", "kh", "kw", "stride_h",
                                       "stride_w", "pad_h", "pad_w", "groups")]


# Every exported symbol of include/frame_b200.h: name -> (restype, argtypes)
_P = c_void_p
_PP = POINTER(c_void_p)
_I64P = POINTER(c_int64)
_IP = POINTER(c_int)
SIGNATURES = {
    "fb200_last_error": (c_char_p, []),
    "fb200_version": (c_char_p, []),
    "fb200_launch_count": (c_int64, []),
    "fb200_kernel_status": (c_int, [c_int, _IP]),
    "fb200_device_count": (c_int, [_IP]),
    "fb200_device_pci_bus_id": (c_int, [c_int, c_char_p, c_int]),
    "fb200_malloc": (c_int, [c_int, c_size_t, c_size_t, _PP]),
    "fb200_free": (c_int, [c_int, _P]),
    "fb200_host_alloc": (c_int, [c_size_t, _PP]),
    "fb200_host_free": (c_int, [_P]),
    "fb200_memcpy": (c_int, [c_int, _P, _P, c_size_t, c_int, _P, c_int]),
    "fb200_memset": (c_int, [c_int, _P, c_int, c_size_t, _P]),
    "fb200_stream_create": (c_int, [c_int, _PP]),
    "fb200_stream_destroy": (c_int, [c_int, _P]),
    "fb200_stream_synchronize": (c_int, [c_int, _P]),
    "fb200_event_create": (c_int, [c_int, c_int, _PP]),
    "fb200_event_destroy": (c_int, [c_int, _P]),
    "fb200_event_record": (c_int, [c_int, _P, _P]),
    "fb200_stream_wait_event": (c_int, [c_int, _P, _P]),
    "fb200_event_query": (c_int, [c_int, _P, _IP]),
    "fb200_event_synchronize": (c_int, [c_int, _P]),
    "fb200_event_elapsed_ms": (c_int, [_P, _P, POINTER(c_float)]),
    "fb200_fused_elementwise": (c_int, [_PP, c_int, _P, c_int64, c_int, _IP, _IP, c_int, _P]),
    "fb200_bias_add": (c_int, [_P, _P, _P, c_int64, c_int64, c_int, _P]),
    "fb200_matmul": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int, c_int,
                             POINTER(Epilogue), _P]),
    "fb200_matmul_split": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int, c_int,
                                   POINTER(Epilogue), _P]),
    "fb200_matmul_colsplit": (c_int, [_P, _P, _PP, c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                                      c_int, c_int, POINTER(Epilogue), _P]),
    "fb200_ipc_export": (c_int, [c_int, _P, _P]),
    "fb200_ipc_import": (c_int, [c_int, _P, _PP]),
    "fb200_ipc_close": (c_int, [c_int, _P]),
    "fb200_matmul_uses_tensor_cores": (c_int, [c_int64, c_int64, c_int64, c_int, c_int]),
    "fb200_matmul_schedule": (c_int, [c_int64, c_int64, c_int64, c_int, c_int, c_int, _I64P]),
    "fb200_conv2d": (c_int, [_P, _P, _P, _P, POINTER(Conv2dParams), c_int, c_int,
                             POINTER(Epilogue), _P]),
    "fb200_conv2d_max_pool": (c_int, [_P, _P, _P, _P, _P, POINTER(Conv2dParams)] + [c_int64] * 6 +
                              [c_int, c_int, POINTER(Epilogue), _P]),
    "fb200_conv1d": (c_int, [_P, _P, _P, _P] + [c_int64] * 8 + [c_int, _P]),
    "fb200_max_pool2d": (c_int, [_P, _P] + [c_int64] * 10 + [c_int, _P]),
    "fb200_avg_pool2d": (c_int, [_P, _P] + [c_int64] * 10 + [c_int, _P]),
    "fb200_max_pool2d_select": (c_int, [_P, _P, _P] + [c_int64] * 10 + [c_int, _P]),
    "fb200_max_pool2d_grad": (c_int, [_P, _P, _P] + [c_int64] * 10 + [c_int, _P]),
    "fb200_avg_pool2d_grad": (c_int, [_P, _P] + [c_int64] * 10 + [c_int, _P]),
    "fb200_conv2d_grad_input": (c_int, [_P, _P, _P, POINTER(Conv2dParams), c_int, _P]),
    "fb200_conv2d_grad_filter": (c_int, [_P, _P, _P, POINTER(Conv2dParams), c_int, _P]),
    "fb200_matmul_grad_lhs": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int, c_int, _P]),
    "fb200_matmul_grad_rhs": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int, c_int, _P]),
    "fb200_mse_loss": (c_int, [_P, _P, _P, c_int64, c_int, _P]),
    "fb200_mse_loss_grad": (c_int, [_P, _P, _P, _P, c_int64, c_int, _P]),
    "fb200_rfft": (c_int, [_P, _P, c_int64, c_int64, c_int, _P]),
    "fb200_irfft": (c_int, [_P, _P, c_int64, c_int64, c_int, _P]),
    "fb200_gather": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int, c_int, _P]),
    "fb200_scatter_add": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int, c_int, _P]),
    "fb200_softmax": (c_int, [_P, _P, c_int64, c_int64, c_int, _P]),
    "fb200_layer_norm": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_double, c_int, _P]),
    "fb200_add_layer_norm": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int64, c_double, c_int, _P]),
    "fb200_selective_scan": (c_int, [_P] * 6 + [c_int64, c_int64, c_int, _P]),
    "fb200_selective_scan_noalloc": (c_int, [_P] * 6 + [c_int64, c_int64, c_int, _P]),
    "fb200_dwconv1d_time_major": (c_int, [_P, c_int64, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int64,
                                          c_int64, c_int64, POINTER(c_int), c_int, c_int, _P]),
    "fb200_attention_fan_supported": (c_int, [c_int64, c_int64, c_int64, c_int]),
    "fb200_attention_fan": (c_int, [_P, c_int64, c_int64, _P, c_int64, c_int64, _P, c_int64, c_int64, _P,
                                    c_int64, _P, c_int64, c_int64, c_int64, c_int64, c_float, c_int, _P]),
    "fb200_mamba_scan": (c_int, [_P] * 8 + [c_int64] * 4 + [_P]),
    "fb200_transpose": (c_int, [_P, _P, c_int, _I64P, _I64P, c_int, _P]),
    "fb200_slice": (c_int, [_P, _P, c_int, _I64P, c_int64, c_int64, c_int64, c_int, _P]),
    "fb200_concat": (c_int, [_PP, c_int, _I64P, _P, c_int, _I64P, c_int64, c_int, _P]),
    "fb200_sum_axes": (c_int, [_P, _P, c_int, _I64P, _I64P, c_int, c_int, _P]),
    "fb200_plan_create": (c_int, [c_char_p, c_int, c_int, c_int, _PP]),
    "fb200_plan_destroy": (c_int, [_P]),
    "fb200_plan_num_inputs": (c_int, [_P]),
    "fb200_plan_num_outputs": (c_int, [_P]),
    "fb200_plan_io_spec": (c_int, [_P, c_int, c_int, _IP, _IP, _I64P]),
    "fb200_plan_arena_bytes": (c_size_t, [_P]),
    "fb200_plan_private_bytes": (c_size_t, [_P]),
    "fb200_plan_launches_per_run": (c_int, [_P]),
    "fb200_plan_run": (c_int, [_P, _PP, _PP, _P]),
    "fb200_plan_run_host": (c_int, [_P, _PP, _PP, _P]),
    "fb200_plan_profile": (c_int, [_P, _PP, _PP, _P, POINTER(c_float), c_int, _IP]),
    "fb200_plan_step_op": (c_char_p, [_P, c_int]),
    "fb200_plan_run_host_async": (c_int, [_P, _PP, _PP, _P]),
    "fb200_plan_host_sync": (c_int, [_P]),
    "fb200_plan_bind_resident": (c_int, [_P, c_int, _P]),
    "fb200_plan_describe": (c_int, [c_char_p, c_int, c_int, _PP]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m frame_public_b200.build` "
                "(there is no CPU fallback)")
        lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise Fb200Error(rc, load().fb200_last_error().decode("utf-8", "replace"))


def device_count() -> int:
    n = c_int(0)
    rc = load().fb200_device_count(byref(n))
    return n.value if rc == 0 else 0


def kernel_status(device: int = 0) -> int:
    code = c_int(0)
    check(load().fb200_kernel_status(device, byref(code)))
    return code.value


def launch_count() -> int:
    return int(load().fb200_launch_count())


class DeviceBuffer:
    """A device allocation made through fb200_malloc, with numpy upload/download."""

    def __init__(self, nbytes: int, device: int = 0):
        self.device = device
        self.nbytes = int(nbytes)
        self.ptr = c_void_p(None)
        if self.nbytes > 0:
            check(load().fb200_malloc(device, self.nbytes, 256, byref(self.ptr)))

    @classmethod
    def from_numpy(cls, arr: np.ndarray, device: int = 0) -> "DeviceBuffer":
        arr = np.ascontiguousarray(arr)
        buf = cls(arr.nbytes, device)
        buf.upload(arr)
        return buf

    def upload(self, arr: np.ndarray) -> None:
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes <= self.nbytes
        if arr.nbytes:
            check(load().fb200_memcpy(self.device, self.ptr, arr.ctypes.data_as(c_void_p),
                                      arr.nbytes, H2D, None, 1))

    def download(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        if out.nbytes:
            check(load().fb200_memcpy(self.device, out.ctypes.data_as(c_void_p), self.ptr,
                                      out.nbytes, D2H, None, 1))
        return out

    def free(self) -> None:
        if self.ptr.value:
            load().fb200_free(self.device, self.ptr)
            self.ptr = c_void_p(None)

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _i64(values):
    arr = (c_int64 * max(1, len(values)))(*[int(v) for v in values])
    return arr


def make_epilogue(steps) -> Epilogue:
    """steps: list of (op_name, operand_ptr_or_None, mode)."""
    e = Epilogue()
    e.n_ops = len(steps)
    for i, (name, operand, mode) in enumerate(steps):
        e.ops[i] = EW[name]
        e.operands[i] = operand.value if isinstance(operand, c_void_p) else operand
        e.modes[i] = mode
    return e


# ---- thin op wrappers over device pointers (c_void_p) ------------------------------------------
def fused_elementwise(inputs, out, numel, dtype, op_names, stream=None):
    n = len(inputs)
    arr = (c_void_p * max(1, n))(*[p.value if isinstance(p, c_void_p) else p for p in inputs])
    ops = (c_int * len(op_names))(*[EW[o] for o in op_names])
    ar = (c_int * len(op_names))(*[EW_ARITY.get(o, 1) for o in op_names])
    check(load().fb200_fused_elementwise(arr, n, out, numel, dtype, ops, ar, len(op_names), stream))


def bias_add(x, bias, out, rows, cols, dtype, stream=None):
    check(load().fb200_bias_add(x, bias, out, rows, cols, dtype, stream))


def matmul(a, b, c, m, n, k, dtype, allow_tf32=False, epilogue=None, stream=None):
    ep = byref(epilogue) if epilogue is not None else None
    check(load().fb200_matmul(a, b, c, m, n, k, dtype, 1 if allow_tf32 else 0, ep, stream))


def matmul_split(a, b, c, c_tail, tail_col, m, n, k, dtype, allow_tf32=False, epilogue=None, stream=None):
    ep = byref(epilogue) if epilogue is not None else None
    check(load().fb200_matmul_split(a, b, c, c_tail, tail_col, m, n, k, dtype, 1 if allow_tf32 else 0, ep, stream))


def matmul_schedule(m, n, k, dtype, light_epilogue=False, compensated=False):
    """Tile shape and last-wave split fb200_matmul uses for a tensor-core product (host logic only)."""
    out = (c_int64 * 6)()
    check(load().fb200_matmul_schedule(m, n, k, dtype, 1 if light_epilogue else 0, 1 if compensated else 0, out))
    keys = ("tile_n", "tile_m", "dp_tiles", "sk_units", "sk_ctas", "k_blocks")
    return dict(zip(keys, (int(v) for v in out)))


def conv2d(x, w, bias, out, params: Conv2dParams, dtype, allow_tf32=False, epilogue=None,
           stream=None):
    ep = byref(epilogue) if epilogue is not None else None
    check(load().fb200_conv2d(x, w, bias, out, byref(params), dtype, 1 if allow_tf32 else 0, ep,
                              stream))


def conv2d_max_pool(x, w, bias, mid, out, params: Conv2dParams, pool, dtype, allow_tf32=False, epilogue=None,
                    stream=None):
    """pool = (kh, kw, stride_h, stride_w, pad_h, pad_w)."""
    ep = byref(epilogue) if epilogue is not None else None
    check(load().fb200_conv2d_max_pool(x, w, bias, mid, out, byref(params), *pool, dtype, 1 if allow_tf32 else 0,
                                       ep, stream))


def conv1d(x, w, bias, out, n, cin, l, cout, k, stride, padding, groups, dtype, stream=None):
    check(load().fb200_conv1d(x, w, bias, out, n, cin, l, cout, k, stride, padding, groups, dtype,
                              stream))


def max_pool2d(x, out, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream=None):
    check(load().fb200_max_pool2d(x, out, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream))


def avg_pool2d(x, out, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream=None):
    check(load().fb200_avg_pool2d(x, out, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream))


def max_pool2d_select(g, x, out, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream=None):
    check(load().fb200_max_pool2d_select(g, x, out, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream))


def max_pool2d_grad(dy, x, dx, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream=None):
    check(load().fb200_max_pool2d_grad(dy, x, dx, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream))


def avg_pool2d_grad(dy, dx, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream=None):
    check(load().fb200_avg_pool2d_grad(dy, dx, n, c, h, w, kh, kw, sh, sw, ph, pw, dtype, stream))


def conv2d_grad_input(dy, w, dx, params: Conv2dParams, dtype, stream=None):
    check(load().fb200_conv2d_grad_input(dy, w, dx, byref(params), dtype, stream))


def conv2d_grad_filter(x, dy, dw, params: Conv2dParams, dtype, stream=None):
    check(load().fb200_conv2d_grad_filter(x, dy, dw, byref(params), dtype, stream))


def matmul_grad_lhs(gy, b, ga, m, n, k, dtype, allow_tf32=False, stream=None):
    check(load().fb200_matmul_grad_lhs(gy, b, ga, m, n, k, dtype, 1 if allow_tf32 else 0, stream))


def matmul_grad_rhs(a, gy, gb, m, n, k, dtype, allow_tf32=False, stream=None):
    check(load().fb200_matmul_grad_rhs(a, gy, gb, m, n, k, dtype, 1 if allow_tf32 else 0, stream))


def mse_loss(pred, target, out, numel, dtype, stream=None):
    check(load().fb200_mse_loss(pred, target, out, numel, dtype, stream))


def mse_loss_grad(pred, target, gy, gpred, numel, dtype, stream=None):
    check(load().fb200_mse_loss_grad(pred, target, gy, gpred, numel, dtype, stream))


def rfft(x, out, rows, n, dtype, stream=None):
    check(load().fb200_rfft(x, out, rows, n, dtype, stream))


def irfft(z, out, rows, n, dtype, stream=None):
    check(load().fb200_irfft(z, out, rows, n, dtype, stream))


def gather(x, indices, out, n, f, k, dtype, index_dtype, stream=None):
    check(load().fb200_gather(x, indices, out, n, f, k, dtype, index_dtype, stream))


def scatter_add(updates, indices, out, k, f, v, dtype, index_dtype, stream=None):
    check(load().fb200_scatter_add(updates, indices, out, k, f, v, dtype, index_dtype, stream))


def softmax(x, out, rows, cols, dtype, stream=None):
    check(load().fb200_softmax(x, out, rows, cols, dtype, stream))


def layer_norm(x, gamma, beta, out, rows, cols, eps, dtype, stream=None):
    check(load().fb200_layer_norm(x, gamma, beta, out, rows, cols, eps, dtype, stream))


def add_layer_norm(x, res, gamma, beta, sum_out, out, rows, cols, eps, dtype, stream=None):
    check(load().fb200_add_layer_norm(x, res, gamma, beta, sum_out, out, rows, cols, eps, dtype, stream))


def selective_scan(x, a, b, c, d, out, rows, steps, dtype, stream=None):
    check(load().fb200_selective_scan(x, a, b, c, d, out, rows, steps, dtype, stream))


def mamba_scan(u, delta, A, B, C, D, z, y, batch, length, dm, nstate, stream=None):
    check(load().fb200_mamba_scan(u, delta, A, B, C, D, z, y, batch, length, dm, nstate, stream))


def dwconv1d_time_major(x, x_ld, w, bias, out, out_ld, batch, length, out_len, channels, k, shift,
                        op_names, dtype, stream=None):
    ops = (c_int * max(1, len(op_names)))(*[EW[n] for n in op_names])
    check(load().fb200_dwconv1d_time_major(x, x_ld, w, bias, out, out_ld, batch, length, out_len, channels,
                                           k, shift, ops, len(op_names), dtype, stream))


HEAD_DTYPE = np.dtype([("q_row", "<i4"), ("q_col", "<i4"), ("k_row", "<i4"), ("k_col", "<i4"),
                       ("v_row", "<i4"), ("v_col", "<i4"), ("o_offset", "<i8")])


def attention_fan(q, q_rows, q_ld, k, k_rows, k_ld, v, v_rows, v_ld, o, o_ld, heads_dev, n_heads,
                  sq, sk, head_dim, dtype, stream=None, scale=1.0):
    """heads_dev: device pointer of an array of HEAD_DTYPE records (fb200_attention_head)."""
    check(load().fb200_attention_fan(q, q_rows, q_ld, k, k_rows, k_ld, v, v_rows, v_ld, o, o_ld,
                                     heads_dev, n_heads, sq, sk, head_dim, scale, dtype, stream))


def transpose(x, out, dims, perm, itemsize, stream=None):
    check(load().fb200_transpose(x, out, len(dims), _i64(dims), _i64(perm), itemsize, stream))


def slice_(x, out, dims, axis, start, stop, itemsize, stream=None):
    check(load().fb200_slice(x, out, len(dims), _i64(dims), axis, start, stop, itemsize, stream))


def concat(inputs, axis_sizes, out, out_dims, axis, itemsize, stream=None):
    n = len(inputs)
    arr = (c_void_p * max(1, n))(*[p.value if isinstance(p, c_void_p) else p for p in inputs])
    check(load().fb200_concat(arr, n, _i64(axis_sizes), out, len(out_dims), _i64(out_dims), axis,
                              itemsize, stream))


def sum_axes(x, out, dims, axes, dtype, stream=None):
    check(load().fb200_sum_axes(x, out, len(dims), _i64(dims), _i64(axes), len(axes), dtype, stream))


def synchronize(device: int = 0, stream=None) -> None:
    check(load().fb200_stream_synchronize(device, stream))
