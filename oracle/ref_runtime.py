"""TEST INFRASTRUCTURE — ctypes driver of oracle/_ref (the UNMODIFIED reference framework built
from its own sources by oracle/build_ref.sh, plus the extern "C" shim of oracle/ref_shim.cpp).

With backend "cpu" this runs the reference's CPU backend: the parity oracle and the timed CPU
baseline.  When the sm_100a backend of this repository has been loaded into the same process
(load_b200_backend), backend "cuda" runs the product end to end through the reference's own
runtime::compile and Executable::run.

Only tests, the smoke check and the benchmark's CPU-baseline / reference arms import this.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, byref, c_char_p, c_double, c_int, c_int32, c_int64, c_void_p, create_string_buffer

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
LIB_REF = os.path.join(REF_DIR, "libframe_ref.so")
LIB_SHIM = os.path.join(REF_DIR, "libframe_ref_shim.so")

NP_STORAGE = {0: np.float32, 1: np.float64, 2: np.uint16, 3: np.uint16, 4: np.int8, 5: np.int16,
              6: np.int32, 7: np.int64, 8: np.uint8, 9: np.uint8}

_shim = None


def available() -> bool:
    return os.path.exists(LIB_REF) and os.path.exists(LIB_SHIM)


def load():
    """Loads the reference framework (RTLD_GLOBAL, so that a backend plugin loaded afterwards
    resolves the framework's symbols) and the shim."""
    global _shim
    if _shim is None:
        if not available():
            raise FileNotFoundError(f"{LIB_REF} not built: run oracle/build_ref.sh where the "
                                    "reference sources are present")
        ctypes.CDLL(LIB_REF, mode=ctypes.RTLD_GLOBAL)
        s = ctypes.CDLL(LIB_SHIM, mode=ctypes.RTLD_GLOBAL)
        s.fref_compile.restype = c_void_p
        s.fref_compile.argtypes = [c_char_p, c_char_p, c_int, c_int, c_char_p, c_int]
        s.fref_free.argtypes = [c_void_p]
        s.fref_num_io.argtypes = [c_void_p, c_int]
        s.fref_io_spec.argtypes = [c_void_p, c_int, c_int, POINTER(c_int), POINTER(c_int),
                                   POINTER(c_int64), c_int]
        s.fref_run.argtypes = [c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_char_p, c_int]
        s.fref_time_run.restype = c_double
        s.fref_time_run.argtypes = [c_void_p, c_int, c_char_p, c_int]
        s.fref_device_buffer.restype = c_void_p
        s.fref_device_buffer.argtypes = [c_void_p, c_int, c_int]
        s.fref_backward_text.restype = c_int64
        s.fref_backward_text.argtypes = [c_char_p, c_int32, POINTER(c_int32), c_int32, c_char_p, c_int64, c_char_p, c_int]
        s.fref_pipeline_text.restype = c_int64
        s.fref_pipeline_text.argtypes = [c_char_p, c_char_p, c_char_p, c_int64, c_char_p, c_int]
        s.fref_nn_graph_text.restype = c_int64
        s.fref_nn_graph_text.argtypes = [c_char_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int,
                                         c_char_p, c_int, c_char_p, c_int64, c_char_p, c_int]
        s.fref_plan_text.restype = c_int64
        s.fref_plan_text.argtypes = [c_char_p, c_char_p, c_int, c_char_p, c_int64, c_char_p, c_int]
        s.fref_fallback_count.restype = c_int64
        s.fref_fallback_count.argtypes = [c_char_p, c_char_p]
        s.fref_has_kernel.argtypes = [c_char_p, c_char_p]
        s.fref_has_backend.argtypes = [c_char_p]
        s.fref_hal_conformance.argtypes = [c_char_p, c_char_p, c_int]
        _shim = s
    return _shim


class Compiled:
    """A graph compiled by the reference's runtime::compile for one backend."""

    def __init__(self, ir_text: str, backend: str = "cpu", device: int = 0, allow_tf32: bool = False):
        s = load()
        err = create_string_buffer(2048)
        self._h = s.fref_compile(ir_text.encode(), backend.encode(), device, 1 if allow_tf32 else 0,
                                 err, len(err))
        if not self._h:
            raise RuntimeError(f"reference compile failed: {err.value.decode('utf-8', 'replace')}")
        self.backend = backend
        self.inputs = [self._spec(0, i) for i in range(s.fref_num_io(self._h, 0))]
        self.outputs = [self._spec(1, i) for i in range(s.fref_num_io(self._h, 1))]

    def _spec(self, is_out: int, i: int):
        dt, rank = c_int(0), c_int(0)
        dims = (c_int64 * 8)()
        load().fref_io_spec(self._h, is_out, i, byref(dt), byref(rank), dims, 8)
        return dt.value, tuple(dims[j] for j in range(rank.value))

    def run(self, arrays):
        """Host arrays in (numpy, storage dtype: uint16 for bf16/f16), host arrays out."""
        s = load()
        assert len(arrays) == len(self.inputs)
        ins = [np.ascontiguousarray(a) for a in arrays]
        for a, (dt, shape) in zip(ins, self.inputs):
            assert a.size == int(np.prod(shape, dtype=np.int64)), (a.shape, shape)
        outs = [np.empty(shape, dtype=NP_STORAGE[dt]) for dt, shape in self.outputs]
        pin = (c_void_p * max(1, len(ins)))(*[a.ctypes.data for a in ins])
        pout = (c_void_p * max(1, len(outs)))(*[o.ctypes.data for o in outs])
        err = create_string_buffer(2048)
        rc = s.fref_run(self._h, pin, pout, err, len(err))
        if rc != 0:
            raise RuntimeError(f"reference run failed ({rc}): {err.value.decode('utf-8', 'replace')}")
        return outs

    def time_run(self, iters: int) -> float:
        err = create_string_buffer(2048)
        t = load().fref_time_run(self._h, iters, err, len(err))
        if t < 0:
            raise RuntimeError(f"reference timed run failed: {err.value.decode('utf-8', 'replace')}")
        return t

    def close(self):
        if self._h:
            load().fref_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def backward_text(ir_text: str, loss_output_index: int, wrt_input_indices) -> str:
    """IR text of the training graph the reference's build_backward_graph derives: the forward
    outputs followed by the gradients w.r.t. the listed graph inputs."""
    s = load()
    err = create_string_buffer(2048)
    wrt = (c_int32 * len(wrt_input_indices))(*wrt_input_indices)
    n = s.fref_backward_text(ir_text.encode(), loss_output_index, wrt, len(wrt_input_indices), None, 0, err, len(err))
    if n < 0:
        raise RuntimeError(f"build_backward_graph failed: {err.value.decode('utf-8', 'replace')}")
    buf = create_string_buffer(int(n))
    s.fref_backward_text(ir_text.encode(), loss_output_index, wrt, len(wrt_input_indices), buf, n, err, len(err))
    return buf.value.decode()


def pipeline_text(ir_text: str, backend: str = "cpu") -> str:
    """IR text after the reference's nine-pass pipeline."""
    s = load()
    err = create_string_buffer(2048)
    n = s.fref_pipeline_text(ir_text.encode(), backend.encode(), None, 0, err, len(err))
    if n < 0:
        raise RuntimeError(f"pipeline failed: {err.value.decode('utf-8', 'replace')}")
    buf = create_string_buffer(int(n))
    s.fref_pipeline_text(ir_text.encode(), backend.encode(), buf, n, err, len(err))
    return buf.value.decode()


def nn_graph_text(kind: str, batch: int, p1: int, p2: int, p3: int, p4: int = 0, with_bias: bool = True,
                  dtype_code: int = 0, backend: str = "cpu", device: int = 0) -> str:
    """IR text of one of the reference's own nn:: modules (include/frame/nn/layers.h:157-234) as its
    builder emits it: "transformer" (batch, seq, embed, heads, ffn), "mha" (batch, seq, embed, heads),
    "mamba" (batch, steps, channels, kernel).  Input 0 is the activation, the parameters follow."""
    s = load()
    err = create_string_buffer(2048)
    args = (kind.encode(), batch, p1, p2, p3, p4, int(with_bias), dtype_code, backend.encode(), device)
    n = s.fref_nn_graph_text(*args, None, 0, err, len(err))
    if n < 0:
        raise RuntimeError(f"nn graph failed: {err.value.decode('utf-8', 'replace')}")
    buf = create_string_buffer(int(n))
    s.fref_nn_graph_text(*args, buf, n, err, len(err))
    return buf.value.decode()


def plan_text(ir_text: str, backend: str = "cpu", run_pipeline: bool = True) -> str:
    """The executable plan (steps, slots, planner offsets) the reference derives for the graph."""
    s = load()
    err = create_string_buffer(2048)
    n = s.fref_plan_text(ir_text.encode(), backend.encode(), 1 if run_pipeline else 0, None, 0, err,
                         len(err))
    if n < 0:
        raise RuntimeError(f"plan failed: {err.value.decode('utf-8', 'replace')}")
    buf = create_string_buffer(int(n))
    s.fref_plan_text(ir_text.encode(), backend.encode(), 1 if run_pipeline else 0, buf, n, err,
                     len(err))
    return buf.value.decode()


def fallback_count(op: str, backend: str) -> int:
    return int(load().fref_fallback_count(op.encode(), backend.encode()))


def has_kernel(op: str, backend: str) -> bool:
    return bool(load().fref_has_kernel(op.encode(), backend.encode()))


def has_backend(backend: str) -> bool:
    return bool(load().fref_has_backend(backend.encode()))


def hal_conformance(backend: str):
    """(failed cases, report lines) of the HAL contract check on the backend's C++ classes."""
    buf = create_string_buffer(4096)
    failed = int(load().fref_hal_conformance(backend.encode(), buf, len(buf)))
    return failed, buf.value.decode().splitlines()


_plugin = None


def load_b200_backend():
    """Loads this repository's Frame plugin (backend "cuda" + new-op registrations) into the
    reference process.  The plugin's static registrars run at load time."""
    global _plugin
    if _plugin is None:
        load()
        path = os.path.join(os.path.dirname(HERE), "frame_public_b200", "lib", "libframe_b200_hal.so")
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} not built: run frame_public_b200/host/build_adapter.sh")
        _plugin = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    return _plugin
