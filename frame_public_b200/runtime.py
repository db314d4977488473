"""Python mirror of the compiled-graph executor: a plan (the step list, slots and memory-planner
offsets the reference pipeline emits for a graph) is handed to fb200_plan_create and run through
the C ABI.  Nothing is computed here; without the shared library or a B200 this raises."""
from __future__ import annotations

import os
from ctypes import byref, c_int, c_int64, c_void_p
from typing import List, Sequence

import numpy as np

from . import capi

PLAN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "plans")


def load_plan_text(name: str) -> str:
    path = os.path.join(PLAN_DIR, name + ".plan")
    with open(path) as f:
        return f.read()


def describe_plan(plan_text: str, opt_level: int = 1, allow_tf32: bool = False):
    """(step names, launches per run) of a plan after the executor's rewrites, without touching a
    GPU (fb200_plan_describe): what would run, not a runnable plan."""
    lib = capi.load()
    h = c_void_p()
    capi.check(lib.fb200_plan_describe(plan_text.encode(), 1 if allow_tf32 else 0, opt_level, byref(h)))
    try:
        names = []
        while True:
            name = lib.fb200_plan_step_op(h, len(names)).decode()
            if not name:
                break
            names.append(name)
        return names, int(lib.fb200_plan_launches_per_run(h))
    finally:
        lib.fb200_plan_destroy(h)


def plan_private_bytes(plan_text: str, opt_level: int = 1, allow_tf32: bool = False) -> int:
    """Bytes of private buffers (per stream workspace, beside the arena) the rewrites of a plan
    ask for; no GPU needed."""
    lib = capi.load()
    h = c_void_p()
    capi.check(lib.fb200_plan_describe(plan_text.encode(), 1 if allow_tf32 else 0, opt_level, byref(h)))
    try:
        return int(lib.fb200_plan_private_bytes(h))
    finally:
        lib.fb200_plan_destroy(h)


class CompiledPlan:
    def __init__(self, plan_text: str, device: int = 0, allow_tf32: bool = False, opt_level: int = 1):
        self.lib = capi.load()
        self.device = device
        self._h = c_void_p()
        capi.check(self.lib.fb200_plan_create(plan_text.encode(), device, 1 if allow_tf32 else 0,
                                              opt_level, byref(self._h)))
        self.inputs = [self._spec(0, i) for i in range(self.lib.fb200_plan_num_inputs(self._h))]
        self.outputs = [self._spec(1, i) for i in range(self.lib.fb200_plan_num_outputs(self._h))]

    def _spec(self, is_out, i):
        dt, rank = c_int(0), c_int(0)
        dims = (c_int64 * 8)()
        capi.check(self.lib.fb200_plan_io_spec(self._h, is_out, i, byref(dt), byref(rank), dims))
        return dt.value, tuple(dims[j] for j in range(rank.value))

    @property
    def arena_bytes(self) -> int:
        return int(self.lib.fb200_plan_arena_bytes(self._h))

    @property
    def private_bytes(self) -> int:
        return int(self.lib.fb200_plan_private_bytes(self._h))

    @property
    def launches_per_run(self) -> int:
        return int(self.lib.fb200_plan_launches_per_run(self._h))

    def run_device(self, in_ptrs: Sequence, out_ptrs: Sequence, stream=None) -> None:
        a = (c_void_p * max(1, len(in_ptrs)))(*[p.value if isinstance(p, c_void_p) else p for p in in_ptrs])
        b = (c_void_p * max(1, len(out_ptrs)))(*[p.value if isinstance(p, c_void_p) else p for p in out_ptrs])
        capi.check(self.lib.fb200_plan_run(self._h, a, b, stream))

    def run_host_ptrs(self, in_ptrs: Sequence[int], out_ptrs: Sequence[int], stream=None) -> None:
        a = (c_void_p * max(1, len(in_ptrs)))(*in_ptrs)
        b = (c_void_p * max(1, len(out_ptrs)))(*out_ptrs)
        capi.check(self.lib.fb200_plan_run_host(self._h, a, b, stream))

    def run_host_async_ptrs(self, in_ptrs: Sequence[int], out_ptrs: Sequence[int], stream=None) -> None:
        """Queues one pipelined run (copy-in, run, copy-out on three streams, two staging sets); the
        host outputs are valid after host_sync()."""
        a = (c_void_p * max(1, len(in_ptrs)))(*in_ptrs)
        b = (c_void_p * max(1, len(out_ptrs)))(*out_ptrs)
        capi.check(self.lib.fb200_plan_run_host_async(self._h, a, b, stream))

    def bind_resident(self, index: int, device_ptr) -> None:
        """Input `index` is a parameter that already lives on the device: the host-buffer entry points
        read it in place instead of copying it in."""
        capi.check(self.lib.fb200_plan_bind_resident(self._h, index, device_ptr))

    def host_sync(self) -> None:
        capi.check(self.lib.fb200_plan_host_sync(self._h))

    def run_host(self, arrays: Sequence[np.ndarray], stream=None) -> List[np.ndarray]:
        ins = [np.ascontiguousarray(a) for a in arrays]
        assert len(ins) == len(self.inputs)
        for a, (dt, shape) in zip(ins, self.inputs):
            assert a.nbytes == int(np.prod(shape, dtype=np.int64)) * capi.ITEMSIZE[dt], (a.shape, shape)
        outs = [np.empty(shape, dtype=capi.NP_STORAGE[dt]) for dt, shape in self.outputs]
        self.run_host_ptrs([a.ctypes.data for a in ins], [o.ctypes.data for o in outs], stream)
        return outs

    def profile(self, in_ptrs: Sequence, out_ptrs: Sequence, stream=None):
        """[(op name, milliseconds)] per step of one eager run."""
        from ctypes import c_float
        a = (c_void_p * max(1, len(in_ptrs)))(*[p.value if isinstance(p, c_void_p) else p for p in in_ptrs])
        b = (c_void_p * max(1, len(out_ptrs)))(*[p.value if isinstance(p, c_void_p) else p for p in out_ptrs])
        ms = (c_float * 4096)()
        n = c_int(0)
        capi.check(self.lib.fb200_plan_profile(self._h, a, b, stream, ms, 4096, byref(n)))
        return [(self.lib.fb200_plan_step_op(self._h, i).decode(), float(ms[i])) for i in range(n.value)]

    def step_names(self) -> List[str]:
        """Op name of every step as the executor will run it ("(absorbed)" for a step folded into
        another launch, "(alias)" for a reshape that became a view)."""
        names = []
        while True:
            name = self.lib.fb200_plan_step_op(self._h, len(names)).decode()
            if not name:
                return names
            names.append(name)

    def close(self):
        if self._h:
            self.lib.fb200_plan_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
