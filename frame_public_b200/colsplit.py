"""Column-split GEMM across the GPUs of one box with the all-gather of C fused into the GEMM
epilogue: rank j multiplies A by its column block of B and its epilogue stores the block into
every rank's copy of C over NVLink (plain peer stores to buffers mapped with CUDA IPC).  The
process group (any backend; gloo is enough) is used only to exchange the 64-byte IPC handles and
for the barrier that closes the exchange."""
from __future__ import annotations

import ctypes
from ctypes import byref, c_void_p
from typing import List

from . import capi


class PeerMatrix:
    """This rank's copy of a device matrix plus every peer's copy mapped into this process."""

    def __init__(self, nbytes: int, rank: int, world: int, device: int, dist):
        self.rank, self.world, self.device = rank, world, device
        self.lib = capi.load()
        self.local = capi.DeviceBuffer(nbytes, device)
        handle = (ctypes.c_char * 64)()
        capi.check(self.lib.fb200_ipc_export(device, self.local.ptr, handle))
        handles: List[bytes] = [None] * world
        dist.all_gather_object(handles, bytes(handle))
        self.ptrs: List[c_void_p] = []
        self._imported: List[c_void_p] = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(self.local.ptr)
            else:
                p = c_void_p()
                buf = ctypes.create_string_buffer(handles[r], 64)
                capi.check(self.lib.fb200_ipc_import(device, buf, byref(p)))
                self.ptrs.append(p)
                self._imported.append(p)

    def close(self):
        for p in self._imported:
            self.lib.fb200_ipc_close(self.device, p)
        self._imported = []


def matmul_colsplit(a, b_local, c: PeerMatrix, m, n_total, k, dtype, allow_tf32=False, epilogue=None,
                    stream=None):
    """C[:, rank*n_local:(rank+1)*n_local] = epilogue(A . B_local), stored on every rank."""
    n_local = n_total // c.world
    dest = (c_void_p * c.world)(*[p.value for p in c.ptrs])
    ep = byref(epilogue) if epilogue is not None else None
    capi.check(c.lib.fb200_matmul_colsplit(a, b_local, dest, c.world, m, n_local, n_total,
                                           c.rank * n_local, k, dtype, 1 if allow_tf32 else 0, ep, stream))
