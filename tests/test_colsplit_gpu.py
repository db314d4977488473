"""Column-split GEMM with the all-gather fused into the epilogue, on 2 GPUs (skipped on a 1-GPU
box): two child processes, one GPU each, gloo for the handle exchange and the barrier; every rank
must end up with the whole C = GELU(A.B + bias), equal to the CPU oracle within the bf16 tier."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest

from frame_public_b200 import capi

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    import numpy as np
    import torch.distributed as dist
    from frame_public_b200 import capi, colsplit
    from oracle import frame_oracle as fo
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    m, k, n = 384, 256, 1024
    rng = np.random.default_rng(5)
    a = fo.from_accum(rng.uniform(-1, 1, (m, k)).astype(np.float32), fo.DT_BF16)
    b = fo.from_accum(rng.uniform(-1, 1, (k, n)).astype(np.float32), fo.DT_BF16)
    bias = fo.from_accum(np.tile(rng.normal(0, 0.1, (1, n)).astype(np.float32), (m, 1)), fo.DT_BF16)
    nl = n // world
    cols = slice(rank * nl, (rank + 1) * nl)
    da = capi.DeviceBuffer.from_numpy(a, rank)
    db = capi.DeviceBuffer.from_numpy(np.ascontiguousarray(b[:, cols]), rank)
    dbias = capi.DeviceBuffer.from_numpy(np.ascontiguousarray(bias[:, cols]), rank)
    c = colsplit.PeerMatrix(m * n * 2, rank, world, rank, dist)
    capi.check(capi.load().fb200_memset(rank, c.local.ptr, 0, m * n * 2, None))
    capi.synchronize(rank)
    dist.barrier()
    epi = capi.make_epilogue([("add", dbias.ptr, capi.OPERAND_FULL), ("gelu", None, 0)])
    colsplit.matmul_colsplit(da.ptr, db.ptr, c, m, n, k, capi.BF16, False, epi)
    capi.synchronize(rank)
    dist.barrier()
    assert capi.kernel_status(rank) == 0
    got = c.local.download(np.uint16, (m, n))
    exp = fo.gelu(fo.add(fo.matmul(a, b, fo.DT_BF16), bias, fo.DT_BF16), fo.DT_BF16)
    assert fo.all_close(got, exp, fo.DT_BF16, rtol=2e-2, atol=2e-2), fo.max_err(got, exp, fo.DT_BF16)
    dist.barrier()
    c.close()
    dist.destroy_process_group()
    print("rank", rank, "colsplit ok")
""" % ROOT)


def test_colsplit_gemm_allgather_two_gpus():
    if capi.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, "-c", CHILD], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out[-3000:]
        assert f"rank {rank} colsplit ok" in out
