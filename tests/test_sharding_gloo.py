"""Multi-process host logic on CPU (gloo, world_size 2): shard ownership, barrier, max/sum over
ranks — the plumbing bench.py uses around the timed region when launched with torchrun."""
import os
import socket
import subprocess
import sys
import textwrap

from frame_public_b200 import sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges_partition_every_unit_once():
    for total in (0, 1, 7, 16, 32768):
        for world in (1, 2, 3, 4, 8):
            owned = []
            for r in range(world):
                b, e = sharding.shard_range(total, r, world)
                assert 0 <= b <= e <= total
                owned.extend(range(b, e))
            assert owned == list(range(total))
            sizes = [sharding.shard_range(total, r, world) for r in range(world)]
            assert max(e - b for b, e in sizes) - min(e - b for b, e in sizes) <= 1


def test_gloo_world_of_two_reduces_max_and_sum():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = textwrap.dedent("""
        import os, sys
        sys.path.insert(0, %r)
        from frame_public_b200 import sharding
        rank, local, world = sharding.env_rank()
        dist = sharding.init_process_group("gloo", local)
        dist.barrier()
        b, e = sharding.shard_range(17, rank, world)
        mx = sharding.max_over_ranks(10.0 + rank, dist)
        sm = sharding.sum_over_ranks(e - b, dist)
        assert mx == 11.0 and sm == 17.0, (mx, sm)
        dist.barrier()
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """ % ROOT)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-c", script], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out
        assert f"rank {rank} ok" in out
