"""Host-side multi-GPU plumbing: one process per GPU, independent shards, no data-path collective.

Every op of the compiled-graph path is row/sample independent, so N GPUs run N independent
executables on contiguous batch ranges (or, for the weak-scaling benchmark, one full batch each).
torch.distributed is used only for the rendezvous, barriers and the max-over-ranks of a timing."""
from __future__ import annotations

import os
from typing import Tuple


def env_rank() -> Tuple[int, int, int]:
    """(rank, local_rank, world_size) from the torchrun environment; (0, 0, 1) when absent."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [begin, end) of `total` units owned by `rank`; the first total % world ranks get
    one unit more, every unit is owned exactly once."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def init_process_group(backend: str, local_rank: int):
    """Initialises torch.distributed from the MASTER_* environment (127.0.0.1 rendezvous)."""
    import torch.distributed as dist
    if dist.is_initialized():
        return dist
    if backend == "nccl":
        import torch
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        dist.init_process_group(backend)
    return dist


def max_over_ranks(value: float, dist=None, device: str = "cpu") -> float:
    """The slowest rank's figure: what a multi-GPU timing reports."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, dist=None, device: str = "cpu") -> float:
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())
