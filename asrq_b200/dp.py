"""Data-parallel plumbing: one process per GPU, no collective on the data path.

Utterances (rows of a batch) are independent and the packed weights are read-only, so
the quantized-linear path shards by giving each rank a contiguous slice of the rows and
a full replica of the weights.  The only communication is control-plane: a barrier
around timed regions and a MAX-reduce of the per-rank device time.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def env_world():
    """(rank, local_rank, world_size) from the torchrun environment; (0, 0, 1) outside it."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def init(backend: str | None = None) -> tuple[int, int, int]:
    """Joins the process group when launched under torchrun.  ``backend`` defaults to nccl on
    CUDA machines and gloo elsewhere."""
    rank, local_rank, world = env_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, local_rank, world


def shard_range(n_items: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of the rows rank ``rank`` owns: contiguous, sizes differ by at most one,
    earlier ranks take the remainder."""
    if not 0 <= rank < world:
        raise ValueError("rank outside [0, world)")
    base, rem = divmod(n_items, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(value: float, device=None) -> float:
    """MAX-reduce of a host float (the per-rank device time of a timed region)."""
    if not dist.is_initialized():
        return float(value)
    dev = device if device is not None else ("cuda" if dist.get_backend() == "nccl" else "cpu")
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device=None) -> float:
    if not dist.is_initialized():
        return float(value)
    dev = device if device is not None else ("cuda" if dist.get_backend() == "nccl" else "cpu")
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def finalize() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
