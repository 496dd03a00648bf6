"""Multi-GPU plumbing: one process per GPU, requests sharded by rank, no collective on the data path.

Requests share nothing (the reference serves one at a time, README.md:215-216), so scaling out is a
partition of the request list plus two tiny host-side collectives that are NOT part of the forward:
the max over ranks of a timing, and the gather of the per-request logits on rank 0. Both run on
whatever backend the process group was created with (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import os

import numpy as np
import torch
import torch.distributed as dist


def env_rank() -> tuple[int, int, int]:
    """(rank, local_rank, world_size) from the launcher's environment; (0, 0, 1) when not launched."""
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def shard(n_items: int, world: int, rank: int) -> range:
    """Contiguous block of items owned by `rank`: sizes differ by at most one, earlier ranks get the extras."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def max_over_ranks(value: float, device=None) -> float:
    """The slowest rank's value; the identity without a process group."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_rows(local: np.ndarray, device=None) -> np.ndarray | None:
    """Concatenates every rank's rows (in rank order) on rank 0; other ranks get None. Row counts may differ."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    world, rank = dist.get_world_size(), dist.get_rank()
    counts = torch.zeros(world, dtype=torch.int64, device=device)
    counts[rank] = local.shape[0]
    dist.all_reduce(counts)
    width = local.shape[1]
    padded = torch.zeros(int(counts.max()), width, dtype=torch.float32, device=device)
    padded[:local.shape[0]] = torch.from_numpy(np.ascontiguousarray(local, dtype=np.float32)).to(padded.device)
    parts = [torch.zeros_like(padded) for _ in range(world)] if rank == 0 else None
    dist.gather(padded, parts, dst=0)
    if rank != 0:
        return None
    return np.concatenate([p[:int(c)].cpu().numpy() for p, c in zip(parts, counts)], axis=0)
