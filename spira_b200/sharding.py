"""Multi-GPU sharding of the hot path: independent scenes, one process per GPU, nothing exchanged on the data path.

A scene's keys, kernel maps and activations never interact with another scene's (the reference has no batch
dimension at all: ``csrc/spira/cuda/kernels/compress.cuh:17-22`` packs ``[N,3]`` coordinates without a batch
column), so scene ``i`` simply goes to rank ``i mod world_size``.  The only collective is the max-reduction of the
per-rank elapsed time that turns local timings into a whole-job throughput; it runs after the timed region.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


def assign_scenes(n_scenes: int, world_size: int, rank: int) -> List[int]:
    """Indices of the scenes rank ``rank`` processes (round robin)."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    return list(range(rank, n_scenes, world_size))


def max_over_ranks(value: float, device: Optional[torch.device] = None) -> float:
    """The slowest rank's value; identity when no process group is initialised."""
    if not (torch.distributed.is_available() and torch.distributed.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def all_ranks(value: float, device: Optional[torch.device] = None) -> list:
    """The value of every rank, in rank order (a one-element list without a process group)."""
    if not (torch.distributed.is_available() and torch.distributed.is_initialized()):
        return [float(value)]
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    out = [torch.zeros_like(t) for _ in range(torch.distributed.get_world_size())]
    torch.distributed.all_gather(out, t)
    return [float(v.item()) for v in out]


def job_throughput(local_ms: float, scenes_per_rank: Sequence[int], device: Optional[torch.device] = None) -> float:
    """Whole-job scenes/s: all ranks' scenes divided by the slowest rank's time."""
    worst = max_over_ranks(local_ms, device)
    return sum(scenes_per_rank) / (worst / 1e3) if worst > 0 else float("inf")
