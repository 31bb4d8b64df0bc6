"""Multi-GPU plumbing of the sequence-sharded operator: who owns which sequences, and the
reductions a benchmark or a serving loop needs around it.  The data path itself never
communicates: every sequence (batch row) is independent for prefill and every (sequence,
channel) state row for decode, so a rank only ever touches its own slice.

Backend-neutral (NCCL on GPUs, gloo on CPUs): nothing here calls into the CUDA library.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def shard_range(batch: int, rank: int, world: int) -> range:
    """Contiguous slice of ``range(batch)`` owned by ``rank``: equal counts, the first
    ``batch % world`` ranks take one extra sequence."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(batch, world)
    start = rank * base + min(rank, rem)
    return range(start, start + base + (1 if rank < rem else 0))


def shard_by_cost(costs: Sequence[float], world: int) -> List[List[int]]:
    """Assign sequences to ranks by descending cost, each to the currently lightest rank
    (longest-processing-time rule).  Use when masked rows are skipped, so that a sequence's
    cost follows its valid length rather than the padded length."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads = [0.0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (loads[k], k))
        out[r].append(i)
        loads[r] += costs[i]
    for rows in out:
        rows.sort()
    return out


def _active(group) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def max_over_ranks(value: float, device: Optional[torch.device] = None, group=None) -> float:
    """Slowest rank's value: the time that counts for a sharded step."""
    if not _active(group):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def sum_over_ranks(value: float, device: Optional[torch.device] = None, group=None) -> float:
    if not _active(group):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return float(t.item())


def barrier(device: Optional[torch.device] = None, group=None) -> None:
    """Host-side rendezvous bracketing a timed region, with the device drained on both sides."""
    if device is not None and device.type == "cuda":
        torch.cuda.synchronize(device)
    if _active(group):
        dist.barrier(group=group)
    if device is not None and device.type == "cuda":
        torch.cuda.synchronize(device)


def aggregate_throughput(units_this_rank: float, seconds_this_rank: float, device=None, group=None) -> float:
    """Whole-job throughput of a sharded step: all units over the slowest rank's time."""
    total = sum_over_ranks(units_this_rank, device, group)
    slowest = max_over_ranks(seconds_this_rank, device, group)
    return total / slowest if slowest > 0 else float("inf")
