"""Sharding of independent cases across ranks and the two tiny reductions the benchmark
needs. The sweep has no data-path collective: ranks share nothing, so the only
communication is a barrier around the timed region, the max of the per-rank times and
the sum of the per-rank unit counts (`torch.distributed`, NCCL on GPUs, gloo on CPU)."""

from __future__ import annotations

from dataclasses import replace
from typing import List, Sequence

import torch


def shard_for_rank(cases: Sequence, rank: int, world: int, mode: str = "weak") -> List:
    """weak: every rank gets a full-size sweep of its own (same shapes, rank-specific
    seeds), so per-GPU work is fixed as the world grows. strong: the one sweep is dealt
    round-robin after sorting by cost, so each rank gets a similar mix of large and small."""
    if mode == "weak":
        return [replace(c, seed=c.seed + 7919 * rank) for c in cases]
    if mode == "strong":
        order = sorted(cases, key=lambda c: -(c.algorithmic_bytes() + c.flops() // 200))
        return order[rank::world]
    raise ValueError(mode)


def _dist_ready() -> bool:
    return torch.distributed.is_available() and torch.distributed.is_initialized()


def _reduce(value: float, op) -> float:
    if not _dist_ready():
        return value
    dev = "cuda" if torch.distributed.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    torch.distributed.all_reduce(t, op=op)
    return float(t.item())


def max_over_ranks(value: float) -> float:
    return _reduce(value, torch.distributed.ReduceOp.MAX) if _dist_ready() else value


def sum_over_ranks(value: float) -> float:
    return _reduce(value, torch.distributed.ReduceOp.SUM) if _dist_ready() else value


def barrier() -> None:
    if _dist_ready():
        torch.distributed.barrier()
