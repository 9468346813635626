"""Sharding of independent cases across ranks and the two tiny reductions the benchmark
needs. The sweep has no data-path collective: ranks share nothing, so the only
communication is a barrier around the timed region, the max of the per-rank times and
the sum of the per-rank unit counts (`torch.distributed`, NCCL on GPUs, gloo on CPU)."""

from __future__ import annotations

from dataclasses import replace
from typing import List, Sequence

import torch


# What a case costs is estimated from the two roofs of the part (HBM stream rate, dense
# bf16 tensor rate; fp32 products are charged the six bf16 plane products they become).
COST_HBM_GBS = 6500.0
COST_BF16_TFLOPS = 1400.0


def estimated_seconds(case, hbm_gbs: float = COST_HBM_GBS, bf16_tflops: float = COST_BF16_TFLOPS) -> float:
    """Lower bound of one launch of `case`: max(algorithmic bytes / HBM rate, FLOP / tensor rate)."""
    flops = case.flops() * (6 if getattr(case, "dtype", "") == "f32" else 1)
    return max(case.algorithmic_bytes() / (hbm_gbs * 1e9), flops / (bf16_tflops * 1e12))


def lpt_order(cases: Sequence) -> List:
    """Longest processing time first: with one shared queue and N workers, handing out the
    costly cases first leaves only small ones for the end, so the workers finish together
    (list scheduling's 4/3 bound). Ties keep the original order."""
    return sorted(cases, key=lambda c: -estimated_seconds(c))


def shard_for_rank(cases: Sequence, rank: int, world: int, mode: str = "weak") -> List:
    """weak: every rank gets a full-size sweep of its own (same shapes, rank-specific
    seeds), so per-GPU work is fixed as the world grows. strong: the one sweep is dealt
    round-robin in longest-first order, so each rank gets a similar mix of large and small."""
    if mode == "weak":
        return [replace(c, seed=c.seed + 7919 * rank) for c in cases]
    if mode == "strong":
        return lpt_order(cases)[rank::world]
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
