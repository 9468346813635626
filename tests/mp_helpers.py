"""Picklable helpers for the multi-process tests (spawned workers import this module)."""

import os
import queue
import time

import torch


def raises_injected_cuda_error(x):
    raise RuntimeError("CUDA error: injected by the test (no GPU involved)")


def raises_plain_error(x):
    raise ValueError("plain failure injected by the test")


def hard_exit(x):
    os._exit(17)  # the process vanishes without posting anything


def doubled_relu(x):
    return torch.relu(x) * 2


def gloo_shard_worker(rank, world, port, out_dir):
    """One rank of the CPU stand-in for `bench.py --gpus N`: shard the cases, barrier,
    'time' the local shard and take the max over ranks -- the same plumbing bench.py uses."""
    import json

    import torch.distributed as dist

    from backendbench_b200.cases import sweep_cases
    from backendbench_b200.sharding import max_over_ranks, shard_for_rank, sum_over_ranks

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cases = sweep_cases(32, seed=0, max_log2=12)
    mine = shard_for_rank(cases, rank, world, mode="weak")
    strong = shard_for_rank(cases, rank, world, mode="strong")
    dist.barrier()
    local_ms = 10.0 * (rank + 1)
    worst = max_over_ranks(local_ms)
    total = sum_over_ranks(len(mine))
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as fh:
        json.dump({"rank": rank, "n_weak": len(mine), "strong_ids": [c.case_id for c in strong], "weak_seeds": [c.seed for c in mine][:4], "max_ms": worst, "total_units": total}, fh)
    dist.barrier()
    dist.destroy_process_group()


def worker_one_dies_idle(worker_id, task_queue, result_queue):
    """Worker target for the liveness test: worker 1 vanishes before it ever takes a task
    (a crash during start-up); every other worker is the ordinary loop."""
    if worker_id == 1:
        os._exit(23)
    from backendbench_b200.multiprocessing_eval import _worker_process

    _worker_process(worker_id, task_queue, result_queue)
