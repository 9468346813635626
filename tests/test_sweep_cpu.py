"""The process-per-GPU evaluator and the rank sharding, exercised on CPU: two spawned
workers, failures injected on the host only (an exception whose text says CUDA, a worker
that exits hard), and a world_size-2 gloo run of the benchmark's sharding plumbing."""

import json
import socket

import pytest
import torch
import torch.multiprocessing as tmp

import mp_helpers
from backendbench_b200.backends import AtenBackend
from backendbench_b200.cases import sweep_cases
from backendbench_b200.multiprocessing_eval import BackendRef, EvalResult, MultiprocessingEvaluator, SpecTest, is_pickleable
from backendbench_b200.opregistry import get_operator
from backendbench_b200.sharding import shard_for_rank
from backendbench_b200.suite import make_smoke_suite

RELU = torch.ops.aten.relu.default


class Case:
    def __init__(self, args, kwargs):
        self.args, self.kwargs = args, kwargs


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_workers_evaluate_smoke_and_descriptor_tasks():
    be = AtenBackend()
    small = [c for c in sweep_cases(64, seed=0, max_log2=14) if c.flops() < 1e8][:8]
    with MultiprocessingEvaluator(2, backend=BackendRef("aten")) as ev:
        for t in make_smoke_suite("cpu"):
            ev.submit_task(t.op, be[t.op], t.correctness_tests, t.performance_tests)
        for c in small:
            ev.submit_task(c.op, BackendRef("aten"), [SpecTest(c, "cpu")], [])
        ev.start_evaluation()
        results = ev.get_results()
    assert [r.task_id for r in results] == list(range(1 + len(small)))  # sorted by task id
    assert all(isinstance(r, EvalResult) and r.correctness_score == 1.0 and r.error is None for r in results)
    assert results[0].performance_score > 0
    assert {r.worker_id for r in results} <= {0, 1}


def test_unpicklable_op_travels_as_spec_name():
    assert not is_pickleable(lambda x: x)
    with MultiprocessingEvaluator(1) as ev:
        ev.submit_task(RELU, mp_helpers.doubled_relu, [Case([torch.tensor([-1.0, 2.0])], {})], [])
        ev.start_evaluation()
        (r,) = ev.get_results()
    assert r.correctness_score == 0.0 and r.correctness_results[0].op_name == "relu.default"
    assert r.correctness_results[0].max_abs_error == pytest.approx(2.0)


def test_cuda_error_escaping_eval_kills_worker_and_it_is_restarted():
    """An error whose text says CUDA and that escapes eval_one_op (here: raised while the
    REFERENCE result is computed, outside the per-case try) makes the worker post a death
    signal and exit; the parent restarts it and the fatal task yields no result
    (BackendBench/multiprocessing_eval.py:130-138, :336-341). Injected on the host."""
    with MultiprocessingEvaluator(1) as ev:
        ev.submit_task(mp_helpers.raises_injected_cuda_error, RELU, [Case([torch.tensor([1.0])], {})], [])
        ev.submit_task(RELU, RELU, [Case([torch.tensor([1.0])], {})], [])
        ev.start_evaluation()
        results = ev.get_results()
        restarts = ev.restarts
    assert [r.task_id for r in results] == [1] and results[0].correctness_score == 1.0 and restarts == 1


def test_cuda_error_inside_impl_is_a_failed_case_not_a_dead_worker():
    with MultiprocessingEvaluator(1) as ev:
        ev.submit_task(RELU, mp_helpers.raises_injected_cuda_error, [Case([torch.tensor([1.0])], {})], [])
        ev.submit_task(RELU, RELU, [Case([torch.tensor([1.0])], {})], [])
        ev.start_evaluation()
        results = ev.get_results()
        restarts = ev.restarts
    # eval_one_op catches the exception per test, so the worker survives and reports a failed case
    assert len(results) == 2 and results[0].correctness_score == 0.0 and results[1].correctness_score == 1.0
    assert "injected" in results[0].correctness_results[0].error_msg and restarts == 0


def test_plain_exception_is_recorded_not_fatal():
    with MultiprocessingEvaluator(1) as ev:
        ev.submit_task(RELU, mp_helpers.raises_plain_error, [Case([torch.tensor([1.0])], {})], [])
        ev.start_evaluation()
        (r,) = ev.get_results()
    assert r.correctness_score == 0.0 and "plain failure" in r.correctness_results[0].error_msg


def test_hard_worker_exit_does_not_stall_and_loses_only_its_task():
    """A worker that disappears (os._exit) posts nothing; the reference would spin forever in
    get_results. Here the liveness check accounts for the lost task and restarts the worker."""
    with MultiprocessingEvaluator(1) as ev:
        ev.submit_task(RELU, mp_helpers.hard_exit, [Case([torch.tensor([1.0])], {})], [])
        ev.submit_task(RELU, RELU, [Case([torch.tensor([-1.0, 1.0])], {})], [])
        ev.start_evaluation()
        results = ev.get_results()
        restarts = ev.restarts
    assert [r.task_id for r in results] == [1] and results[0].correctness_score == 1.0
    assert restarts >= 1


def test_shard_for_rank_weak_and_strong():
    cases = sweep_cases(32, seed=0, max_log2=12)
    w0, w1 = shard_for_rank(cases, 0, 2, "weak"), shard_for_rank(cases, 1, 2, "weak")
    assert len(w0) == len(w1) == 32 and [c.shape for c in w0] == [c.shape for c in w1]
    assert all(a.seed != b.seed for a, b in zip(w0, w1))
    s0, s1 = shard_for_rank(cases, 0, 2, "strong"), shard_for_rank(cases, 1, 2, "strong")
    assert sorted(c.case_id for c in s0 + s1) == list(range(32)) and abs(len(s0) - len(s1)) <= 1


def test_gloo_world_size_two_sharding_and_reductions(tmp_path):
    port = _free_port()
    tmp.spawn(mp_helpers.gloo_shard_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = json.load(open(tmp_path / "rank0.json"))
    r1 = json.load(open(tmp_path / "rank1.json"))
    assert r0["max_ms"] == r1["max_ms"] == 20.0  # the slower rank's time, on both
    assert r0["total_units"] == r1["total_units"] == 64.0  # units all ranks processed
    assert r0["n_weak"] == r1["n_weak"] == 32 and r0["weak_seeds"] != r1["weak_seeds"]
    assert sorted(r0["strong_ids"] + r1["strong_ids"]) == list(range(32))


def test_worker_that_dies_idle_costs_no_task():
    """Only a worker that HELD a task takes one with it. Worker 1 exits during start-up,
    over and over (it is restarted while tasks remain); every task must still be answered
    by worker 0 and none may be booked as lost."""
    with MultiprocessingEvaluator(2, worker_target=mp_helpers.worker_one_dies_idle) as ev:
        for v in (1.0, 2.0, 3.0, 4.0):
            ev.submit_task(RELU, RELU, [Case([torch.tensor([-v, v])], {})], [])
        ev.start_evaluation()
        results = ev.get_results()
        lost, restarts = list(ev.lost_tasks), ev.restarts
    assert [r.task_id for r in results] == [0, 1, 2, 3] and all(r.correctness_score == 1.0 for r in results)
    assert lost == [] and restarts >= 0  # (restarted only if the parent looked while tasks were still open)
    assert {r.worker_id for r in results} == {0}


def test_fatal_task_is_booked_once_and_timeline_reports_the_run():
    with MultiprocessingEvaluator(1) as ev:
        ev.submit_task(mp_helpers.raises_injected_cuda_error, RELU, [Case([torch.tensor([1.0])], {})], [])
        for v in (1.0, 2.0, 3.0):
            ev.submit_task(RELU, RELU, [Case([torch.tensor([-v, v])], {})], [])
        ev.start_evaluation()
        results = ev.get_results()
        assert ev.lost_tasks == [0] and ev.restarts == 1 and ev.completed_tasks == ev.total_tasks == 4
        # a second batch on the same (restarted) worker: get_results can be called again
        ev.submit_task(RELU, RELU, [Case([torch.tensor([5.0])], {})], [])
        more = ev.get_results()
        tl = ev.timeline()
    assert [r.task_id for r in results] == [1, 2, 3] and [r.task_id for r in more] == [4]
    assert tl["results"] == 4 and tl["lost_tasks"] == [0] and tl["wall_s"] > 0 and tl["per_worker_tasks"] == {0: 4}
    assert tl["first_worker_ready_s"] is not None and tl["worker_startup_s"][0] > 0


def test_sweep_tasks_are_per_case_and_longest_first():
    from backendbench_b200.backends import AtenBackend as Aten
    from backendbench_b200.scripts.main import build_suite, task_units
    from backendbench_b200.sharding import estimated_seconds, lpt_order

    cases = sweep_cases(64, seed=0)
    order = lpt_order(cases)
    costs = [estimated_seconds(c) for c in order]
    assert costs == sorted(costs, reverse=True) and sorted(c.case_id for c in order) == list(range(64))
    units = task_units(build_suite("sweep", "cpu", None, 64), Aten())
    assert sum(len(c) for _, c, _ in units) == 64 and all(len(c) <= 1 for _, c, _ in units)  # one case per task
    untimed = [estimated_seconds(c[0].spec) for _, c, q in units if c and not q]
    assert untimed == sorted(untimed, reverse=True)
