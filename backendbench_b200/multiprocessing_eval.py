"""Process-per-GPU evaluation of independent tasks (no collective: tasks share nothing).

Same interface as BackendBench/multiprocessing_eval.py:36-395 --
`MultiprocessingEvaluator(num_workers)`, `submit_task(op, impl, correctness_tests,
performance_tests)`, `start_evaluation()`, `get_results()`, `shutdown()`, context
manager; worker *i* owns GPU *i* (`torch.cuda.set_device(i)`, :82); a worker that hits
a CUDA error posts a `ProcessDeathSignal` and is restarted on the same GPU (:130-138,
:299-318), and the task that killed it yields no result (:336-341).

What is different, because the machine is 8 GPUs with 180 GB each rather than one T4:

* Tasks may carry `CaseSpec` descriptors instead of tensors. The worker generates the
  inputs on its own GPU from the seed, so nothing is pickled through a pipe and nothing
  crosses PCIe; tensor-carrying tests still work (moved to the CPU for the queue and
  back on the worker, as the reference does at :256-271 and :107-112).
* Implementations travel as `(backend name, ops directory)` plus the operator's spec
  name and are re-loaded in the worker. (Functions loaded from a kernel directory do not
  pickle; the reference then ships the operator's own name and ends up evaluating aten
  against aten, :246-249.)
* Queues block with a timeout instead of 0.1 s sleep-polling, the parent watches
  `Process.is_alive()` so a hard crash (segfault, SIGKILL, `os._exit`) cannot stall
  `get_results` forever, and a per-task wall-clock limit bounds a wedged worker.
"""

from __future__ import annotations

import logging
import multiprocessing as mp
import os
import queue
import time
import traceback
from dataclasses import dataclass, field
from typing import Any, List, Optional, Tuple

import torch

from .eval import CorrectnessTestResult, PerformanceTestResult, eval_one_op
from .opregistry import _extract_spec_name_from_op, get_operator

logger = logging.getLogger(__name__)


@dataclass
class EvalTask:
    task_id: int
    op: Any
    impl: Any
    correctness_tests: List[Any]
    performance_tests: List[Any]
    device: str
    tolerances: Any = None


@dataclass
class EvalResult:
    task_id: int
    correctness_score: float
    performance_score: float
    correctness_results: List[CorrectnessTestResult]
    performance_results: List[PerformanceTestResult]
    error: Optional[str] = None
    worker_id: int = -1
    seconds: float = 0.0


@dataclass
class ProcessDeathSignal:
    worker_id: int
    error_msg: str
    task_id: int = -1


@dataclass(frozen=True)
class BackendRef:
    """How a worker rebuilds the implementation table: `make_backend(name, ops_directory)`."""

    name: str
    ops_directory: Optional[str] = None


class SpecTest:
    """A test whose arguments are generated from a `CaseSpec` on first use, on `device`."""

    def __init__(self, spec, device="cuda", gen_device=None):
        self.spec, self.device, self.gen_device = spec, device, gen_device
        self._built = None

    def _build(self):
        if self._built is None:
            self._built = self.spec.build(self.device, self.gen_device)
        return self._built

    @property
    def args(self):
        return self._build()[0]

    @property
    def kwargs(self):
        return self._build()[1]

    def __getstate__(self):  # tensors never travel
        return {"spec": self.spec, "device": self.device, "gen_device": self.gen_device, "_built": None}


def is_pickleable(obj) -> bool:
    import io
    import pickle

    try:
        pickle.dump(obj, io.BytesIO())
        return True
    except Exception:
        return False


def args_to_device(value, device):
    if isinstance(value, torch.Tensor):
        return value.to(device)
    if isinstance(value, list):
        return [args_to_device(v, device) for v in value]
    if isinstance(value, tuple):
        return tuple(args_to_device(v, device) for v in value)
    if isinstance(value, dict):
        return {k: args_to_device(v, device) for k, v in value.items()}
    return value


def find_device(test):
    """Device of the first tensor found in a test's args (None when it has no tensors)."""
    if isinstance(test, torch.Tensor):
        return test.device
    if isinstance(test, (list, tuple)):
        for item in test:
            d = find_device(item)
            if d is not None:
                return d
    if isinstance(test, dict):
        return find_device(list(test.values()))
    if hasattr(test, "args") and not isinstance(test, SpecTest):
        return find_device(test.args)
    return None


class _MaterialisedTest:
    """Plain (args, kwargs) holder: what a thunk-based test becomes before it is queued."""

    def __init__(self, args, kwargs):
        self.args, self.kwargs = args, kwargs


def test_to_device(test, device):
    if isinstance(test, SpecTest):  # nothing to move: the tensors do not exist yet
        return SpecTest(test.spec, str(device), test.gen_device)
    return _MaterialisedTest(args_to_device(test.args, device), args_to_device(test.kwargs, device))


test_to_device.__test__ = False  # not a pytest test despite the name


def _worker_device(worker_id: int) -> str:
    if torch.cuda.is_available():
        torch.cuda.set_device(worker_id)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        return f"cuda:{worker_id}"
    return "cpu"


def _resolve_impl(impl, op, backends_cache):
    if isinstance(impl, BackendRef):
        from .backends import make_backend

        be = backends_cache.get(impl)
        if be is None:
            be = backends_cache[impl] = make_backend(impl.name, impl.ops_directory)
        return be[op]
    if isinstance(impl, str):
        return get_operator(impl)
    return impl


def _worker_process(worker_id, task_queue, result_queue, poll_s=0.5):
    backends_cache = {}
    try:
        own_device = _worker_device(worker_id)
        while True:
            try:
                task = task_queue.get(timeout=poll_s)
            except queue.Empty:
                continue
            if task is None:
                logger.info(f"Worker {worker_id} received shutdown signal")
                break
            t0 = time.perf_counter()
            op = task.op
            try:
                if isinstance(op, str):
                    op = get_operator(op)
                impl = _resolve_impl(task.impl, op, backends_cache)
                device = own_device if (task.device.startswith("cuda") and own_device != "cpu") else task.device
                if device.startswith("cuda") and own_device == "cpu":
                    device = "cpu"
                ctests = (test_to_device(t, torch.device(device)) for t in task.correctness_tests)
                ptests = (test_to_device(t, torch.device(device)) for t in task.performance_tests)
                cs, ps, cr, pr = eval_one_op(op, impl, ctests, ptests, task.tolerances)
                if device.startswith("cuda"):
                    from .ops import check_device_status

                    check_device_status(torch.device(device))
                result = EvalResult(task.task_id, float(cs), float(ps), cr, pr, None, worker_id, time.perf_counter() - t0)
            except Exception as e:
                msg = f"Error in eval_one_op: {e}\n{traceback.format_exc()}"
                logger.warning(f"Worker {worker_id} task {task.task_id} failed: {msg}")
                if "cuda" in str(e).lower():
                    # a CUDA error may have poisoned the context: die and let the parent restart us
                    result_queue.put(ProcessDeathSignal(worker_id, f"Worker {worker_id} CUDA error: {msg}", task.task_id))
                    break
                name = getattr(op, "__name__", str(op))
                result = EvalResult(
                    task.task_id, 0.0, 1.0,
                    [CorrectnessTestResult(op_name=name, args="", is_correct=False, error_msg=msg) for _ in task.correctness_tests],
                    [PerformanceTestResult(op_name=name, args="", speedup=None, benchmark_time_ms=None, reference_time_ms=None, error_msg=msg) for _ in task.performance_tests],
                    msg, worker_id, time.perf_counter() - t0,
                )
            result_queue.put(result)
    except Exception as e:
        result_queue.put(ProcessDeathSignal(worker_id, f"Worker {worker_id} fatal error: {e}\n{traceback.format_exc()}"))
    finally:
        if torch.cuda.is_available():
            try:
                torch.cuda.synchronize()
            except Exception:
                pass
    logger.info(f"Worker {worker_id} exiting")


class MultiprocessingEvaluator:
    def __init__(self, num_workers: int = 1, daemon: bool = True, backend: Optional[BackendRef] = None, task_timeout_s: float = 600.0, worker_target=None):
        if torch.cuda.is_available():
            assert num_workers <= torch.cuda.device_count(), "performance will be suboptimal"
        self.mp_context = mp.get_context("spawn")
        self.num_workers = num_workers
        self.task_queue = self.mp_context.Queue()
        self.result_queue = self.mp_context.Queue()
        self.workers = {}
        self.next_task_id = 0
        self.total_tasks = 0
        self.completed_tasks = 0
        self.daemon = daemon
        self.backend = backend
        self.task_timeout_s = task_timeout_s
        self.restarts = 0
        self._worker_target = worker_target or _worker_process
        self._last_progress = time.monotonic()

    # ---------------------------------------------------------------- submission
    def submit_task(self, op, impl, correctness_tests, performance_tests, tolerances=None) -> int:
        task_id = self.next_task_id
        self.next_task_id += 1
        if not isinstance(op, str) and not is_pickleable(op):
            op = _extract_spec_name_from_op(op)
        if not isinstance(impl, (str, BackendRef)) and not is_pickleable(impl):
            # a function loaded from a kernel directory: rebuild it in the worker when we
            # know where it came from; otherwise ship the operator's name like the reference
            impl = self.backend if self.backend is not None else _extract_spec_name_from_op(impl)
        orig_device = None
        ctests, ptests = [], []
        for src, dst in ((correctness_tests, ctests), (performance_tests, ptests)):
            for t in src:
                if isinstance(t, SpecTest):  # descriptor: travels as is, built on the worker
                    if orig_device is None:
                        orig_device = torch.device(t.device)
                    dst.append(SpecTest(t.spec, t.device, t.gen_device))
                else:  # tensors: park them on the CPU for the queue
                    cpu_t = test_to_device(t, torch.device("cpu"))
                    if orig_device is None:
                        orig_device = find_device(t.args if hasattr(t, "args") else t)
                    dst.append(cpu_t)
        if orig_device is None:
            orig_device = torch.device("cuda")
        self.task_queue.put(EvalTask(task_id, op, impl, ctests, ptests, str(orig_device), tolerances))
        self.total_tasks += 1
        return task_id

    # ---------------------------------------------------------------- workers
    def _start_worker(self, worker_id):
        p = self.mp_context.Process(target=self._worker_target, args=(worker_id, self.task_queue, self.result_queue), daemon=self.daemon)
        p.start()
        self.workers[worker_id] = p
        logger.info(f"Started worker {worker_id} (PID: {p.pid}, GPU: {worker_id})")

    def _restart_worker(self, worker_id):
        old = self.workers.pop(worker_id, None)
        if old is not None:
            if old.is_alive():
                old.terminate()
            old.join(timeout=5)
        self.restarts += 1
        self._start_worker(worker_id)
        logger.warning(f"Restarted worker {worker_id}")

    def start_evaluation(self) -> None:
        self._last_progress = time.monotonic()
        for i in range(self.num_workers):
            self._start_worker(i)

    # ---------------------------------------------------------------- results
    def get_results(self):
        results = []
        while self.completed_tasks < self.total_tasks:
            try:
                item = self.result_queue.get(timeout=0.2)
            except queue.Empty:
                self._check_liveness()
                continue
            self._last_progress = time.monotonic()
            if isinstance(item, ProcessDeathSignal):
                self.completed_tasks += 1  # the task that killed the worker yields no result
                logger.error(f"Worker {item.worker_id} died: {item.error_msg}")
                self._restart_worker(item.worker_id)
            elif isinstance(item, EvalResult):
                results.append(item)
                self.completed_tasks += 1
                if item.error:
                    logger.warning(f"Task {item.task_id} completed with error: {item.error}")
        results.sort(key=lambda r: r.task_id)
        return results

    def _check_liveness(self):
        """A worker that vanished without a signal took one task with it: account for the
        task and restart the worker. A worker silent for `task_timeout_s` is replaced too."""
        for wid, p in list(self.workers.items()):
            if not p.is_alive() and self.completed_tasks < self.total_tasks:
                logger.error(f"Worker {wid} exited unexpectedly (exit code {p.exitcode})")
                self.completed_tasks += 1
                self._last_progress = time.monotonic()
                self._restart_worker(wid)
        if time.monotonic() - self._last_progress > self.task_timeout_s:
            logger.error(f"No result for {self.task_timeout_s} s: restarting all workers")
            self.completed_tasks += len(self.workers)
            self._last_progress = time.monotonic()
            for wid in list(self.workers):
                self._restart_worker(wid)

    # ---------------------------------------------------------------- shutdown
    def shutdown(self) -> None:
        for _ in range(len(self.workers)):
            self.task_queue.put(None)
        for wid, p in list(self.workers.items()):
            try:
                p.join(timeout=5)
                if p.is_alive():
                    logger.warning(f"Force terminating worker {wid}")
                    p.terminate()
                    p.join(timeout=2)
            except Exception as e:
                logger.error(f"Error shutting down worker {wid}: {e}")
        self.workers.clear()

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.shutdown()
