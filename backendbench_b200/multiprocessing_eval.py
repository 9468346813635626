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
* The parent knows which task every worker holds (workers post `TaskStarted` the moment
  they take one), so a lost task is booked exactly once and only for a worker that held
  one: a worker that dies idle costs nothing, and a death signal that arrives after the
  liveness check already replaced its sender restarts nobody.
* Workers post `WorkerReady` once their CUDA context and the kernel library are loaded;
  `timeline()` reports start-up, steady-state rate and per-worker busy time, which is
  what the sharded-sweep figure of the benchmark is made of.
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
    pid: int = -1


@dataclass
class TaskStarted:
    """Posted by a worker the moment it takes a task off the queue."""

    worker_id: int
    task_id: int
    pid: int = -1


@dataclass
class WorkerReady:
    """Posted once per worker process when its device and the backend library are usable."""

    worker_id: int
    pid: int
    seconds: float  # from process entry to ready (imports, CUDA context, library load)


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
    """Bind this worker to GPU `worker_id` (the reference: `torch.cuda.set_device(worker_id)`,
    BackendBench/multiprocessing_eval.py:82). When CUDA has not been initialised in this
    process yet -- the normal case in a freshly spawned worker -- the binding is made by
    narrowing CUDA_VISIBLE_DEVICES to that one GPU first: the driver then enumerates one device
    instead of every GPU of the node while N workers start at once, and the worker cannot touch
    a neighbour's GPU by accident. The GPU is then `cuda:0` in this process."""
    narrowed = False
    if not torch.cuda.is_initialized():  # a Python-side flag: no driver call yet, so the variable still counts
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        ids = [v.strip() for v in visible.split(",") if v.strip()] if visible else None
        if ids is None or worker_id < len(ids):
            os.environ["CUDA_VISIBLE_DEVICES"] = ids[worker_id] if ids else str(worker_id)
            narrowed = True
    if not torch.cuda.is_available():
        return "cpu"
    if narrowed:
        torch.cuda.set_device(0)
        torch.cuda.synchronize()
        return "cuda:0"
    torch.cuda.set_device(worker_id)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return f"cuda:{worker_id}"


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


def _worker_process(worker_id, task_queue, result_queue, poll_s=0.5, warm_backend=None):
    t_entry = time.perf_counter()
    pid = os.getpid()
    backends_cache = {}
    try:
        own_device = _worker_device(worker_id)
        if warm_backend is not None:  # load the kernel table (and the shared library) before the first task
            from .backends import make_backend

            backends_cache[warm_backend] = make_backend(warm_backend.name, warm_backend.ops_directory)
        result_queue.put(WorkerReady(worker_id, pid, time.perf_counter() - t_entry))
        while True:
            try:
                task = task_queue.get(timeout=poll_s)
            except queue.Empty:
                continue
            if task is None:
                logger.info(f"Worker {worker_id} received shutdown signal")
                break
            result_queue.put(TaskStarted(worker_id, task.task_id, pid))
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
                error = None
                if device.startswith("cuda"):
                    # backstop: the per-test check in eval_correctness_test normally clears the word
                    from .ops import check_device_status

                    try:
                        check_device_status(torch.device(device))
                    except IndexError as e:
                        error = f"device status after the task: {e}"
                result = EvalResult(task.task_id, float(cs), float(ps), cr, pr, error, worker_id, time.perf_counter() - t0)
            except Exception as e:
                msg = f"Error in eval_one_op: {e}\n{traceback.format_exc()}"
                logger.warning(f"Worker {worker_id} task {task.task_id} failed: {msg}")
                if "cuda" in str(e).lower():
                    # a CUDA error may have poisoned the context: die and let the parent restart us
                    result_queue.put(ProcessDeathSignal(worker_id, f"Worker {worker_id} CUDA error: {msg}", task.task_id, pid))
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
        result_queue.put(ProcessDeathSignal(worker_id, f"Worker {worker_id} fatal error: {e}\n{traceback.format_exc()}", -1, pid))
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
        self.lost_tasks: List[int] = []  # task ids that died with their worker (no result)
        self._worker_target = worker_target or _worker_process
        self._last_progress = time.monotonic()
        self._holding = {}  # worker id -> task id it took and has not answered yet
        self._accounted = set()  # task ids already counted as completed
        # timeline (time.monotonic): start of evaluation, per-worker ready, first / last result
        self._t_start = None
        self._t_ready = {}
        self._t_spawn = {}
        self._startup_s = {}
        self._t_results: List[float] = []
        self._busy_s = {}
        self._tasks_by_worker = {}

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
        args = (worker_id, self.task_queue, self.result_queue)
        if self._worker_target is _worker_process:
            args = args + (0.5, self.backend)
        p = self.mp_context.Process(target=self._worker_target, args=args, daemon=self.daemon)
        self._t_spawn[worker_id] = time.monotonic()
        p.start()
        self.workers[worker_id] = p
        logger.info(f"Started worker {worker_id} (PID: {p.pid}, GPU: {worker_id})")

    def _restart_worker(self, worker_id):
        old = self.workers.pop(worker_id, None)
        if old is not None:
            if old.is_alive():
                old.terminate()
            old.join(timeout=5)
        self._holding.pop(worker_id, None)
        self.restarts += 1
        self._start_worker(worker_id)
        logger.warning(f"Restarted worker {worker_id}")

    def start_evaluation(self) -> None:
        self._last_progress = time.monotonic()
        self._t_start = time.monotonic()
        for i in range(self.num_workers):
            self._start_worker(i)

    # ---------------------------------------------------------------- accounting
    def _account(self, task_id, lost=False) -> bool:
        """Count `task_id` as completed, once. Returns False when it was counted before."""
        if task_id is None or task_id < 0 or task_id in self._accounted:
            return False
        self._accounted.add(task_id)
        self.completed_tasks += 1
        if lost:
            self.lost_tasks.append(task_id)
        return True

    def _is_current(self, worker_id, pid) -> bool:
        """Whether a message's sender is the process that now owns `worker_id` (a message of a
        process that was already replaced must not touch its successor)."""
        p = self.workers.get(worker_id)
        return p is not None and (pid is None or pid < 0 or p.pid == pid)

    def _handle(self, item, results) -> None:
        now = time.monotonic()
        self._last_progress = now
        if isinstance(item, WorkerReady):
            if self._is_current(item.worker_id, item.pid):
                self._t_ready.setdefault(item.worker_id, now)
                # spawn -> ready as the parent sees it: interpreter start, imports, CUDA context, library load
                self._startup_s.setdefault(item.worker_id, now - self._t_spawn.get(item.worker_id, now))
        elif isinstance(item, TaskStarted):
            if self._is_current(item.worker_id, item.pid) and item.task_id not in self._accounted:
                self._holding[item.worker_id] = item.task_id
        elif isinstance(item, ProcessDeathSignal):
            logger.error(f"Worker {item.worker_id} died: {item.error_msg}")
            task_id = item.task_id if item.task_id >= 0 else (self._holding.get(item.worker_id) if self._is_current(item.worker_id, item.pid) else None)
            self._account(task_id, lost=True)  # the task that killed the worker yields no result
            if self._is_current(item.worker_id, item.pid):
                self._restart_worker(item.worker_id)
        elif isinstance(item, EvalResult):
            if self._account(item.task_id):
                results.append(item)
                self._t_results.append(now)
                self._busy_s[item.worker_id] = self._busy_s.get(item.worker_id, 0.0) + item.seconds
                self._tasks_by_worker[item.worker_id] = self._tasks_by_worker.get(item.worker_id, 0) + 1
            if self._holding.get(item.worker_id) == item.task_id:
                del self._holding[item.worker_id]
            if item.error:
                logger.warning(f"Task {item.task_id} completed with error: {item.error}")

    def _drain(self, results, wait_s=0.05) -> None:
        """Handle every message already in the result queue (a worker that posted and then
        exited may be seen dead before its last message is read)."""
        while True:
            try:
                item = self.result_queue.get(timeout=wait_s)
            except queue.Empty:
                return
            self._handle(item, results)

    # ---------------------------------------------------------------- results
    def get_results(self):
        """Block until every submitted task is accounted for; results sorted by task id. May be
        called again after further `submit_task` calls: the workers stay up in between."""
        results = []
        if self._t_start is None:
            self._t_start = time.monotonic()
        while self.completed_tasks < self.total_tasks:
            try:
                item = self.result_queue.get(timeout=0.2)
            except queue.Empty:
                self._check_liveness(results)
                continue
            self._handle(item, results)
        results.sort(key=lambda r: r.task_id)
        return results

    def _check_liveness(self, results):
        """A worker that vanished without a signal took the task it held (if any) with it:
        book that task once and restart the worker. When nothing at all has arrived for
        `task_timeout_s`, the tasks in flight are booked as lost and their workers replaced."""
        dead = [wid for wid, p in self.workers.items() if not p.is_alive()]
        if dead:
            self._drain(results)  # their last messages first
        for wid in dead:
            p = self.workers.get(wid)
            if p is None or p.is_alive():
                continue  # replaced while draining
            logger.error(f"Worker {wid} exited unexpectedly (exit code {p.exitcode})")
            self._account(self._holding.pop(wid, None), lost=True)
            self._last_progress = time.monotonic()
            if self.completed_tasks < self.total_tasks:
                self._restart_worker(wid)
            else:
                self.workers.pop(wid, None)
        if time.monotonic() - self._last_progress > self.task_timeout_s:
            logger.error(f"No message for {self.task_timeout_s} s: replacing the workers that hold a task")
            held = list(self._holding.items())
            for wid, task_id in held:
                self._account(task_id, lost=True)
                self._restart_worker(wid)
            if not held:
                # nothing is known to be in flight, yet tasks are missing (one vanished between a
                # worker's queue read and its TaskStarted message): give up on the remainder
                missing = [t for t in range(self.next_task_id) if t not in self._accounted]
                logger.error(f"Giving up on tasks nobody holds: {missing}")
                for t in missing:
                    self._account(t, lost=True)
            self._last_progress = time.monotonic()

    def timeline(self) -> dict:
        """Wall-clock anatomy of the evaluation so far (seconds, `time.monotonic` of the parent)."""
        t0 = self._t_start
        if t0 is None or not self._t_results:
            return {}
        ready = sorted(self._t_ready.values())
        last = max(self._t_results)
        first = min(self._t_results)
        all_ready = ready[-1] if len(ready) >= self.num_workers else None
        out = {
            "wall_s": last - t0,
            "first_result_s": first - t0,
            "first_worker_ready_s": (ready[0] - t0) if ready else None,
            "all_workers_ready_s": (all_ready - t0) if all_ready is not None else None,
            "worker_startup_s": {int(k): round(v, 3) for k, v in sorted(self._startup_s.items())},
            "per_worker_busy_s": {int(k): round(v, 3) for k, v in sorted(self._busy_s.items())},
            "per_worker_tasks": {int(k): v for k, v in sorted(self._tasks_by_worker.items())},
            "results": len(self._t_results),
            "lost_tasks": list(self.lost_tasks),
            "restarts": self.restarts,
        }
        if all_ready is not None:
            after = [t for t in self._t_results if t >= all_ready]
            out["results_after_all_ready"] = len(after)
            out["steady_s"] = (last - all_ready) if after else 0.0
        return out

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
