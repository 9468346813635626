"""Correctness and timing of one operator implementation against aten.

Same contract as BackendBench/eval.py (result records :18-40, `allclose` :68-90,
`eval_correctness[_test]` :93-146, `cpu_bench` :149-159, `eval_performance` :162-224,
`eval_one_op` :227-271, `perf_at_p` :274-282), rebuilt around the GPU:

* closeness and error magnitudes of CUDA tensors come from ONE fused device pass
  (`b200_allclose`) and one 32-byte read-back, instead of several elementwise aten
  passes, two `.item()` syncs and an exception used as control flow;
* tolerances are forwarded (the reference's `allclose` accepts atol/rtol but compares
  with 1e-2 regardless) and can be chosen per dtype with `tolerances_for`;
* CUDA timing uses CUDA events around single launches with an L2 flush before each,
  a few dozen launches per case, instead of do_bench's fixed 25 ms + 100 ms windows.
"""

from __future__ import annotations

import logging
import math
import struct
import time
import traceback
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from . import _abi
from .utils import compute_errors, serialize_args, uses_cuda_stream

logger = logging.getLogger(__name__)


@dataclass
class CorrectnessTestResult:
    op_name: str
    args: str
    is_correct: bool = False
    error_msg: str = ""
    error_type: str = ""
    traceback: str = ""
    max_abs_error: float = -math.inf
    max_rel_error: float = -math.inf
    test_type: str = "correctness"


@dataclass
class PerformanceTestResult:
    op_name: str
    args: str
    speedup: float
    benchmark_time_ms: float
    reference_time_ms: float
    error_msg: str = ""
    successfully_ran: bool = False
    test_type: str = "performance"


EXC_MSG = """
Exception raised for {op}:
    args: {args}
    exc: {exc}
    traceback: {traceback}
"""


def format_exception(e, op, args, kwargs, traceback=None):
    op_name = getattr(op, "__name__", str(op))
    return EXC_MSG.format(op=op_name, args=serialize_args(args, kwargs), exc=e, traceback=traceback)


# ------------------------------------------------------------------ tolerances
HARNESS_ATOL = HARNESS_RTOL = 1e-2  # BackendBench/eval.py:68, applied there to every dtype

_ELEMENTWISE = ("relu", "add", "mul", "where")


def tolerances_for(op, dtype) -> Tuple[float, float]:
    """(atol, rtol) for `op` producing `dtype`: the harness's 1e-2 for bf16/fp16, 1e-5 for
    fp32 elementwise results, 1e-4 for fp32 reductions / normalisations / contractions
    (summation order differs from aten's), 0 for integer and bool results."""
    if dtype in (torch.bfloat16, torch.float16):
        return HARNESS_ATOL, HARNESS_RTOL
    if dtype == torch.float32 or dtype == torch.float64:
        name = getattr(op, "__name__", str(op)).split(".")[0]
        return (1e-5, 1e-5) if name in _ELEMENTWISE else (1e-4, 1e-4)
    return 0.0, 0.0


# ------------------------------------------------------------------ device compare
_records = {}
_KERNEL_DTYPES = {
    torch.float32: _abi.F32, torch.bfloat16: _abi.BF16, torch.float16: _abi.F16, torch.int64: _abi.I64,
    torch.int32: _abi.I32, torch.int16: _abi.I16, torch.int8: _abi.I8, torch.uint8: _abi.U8, torch.bool: _abi.BOOL,
}


def _record(device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    rec = _records.get(key)
    if rec is None:
        rec = torch.zeros(8, dtype=torch.int32, device=device)
        _records[key] = rec
    return rec


class _Compare:
    """Accumulates the verdict over every tensor pair of one (reference, result) structure."""

    def __init__(self, atol, rtol, rec=None):
        self.atol, self.rtol = atol, rtol
        self.ok = True
        self.max_abs = None
        self.max_rel = None
        self.nan = False
        self.rec = rec  # caller-owned 8 x int32 device record, or None for the shared one
        self.rec_used = False
        self.saw_tensor_ref = self.saw_tensor_res = False

    def _host_pair(self, r, s):
        if r.numel() == 0:
            self._merge(0.0, 0.0)
            return
        if r.is_sparse or s.is_sparse:
            self.ok = self.ok and bool(torch.equal(r.to_dense(), s.to_dense()))
            return
        rf, sf = r.detach().double(), s.detach().double()
        close = torch.isclose(rf, sf, rtol=self.rtol, atol=self.atol, equal_nan=True)
        self.ok = self.ok and bool(close.all().item())
        a, b = compute_errors(r, s)
        if a is not None:
            self._merge(a, b)

    def _merge(self, a, b):
        if a != a or b != b:
            self.nan = True
            return
        self.max_abs = a if self.max_abs is None else max(self.max_abs, a)
        self.max_rel = b if self.max_rel is None else max(self.max_rel, b)

    def tensor_pair(self, r, s):
        if not isinstance(s, torch.Tensor) or r.shape != s.shape or r.dtype != s.dtype or r.device != s.device or r.layout != s.layout:
            self.ok = False  # assert_close checks shape, dtype, device and layout before values
            if isinstance(s, torch.Tensor) and r.shape == s.shape and r.device == s.device and not r.is_sparse:
                a, b = compute_errors(r, s)
                if a is not None:
                    self._merge(a, b)
            return
        code = _KERNEL_DTYPES.get(r.dtype)
        if not r.is_cuda or code is None or r.is_sparse:
            self._host_pair(r, s)
            return
        if r.numel() == 0:
            self._merge(0.0, 0.0)
            return
        from . import ops  # strided copies go through our own kernel

        rc, sc = ops._contig(r.detach()), ops._contig(s.detach())
        if self.rec is None:
            self.rec = _record(r.device)
        _abi.check(
            _abi.lib().b200_allclose(rc.data_ptr(), sc.data_ptr(), rc.numel(), code, self.rtol, self.atol, self.rec.data_ptr(), 0 if self.rec_used else 1, torch.cuda.current_stream().cuda_stream),
            "b200_allclose",
        )
        self.rec_used = True

    def walk(self, a, b):
        stack = [(a, b)]
        while stack:
            x, y = stack.pop()
            if isinstance(x, torch.Tensor):
                self.saw_tensor_ref = True
                self.saw_tensor_res = self.saw_tensor_res or isinstance(y, torch.Tensor)
                self.tensor_pair(x, y)
            elif isinstance(x, (list, tuple)):
                if not isinstance(y, (list, tuple)) or len(x) != len(y):
                    self.ok = False
                    continue
                stack.extend(reversed(list(zip(x, y))))
            else:
                try:
                    self.ok = self.ok and bool(x == y)
                except Exception:
                    self.ok = False

    def finish(self):
        """(is_close, max_abs_error, max_rel_error); errors are None when no tensors were compared."""
        if self.rec_used:
            words = self.rec.tolist()  # the single device->host read of the comparison
            raw = struct.pack("8i", *words)
            mism, mabs, mrel, nan_seen = struct.unpack("<QffI", raw[:20])
            if mism:
                self.ok = False
            if nan_seen:
                self.nan = True
            self._merge(mabs, mrel)
        if self.nan:
            return self.ok, math.nan, math.nan
        return self.ok, self.max_abs, self.max_rel


def compare(ref, res, atol=HARNESS_ATOL, rtol=HARNESS_RTOL):
    """(is_close, max_abs_error, max_rel_error) of a result structure against a reference
    structure: tensors by assert_close's rule (equal_nan), sequences pairwise, anything
    else by `==`."""
    c = _Compare(atol, rtol)
    c.walk(ref, res)
    return c.finish()


def compare_enqueue(ref, res, atol, rtol, rec: torch.Tensor) -> bool:
    """Queue the comparison of CUDA structures into the caller's 8 x int32 device record
    without reading anything back (many cases, one read at the end: `decode_record`).
    Returns False when the structures already differ in shape / dtype / length."""
    c = _Compare(atol, rtol, rec)
    c.walk(ref, res)
    if not c.rec_used:  # nothing was queued (empty tensors): leave a clean record behind
        rec.zero_()
    return c.ok


def decode_record(words) -> Tuple[int, float, float, bool]:
    """(mismatches, max_abs, max_rel, nan_seen) from the 8 int32 words of one record."""
    mism, mabs, mrel, nan_seen = struct.unpack("<QffI", struct.pack("8i", *words)[:20])
    return mism, mabs, mrel, bool(nan_seen)


def allclose(a, b, atol=HARNESS_ATOL, rtol=HARNESS_RTOL) -> bool:
    try:
        return compare(a, b, atol, rtol)[0]
    except Exception:
        return False


def _first_dtype(x):
    if isinstance(x, torch.Tensor):
        return x.dtype
    if isinstance(x, (list, tuple)):
        for y in x:
            d = _first_dtype(y)
            if d is not None:
                return d
    return None


def _first_cuda_device(x):
    if isinstance(x, torch.Tensor):
        return x.device if x.is_cuda else None
    if isinstance(x, (list, tuple)):
        for y in x:
            d = _first_cuda_device(y)
            if d is not None:
                return d
    return None


def _raise_device_status(res) -> None:
    """Read (and clear) the status word of the device a CUDA result lives on; raises what
    `ops.check_device_status` raises (IndexError for an out-of-range index). The comparison
    before it has already synchronised, so this costs one 4-byte read."""
    dev = _first_cuda_device(res)
    if dev is not None:
        from .ops import check_device_status

        check_device_status(dev)


# ------------------------------------------------------------------ correctness
def eval_correctness_test(op, impl, test, tolerances=None) -> CorrectnessTestResult:
    """Run `impl` on the test's arguments and compare with `op` on the same arguments.
    `tolerances`: None -> harness 1e-2; "dtype" -> `tolerances_for`; or an (atol, rtol) pair."""
    args, kwargs = test.args, test.kwargs
    ref = op(*args, **kwargs)
    op_name = getattr(op, "__name__", str(op))
    try:
        res = impl(*args, **kwargs)
        if tolerances is None:
            atol, rtol = HARNESS_ATOL, HARNESS_RTOL
        elif tolerances == "dtype":
            atol, rtol = tolerances_for(op, _first_dtype(ref))
        else:
            atol, rtol = tolerances
        ok, abs_err, rel_err = compare(ref, res, atol, rtol)
        _raise_device_status(res)  # a kernel that zero-filled on a bad index fails THIS test, with the reason
        return CorrectnessTestResult(op_name=op_name, args=serialize_args(args, kwargs), is_correct=ok, max_abs_error=abs_err, max_rel_error=rel_err)
    except Exception as e:
        tb = traceback.format_exc()
        msg = format_exception(e, op, args, kwargs, tb)
        logger.warning(msg)
        return CorrectnessTestResult(op_name=op_name, args=serialize_args(args, kwargs), is_correct=False, error_msg=msg, error_type=str(type(e)), traceback=tb)


def eval_correctness(op, impl, tests, tolerances=None) -> Tuple[float, List[CorrectnessTestResult]]:
    results = [eval_correctness_test(op, impl, t, tolerances) for t in tests]
    if not results:
        logger.warning(f"No correctness tests available for {str(op)}")
        return 0.0, []
    return sum(r.is_correct for r in results) / len(results), results


# ------------------------------------------------------------------ timing
def cpu_bench(fn, num_runs=100):
    """10 warm-up calls, then the mean wall time of `num_runs` calls, in SECONDS."""
    for _ in range(10):
        fn()
    t0 = time.perf_counter()
    for _ in range(num_runs):
        fn()
    return (time.perf_counter() - t0) / num_runs


_flush_buffers = {}
L2_FLUSH_BYTES = 256 << 20  # twice the 126 MB L2


def l2_flush(device=None):
    """Overwrite a 256 MiB scratch buffer on the current stream so the next launch starts cold."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = device.index if device.index is not None else torch.cuda.current_device()
    buf = _flush_buffers.get(key)
    if buf is None:
        buf = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
        _flush_buffers[key] = buf
    _abi.check(_abi.lib().b200_l2_flush(buf.data_ptr(), buf.numel(), torch.cuda.current_stream().cuda_stream), "b200_l2_flush")


def cuda_bench(fn, warmup=3, reps=20, flush=True, return_all=False):
    """Median device time of one call of `fn` in MILLISECONDS: `warmup` untimed calls,
    then `reps` calls each bracketed by CUDA events on the current stream, with an L2
    flush queued before each so every launch reads its inputs from HBM."""
    for _ in range(warmup):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    for i in range(reps):
        if flush:
            l2_flush()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    times = sorted(s.elapsed_time(e) for s, e in zip(starts, ends))
    if return_all:
        return times
    return times[len(times) // 2]


def cuda_bench_rotating(fns, reps=30, warmup=None, graph=False, replays=5):
    """Mean device time per call in MILLISECONDS over `reps` back-to-back launches that
    cycle through `fns` -- closures over DISTINCT input sets whose total footprint exceeds
    L2, so every launch reads its inputs from HBM and evicts its predecessors' outputs, as
    in steady state. One pair of CUDA events brackets the whole loop (no per-launch event or
    flush overhead); the last len(fns) results are kept alive so outputs rotate too.

    `graph=True`: the loop is captured once in a CUDA graph on a side stream (after warm-up
    calls on that stream, which also size its scratch buffers) and the REPLAY is timed, median
    of `replays`. Launched from Python, a call of this package costs the host about 20 us, more
    than several of the kernels take (sum over 64 MiB: 14 us), so an eager loop measures the
    interpreter; the replay measures the device."""
    n = len(fns)
    ring = [None] * n
    if not graph:
        for i in range(warmup if warmup is not None else max(3, n)):
            ring[i % n] = fns[i % n]()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(reps):
            ring[i % n] = fns[i % n]()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / reps
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(warmup if warmup is not None else max(3, n)):
            ring[i % n] = fns[i % n]()
    side.synchronize()
    ring = [None] * n
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for i in range(reps):
            ring[i % n] = fns[i % n]()
    times = []
    for _ in range(replays + 1):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        g.replay()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / reps)
    del ring, g
    times = sorted(times[1:])
    return times[len(times) // 2]


def _on_cuda(x) -> bool:
    if isinstance(x, torch.Tensor):
        return x.is_cuda
    if isinstance(x, (list, tuple)):
        return any(_on_cuda(y) for y in x)
    if isinstance(x, dict):
        return any(_on_cuda(y) for y in x.values())
    return False


def eval_performance(op, impl, tests, tolerances=None) -> Tuple[float, List[PerformanceTestResult]]:
    """Per case: time aten, re-verify the implementation, time it; score = geomean speedup.
    A case whose implementation fails or is wrong counts as speedup 1.0 in the score.
    CUDA cases report milliseconds; CPU cases report what `cpu_bench` returns (seconds)."""
    base_times, test_times, results = [], [], []
    op_name = getattr(op, "__name__", str(op))
    for test in tests:
        args, kwargs = test.args, test.kwargs  # cached: both sides must see the same tensors
        args_str = serialize_args(args, kwargs)
        bench = cuda_bench if (_on_cuda(args) or _on_cuda(kwargs)) else cpu_bench
        base = bench(lambda: op(*args, **kwargs))
        base_times.append(base)
        t = base
        try:
            ref = op(*args, **kwargs)
            res = impl(*args, **kwargs)
            if tolerances is None:
                atol, rtol = HARNESS_ATOL, HARNESS_RTOL
            elif tolerances == "dtype":
                atol, rtol = tolerances_for(op, _first_dtype(ref))
            else:
                atol, rtol = tolerances
            ok, abs_err, rel_err = compare(ref, res, atol, rtol)
            _raise_device_status(res)
            if not ok:
                raise ValueError(f"Reference and result tensors are not close: max absolute error {abs_err}, max relative error {rel_err}")
            t = bench(lambda: impl(*args, **kwargs))
            results.append(PerformanceTestResult(op_name=op_name, args=args_str, speedup=base / t, successfully_ran=True, benchmark_time_ms=t, reference_time_ms=base))
        except Exception as e:
            msg = format_exception(e, op, args, kwargs, traceback.format_exc())
            results.append(PerformanceTestResult(op_name=op_name, args=args_str, successfully_ran=False, speedup=None, benchmark_time_ms=None, reference_time_ms=base, error_msg=msg))
        finally:
            test_times.append(t)
    speedups = torch.tensor(base_times, dtype=torch.float64) / torch.tensor(test_times, dtype=torch.float64)
    return speedups.log().mean().exp().float(), results


_stream_screen = {}


def _creates_streams(impl) -> bool:
    """`uses_cuda_stream(impl)`, remembered per callable (reading and parsing the source of
    the same function for each of thousands of per-case tasks is pure overhead)."""
    try:
        return _stream_screen[impl]
    except KeyError:
        verdict = _stream_screen[impl] = uses_cuda_stream(impl)
        return verdict
    except TypeError:  # unhashable callable
        return uses_cuda_stream(impl)


def eval_one_op(op, impl, correctness_tests, performance_tests, tolerances=None):
    """(correctness score, performance score, correctness results, performance results).
    Implementations whose source creates CUDA streams are not evaluated (score 0 / 1.0)."""
    op_name = getattr(op, "__name__", str(op))
    if _creates_streams(impl):
        logger.warning(f"Skipping {op_name} because it uses CUDA stream")
        why = "Skipped: uses CUDA stream"
        cres = [CorrectnessTestResult(op_name=op_name, args=serialize_args(t.args, t.kwargs), is_correct=False, error_msg=why) for t in correctness_tests]
        pres = [PerformanceTestResult(op_name=op_name, args=serialize_args(t.args, t.kwargs), speedup=0, benchmark_time_ms=0, reference_time_ms=0, error_msg=why) for t in performance_tests]
        return 0, 1.0, cres, pres
    cscore, cres = eval_correctness(op, impl, correctness_tests, tolerances)
    pscore, pres = eval_performance(op, impl, performance_tests, tolerances)
    return cscore, pscore, cres, pres


def perf_at_p(correctness, performance, p=1.0):
    """Fraction of operators that are correct AND faster than p x the reference."""
    assert len(correctness) == len(performance), "correctness and performance must have the same length"
    return torch.where(torch.tensor(correctness).bool(), torch.tensor(performance) > p, 0).float().mean()
