"""Benchmark of the B200 operator backend on the 512-case sharded sweep.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One STEP is one correctness pass of the sweep on each rank: for each of the 512 seeded
(op, shape, dtype) cases the backend kernel is launched on inputs resident in HBM and its
result is checked on the device against the resident aten reference result by the fused
allclose kernel; the 512 verdict records are read back once at the end of the step.
Ranks share nothing (weak scaling: every rank owns a full sweep with its own seeds), so
the only communication is the barrier around the timed region and the max over ranks of
the device time. `value` = cases all ranks processed / that time.

The JSON line also carries:
* `e2e`: the same pass through the public plugin call with the inputs in pinned HOST memory,
  H2D copies and the verdict read-back inside the timed region, next to an H2D-only pass over
  the same buffers (the box's copy ceiling);
* `full_eval`: the pass as the harness itself runs a case (`eval_correctness_test`: aten CUDA
  reference computed inside the timed region, backend call, compare, one read-back per case),
  wall clock;
* `sharded_sweep`: the 512 cases as per-case tasks, longest first, through ONE shared queue
  of `MultiprocessingEvaluator` with one worker process per GPU (N = --gpus); wall clock from
  the first dispatch to the last result, start-up and steady state apart; rank 0 owns the
  evaluator, the other ranks wait on a host-side barrier;
* `strong_scaling`: the ONE sweep dealt over the ranks longest-first and replayed from a graph;
* `roofline`: the kernel with the largest share of the sweep's device time (the fused fp32
  compare kernel), algorithmic bytes / CUDA-event time over all its launches of one pass;
* `per_op`: every named operator configuration: GB/s or TFLOP/s against the measured and
  nominal peaks, speed-up over aten CUDA, and the aten-CPU time by the harness's `cpu_bench`
  protocol with the core count; `geomean_speedup_vs_aten` over that table;
* `cpu_baseline` (the reference's aten-CPU path on a bounded sample, host cores), `clocks`
  and `gpu_launches`.

`--impl reference` times the reference's own CPU path (AtenBackend + the reference's
correctness evaluation, restated in oracle/aten_cpu_path.py) over the same 512 cases per step.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

N_CASES = 512
SWEEP_SEED = 0
NOMINAL_HBM_GBS = 8000.0
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
WORKLOAD = "sharded sweep: 512 seeded (op, shape, dtype) cases over 16 aten overloads, 2^8..2^26 elements, 15% edge cases; one correctness pass over all 512 cases per step"
# DRAM bytes moved per algorithmic byte by the fp32 compare kernel, from its profiler capture
# of one launch on two 4096 x 4096 fp32 tensors: 134.2 MB read + 4.1 MB written for 134.2 MB of operands
ALLCLOSE_F32_DRAM_PER_ALGORITHMIC_BYTE = 1.031
EXACT_VS_CPU = ("scatter_add.default",)  # aten CUDA scatter_add is order-nondeterministic: its reference comes from aten CPU


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def _dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, local, world


def _host_memory_allows(bytes_per_rank: int, ranks: int) -> bool:
    """Whether every rank of this node can hold a pinned host copy of its inputs (plus the
    pageable staging copy of one tensor at a time), by the free memory the OS reports and by
    the container's cgroup limit when there is one."""
    need = 1.3 * bytes_per_rank * max(ranks, 1)
    try:
        import psutil

        if psutil.virtual_memory().available < need:
            return False
    except Exception:
        pass
    for path in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            raw = open(path).read().strip()
            if raw.isdigit() and int(raw) < need:
                return False
        except OSError:
            pass
    return True


def common_config(cases_per_rank=N_CASES):
    """The workload description both arms print (what is measured is the same list of cases)."""
    return {"workload": WORKLOAD, "cases_per_step": cases_per_rank, "sweep_seed": SWEEP_SEED,
            "cache": "the inputs of one pass exceed L2 many times over (about 10 GB); no flush between steps"}


def _bytes_of(args):
    return sum(a.numel() * a.element_size() for a in args if isinstance(a, torch.Tensor))


# ------------------------------------------------------------------------- b200 arm
def prepare_cases(cases, backend, device):
    """Inputs generated on the device from each case's seed, aten reference results resident."""
    from backendbench_b200.eval import tolerances_for
    from backendbench_b200.opregistry import get_operator

    prepared = []
    for c in cases:
        op = get_operator(c.op)
        args, kwargs = c.build(device)
        if c.op in EXACT_VS_CPU:
            cpu_args = [a.cpu() if isinstance(a, torch.Tensor) else a for a in args]
            ref = op(*cpu_args, **kwargs).to(device)
            atol = rtol = 0.0
        else:
            ref = op(*args, **kwargs)
            first = ref[0] if isinstance(ref, (tuple, list)) else ref
            atol, rtol = tolerances_for(op, first.dtype)
            if c.op in ("embedding.default", "index_select.default", "gather.default", "where.self", "argmax.default"):
                atol = rtol = 0.0
        prepared.append({"case": c, "op": op, "impl": backend[op], "args": args, "kwargs": kwargs, "ref": ref, "atol": atol, "rtol": rtol})
    torch.cuda.synchronize()
    return prepared


def sweep_enqueue(prepared, records, streams=None):
    """Queue one correctness pass (backend launch + fused compare per case); no read-back.
    With `streams`, case i goes to streams[i % len(streams)]: the cases are independent (own
    inputs, own output, own verdict record, per-stream scratch), so their launch chains can
    run side by side -- most cases are too small to fill the GPU and their cost is the launch
    gap, not the kernel. The current stream forks to the side streams and joins them again,
    which under graph capture yields a graph with that many parallel branches."""
    from backendbench_b200.eval import compare_enqueue

    structural = []
    if not streams:
        for i, p in enumerate(prepared):
            res = p["impl"](*p["args"], **p["kwargs"])
            structural.append(compare_enqueue(p["ref"], res, p["atol"], p["rtol"], records[i]))
        return structural
    cur = torch.cuda.current_stream()
    fork = torch.cuda.Event()
    fork.record(cur)
    for s in streams:
        s.wait_event(fork)
    for i, p in enumerate(prepared):
        with torch.cuda.stream(streams[i % len(streams)]):
            res = p["impl"](*p["args"], **p["kwargs"])
            structural.append(compare_enqueue(p["ref"], res, p["atol"], p["rtol"], records[i]))
            del res
    for s in streams:
        join = torch.cuda.Event()
        join.record(s)
        cur.wait_event(join)
    return structural


def sweep_pass(prepared, records, host_inputs=None, device=None):
    """One correctness pass; returns the (n, 8) int32 verdict records on the host. With
    `host_inputs` (pinned host tensors) every case's inputs are copied host->device first, on
    a copy stream that runs a few cases ahead of the compute stream."""
    from backendbench_b200.eval import compare_enqueue

    structural = []
    if host_inputs is None:
        for i, p in enumerate(prepared):
            res = p["impl"](*p["args"], **p["kwargs"])
            structural.append(compare_enqueue(p["ref"], res, p["atol"], p["rtol"], records[i]))
        return records.cpu(), structural  # the step's single device->host read

    main = torch.cuda.current_stream()
    copier = _copy_stream(device)
    copier.wait_stream(main)
    ahead, n, staged = 4, len(prepared), {}

    def stage(i):
        with torch.cuda.stream(copier):
            args = [a.to(device, non_blocking=True) if isinstance(a, torch.Tensor) else a for a in host_inputs[i]]
            ev = torch.cuda.Event()
            ev.record(copier)
        staged[i] = (args, ev)

    for i in range(min(ahead, n)):
        stage(i)
    for i, p in enumerate(prepared):
        args, ev = staged.pop(i)
        main.wait_event(ev)
        for a in args:
            if isinstance(a, torch.Tensor):
                a.record_stream(main)  # allocated on the copy stream, consumed here
        res = p["impl"](*args, **p["kwargs"])
        structural.append(compare_enqueue(p["ref"], res, p["atol"], p["rtol"], records[i]))
        if i + ahead < n:
            stage(i + ahead)
    host = records.cpu()
    return host, structural


_copy_streams = {}


def _copy_stream(device):
    st = _copy_streams.get(str(device))
    if st is None:
        st = _copy_streams[str(device)] = torch.cuda.Stream(device=device)
    return st


def count_correct(host_records, structural):
    from backendbench_b200.eval import decode_record

    ok, bad = 0, []
    rows = host_records.tolist()
    for i, (row, s) in enumerate(zip(rows, structural)):
        mism = decode_record(row)[0]
        if s and mism == 0:
            ok += 1
        else:
            bad.append(i)
    return ok, bad


def time_steps(fn, steps, warmup):
    """`warmup` untimed calls, then `steps` calls between a barrier + synchronize on both
    sides, timed on the device with CUDA events on the current stream; max over ranks."""
    from backendbench_b200.sharding import barrier, max_over_ranks

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    last = None
    for _ in range(steps):
        last = fn()
    end.record()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    return max_over_ranks(start.elapsed_time(end)), last


def per_kernel_profile(prepared, step_ms, repeats=3):
    """Device time of every case's backend launch (CUDA events, L2 flushed before each;
    median of `repeats` passes) aggregated per operator: the share table of the sweep. A case
    whose event time exceeds a whole step caught a host stall between its two events, not
    kernel time, and is left out (and counted)."""
    from backendbench_b200.eval import l2_flush

    n = len(prepared)
    samples = [[] for _ in range(n)]
    for _ in range(repeats):
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        for i, p in enumerate(prepared):
            l2_flush()
            starts[i].record()
            p["impl"](*p["args"], **p["kwargs"])
            ends[i].record()
        torch.cuda.synchronize()
        for i in range(n):
            samples[i].append(starts[i].elapsed_time(ends[i]))
    by_op, per_case, dropped = {}, [], 0
    for i, p in enumerate(prepared):
        c = p["case"]
        ms = statistics.median(samples[i])
        if ms > step_ms:
            dropped += 1
            continue
        per_case.append((ms, c.label() + (" " + str(dict(c.extra)) if c.extra else "")))
        d = by_op.setdefault(c.op, {"ms": 0.0, "bytes": 0, "flops": 0, "launches": 0})
        d["ms"] += ms
        d["bytes"] += c.algorithmic_bytes()
        d["flops"] += c.flops()
        d["launches"] += 1
    per_case.sort(reverse=True)
    return by_op, [{"ms": round(ms, 3), "case": label} for ms, label in per_case[:12]], round(sum(ms for ms, _ in per_case), 3), dropped


def _f32_pairs(ref, res, out):
    """Contiguous fp32 CUDA tensor pairs of a (reference, result) structure, in order."""
    if isinstance(ref, torch.Tensor):
        if isinstance(res, torch.Tensor) and ref.dtype == torch.float32 and res.dtype == torch.float32 and ref.shape == res.shape and ref.numel() and ref.is_contiguous() and res.is_contiguous():
            out.append((ref, res))
    elif isinstance(ref, (list, tuple)) and isinstance(res, (list, tuple)):
        for r, s in zip(ref, res):
            _f32_pairs(r, s, out)


def compare_kernel_roofline(prepared, peaks, repeats=5):
    """Roofline of the kernel that holds the largest share of the sweep's device time: the fused
    fp32 compare (`allclose_kernel<float>`, ahead of every operator kernel in the profiler's
    launch list of one pass). Every fp32 (reference, result) pair of one pass is compared back
    to back -- its launches exactly as the sweep makes them, gigabytes of operands in total, so
    nothing stays in L2 from one launch to the next. The launches are captured in a CUDA graph
    (as the timed step is) and the replay is bracketed by one pair of CUDA events on the
    launching stream; median of `repeats`. Algorithmic bytes of a launch: both operands read
    once, 2 x 4 x numel (the 32-byte verdict record is noise)."""
    from backendbench_b200 import _abi
    from backendbench_b200.eval import compare_enqueue

    pairs = []
    for p in prepared:
        res = p["impl"](*p["args"], **p["kwargs"])
        _f32_pairs(p["ref"], res, pairs)
    if not pairs:
        return None
    rec = torch.zeros(8, dtype=torch.int32, device=pairs[0][0].device)

    def timed(subset):
        for r, s in subset:  # warm-up, and the launch count
            compare_enqueue(r, s, 1e-4, 1e-4, rec)
        torch.cuda.synchronize()
        n0 = _abi.lib().b200_launch_count()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for r, s in subset:
                compare_enqueue(r, s, 1e-4, 1e-4, rec)
        launches = _abi.lib().b200_launch_count() - n0
        times = []
        for _ in range(repeats + 1):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        return statistics.median(times[1:]), launches

    nbytes = sum(2 * 4 * r.numel() for r, _ in pairs)
    ms, launches = timed(pairs)
    everything = {"launches": int(launches), "achieved": round(nbytes / (ms * 1e-3) / 1e9, 1), "frac": round(nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                  "avg_launch_ms": round(ms / max(launches, 1), 5), "algorithmic_bytes_per_launch": int(nbytes / max(launches, 1)),
                  "note": "most of these launches move under a megabyte and cost a launch, not bandwidth"}
    # The launch class the roofline line describes: operands of 32 MiB or more in total, the
    # launches that hold nine tenths of the kernel's bytes and are bound by HBM, not by launch latency
    big = [(r, s) for r, s in pairs if 2 * 4 * r.numel() >= (32 << 20)] or pairs
    bb = sum(2 * 4 * r.numel() for r, _ in big)
    bms, bl = timed(big)
    ach = bb / (bms * 1e-3) / 1e9
    per_launch = bb / max(bl, 1)
    return {"bound": "hbm", "kernel": "b200::allclose_kernel<float>", "launch_class": "fp32 operand pairs of 32 MiB or more", "achieved": round(ach, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(ach / peaks["hbm_gbs"], 4), "peak_source": peaks["source"], "launches": int(bl), "avg_launch_ms": round(bms / max(bl, 1), 5),
            "algorithmic_bytes_per_launch": int(per_launch), "traffic": int(per_launch * ALLCLOSE_F32_DRAM_PER_ALGORITHMIC_BYTE) if ALLCLOSE_F32_DRAM_PER_ALGORITHMIC_BYTE else None,
            "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one captured launch (128 MiB of operands) scaled by the bytes of the average launch of the class",
            "share_of_kernel_bytes": round(bb / nbytes, 4), "share_of_kernel_time": round(bms / ms, 4),
            "timing": f"the {bl} launches of the class replayed from a CUDA graph between one CUDA-event pair, median of {repeats}", "all_launches": everything}


def cpu_bench_bounded(fn, budget_s=2.0):
    """The harness's CPU timing protocol (BackendBench/eval.py:149-159: 10 warm-up calls, then
    the mean wall time of 100 calls, perf_counter) -- cut down for calls too slow for it: one
    probe call sizes the run so that it stays near `budget_s`, never under 1 warm-up + 3
    timed calls. Returns (seconds per call, warm-up calls, timed calls)."""
    t0 = time.perf_counter()
    fn()
    probe = max(time.perf_counter() - t0, 1e-7)
    runs = int(max(3, min(100, budget_s / probe)))
    warm = int(max(1, min(10, runs // 10)))
    for _ in range(warm - 1):  # the probe was the first warm-up call
        fn()
    t0 = time.perf_counter()
    for _ in range(runs):
        fn()
    return (time.perf_counter() - t0) / runs, warm, runs


def named_config_table(backend, device, peaks, reps, with_cpu=False):
    """Throughput of every named operator configuration, next to aten CUDA on the same
    tensors. Each configuration is instantiated several times (different seeds) until the
    input sets exceed twice the L2 size; `reps` back-to-back launches rotate through the
    sets, captured in a CUDA graph whose replay is timed between one pair of CUDA events (`ms`,
    `aten_cuda_ms`: device time of both); `eager_ms` is the same loop launched from Python. With `with_cpu`, the aten CPU operator is timed on a
    host copy of the first input set by the harness's cpu_bench protocol (all host threads)."""
    from dataclasses import replace

    from backendbench_b200.cases import named_cases
    from backendbench_b200.eval import cuda_bench_rotating
    from backendbench_b200.opregistry import get_operator

    l2_bytes = 126 << 20
    rows = []
    for c in named_cases():
        op = get_operator(c.op)
        impl = backend[op]
        nsets = max(2, min(8, -(-2 * l2_bytes // max(c.algorithmic_bytes(), 1))))
        try:
            sets = [replace(c, seed=c.seed + i).build(device) for i in range(nsets)]
            ms = cuda_bench_rotating([(lambda a=a, k=k: impl(*a, **k)) for a, k in sets], reps=reps, graph=True)
            aten_ms = cuda_bench_rotating([(lambda a=a, k=k: op(*a, **k)) for a, k in sets], reps=reps, graph=True)
            eager_ms = cuda_bench_rotating([(lambda a=a, k=k: impl(*a, **k)) for a, k in sets], reps=reps)
        except Exception as e:  # a failing configuration must not hide the others
            rows.append({"name": c.name, "error": repr(e)[:200]})
            continue
        tensor_bound = c.op in ("mm.default", "addmm.default")
        row = {"name": c.name, "ms": round(ms, 5), "aten_cuda_ms": round(aten_ms, 5), "speedup_vs_aten_cuda": round(aten_ms / ms, 4), "eager_ms": round(eager_ms, 5),
               "bound": "tensor" if tensor_bound else "hbm", "input_sets": nsets}
        gbs = c.algorithmic_bytes() / (ms * 1e-3) / 1e9
        row["gbs"] = round(gbs, 1)
        if c.flops():
            row["tflops"] = round(c.flops() / (ms * 1e-3) / 1e12, 2)
        if tensor_bound:
            row["frac_measured"] = round(row["tflops"] / peaks["bf16_tflops"], 4)
            row["frac_nominal"] = round(row["tflops"] / NOMINAL_BF16_TFLOPS, 4)
        else:
            row["frac_measured"] = round(gbs / peaks["hbm_gbs"], 4)
            row["frac_nominal"] = round(gbs / NOMINAL_HBM_GBS, 4)
        if c.op == "bmm.default" and peaks.get("hbm_write_gbs"):
            # 89 % of this product's bytes are the output: the write-only stream rate is its roof
            row["frac_write_roof"] = round(gbs / peaks["hbm_write_gbs"], 4)
        if with_cpu:
            try:
                cargs = [a.cpu() if isinstance(a, torch.Tensor) else a for a in sets[0][0]]
                ckw = sets[0][1]
                sec, warm, runs = cpu_bench_bounded(lambda: op(*cargs, **ckw))
                row.update({"cpu_ms": round(sec * 1e3, 4), "cpu_protocol": f"{warm} warm-up + {runs} timed calls", "speedup_vs_aten_cpu": round(sec * 1e3 / ms, 1)})
                del cargs
            except Exception as e:
                row["cpu_error"] = repr(e)[:120]
        rows.append(row)
        del sets
        torch.cuda.empty_cache()
    return rows


def geomean(values):
    vals = [v for v in values if v and v > 0]
    if not vals:
        return None
    import math

    return round(math.exp(sum(math.log(v) for v in vals) / len(vals)), 4)


def write_only_stream_gbs(device, nbytes=1 << 30, reps=10):
    """HBM write-only stream rate: this library's own fill kernel (`b200_l2_flush`: 16-byte
    stores, nothing read) over a 1 GiB buffer, best of `reps`, CUDA events."""
    from backendbench_b200 import _abi

    buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream().cuda_stream
    best = None
    for _ in range(reps + 2):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        _abi.check(_abi.lib().b200_l2_flush(buf.data_ptr(), nbytes, stream), "b200_l2_flush")
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        best = ms if best is None else min(best, ms)
    del buf
    return nbytes / (best * 1e-3) / 1e9


_cpu_built = {}


def cpu_reference_cases(cases, stride=1):
    """CPU inputs of every `stride`-th case, built once per process and kept."""
    from backendbench_b200.opregistry import get_operator

    key = (id(cases), stride)
    if key not in _cpu_built:
        _cpu_built[key] = [(get_operator(c.op), *c.build("cpu")) for c in cases[::stride]]
    return _cpu_built[key]


def cpu_reference_pass(built, budget_s=None):
    """The reference's aten-CPU path (AtenBackend through the reference's correctness
    evaluation) over `built` cases, in order, all host threads; stops early only when
    `budget_s` is given and spent. Returns (cases done, seconds)."""
    from oracle.aten_cpu_path import eval_case_cpu

    done, t0 = 0, time.perf_counter()
    for op, args, kwargs in built:
        eval_case_cpu(op, args, kwargs)
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    return done, time.perf_counter() - t0


def full_eval_pass(prepared):
    """The sweep as the harness itself evaluates a case (BackendBench/eval.py:93-126): per case
    the aten reference computed on the device INSIDE the timed region, the backend call, the
    comparison, and one read-back of the verdict, through this package's
    `eval_correctness_test`. Wall clock. Returns (cases/s, passed)."""
    from backendbench_b200.eval import eval_correctness_test

    class Resident:
        def __init__(self, args, kwargs):
            self.args, self.kwargs = args, kwargs

    tests = [(p["op"], p["impl"], Resident(p["args"], p["kwargs"])) for p in prepared]
    for op, impl, t in tests[:: max(len(tests) // 32, 1)]:  # warm both sides' lazy initialisations
        eval_correctness_test(op, impl, t, "dtype")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    passed = sum(bool(eval_correctness_test(op, impl, t, "dtype").is_correct) for op, impl, t in tests)
    torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    return len(tests) / secs, passed


def h2d_only_pass(host_inputs, device):
    """Only the host->device copies of one e2e pass (same pinned buffers, same copy stream, no
    kernels): what the box lets one rank copy while the other ranks do the same."""
    copier = _copy_stream(device)
    copier.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(copier):
        for args in host_inputs:
            for a in args:
                if isinstance(a, torch.Tensor):
                    a.to(device, non_blocking=True)
    torch.cuda.current_stream().wait_stream(copier)


def sharded_sweep(n_workers, cases, timing=True, task_timeout_s=300.0):
    """The 512 cases as per-case tasks in longest-first order through the ONE shared queue of
    `MultiprocessingEvaluator`, worker i on GPU i; each worker generates a case's inputs on its
    own GPU from the seed, computes the aten reference there, runs the backend and compares
    (BackendBench/multiprocessing_eval.py:226-395 driven as scripts/main.py:266-287 drives it).
    Pass 1: correctness only, wall clock from the first dispatch (workers not yet started) to
    the last result. Pass 2, on the same, now warm, workers: correctness + timing of every case."""
    from backendbench_b200.multiprocessing_eval import BackendRef, MultiprocessingEvaluator, SpecTest
    from backendbench_b200.sharding import lpt_order

    order = lpt_order(cases)
    ref = BackendRef("b200")
    out = {"workers": n_workers, "tasks": len(order), "order": "longest first by max(bytes / HBM rate, FLOP / tensor rate)"}
    with MultiprocessingEvaluator(n_workers, backend=ref, task_timeout_s=task_timeout_s) as ev:
        for c in order:
            ev.submit_task(c.op, ref, [SpecTest(c, "cuda")], [], "dtype")
        ev.start_evaluation()
        results = ev.get_results()
        tl = ev.timeline()
        wrong = [order[r.task_id].label() for r in results if r.correctness_score != 1.0]
        steady_n, steady_s = tl.get("results_after_all_ready", 0), tl.get("steady_s", 0.0)
        busy = tl.get("per_worker_busy_s", {})
        out.update({
            "cases_per_sec_wall": round(len(results) / tl["wall_s"], 2), "wall_s": round(tl["wall_s"], 3),
            "startup_s": round(tl["all_workers_ready_s"], 3) if tl.get("all_workers_ready_s") is not None else None,
            "first_result_s": round(tl["first_result_s"], 3),
            "steady_cases_per_sec": round(steady_n / steady_s, 2) if steady_s > 0 else None, "steady_cases": steady_n,
            "per_worker_busy_s": busy, "per_worker_tasks": tl.get("per_worker_tasks", {}),
            "busy_imbalance": round(max(busy.values()) / (sum(busy.values()) / len(busy)), 3) if busy else None,
            "results": len(results), "lost_tasks": len(tl.get("lost_tasks", [])), "restarts": tl.get("restarts", 0),
            "correct": len(results) - len(wrong), "not_close_vs_aten_cuda": wrong[:8],
        })
        if timing:
            t0 = time.monotonic()
            first = ev.next_task_id
            for c in order:
                ev.submit_task(c.op, ref, [SpecTest(c, "cuda")], [SpecTest(c, "cuda")], "dtype")
            timed = ev.get_results()
            secs = time.monotonic() - t0
            sp = [float(q.speedup) for r in timed for q in r.performance_results if q.successfully_ran and q.speedup]
            busy2 = {}
            for r in timed:
                busy2[r.worker_id] = busy2.get(r.worker_id, 0.0) + r.seconds
            out["timed_pass"] = {"cases_per_sec_wall": round(len(timed) / secs, 2), "wall_s": round(secs, 3), "cases": len(timed), "timed_ok": len(sp),
                                 "geomean_speedup_vs_aten_cuda": geomean(sp), "per_worker_busy_s": {int(k): round(v, 3) for k, v in sorted(busy2.items())},
                                 "protocol": "warm workers; per case correctness, then 3 warm-up + 20 timed launches of aten and of the backend, L2 flushed before each"}
            assert first == len(order)
    return out


def run_b200(args):
    from datetime import timedelta

    from backendbench_b200 import _abi
    from backendbench_b200.backends import B200Backend
    from backendbench_b200.cases import sweep_cases
    from backendbench_b200.ops import check_device_status
    from backendbench_b200.sharding import barrier, lpt_order, max_over_ranks, shard_for_rank, sum_over_ranks

    rank, local, world = _dist_env()
    host_group = None
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
        # a host-side group: ranks that only wait (while rank 0 drives the worker processes of the
        # sharded sweep) must not sit in an NCCL kernel on a GPU a worker is using
        host_group = torch.distributed.new_group(backend="gloo", timeout=timedelta(minutes=30))
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    peaks = measured_peaks()
    backend = B200Backend()
    _abi.lib()  # fail loudly here if the CUDA library is missing

    cases = sweep_cases(N_CASES, SWEEP_SEED)
    mine = shard_for_rank(cases, rank, world, "weak")
    prepared = prepare_cases(mine, backend, device)
    records = torch.zeros(len(prepared), 8, dtype=torch.int32, device=device)

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    # Warm up eagerly (also sizes every scratch buffer), then capture the launch sequence of
    # one pass -- ~1100 small kernels whose eager cost is host dispatch, not GPU time -- in a
    # CUDA graph; a timed step replays the graph and reads the verdict records back.
    eager_ms, _ = time_steps(lambda: sweep_pass(prepared, records), 1, max(args.warmup, 2))
    streams = [torch.cuda.Stream(device=device) for _ in range(args.sweep_streams)] if args.sweep_streams > 1 else None

    def capture(subset, recs):
        if args.no_graph:
            return None, None
        try:
            if streams:  # one eager multi-stream pass sizes the per-stream scratch buffers
                sweep_enqueue(subset, recs, streams)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                st = sweep_enqueue(subset, recs, streams)
            torch.cuda.synchronize()
            return g, st
        except Exception as e:  # capture is an optimisation: fall back to eager launches
            print(f"[bench] CUDA graph capture failed, timing eager launches: {e!r}", file=sys.stderr)
            torch.cuda.synchronize()
            return None, None

    graph, structural = capture(prepared, records)

    def graph_step():
        graph.replay()
        return records.cpu(), structural

    step = graph_step if graph is not None else (lambda: sweep_pass(prepared, records))
    total_ms, last = time_steps(step, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    launches0 = _abi.lib().b200_launch_count()  # one more (untimed) pass, only to count its launches
    sweep_pass(prepared, records)
    launches = (_abi.lib().b200_launch_count() - launches0) * args.steps
    check_device_status(torch.device(device))
    n_ok, bad = count_correct(*last)
    units = sum_over_ranks(float(len(prepared) * args.steps))
    value = units / (total_ms * 1e-3)
    step_ms = total_ms / args.steps

    # ---- strong scaling: the ONE sweep dealt over the ranks, longest first (rank r replays
    # cases r, r+N, ... of that order); time = max over ranks, units = 512 per step
    strong = None
    if not args.sweep_only:
        by_id = {p["case"].case_id: p for p in prepared}
        my_part = [by_id[c.case_id] for c in lpt_order(cases)[rank::world]]
        part_records = torch.zeros(len(my_part), 8, dtype=torch.int32, device=device)
        g2, st2 = capture(my_part, part_records) if world > 1 else (graph, structural)

        def part_step():
            g2.replay()
            return part_records.cpu(), st2

        if world == 1:
            strong_ms = total_ms
        else:
            strong_ms, _ = time_steps(part_step if g2 is not None else (lambda: sweep_pass(my_part, part_records)), args.steps, args.warmup)
        strong = {"value": round(N_CASES * args.steps / (strong_ms * 1e-3), 2), "unit": "cases/s", "ms_per_step": round(strong_ms / args.steps, 3), "cases_this_rank": len(my_part),
                  "what": "512 cases in total, dealt longest-first round-robin over the ranks; device time, max over ranks"}
        del g2, part_records

    # ---- the harness's own per-case evaluation (reference computed inside the timed region)
    full_eval = None
    if not args.sweep_only:
        rate, passed = full_eval_pass(prepared)
        rate_sum = sum_over_ranks(rate)
        full_eval = {"value": round(rate_sum, 2), "unit": "cases/s", "passed_rank0": f"{passed}/{len(prepared)}",
                     "what": "eval_correctness_test per case: aten CUDA reference inside the timed region + backend + compare + one read-back per case; wall clock, inputs resident; sum over ranks"}

    # ---- end to end: pinned host inputs, H2D inside the timed region
    e2e = None
    need_host = sum(_bytes_of(p["args"]) for p in prepared)
    # one decision for all ranks (each looks at the free memory at a slightly different moment;
    # a split decision would leave some ranks alone in the collectives of the timed passes)
    host_ok = args.sweep_only or sum_over_ranks(1.0 if _host_memory_allows(need_host, world) else 0.0) == float(world)
    if not args.sweep_only and not host_ok:
        e2e = {"skipped": f"host memory: {world} rank(s) x {need_host} bytes of pinned inputs do not fit what this box offers"}
    elif not args.sweep_only:
        host_inputs = [[a.cpu().pin_memory() if isinstance(a, torch.Tensor) else a for a in p["args"]] for p in prepared]
        h2d = sum(_bytes_of(h) for h in host_inputs)
        e2e_steps = max(1, min(args.steps, 3))
        e2e_ms, _ = time_steps(lambda: sweep_pass(prepared, records, host_inputs, device), e2e_steps, 1)
        e2e_units = sum_over_ranks(float(len(prepared) * e2e_steps))
        copy_ms, _ = time_steps(lambda: h2d_only_pass(host_inputs, device), e2e_steps, 1)
        agg_gbs = sum_over_ranks(float(h2d)) * e2e_steps / (copy_ms * 1e-3) / 1e9
        e2e = {"value": round(e2e_units / (e2e_ms * 1e-3), 2), "unit": "cases/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(records.numel() * 4), "steps": e2e_steps,
               "h2d_gbs_all_ranks": round(sum_over_ranks(float(h2d)) * e2e_steps / (e2e_ms * 1e-3) / 1e9, 1),
               "h2d_only_gbs_all_ranks": round(agg_gbs, 1), "frac_of_copy_ceiling": round(copy_ms / e2e_ms, 4),
               "copy_ceiling": "the same pinned buffers copied on the same stream with no kernels queued, all ranks at once"}
        del host_inputs

    line = {
        "metric": "sweep_cases_per_sec", "value": round(value, 2), "unit": "cases/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(step_ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32/bf16/f16 (fp32 accumulate)",
        "data": "synthetic", "impl": "b200",
        "config": common_config(len(prepared)),
        "arm": {"launches": f"one pass captured in a CUDA graph of {len(streams) if streams else 1} parallel branch(es) (case i on branch i mod n) and replayed per step (eager_cases_per_sec: the same pass launched from Python on one stream)",
                "inputs": "resident in HBM (about 10 GB per rank)", "reference_results": "aten CUDA (aten CPU for scatter_add), PRECOMPUTED and resident: `value` times backend + compare only; `full_eval` computes the reference inside its timed region",
                "parallelism": f"{world} independent rank(s), every rank a full sweep of its own (weak), no collective"},
        "sweep_correct": f"{n_ok}/{len(prepared)}", "launch_mode": "cuda_graph_replay" if graph is not None else "eager", "eager_cases_per_sec": round(len(prepared) / (eager_ms * 1e-3), 2),
        "e2e": e2e, "full_eval": full_eval, "strong_scaling": strong, "gpu_launches": int(launches), "clocks": clocks,
    }
    if bad:
        line["sweep_failed_cases"] = [prepared[i]["case"].label() for i in bad[:12]]

    if rank == 0 and not args.sweep_only:
        by_op, slowest, total_dev_ms, dropped = per_kernel_profile(prepared, step_ms)
        line["sweep_slowest_cases"] = slowest
        line["sweep_device_ms_sum"] = total_dev_ms
        if dropped:
            line["sweep_profile_dropped_cases"] = dropped
        total = sum(d["ms"] for d in by_op.values()) or 1.0
        line["sweep_time_share_by_op"] = {op: round(d["ms"] / total, 4) for op, d in sorted(by_op.items(), key=lambda kv: -kv[1]["ms"])}
        line["roofline"] = compare_kernel_roofline(prepared, peaks)
        peaks["hbm_write_gbs"] = write_only_stream_gbs(device)
        line["hbm_write_only_gbs"] = round(peaks["hbm_write_gbs"], 1)
        line["per_op"] = named_config_table(backend, device, peaks, reps=40, with_cpu=(world == 1))
        line["geomean_speedup_vs_aten"] = geomean([r.get("speedup_vs_aten_cuda") for r in line["per_op"]])
        if world == 1:
            line["geomean_speedup_vs_aten_cpu"] = geomean([r.get("speedup_vs_aten_cpu") for r in line["per_op"]])
            line["cpu_cores"] = torch.get_num_threads()
            built = cpu_reference_cases(cases, stride=8)
            done, secs = cpu_reference_pass(built, budget_s=25.0)
            line["cpu_baseline"] = {"value": round(done / secs, 2), "unit": "cases/s", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"every 8th sweep case in order ({done} of {len(built)} run within 25 s), aten CPU through the reference's correctness evaluation, {torch.get_num_threads()} threads"}

    # ---- the sharded sweep proper: rank 0 drives one worker process per GPU; the other ranks
    # release their memory and wait on the host
    if not args.sweep_only and not args.no_sharded:
        del prepared, graph, records
        torch.cuda.empty_cache()
        if host_group is not None:
            torch.distributed.barrier(group=host_group)
        if rank == 0:
            try:
                line["sharded_sweep"] = sharded_sweep(world, cases)
                line["sharded_sweep"]["efficiency_note"] = "efficiency_vs_1 = value at N / (N x value at 1): computed by whoever holds the per-N lines"
            except Exception as e:
                line["sharded_sweep"] = {"error": repr(e)[:300]}
        if host_group is not None:
            torch.distributed.barrier(group=host_group)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


# ------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The reference's own CPU path over the SAME 512 cases per step as the b200 arm: inputs
    built once on the CPU from the same seeds, then per step every case through AtenBackend +
    the reference's correctness evaluation on all host threads. A wall-clock budget bounds the
    run: when W + K full passes would not fit, fewer are run and the line says so."""
    rank, _, world = _dist_env()
    if rank != 0:
        return  # the CPU arm runs once per job
    from backendbench_b200.cases import sweep_cases

    # torchrun exports OMP_NUM_THREADS=1 for its ranks; this arm runs on rank 0 alone and is
    # meant to use every host core the box has
    torch.set_num_threads(max(os.cpu_count() or 1, 1))
    t_begin = time.perf_counter()
    cases = sweep_cases(N_CASES, SWEEP_SEED)
    built = cpu_reference_cases(cases)
    budget_s = args.reference_budget_s
    warm_done = 0
    last = None
    for _ in range(args.warmup):
        if last is not None and time.perf_counter() - t_begin + (args.steps + 1) * last > budget_s:
            break  # keep the budget for the timed passes
        _, last = cpu_reference_pass(built)
        warm_done += 1
    steps_done, done_total, t_total = 0, 0, 0.0
    for _ in range(args.steps):
        if steps_done and time.perf_counter() - t_begin + 1.1 * (t_total / steps_done) > budget_s:
            break
        done, secs = cpu_reference_pass(built)
        steps_done += 1
        done_total += done
        t_total += secs
    value = done_total / t_total
    cores = torch.get_num_threads()
    sample = f"all {len(built)} sweep cases per step, {steps_done} timed + {warm_done} warm-up passes" + ("" if steps_done == args.steps and warm_done == args.warmup else f" (of {args.steps} + {args.warmup} asked: bounded by a {budget_s:.0f} s budget)") + f", aten CPU through the reference's correctness evaluation, {cores} threads"
    line = {
        "metric": "sweep_cases_per_sec", "value": round(value, 2), "unit": "cases/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "steps_run": steps_done, "warmup_run": warm_done,
        "ms_per_step": round(t_total / steps_done * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32/bf16/f16 (fp32 accumulate)", "data": "synthetic", "impl": "reference",
        "config": common_config(len(built)),
        "arm": {"parallelism": f"host cores, one process, {cores} threads", "inputs": "resident in host memory", "reference_results": "computed inside the timed region, twice per case (reference and AtenBackend implementation), as the harness does"},
        "cpu_baseline": {"value": round(value, 2), "unit": "cases/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 2), "unit": "cases/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of replaying a CUDA graph of the pass")
    ap.add_argument("--sweep-streams", type=int, default=8, help="parallel branches of the captured sweep graph (1 = one chain)")
    ap.add_argument("--no-sharded", action="store_true", help="skip the MultiprocessingEvaluator pass (one worker process per GPU)")
    ap.add_argument("--reference-budget-s", type=float, default=900.0, help="wall-clock bound of the --impl reference run")
    ap.add_argument("--sweep-only", action="store_true", help="time the sweep only (no e2e pass, per-op table or CPU sample): the short run used for profiler launch lists")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl b200 needs a CUDA device; there is no CPU fallback")
    run_b200(args)


if __name__ == "__main__":
    main()
