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

The JSON line also carries: `e2e` (the same pass through the public plugin call with the
inputs in pinned HOST memory, H2D copies and the verdict read-back inside the timed
region), `roofline` (the operator with the largest share of device time in the sweep, its
cases classed by the roof that binds them),
`per_op` (every named operator configuration: GB/s or TFLOP/s against the measured and
nominal peaks, and the speed-up over aten CUDA), `cpu_baseline` (the reference's aten-CPU
path on a bounded sample, host cores), `clocks` and `gpu_launches`.

`--impl reference` times the reference's own CPU path (AtenBackend + the reference's
correctness evaluation, restated in oracle/aten_cpu_path.py) on a bounded sample.
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
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu_index)],
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


def per_kernel_profile(prepared):
    """Device time of every case's backend launch (CUDA events, L2 flushed before each)
    aggregated per operator: the share table and the dominant kernel's roofline input."""
    from backendbench_b200.eval import l2_flush

    by_op = {}
    n = len(prepared)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
    for i, p in enumerate(prepared):
        l2_flush()
        starts[i].record()
        p["impl"](*p["args"], **p["kwargs"])
        ends[i].record()
    torch.cuda.synchronize()
    per_case = []
    for i, p in enumerate(prepared):
        c = p["case"]
        per_case.append((starts[i].elapsed_time(ends[i]), c.label() + (" " + str(dict(c.extra)) if c.extra else "")))
        d = by_op.setdefault(c.op, {"ms": 0.0, "bytes": 0, "flops": 0, "launches": 0, "cases": []})
        d["ms"] += starts[i].elapsed_time(ends[i])
        d["bytes"] += c.algorithmic_bytes()
        d["flops"] += c.flops()
        d["launches"] += 1
        d["cases"].append((starts[i].elapsed_time(ends[i]), c.algorithmic_bytes(), c.flops()))
    per_case.sort(reverse=True)
    by_op["__slowest__"] = [{"ms": round(ms, 3), "case": label} for ms, label in per_case[:12]]
    by_op["__total_ms__"] = round(sum(ms for ms, _ in per_case), 3)
    return by_op


def named_config_table(backend, device, peaks, reps):
    """Throughput of every named operator configuration, next to aten CUDA on the same
    tensors. Each configuration is instantiated several times (different seeds) until the
    input sets exceed twice the L2 size; `reps` back-to-back launches rotate through the
    sets between one pair of CUDA events."""
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
            ms = cuda_bench_rotating([(lambda a=a, k=k: impl(*a, **k)) for a, k in sets], reps=reps)
            aten_ms = cuda_bench_rotating([(lambda a=a, k=k: op(*a, **k)) for a, k in sets], reps=reps)
        except Exception as e:  # a failing configuration must not hide the others
            rows.append({"name": c.name, "error": repr(e)[:200]})
            continue
        tensor_bound = c.op in ("mm.default", "addmm.default")
        row = {"name": c.name, "ms": round(ms, 5), "aten_cuda_ms": round(aten_ms, 5), "speedup_vs_aten_cuda": round(aten_ms / ms, 4), "bound": "tensor" if tensor_bound else "hbm", "input_sets": nsets}
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
        rows.append(row)
        del sets
        torch.cuda.empty_cache()
    return rows


def cpu_reference_sample(cases, budget_s):
    """The reference's aten-CPU path over a bounded sample of the sweep (every 8th case, in
    order, until `budget_s` of CPU time is spent). Returns (cases done, seconds, description)."""
    from backendbench_b200.opregistry import get_operator
    from oracle.aten_cpu_path import eval_case_cpu, host_threads

    sample = cases[::8]
    built = []
    for c in sample:
        if c.flops() > 4e10 or c.algorithmic_bytes() > (1 << 28):
            continue  # bounded: skip the few cases that alone would take the CPU many seconds
        built.append((get_operator(c.op), *c.build("cpu")))
    done, t0 = 0, time.perf_counter()
    for op, args, kwargs in built:
        eval_case_cpu(op, args, kwargs)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    secs = time.perf_counter() - t0
    desc = f"every 8th sweep case in order, skipping cases above 4e10 FLOP or 256 MiB ({done} of {len(built)} eligible run within {budget_s:.0f} s), aten CPU, {host_threads()} threads"
    return done, secs, desc, host_threads()


def run_b200(args):
    from backendbench_b200 import _abi
    from backendbench_b200.backends import B200Backend
    from backendbench_b200.cases import sweep_cases
    from backendbench_b200.ops import check_device_status
    from backendbench_b200.sharding import shard_for_rank, sum_over_ranks

    rank, local, world = _dist_env()
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
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
    graph, structural = None, None
    streams = [torch.cuda.Stream(device=device) for _ in range(args.sweep_streams)] if args.sweep_streams > 1 else None
    if not args.no_graph:
        try:
            if streams:  # one eager multi-stream pass sizes the per-stream scratch buffers
                sweep_enqueue(prepared, records, streams)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                structural = sweep_enqueue(prepared, records, streams)
            torch.cuda.synchronize()
        except Exception as e:  # capture is an optimisation: fall back to eager launches
            print(f"[bench] CUDA graph capture failed, timing eager launches: {e!r}", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

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

    # ---- end to end: pinned host inputs, H2D inside the timed region
    e2e = None
    need_host = sum(_bytes_of(p["args"]) for p in prepared)
    if not args.sweep_only and not _host_memory_allows(need_host, world):
        e2e = {"skipped": f"host memory: {world} rank(s) x {need_host} bytes of pinned inputs do not fit what this box offers"}
    elif not args.sweep_only:
        host_inputs = [[a.cpu().pin_memory() if isinstance(a, torch.Tensor) else a for a in p["args"]] for p in prepared]
        h2d = sum(_bytes_of(h) for h in host_inputs)
        e2e_steps = max(1, min(args.steps, 3))
        e2e_ms, _ = time_steps(lambda: sweep_pass(prepared, records, host_inputs, device), e2e_steps, 1)
        e2e_units = sum_over_ranks(float(len(prepared) * e2e_steps))
        e2e = {"value": round(e2e_units / (e2e_ms * 1e-3), 2), "unit": "cases/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(records.numel() * 4), "steps": e2e_steps}
        del host_inputs

    line = {
        "metric": "sweep_cases_per_sec", "value": round(value, 2), "unit": "cases/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(total_ms / args.steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32/bf16/f16 (fp32 accumulate)",
        "data": "synthetic", "impl": "b200",
        "config": {"workload": "sharded sweep: 512 seeded (op, shape, dtype) cases over 16 aten overloads, 2^8..2^26 elements, 15% edge cases; one correctness pass per step",
                   "cases_per_rank": len(prepared), "launches": f"one pass captured in a CUDA graph of {len(streams) if streams else 1} parallel branch(es) (case i on branch i mod n) and replayed per step (eager_cases_per_sec: the same pass launched from Python on one stream)", "inputs": "resident in HBM, larger than L2 in total (about 10 GB per rank)", "reference_results": "aten CUDA (aten CPU for scatter_add), precomputed, resident",
                   "parallelism": f"{world} independent rank(s), no collective"},
        "sweep_correct": f"{n_ok}/{len(prepared)}", "launch_mode": "cuda_graph_replay" if graph is not None else "eager", "eager_cases_per_sec": round(len(prepared) / (eager_ms * 1e-3), 2), "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
    }
    if bad:
        line["sweep_failed_cases"] = [prepared[i]["case"].label() for i in bad[:12]]

    if rank == 0:
        by_op = per_kernel_profile(prepared)
        line["sweep_slowest_cases"] = by_op.pop("__slowest__")
        line["sweep_device_ms_sum"] = by_op.pop("__total_ms__")
        total = sum(d["ms"] for d in by_op.values()) or 1.0
        shares = {op: round(d["ms"] / total, 4) for op, d in sorted(by_op.items(), key=lambda kv: -kv[1]["ms"])}
        top_op, top = max(by_op.items(), key=lambda kv: kv[1]["ms"])
        # The dominant operator's cases are a mix of shapes: each case is bound by whichever
        # roof it would hit first (its algorithmic bytes at the HBM peak or its FLOP at the
        # tensor peak). The roofline line describes the class that holds more of the
        # operator's device time; the other class is listed beside it.
        classes = {"hbm": {"ms": 0.0, "units": 0.0, "launches": 0}, "tensor": {"ms": 0.0, "units": 0.0, "launches": 0}}
        for ms, nbytes, flops in top["cases"]:
            t_hbm, t_tc = nbytes / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12)
            k = "tensor" if t_tc > t_hbm else "hbm"
            classes[k]["ms"] += ms
            classes[k]["units"] += flops if k == "tensor" else nbytes
            classes[k]["launches"] += 1
        bound = max(classes, key=lambda k: classes[k]["ms"])

        def describe(k):
            c = classes[k]
            if not c["launches"]:
                return None
            scale, peak, unit = (1e12, peaks["bf16_tflops"], "TFLOP/s") if k == "tensor" else (1e9, peaks["hbm_gbs"], "GB/s")
            ach = c["units"] / (c["ms"] * 1e-3) / scale
            return {"bound": k, "achieved": round(ach, 2), "peak": peak, "unit": unit, "frac": round(ach / peak, 4), "launches": c["launches"], "avg_launch_ms": round(c["ms"] / c["launches"], 4),
                    "share_of_op_time": round(c["ms"] / top["ms"], 4)}

        roof = describe(bound)
        other = describe("hbm" if bound == "tensor" else "tensor")
        roof.update({"kernel": top_op, "peak_source": peaks["source"], "traffic": None, "other_class": other})
        line["roofline"] = roof
        line["sweep_time_share_by_op"] = shares
        if not args.sweep_only:
            line["per_op"] = named_config_table(backend, device, peaks, reps=40)
        if world == 1 and not args.sweep_only:
            done, secs, desc, cores = cpu_reference_sample(cases, budget_s=20.0)
            line["cpu_baseline"] = {"value": round(done / secs, 2), "unit": "cases/s", "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


# ------------------------------------------------------------------------- reference arm
def run_reference(args):
    rank, _, world = _dist_env()
    if rank != 0:
        return  # the CPU arm runs once per job
    from backendbench_b200.cases import sweep_cases

    # torchrun exports OMP_NUM_THREADS=1 for its ranks; this arm runs on rank 0 alone and is
    # meant to use every host core the box has
    torch.set_num_threads(max(os.cpu_count() or 1, 1))
    cases = sweep_cases(N_CASES, SWEEP_SEED)
    per_step_budget = max(5.0, min(30.0, 150.0 / max(args.steps + args.warmup, 1)))
    for _ in range(args.warmup):
        cpu_reference_sample(cases, per_step_budget)
    done_total, t_total, desc, cores = 0, 0.0, "", 0
    for _ in range(args.steps):
        done, secs, desc, cores = cpu_reference_sample(cases, per_step_budget)
        done_total += done
        t_total += secs
    value = done_total / t_total
    line = {
        "metric": "sweep_cases_per_sec", "value": round(value, 2), "unit": "cases/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(t_total / args.steps * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32/bf16/f16", "data": "synthetic", "impl": "reference",
        "config": {"workload": "sharded sweep: 512 seeded (op, shape, dtype) cases; bounded CPU sample per step", "parallelism": "host cores, one process"},
        "cpu_baseline": {"value": round(value, 2), "unit": "cases/s", "cores": cores, "kind": "port", "sample": desc},
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
