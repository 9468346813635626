"""Command line driver: build a suite and a backend, evaluate every operator the backend
implements (serially or one process per GPU) and print the three summary scores.

Mirrors the hot-path part of BackendBench/scripts/main.py:186-303 with the same flag names
(`--suite --backend --ops --ops-directory --num-workers --p --log-level --log-dir
--daemon/--no-daemon`).
Suites here are the seeded ones this package can generate offline, plus `torchbench` over a
LOCAL trace / parquet file (`--alternative-torchbench-data-path`): `smoke` (one relu case,
as the reference's smoke suite), `named` (the per-operator configurations throughput is
quoted on) and `sweep` (the 512-case sharded sweep). Backends: `aten`, `directory`
(`--ops-directory`), `b200` (the kernels shipped with this package).

    python -m backendbench_b200.scripts.main --suite sweep --backend b200 --num-workers 8
"""

from __future__ import annotations

import json
import logging
import os
import sys
from dataclasses import asdict

import click
import torch

from .. import eval as evaluation
from ..backends import make_backend
from ..cases import named_cases, sweep_cases
from ..multiprocessing_eval import BackendRef, MultiprocessingEvaluator, SpecTest
from ..opregistry import get_operator
from ..sharding import estimated_seconds
from ..suite import OpTest, TestSuite, make_smoke_suite

logger = logging.getLogger(__name__)


def build_suite(name: str, device: str, ops=None, n_cases: int = 512) -> TestSuite:
    """`smoke`: thunk-based tensors on `device`; `named` / `sweep`: one OpTest per operator whose
    tests are `SpecTest` descriptors (inputs generated on the evaluating device from the seed)."""
    if name == "smoke":
        return make_smoke_suite(device)
    specs = named_cases() if name == "named" else sweep_cases(n_cases)
    by_op = {}
    for c in specs:
        if ops and c.op not in ops and c.op.split(".")[0] not in ops:
            continue
        by_op.setdefault(c.op, []).append(c)
    optests = []
    for op_name, cs in by_op.items():
        tests = [SpecTest(c, device) for c in cs]
        perf = tests if name == "named" else tests[:: max(len(tests) // 4, 1)][:4]
        optests.append(OpTest(get_operator(op_name), tests, perf))
    return TestSuite(name, optests)


def task_units(suite, backend):
    """(op, correctness tests, performance tests) per task for the multi-worker run. An
    operator whose tests are all `SpecTest` descriptors is cut into one task per CASE and
    the tasks of all operators are ordered longest first (estimated from the case's bytes
    and FLOP), so the shared queue balances the GPUs; other operators stay one task each,
    at the front (their cost is unknown), as BackendBench/scripts/main.py:266-287 submits them."""
    whole, units = [], []
    for test in suite:
        if test.op not in backend:
            continue
        ctests, ptests = list(test.correctness_tests), list(test.performance_tests)
        if ctests and all(isinstance(t, SpecTest) for t in ctests + ptests):
            timed = {t.spec for t in ptests}
            seen = set()
            for t in ctests:
                seen.add(t.spec)
                units.append((estimated_seconds(t.spec) * (50 if t.spec in timed else 1), test.op, [t], [t] if t.spec in timed else []))
            for t in ptests:
                if t.spec not in seen:
                    units.append((estimated_seconds(t.spec) * 50, test.op, [], [t]))
        else:
            whole.append((test.op, ctests, ptests))
    units.sort(key=lambda u: -u[0])
    return whole + [(op, c, q) for _, op, c, q in units]


def _unit_key(op, ctests, ptests) -> str:
    """What identifies a unit of work across runs: the operator and its test descriptors."""
    def one(t):
        if isinstance(t, SpecTest):
            return f"{t.spec.label()}#{t.spec.seed}"
        return getattr(t, "serialized", None) or repr(type(t).__name__)

    name = getattr(op, "__name__", str(op))
    return name + "|" + ";".join(one(t) for t in ctests) + "|" + ";".join(one(t) for t in ptests)


class Checkpoint:
    """One JSON line per finished unit of work (an operator, or one case of a descriptor
    suite): its key, the operator's name and its result records. The reference writes its
    results once, at the end of the run (BackendBench/scripts/main.py:315); a 512-case sweep on
    eight GPUs that dies at case 500 should not start over. `--resume` reads the file back and
    evaluates only the units that are not in it."""

    def __init__(self, path, resume=False):
        self.path = path
        self.done = {}
        if resume and path and os.path.exists(path):
            with open(path) as fh:
                for line in fh:
                    line = line.strip()
                    if not line:
                        continue
                    try:
                        row = json.loads(line)
                    except ValueError:  # a line cut short by the crash that made the resume necessary
                        continue
                    self.done[row["key"]] = row
        elif path:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            open(path, "w").close()

    def record(self, key, op_name, performance_score, cres, pres):
        row = {"key": key, "op": op_name, "performance_score": performance_score, "correctness": [asdict(c) for c in cres], "performance": [asdict(q) for q in pres]}
        self.done[key] = row
        if self.path:
            with open(self.path, "a") as fh:
                fh.write(json.dumps(row, default=str) + "\n")

    @staticmethod
    def results_of(row):
        cres = [evaluation.CorrectnessTestResult(**c) for c in row["correctness"]]
        pres = [evaluation.PerformanceTestResult(**q) for q in row["performance"]]
        return row["performance_score"], cres, pres


def run(suite, backend, backend_ref, num_workers=None, daemon=True, p=1.0, tolerances=None, checkpoint=None):
    """Evaluate `suite` on `backend`; returns (mean correctness, geomean perf, perf@p, results).
    With a `Checkpoint`, finished units are appended to its file as they come in and units
    already in it (a resumed run) are not evaluated again."""
    overall_correctness, overall_performance, all_c, all_p = [], [], [], []
    ck = checkpoint or Checkpoint(None)
    by_op = {}  # operator -> [(performance score, correctness results, performance results)]
    if num_workers is None:
        for test in suite:
            if test.op not in backend:
                continue
            ctests, ptests = list(test.correctness_tests), list(test.performance_tests)
            key = _unit_key(test.op, ctests, ptests)
            if key in ck.done:
                by_op.setdefault(test.op, []).append(Checkpoint.results_of(ck.done[key]))
                continue
            _, perf, cres, pres = evaluation.eval_one_op(test.op, backend[test.op], ctests, ptests, tolerances)
            ck.record(key, getattr(test.op, "__name__", str(test.op)), float(perf), cres, pres)
            by_op.setdefault(test.op, []).append((float(perf), cres, pres))
    else:
        units = task_units(suite, backend)
        pending = []
        for op, ctests, ptests in units:
            key = _unit_key(op, ctests, ptests)
            if key in ck.done:
                by_op.setdefault(op, []).append(Checkpoint.results_of(ck.done[key]))
            else:
                pending.append((key, op, ctests, ptests))
        if pending:
            with MultiprocessingEvaluator(num_workers, daemon=daemon, backend=backend_ref) as evaluator:
                unit_of_task = {}
                for key, op, ctests, ptests in pending:
                    tid = evaluator.submit_task(op, backend_ref if backend_ref is not None else backend[op], ctests, ptests, tolerances)
                    unit_of_task[tid] = (key, op)
                evaluator.start_evaluation()
                results = evaluator.get_results()
            for r in results:  # one task per CASE for descriptor suites: put the operator back together
                key, op = unit_of_task[r.task_id]
                ck.record(key, getattr(op, "__name__", str(op)), float(r.performance_score), r.correctness_results, r.performance_results)
                by_op.setdefault(op, []).append((float(r.performance_score), r.correctness_results, r.performance_results))
    for op, rs in by_op.items():
        cres = [c for _, cs, _ in rs for c in cs]
        pres = [q for _, _, ps in rs for q in ps]
        overall_correctness.append(all(c.is_correct for c in cres))
        if len(rs) == 1:
            overall_performance.append(float(rs[0][0]))
        elif pres:  # as eval_performance scores an operator: geomean over its cases, a failed case counts 1.0
            sp = torch.tensor([float(q.speedup) if (q.successfully_ran and q.speedup) else 1.0 for q in pres], dtype=torch.float64)
            overall_performance.append(float(sp.log().mean().exp()))
        else:
            overall_performance.append(float("nan"))
        all_c.extend(cres)
        all_p.extend(pres)
    if not overall_correctness:
        return 0.0, 1.0, 0.0, (all_c, all_p)
    mean_correctness = torch.tensor(overall_correctness).float().mean().item()
    perf_t = torch.tensor(overall_performance, dtype=torch.float64)
    perf_t = torch.where(torch.isnan(perf_t), torch.ones_like(perf_t), perf_t)  # operators without performance cases
    geomean_perf = perf_t.log().mean().exp().item()
    perf_at_p = float(evaluation.perf_at_p(overall_correctness, perf_t.tolist(), p))
    return mean_correctness, geomean_perf, perf_at_p, (all_c, all_p)


@click.command()
@click.option("--log-level", default=os.getenv("LOG_LEVEL", "INFO"), type=click.Choice(["DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"], case_sensitive=False), help="Set the logging level")
@click.option("--suite", default="smoke", type=click.Choice(["smoke", "named", "sweep", "torchbench"]), help="Which suite to run")
@click.option("--alternative-torchbench-data-path", default=None, type=str, help="Local .txt trace or .parquet table for --suite torchbench (nothing is downloaded)")
@click.option("--topn-inputs", "--topn", default=None, type=int, help="Largest N recorded inputs per operator (torchbench suite)")
@click.option("--backend", default="aten", type=click.Choice(["aten", "directory", "b200"]), help="Which backend to run")
@click.option("--ops", default=None, type=str, help="Comma-separated list of ops to run")
@click.option("--ops-directory", default="generated_kernels", type=str, help="Path to directory containing kernels (directory backend)")
@click.option("--num-workers", default=None, type=int, help="Number of worker processes (one per GPU); default: evaluate in this process")
@click.option("--p", default=1.0, type=float, help="Performance score threshold for the perf@p score")
@click.option("--device", default=None, type=str, help="Device for the generated inputs (default: cuda when available, else cpu)")
@click.option("--cases", default=512, type=int, help="Number of cases of the sweep suite")
@click.option("--dtype-tolerances/--harness-tolerances", default=False, help="Per-dtype tolerances instead of the harness's 1e-2 for everything")
@click.option("--daemon/--no-daemon", default=True, help="Use daemon worker processes")
@click.option("--log-dir", default=None, type=str, help="Directory for the report artefacts (full_results.json, operator_summary.csv, failed_tests.json, OVERALL_SUMMARY.md); none written when omitted")
@click.option("--checkpoint", default=None, type=str, help="Append one JSON line per finished unit of work to this file (with --resume and --log-dir the default is <log-dir>/results.jsonl)")
@click.option("--resume/--no-resume", default=False, help="Skip the units already recorded in the checkpoint file and merge their results")
def cli(log_level, suite, alternative_torchbench_data_path, topn_inputs, backend, ops, ops_directory, num_workers, p, device, cases, dtype_tolerances, daemon, log_dir, checkpoint, resume):
    logging.basicConfig(level=getattr(logging, log_level.upper()), format="[%(asctime)s][%(levelname)s][%(filename)s] %(message)s", datefmt="%Y-%m-%d %H:%M:%S")
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    op_filter = [o.strip() for o in ops.split(",")] if ops else None
    if suite == "torchbench":
        if not alternative_torchbench_data_path:
            raise click.UsageError("--suite torchbench needs --alternative-torchbench-data-path FILE (a local .txt trace or .parquet table; the public dataset is not fetched)")
        from ..trace_suite import TraceTestSuite

        test_suite = TraceTestSuite("torchbench", alternative_torchbench_data_path, op_filter, topn_inputs)
    else:
        test_suite = build_suite(suite, device, op_filter, cases)
    be = make_backend(backend, ops_directory)
    ref = BackendRef(backend, ops_directory if backend == "directory" else None)
    if checkpoint is None and log_dir and resume:
        checkpoint = os.path.join(log_dir, "results.jsonl")
    ck = Checkpoint(checkpoint, resume) if checkpoint else None
    if ck is not None and resume:
        print(f"resuming: {len(ck.done)} finished unit(s) found in {checkpoint}")
    mean_correctness, geomean_perf, perf_at_p, (all_c, all_p) = run(test_suite, be, ref, num_workers, daemon, p, "dtype" if dtype_tolerances else None, ck)
    if log_dir:
        from ..output import save_results

        save_results(all_c, all_p, log_dir, "python -m backendbench_b200.scripts.main " + " ".join(sys.argv[1:]), mean_correctness, geomean_perf, perf_at_p, p)
    print(f"correctness score (mean pass rate over all operators): {mean_correctness:.2f}")
    print(f"performance score (geomean speedup over all operators): {geomean_perf:.2f}")
    print(f"perf@p score (rate of correct samples with a speedup greater than p, p={p}): {perf_at_p:.2f}")


if __name__ == "__main__":
    cli()
