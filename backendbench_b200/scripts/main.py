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

import logging
import os
import sys

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


def run(suite, backend, backend_ref, num_workers=None, daemon=True, p=1.0, tolerances=None):
    """Evaluate `suite` on `backend`; returns (mean correctness, geomean perf, perf@p, results)."""
    overall_correctness, overall_performance, all_c, all_p = [], [], [], []
    if num_workers is None:
        for test in suite:
            if test.op not in backend:
                continue
            _, perf, cres, pres = evaluation.eval_one_op(test.op, backend[test.op], test.correctness_tests, test.performance_tests, tolerances)
            overall_correctness.append(all(r.is_correct for r in cres))
            overall_performance.append(float(perf))
            all_c.extend(cres)
            all_p.extend(pres)
    else:
        with MultiprocessingEvaluator(num_workers, daemon=daemon, backend=backend_ref) as evaluator:
            op_of_task = {}
            for op, ctests, ptests in task_units(suite, backend):
                tid = evaluator.submit_task(op, backend_ref if backend_ref is not None else backend[op], ctests, ptests, tolerances)
                op_of_task[tid] = op
            evaluator.start_evaluation()
            results = evaluator.get_results()
        by_op = {}
        for r in results:  # one task per CASE for descriptor suites: put the operator back together
            by_op.setdefault(op_of_task[r.task_id], []).append(r)
        for op, rs in by_op.items():
            cres = [c for r in rs for c in r.correctness_results]
            pres = [q for r in rs for q in r.performance_results]
            overall_correctness.append(all(c.is_correct for c in cres))
            if len(rs) == 1:
                overall_performance.append(float(rs[0].performance_score))
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
def cli(log_level, suite, alternative_torchbench_data_path, topn_inputs, backend, ops, ops_directory, num_workers, p, device, cases, dtype_tolerances, daemon, log_dir):
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
    mean_correctness, geomean_perf, perf_at_p, (all_c, all_p) = run(test_suite, be, ref, num_workers, daemon, p, "dtype" if dtype_tolerances else None)
    if log_dir:
        from ..output import save_results

        save_results(all_c, all_p, log_dir, "python -m backendbench_b200.scripts.main " + " ".join(sys.argv[1:]), mean_correctness, geomean_perf, perf_at_p, p)
    print(f"correctness score (mean pass rate over all operators): {mean_correctness:.2f}")
    print(f"performance score (geomean speedup over all operators): {geomean_perf:.2f}")
    print(f"perf@p score (rate of correct samples with a speedup greater than p, p={p}): {perf_at_p:.2f}")


if __name__ == "__main__":
    cli()
