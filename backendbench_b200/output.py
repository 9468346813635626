"""Report artefacts of a run, readable by tooling written for the reference.

BackendBench/output.py:116-196,236-329 writes four files per run; this module writes files
of the same names with the same keys, so scripts that parse a reference run parse these:

    <dir>/full_results.json     every CorrectnessTestResult / PerformanceTestResult as a dict,
                                sorted by (op_name, args)
    <dir>/failed_tests.json     the incorrect / not-run subset, same order
    <dir>/operator_summary.csv  one row per operator; the reference's thirteen columns first,
                                then the columns this package adds (device time and, where
                                the case names its algorithmic bytes / FLOP, achieved GB/s or
                                TFLOP/s and the fraction of the measured peak)
    <dir>/OVERALL_SUMMARY.md    command, the three headline scores, per-operator table

The extra columns are appended, never interleaved: a reader that indexes by header name or
takes the first thirteen columns sees exactly the reference layout.
"""

from __future__ import annotations

import csv
import json
import math
import os
from dataclasses import asdict
from typing import Dict, Iterable, List, Optional, Sequence

REFERENCE_COLUMNS = [
    "operator", "total_tests", "correctness_tests", "performance_tests", "passed_correctness_tests", "passed_performance_tests",
    "failed_correctness_tests", "failed_performance_tests", "correctness_rate", "avg_speedup", "geomean_speedup", "max_absolute_error",
    "max_relative_error",
]
EXTRA_COLUMNS = ["mean_benchmark_time_ms", "mean_reference_time_ms", "achieved_gbs", "achieved_tflops", "frac_of_measured_peak"]


def _geomean(xs: Sequence[float]) -> float:
    xs = [float(x) for x in xs if x and x > 0 and math.isfinite(x)]
    return math.exp(sum(math.log(x) for x in xs) / len(xs)) if xs else 0.0


def _by_operator(results: Iterable) -> Dict[str, list]:
    groups: Dict[str, list] = {}
    for r in results:
        groups.setdefault(r.op_name, []).append(r)
    return groups


def summarize_operators(correctness_results: List, performance_results: List, roofline: Optional[Dict[str, dict]] = None) -> Dict[str, dict]:
    """Per-operator rows. `roofline` (optional): op_name -> {"gbs", "tflops", "frac"} measured
    by the caller for that operator's performance cases."""
    c_by, p_by = _by_operator(correctness_results), _by_operator(performance_results)
    rows: Dict[str, dict] = {}
    for op in list(c_by) + [o for o in p_by if o not in c_by]:
        cs, ps = c_by.get(op, []), p_by.get(op, [])
        passed_c = sum(1 for r in cs if r.is_correct)
        ran_p = sum(1 for r in ps if r.successfully_ran)
        errs = [(float(r.max_abs_error), float(r.max_rel_error)) for r in cs if r.max_abs_error and r.max_rel_error]
        speedups = [float(r.speedup) for r in ps if r.speedup]
        row = {
            "operator": op,
            # the reference stores the number of OPERATORS in this column (output.py:89 takes the
            # length of its per-operator dict); kept, since tooling reads it as written
            "total_tests": len(set(c_by) | set(p_by)),
            "correctness_tests": len(cs),
            "performance_tests": len(ps),
            "passed_correctness_tests": passed_c,
            "passed_performance_tests": ran_p,
            "failed_correctness_tests": len(cs) - passed_c,
            "failed_performance_tests": len(ps) - ran_p,
            "correctness_rate": passed_c / len(cs) if cs else 0.0,
            "avg_speedup": sum(speedups) / len(speedups) if speedups else 0.0,
            "geomean_speedup": _geomean(speedups),
            "max_absolute_error": max((e[0] for e in errs), default=0.0),
            "max_relative_error": max((e[1] for e in errs), default=0.0),
        }
        timed = [r for r in ps if r.successfully_ran]
        row["mean_benchmark_time_ms"] = sum(float(r.benchmark_time_ms) for r in timed) / len(timed) if timed else 0.0
        row["mean_reference_time_ms"] = sum(float(r.reference_time_ms) for r in timed) / len(timed) if timed else 0.0
        extra = (roofline or {}).get(op, {})
        row["achieved_gbs"] = extra.get("gbs", "")
        row["achieved_tflops"] = extra.get("tflops", "")
        row["frac_of_measured_peak"] = extra.get("frac", "")
        rows[op] = row
    return rows


def _sorted_dicts(results: Iterable) -> List[dict]:
    return sorted((asdict(r) for r in results), key=lambda d: (d["op_name"], d["args"]))


def overall_summary_markdown(command: str, mean_correctness: float, geomean_perf: float, perf_at_p_score: float, p: float, correctness_results: List, performance_results: List) -> str:
    c_by, p_by = _by_operator(correctness_results), _by_operator(performance_results)
    table = []
    for op in sorted(set(c_by) | set(p_by)):
        cs, ps = c_by.get(op, []), p_by.get(op, [])
        ratio = f"{100.0 * sum(1 for r in cs if r.is_correct) / len(cs):.4f}%" if cs else "N/A"
        # a case that did not run counts as eager speed, as in the reference's summary
        sp = _geomean([r.speedup if r.successfully_ran else 1.0 for r in ps])
        table.append((op, ratio, f"{sp:.4f}x" if ps else "N/A", sp if ps else -1.0))
    table.sort(key=lambda t: -t[3])
    lines = [
        "# BackendBench Run Summary\n", "## Command", "```bash", command, "```\n", "## Results\n", "| Metric | Value |", "|--------|-------|",
        f"| Correctness Score | {mean_correctness:.2f} |", f"| Performance Score (geomean speedup) | {geomean_perf:.2f} |", f"| Perf@{p} Score | {perf_at_p_score:.2f} |", "",
        "### Metric Descriptions\n", "- **Correctness Score**: Mean pass rate over all operators", "- **Performance Score**: Geometric mean speedup over all operators",
        f"- **Perf@{p} Score**: Rate of correct samples with a speedup greater than {p}", "", "## Output Files\n", "The following files are saved in this directory:\n",
        "- `full_results.json`: Complete test results for all operators", "- `operator_summary.csv`: Operator-level summary statistics (reference columns, then device-time and roofline columns)",
        "- `failed_tests.json`: Log of failed tests (if any)", "- `OVERALL_SUMMARY.md`: This file", "### Operator Speedups vs Eager in Descending Order\n",
        "| Operator | Correctness Ratio | Speedup vs Eager |", "|----------|-----------|----------------|",
    ]
    lines += [f"| {op} | {ratio} | {sp}|" for op, ratio, sp, _ in table]
    lines.append("")
    return "\n".join(lines)


def save_results(correctness_results: List, performance_results: List, output_path: str, command: str, mean_correctness: float, geomean_perf: float, perf_at_p_score: float,
                 p: float = 1.0, roofline: Optional[Dict[str, dict]] = None) -> None:
    """Write the four artefacts under `output_path` (created if needed)."""
    os.makedirs(output_path, exist_ok=True)
    with open(os.path.join(output_path, "full_results.json"), "w") as fh:
        json.dump(_sorted_dicts(list(correctness_results) + list(performance_results)), fh, indent=2)
    failed = [r for r in correctness_results if not r.is_correct] + [r for r in performance_results if not r.successfully_ran]
    with open(os.path.join(output_path, "failed_tests.json"), "w") as fh:
        json.dump(_sorted_dicts(failed), fh, indent=2)
    rows = summarize_operators(correctness_results, performance_results, roofline)
    if rows:
        with open(os.path.join(output_path, "operator_summary.csv"), "w", newline="") as fh:
            writer = csv.DictWriter(fh, fieldnames=REFERENCE_COLUMNS + EXTRA_COLUMNS)
            writer.writeheader()
            for row in rows.values():
                writer.writerow(row)
    if all(v is not None for v in (command, mean_correctness, geomean_perf, perf_at_p_score)):
        with open(os.path.join(output_path, "OVERALL_SUMMARY.md"), "w") as fh:
            fh.write(overall_summary_markdown(command, mean_correctness, geomean_perf, perf_at_p_score, p, correctness_results, performance_results))
    print(f"Results saved to directory: {os.path.abspath(output_path)}")
