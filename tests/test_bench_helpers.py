"""Host-side pieces of bench.py that need no GPU: the CPU timing protocol of the per-op table
(BackendBench/eval.py:149-159, cut down for slow calls), the geomean, the workload description
both arms print, and the reference arm's pass over built cases."""

import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_cpu_protocol_is_the_harness_one_until_calls_get_slow():
    calls = {"n": 0}

    def fast():
        calls["n"] += 1

    sec, warm, runs = bench.cpu_bench_bounded(fast)
    assert (warm, runs) == (10, 100) and calls["n"] == 110 and sec < 1e-3  # 10 warm-up + 100 timed, as cpu_bench
    sec, warm, runs = bench.cpu_bench_bounded(lambda: time.sleep(0.05), budget_s=0.2)
    assert warm == 1 and runs in (3, 4) and 0.04 < sec < 0.2  # too slow for 110 calls: sized to the budget, never under 1 + 3


def test_geomean_and_common_config():
    assert bench.geomean([1.0, 4.0]) == 2.0 and bench.geomean([None, 0, 9.0]) == 9.0 and bench.geomean([]) is None
    a, b = bench.common_config(), bench.common_config()
    assert a == b and a["workload"] == bench.WORKLOAD and a["cases_per_step"] == 512  # what both arms print


def test_reference_pass_runs_built_cases_in_order():
    from backendbench_b200.cases import sweep_cases

    cases = [c for c in sweep_cases(64, seed=0, max_log2=12)][:6]
    built = bench.cpu_reference_cases(cases)
    assert len(built) == 6 and bench.cpu_reference_cases(cases) is built  # built once
    done, secs = bench.cpu_reference_pass(built)
    assert done == 6 and secs > 0
    done, _ = bench.cpu_reference_pass(built, budget_s=0.0)
    assert done == 1  # a spent budget stops after the case in flight
