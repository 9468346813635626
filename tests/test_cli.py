"""The command line driver (flags and summary lines of BackendBench/scripts/main.py:186-303)."""

import pytest
import torch
from click.testing import CliRunner

from backendbench_b200.scripts.main import build_suite, cli


def _scores(output):
    lines = [ln for ln in output.splitlines() if "score" in ln]
    assert len(lines) == 3, output
    return [float(ln.rsplit(":", 1)[1]) for ln in lines]


def test_cli_smoke_suite_with_aten_backend_on_cpu():
    # the reference's own CLI check: `--suite smoke --backend aten` exits 0 (test_backend_evaluation.py:97-115)
    r = CliRunner().invoke(cli, ["--suite", "smoke", "--backend", "aten", "--device", "cpu"])
    assert r.exit_code == 0, r.output
    correctness, geomean, _ = _scores(r.output)
    assert correctness == 1.0 and geomean > 0.1


def test_cli_sweep_subset_with_two_cpu_workers():
    r = CliRunner().invoke(cli, ["--suite", "sweep", "--cases", "16", "--backend", "aten", "--device", "cpu", "--ops", "relu,mul.Tensor,sum", "--num-workers", "2"])
    assert r.exit_code == 0, r.output
    assert _scores(r.output)[0] == 1.0


def test_cli_log_dir_writes_the_four_report_files(tmp_path):
    """`--log-dir`: the artefacts of BackendBench/output.py:116-196 by name, with the
    reference's columns first in the operator summary."""
    import csv
    import json

    from backendbench_b200.output import EXTRA_COLUMNS, REFERENCE_COLUMNS

    out = tmp_path / "report"
    r = CliRunner().invoke(cli, ["--suite", "sweep", "--cases", "16", "--backend", "aten", "--device", "cpu", "--ops", "relu,add.Tensor", "--log-dir", str(out)])
    assert r.exit_code == 0, r.output
    assert sorted(p.name for p in out.iterdir()) == ["OVERALL_SUMMARY.md", "failed_tests.json", "full_results.json", "operator_summary.csv"]
    full = json.load(open(out / "full_results.json"))
    assert full and {"op_name", "args", "test_type"} <= set(full[0]) and full == sorted(full, key=lambda d: (d["op_name"], d["args"]))
    assert json.load(open(out / "failed_tests.json")) == []
    rows = list(csv.DictReader(open(out / "operator_summary.csv")))
    assert list(rows[0]) == REFERENCE_COLUMNS + EXTRA_COLUMNS and {r_["operator"] for r_ in rows} == {"relu.default", "add.Tensor"}
    assert all(float(r_["correctness_rate"]) == 1.0 for r_ in rows)
    assert "| Correctness Score | 1.00 |" in open(out / "OVERALL_SUMMARY.md").read()


def test_build_suite_filters_and_descriptor_tests():
    s = build_suite("named", "cpu", ["relu", "mm.default"])
    ops = {t.op for t in s}
    assert ops == {torch.ops.aten.relu.default, torch.ops.aten.mm.default}
    assert all(len(t.correctness_tests) >= 1 for t in s)
    assert len(list(build_suite("sweep", "cpu", None, 512))) == 16  # all sixteen overloads appear in the sweep


def test_cli_rejects_unknown_backend():
    r = CliRunner().invoke(cli, ["--backend", "flag_gems"])
    assert r.exit_code != 0


@pytest.mark.gpu
def test_cli_sweep_with_b200_backend_on_gpu():
    r = CliRunner().invoke(cli, ["--suite", "sweep", "--cases", "64", "--backend", "b200", "--dtype-tolerances"])
    assert r.exit_code == 0, r.output
    correctness, geomean, _ = _scores(r.output)
    # scatter_add is compared with aten CUDA here (unordered atomics): tolerance-level agreement only
    assert correctness >= 0.9 and geomean > 0.05
