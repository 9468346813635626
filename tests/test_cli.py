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


def test_checkpoint_and_resume(tmp_path):
    """One JSON line per finished unit; a resumed run evaluates only what is missing and ends
    with the same scores (the reference writes results once, at the end: scripts/main.py:315)."""
    import json

    from backendbench_b200.backends import AtenBackend
    from backendbench_b200.scripts import main as cli_main

    ck_path = str(tmp_path / "results.jsonl")
    suite = cli_main.build_suite("sweep", "cpu", ["relu", "add"], 48)
    full = cli_main.run(suite, AtenBackend(), None, None, True, 1.0, None, cli_main.Checkpoint(ck_path))
    rows = [json.loads(line) for line in open(ck_path)]
    assert len(rows) == len(list(suite)) and all(r["correctness"] for r in rows)
    # drop the last unit (and leave a torn line behind, as a crash would) and resume
    with open(ck_path, "w") as fh:
        for r in rows[:-1]:
            fh.write(json.dumps(r) + "\n")
        fh.write('{"key": "torn')
    calls = {"n": 0}
    real = cli_main.evaluation.eval_one_op

    def counting(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    cli_main.evaluation.eval_one_op = counting
    try:
        ck = cli_main.Checkpoint(ck_path, resume=True)
        assert len(ck.done) == len(rows) - 1
        again = cli_main.run(suite, AtenBackend(), None, None, True, 1.0, None, ck)
    finally:
        cli_main.evaluation.eval_one_op = real
    assert calls["n"] == 1  # only the missing unit was evaluated
    assert again[0] == full[0] and len(again[3][0]) == len(full[3][0])
    assert len([line for line in open(ck_path) if line.strip().endswith("}")]) == len(rows)
