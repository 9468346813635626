"""TorchBench-format ingestion (BackendBench/suite/torchbench.py:45-105, trace grammar
data_loaders.py:43-91): a local trace or parquet file becomes per-operator tests, largest
inputs first. The trace below is written for this test (made-up shapes in the documented
grammar); the public dataset is not reproduced."""

import pytest
import torch
from click.testing import CliRunner

from backendbench_b200 import trace_suite
from backendbench_b200.scripts.main import cli

TRACE = """Operator: aten.relu.default
cnt: 3, ((T([4, 16], f32),), {})
cnt: 1, ((T([2, 8, 8], f16),), {})
cnt: 0, ((T([64, 64], f32),), {})
Operator: aten.add.Tensor
cnt: 7, ((T([8, 32], f32), T([32], f32)), {})
cnt: 2, ((T([8, 32], f32), T([8, 32], f32)), {'alpha': 2})
cnt: 2, ((T([8, 32], f32), T([8, 32], f32)), {'alpha': 2})
Operator: aten.sum.SymInt
cnt: 5, ((T([6, 10], f32), [1], True), {})
Operator: aten.mm.default
cnt: 1, ((T([16, 24], f32), T([24, 8], f32, [1, 24])), {})
"""


@pytest.fixture()
def trace_file(tmp_path):
    p = tmp_path / "trace.txt"
    p.write_text(TRACE)
    return str(p)


def test_parse_records_filter_limit_and_rename(trace_file):
    recs = trace_suite.load_ops_from_source(trace_file)
    assert [r["op_name"] for r in recs] == ["aten.relu.default"] * 3 + ["aten.add.Tensor"] * 3 + ["aten.sum.dim_IntList", "aten.mm.default"]
    assert [r["count"] for r in recs] == [3, 1, 0, 7, 2, 2, 5, 1] and [r["is_synthetic"] for r in recs] == [False, False, True] + [False] * 5
    assert recs[0]["args"] == "((T([4, 16], f32),), {})" and len(recs[0]["uuid"]) == 64 and recs[4]["uuid"] == recs[5]["uuid"] != recs[3]["uuid"]
    assert {r["op_name"] for r in trace_suite.load_ops_from_source(trace_file, filter=["add", "mm"])} == {"aten.add.Tensor", "aten.mm.default"}
    assert {r["op_name"] for r in trace_suite.load_ops_from_source(trace_file, limit=2)} == {"aten.relu.default", "aten.add.Tensor"}
    with pytest.raises(ValueError):
        trace_suite.load_ops_from_source("https://example.invalid/trace.txt")
    with pytest.raises(ValueError):
        trace_suite.parse_trace_lines(["cnt: 1, ((), {})\n"])


def test_suite_deduplicates_orders_by_size_and_takes_topn(trace_file):
    suite = trace_suite.TraceTestSuite("torchbench", trace_file, topn=2)
    by_op = {t.op: t for t in suite}
    assert set(by_op) == {torch.ops.aten.relu.default, torch.ops.aten.add.Tensor, torch.ops.aten.sum.dim_IntList, torch.ops.aten.mm.default}
    relu = [t.serialized for t in by_op[torch.ops.aten.relu.default].correctness_tests]
    assert relu == ["((T([64, 64], f32),), {})", "((T([4, 16], f32),), {})"]  # 16 KiB, then the two 256-byte cases by descending string; topn cuts the last
    add = list(by_op[torch.ops.aten.add.Tensor].performance_tests)
    assert len(add) == 2 and add[0].kwargs == {"alpha": 2} and add[0].args[0].shape == (8, 32)
    mm = next(iter(by_op[torch.ops.aten.mm.default].correctness_tests))
    assert mm.args[1].stride() == (1, 24) and mm.args[0].dtype == torch.float32
    import pickle

    again = pickle.loads(pickle.dumps(mm))
    assert again.serialized == mm.serialized and again.args[1].shape == (24, 8)


def test_parquet_table_with_inclusion_flag(tmp_path, trace_file):
    import pyarrow as pa
    import pyarrow.parquet as pq

    recs = trace_suite.load_ops_from_source(trace_file)
    for i, r in enumerate(recs):
        r["included_in_benchmark"] = i != 0
    path = str(tmp_path / "ops.parquet")
    pq.write_table(pa.Table.from_pylist(recs), path)
    suite = trace_suite.TraceTestSuite("torchbench", path, filter=["relu"])
    (optest,) = list(suite)
    assert [t.serialized for t in optest.correctness_tests] == ["((T([64, 64], f32),), {})", "((T([2, 8, 8], f16),), {})"]


def test_cli_runs_a_local_trace_with_the_aten_backend(trace_file, tmp_path):
    r = CliRunner().invoke(cli, ["--suite", "torchbench", "--alternative-torchbench-data-path", trace_file, "--backend", "aten", "--device", "cpu", "--log-dir", str(tmp_path / "out")])
    assert r.exit_code == 0, r.output
    assert "correctness score (mean pass rate over all operators): 1.00" in r.output
    assert (tmp_path / "out" / "operator_summary.csv").exists()
    r = CliRunner().invoke(cli, ["--suite", "torchbench", "--backend", "aten"])
    assert r.exit_code != 0 and "alternative-torchbench-data-path" in r.output
