"""Drop-in proof against the reference's own loader, run only where the reference checkout
is present (it does not travel to the GPU box): BackendBench's DirectoryBackend loads the
kernels directory of this package unmodified, and the reference's name/serialisation
helpers agree with ours on the spot."""

import os
import sys

import pytest
import torch

# the reference checkout: named by the environment, else a `reference` folder beside this repository
REF = os.environ.get("BACKENDBENCH_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "BackendBench")), reason="reference checkout not present")


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, REF)
    try:
        import BackendBench
        from BackendBench import eval as ref_eval
        from BackendBench import utils as ref_utils
        from BackendBench.backends import DirectoryBackend

        yield {"pkg": BackendBench, "eval": ref_eval, "utils": ref_utils, "DirectoryBackend": DirectoryBackend}
    finally:
        sys.path.remove(REF)


def test_reference_directory_backend_loads_our_kernels(ref):
    from backendbench_b200.backends import KERNELS_DIR
    from backendbench_b200.ops import OP_TABLE

    from backendbench_b200.backward import BACKWARD_TABLE
    from backendbench_b200.variants import VARIANT_TABLE

    be = ref["DirectoryBackend"](KERNELS_DIR)
    assert len(be.compiled_kernels) == 16 + len(VARIANT_TABLE) + len(BACKWARD_TABLE)
    for spec in list(OP_TABLE) + list(VARIANT_TABLE) + list(BACKWARD_TABLE):
        op = ref["utils"].get_pytorch_op(spec)
        assert op in be and callable(be[op])
        assert not ref["utils"].uses_cuda_stream(be[op])  # the reference would refuse to evaluate it otherwise


def test_reference_and_local_helpers_agree(ref):
    from backendbench_b200 import eval as ev
    from backendbench_b200 import utils

    for name in ["add.Tensor", "relu.default", "add_.Tensor", "_log_softmax.default", "sum.dim_IntList"]:
        folder = ref["utils"].op_name_to_folder_name(name)
        assert utils.op_name_to_folder_name(name) == folder
        assert utils.folder_name_to_op_name(folder) == ref["utils"].folder_name_to_op_name(folder) == name
    args = [torch.zeros(3, 4, dtype=torch.float16).t(), [1, 2]]
    assert utils.serialize_args(args, {"k": 1.5}) == ref["utils"].serialize_args(args, {"k": 1.5})
    g = torch.Generator().manual_seed(0)
    a = torch.randn(64, generator=g)
    b = a + torch.randn(64, generator=g) * 0.01
    assert ev.allclose(a, b) == ref["eval"].allclose(a, b)
    ours, theirs = ev.compare(a, b)[1:], ref["utils"].compute_errors(a, b)
    assert ours[0] == pytest.approx(theirs[0]) and ours[1] == pytest.approx(theirs[1])


def test_reference_eval_accepts_our_result_records(ref):
    """The reference's eval_one_op drives an implementation from our directory through its
    own loop on CPU: the kernel refuses CPU tensors loudly, which the harness records as a
    failed case rather than crashing (BackendBench/eval.py:114-125)."""
    from backendbench_b200.backends import KERNELS_DIR

    be = ref["DirectoryBackend"](KERNELS_DIR)
    op = torch.ops.aten.relu.default

    class Case:
        def __init__(self, a):
            self.args, self.kwargs = a, {}

    score, _, cres, _ = ref["eval"].eval_one_op(op, be[op], [Case([torch.randn(4)])], [])
    assert score == 0.0 and "no CPU path" in cres[0].error_msg


def test_report_artefacts_match_the_reference_writer(ref, tmp_path):
    """full_results.json / failed_tests.json are identical, the first thirteen columns of
    operator_summary.csv carry the reference's values, OVERALL_SUMMARY.md the same scores."""
    import csv
    import json

    from BackendBench import output as ref_output
    from backendbench_b200 import output
    from backendbench_b200.eval import CorrectnessTestResult, PerformanceTestResult

    cs = [CorrectnessTestResult("relu.default", "a1", True, max_abs_error=0.1, max_rel_error=0.2), CorrectnessTestResult("relu.default", "a0", False, error_msg="boom", error_type="RuntimeError"),
          CorrectnessTestResult("add.Tensor", "b", True, max_abs_error=1e-3, max_rel_error=2e-3)]
    ps = [PerformanceTestResult("relu.default", "a1", 2.0, 1.0, 2.0, successfully_ran=True), PerformanceTestResult("relu.default", "a0", 8.0, 0.5, 4.0, successfully_ran=True),
          PerformanceTestResult("add.Tensor", "b", 0.5, 2.0, 1.0, error_msg="did not run", successfully_ran=False)]
    rcs = [ref["eval"].CorrectnessTestResult(**vars(c)) for c in cs]
    rps = [ref["eval"].PerformanceTestResult(**vars(p)) for p in ps]
    mine, theirs = tmp_path / "mine", tmp_path / "theirs"
    output.save_results(cs, ps, str(mine), "cmd --x", 0.5, 1.25, 0.3, 1.0, roofline={"relu.default": {"gbs": 5000.0, "frac": 0.77}})
    ref_output.save_results(rcs, rps, str(theirs), "cmd --x", 0.5, 1.25, 0.3, 1.0)
    for name in ("full_results.json", "failed_tests.json"):
        assert json.load(open(mine / name)) == json.load(open(theirs / name))
    a, b = list(csv.DictReader(open(mine / "operator_summary.csv"))), list(csv.DictReader(open(theirs / "operator_summary.csv")))
    assert list(a[0])[:13] == list(b[0]) == output.REFERENCE_COLUMNS and len(a) == len(b)
    for ra, rb in zip(a, b):
        for k in rb:
            assert ra[k] == rb[k] or float(ra[k]) == pytest.approx(float(rb[k])), (ra["operator"], k)
    assert a[0]["achieved_gbs"] == "5000.0" and a[0]["frac_of_measured_peak"] == "0.77"
    ma, mb = open(mine / "OVERALL_SUMMARY.md").read().splitlines(), open(theirs / "OVERALL_SUMMARY.md").read().splitlines()
    assert len(ma) == len(mb) and [i for i, (x, y) in enumerate(zip(ma, mb)) if x != y] == [ma.index(next(x for x in ma if x.startswith("- `operator_summary.csv`")))]


def test_trace_parser_and_ordering_match_the_reference(ref, tmp_path):
    """The same local trace through the reference's parser / TorchBenchOpTest and through
    ours: equal records, equal per-operator test order."""
    import importlib.util

    from BackendBench import data_loaders as ref_loaders
    from backendbench_b200 import trace_suite

    # the module by path: importing the `suite` package pulls in OpInfo, whose dependencies are not installed here
    spec = importlib.util.spec_from_file_location("ref_torchbench_suite", os.path.join(REF, "BackendBench", "suite", "torchbench.py"))
    ref_suite = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_suite)
    TorchBenchOpTest = ref_suite.TorchBenchOpTest
    from test_trace_suite import TRACE

    path = tmp_path / "trace.txt"
    path.write_text(TRACE)
    theirs = ref_loaders._parse_trace_file(str(path))
    assert trace_suite.load_ops_from_source(str(path)) == theirs
    assert trace_suite.load_ops_from_source(str(path), filter=["add"]) == ref_loaders._parse_trace_file(str(path), filter=["add"])
    mine = trace_suite.ops_to_benchmark_dict(trace_suite.load_ops_from_source(str(path)))
    for op_name, inputs in mine.items():
        for topn in (None, 1, 2):
            want = TorchBenchOpTest(op_name, inputs, topn).tests()
            assert [t.serialized for t in trace_suite.TraceOpTest(op_name, inputs, topn).correctness_tests] == want
