"""Host-side logic of the plugin and evaluation API on CPU: name mapping, case grammar,
error metrics, closeness rule, scoring, registry, directory loading -- checked against
the known answers recorded from the reference harness (tests/golden/harness_golden.json)
and against the literal vectors the reference's own tests pin."""

import math
import os
import sys
import textwrap

import pytest
import torch

import backendbench_b200 as bb
from backendbench_b200 import eval as ev
from backendbench_b200 import utils
from backendbench_b200.backends import KERNELS_DIR, AtenBackend, B200Backend, DirectoryBackend, make_backend
from backendbench_b200.opregistry import _extract_spec_name_from_op, get_operator, get_registry
from backendbench_b200.ops import OP_TABLE, UnsupportedByB200
from backendbench_b200.suite import SmokeTestSuite, Test


class Case:
    def __init__(self, args, kwargs):
        self.args, self.kwargs = args, kwargs


# ------------------------------------------------------------------ names and registry
def test_name_mapping_matches_reference(harness_golden):
    for op, folder in harness_golden["op_to_folder"].items():
        assert utils.op_name_to_folder_name(op) == folder
    for folder, op in harness_golden["folder_to_op"].items():
        assert utils.folder_name_to_op_name(folder) == op
    for s, want in harness_golden["extract_operator_name"].items():
        assert utils.extract_operator_name(s) == want
    assert utils.folder_name_to_op_name("add___Tensor") == "add_.Tensor"  # right-to-left parse


def test_spec_names_and_operator_resolution(harness_golden):
    for name, spec in harness_golden["spec_names"].items():
        op = utils.get_pytorch_op(name)
        assert op is not None and _extract_spec_name_from_op(op) == spec
        assert op.__name__ == harness_golden["op_dunder_name"][name]
        assert get_operator(spec) is get_operator(op)  # one canonical object per name
    assert get_operator("relu") is torch.ops.aten.relu.default
    assert utils.get_pytorch_op("not_an_op.default") is None
    assert "add.Tensor" in get_registry()


def test_serialize_args_matches_reference(harness_golden):
    inputs = {
        "plain": ([torch.zeros(2, 3)], {}),
        "kw": ([torch.zeros(2, 3, dtype=torch.bfloat16), 1], {"dim": 1, "keepdim": True}),
        "strided": ([torch.zeros(4, 6).t()], {}),
        "list": ([[torch.zeros(2), torch.zeros(3, dtype=torch.int64)], 2.5], {}),
        "empty": ([], {}),
        "scalars": ([1, 2.0, None, "s"], {"x": [1, 2]}),
    }
    for k, (a, kw) in inputs.items():
        assert utils.serialize_args(a, kw) == harness_golden["serialize_args"][k]
    assert utils.serialize_args(None, None) == harness_golden["serialize_none"]


def test_deserialize_round_trip():
    args, kwargs = utils.deserialize_args("((T([8, 4], bf16), T([4, 8], f32, [1, 4]), 2,), {'dim': 1})")
    assert args[0].shape == (8, 4) and args[0].dtype == torch.bfloat16
    assert args[1].shape == (4, 8) and args[1].stride() == (1, 4)
    assert args[2] == 2 and kwargs == {"dim": 1}
    assert 0 <= float(args[1].min()) and float(args[1].max()) <= 1  # floats are U[0,1)
    assert utils.serialize_args(args, kwargs) == "((T([8, 4], bf16), T([4, 8], f32, [1, 4]), 2,), {'dim': 1})"


# ------------------------------------------------------------------ error metrics, closeness
def test_compute_errors_matches_reference(harness_golden):
    pairs = {
        "identical": ([1.0, 2.0, 3.0, 4.0], [1.0, 2.0, 3.0, 4.0]),
        "ten_percent": ([2.0, 4.0, 6.0, 8.0], [2.2, 4.4, 6.6, 8.8]),
        "zero_ref": ([0.0, 1.0], [0.1, 1.1]),
        "with_nan": ([1.0, math.nan], [1.0, math.nan]),
        "with_inf": ([math.inf, 1.0], [math.inf, 1.5]),
    }
    for k, (a, b) in pairs.items():
        for fn in (utils.compute_errors, lambda r, s: ev.compare(r, s)[1:]):
            got = fn(torch.tensor(a), torch.tensor(b))
            for g, w in zip(got, harness_golden["compute_errors"][k]):
                w = float(w)
                assert (math.isnan(g) and math.isnan(w)) or g == pytest.approx(w, rel=1e-6), (k, got)
    la = [torch.tensor([1.0, 2.0]), torch.tensor([3.0, 4.0])]
    lb = [torch.tensor([1.1, 2.2]), torch.tensor([3.3, 4.4])]
    got = utils.compute_errors(la, lb)
    assert got[0] == pytest.approx(float(harness_golden["compute_errors_list"][0]), rel=1e-6)
    assert utils.compute_errors(1.0, 2.0) == (None, None)
    assert utils.compute_errors(torch.ones(3, 4), torch.ones(3, 5)) == (None, None)
    # eps is honoured (test/test_utils.py:576-583): [0.1/(0+1), 0.1/(1+1)] -> 0.1
    a, r = utils.compute_errors(torch.tensor([0.0, 1.0]), torch.tensor([0.1, 1.1]), eps=1.0)
    assert a == pytest.approx(0.1, rel=1e-5) and r == pytest.approx(0.1, rel=1e-5)


def test_allclose_truth_table_matches_reference(harness_golden):
    t = torch.tensor
    table = {
        "equal": (t([1.0, 2.0, 3.0]), t([1.0, 2.0, 3.0])),
        "within": (t([1.0, 2.0, 3.0]), t([1.0, 2.0, 3.01])),
        "outside": (t([1.0, 2.0]), t([1.1, 2.1])),
        "nan_nan": (t([1.0, math.nan]), t([1.0, math.nan])),
        "nan_vs_number": (t([1.0, math.nan]), t([1.0, 2.0])),
        "inf_inf": (t([math.inf, -math.inf]), t([math.inf, -math.inf])),
        "inf_vs_neg_inf": (t([math.inf]), t([-math.inf])),
        "inf_vs_big": (t([math.inf]), t([3e38])),
        "dtype_mismatch": (t([1.0]), t([1.0], dtype=torch.float64)),
        "shape_mismatch": (t([1.0, 2.0]), t([[1.0, 2.0]])),
        "int_equal": (t([1, 2, 3]), t([1, 2, 3])),
        "int_off_by_one": (t([1, 2, 3]), t([1, 2, 4])),
        "bool_diff": (t([True, False]), t([True, True])),
        "nested_ok": ([[t([1.0])], (t([2.0]), t([3.0]))], [[t([1.01])], (t([2.01]), t([3.01]))]),
        "length_mismatch": ([t([1.0]), t([2.0])], [t([1.0])]),
        "scalars_equal": (1, 1),
        "scalars_differ": (1, 2),
        "strings": ("test", "test"),
        "near_zero_atol": (t([0.0]), t([0.009])),
        "near_zero_outside": (t([0.0]), t([0.011])),
        "rtol_on_second_operand": (t([100.0]), t([101.015])),
    }
    assert set(table) == set(harness_golden["allclose"])
    for k, (a, b) in table.items():
        assert ev.allclose(a, b) is harness_golden["allclose"][k], k


def test_allclose_forwards_tolerances():
    a, b = torch.tensor([1.0]), torch.tensor([1.001])
    assert ev.allclose(a, b) is True
    assert ev.allclose(a, b, atol=1e-5, rtol=1e-5) is False  # the reference ignores these
    assert ev.tolerances_for(torch.ops.aten.relu.default, torch.float32) == (1e-5, 1e-5)
    assert ev.tolerances_for(torch.ops.aten.relu.default, torch.bfloat16) == (1e-2, 1e-2)
    assert ev.tolerances_for(torch.ops.aten.mm.default, torch.float32) == (1e-4, 1e-4)
    assert ev.tolerances_for(torch.ops.aten.argmax.default, torch.int64) == (0.0, 0.0)


def test_perf_at_p_matches_reference(harness_golden):
    assert float(ev.perf_at_p([1, 1, 0, 1], [2.0, 0.5, 3.0, 1.0], 1.0)) == pytest.approx(harness_golden["perf_at_p"]["basic"])
    assert float(ev.perf_at_p([1, 0], [0.2, 5.0], 0.0)) == pytest.approx(harness_golden["perf_at_p"]["p0"])
    assert float(ev.perf_at_p([True, True, True], [2.5, 2.0, 1.9], 2.0)) == pytest.approx(harness_golden["perf_at_p"]["p2"])


def test_uses_cuda_stream_matches_reference(harness_golden, tmp_path):
    import importlib.util

    for k, src in harness_golden["uses_cuda_stream_sources"].items():
        f = tmp_path / f"snip_{k}.py"
        f.write_text("import torch\n" + src)
        spec = importlib.util.spec_from_file_location(f"snip_{k}", f)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        assert utils.uses_cuda_stream(mod.f) is harness_golden["uses_cuda_stream"][k], k
    assert utils.uses_cuda_stream(torch.ops.aten.relu.default) is False
    for fn in OP_TABLE.values():  # none of our own host wrappers may trip the screen
        assert utils.uses_cuda_stream(fn) is False
    for op, impl in B200Backend().compiled_kernels.items():
        assert utils.uses_cuda_stream(impl) is False


# ------------------------------------------------------------------ evaluation on CPU
def test_eval_correctness_pass_fail_exception():
    ok = ev.eval_correctness_test(torch.relu, torch.relu, Case([torch.tensor([-1.0, 0.0, 1.0])], {}))
    assert ok.is_correct and ok.max_abs_error == 0.0
    bad = ev.eval_correctness_test(torch.relu, lambda x: x * 2, Case([torch.tensor([1.0, 2.0, 3.0])], {}))
    assert not bad.is_correct and bad.max_abs_error == pytest.approx(3.0)

    def boom(x):
        raise RuntimeError("Test error")

    exc = ev.eval_correctness_test(torch.relu, boom, Case([torch.tensor([1.0])], {}))
    assert not exc.is_correct and "Test error" in exc.error_msg and "RuntimeError" in exc.error_type
    score, results = ev.eval_correctness(torch.abs, torch.abs, [Case([torch.tensor([float(i) - 2.5])], {}) for i in range(5)])
    assert score == 1.0 and len(results) == 5
    assert ev.eval_correctness(torch.abs, torch.abs, []) == (0.0, [])


def test_format_exception_mentions_op_and_args():
    msg = ev.format_exception(ValueError("Test error"), torch.ops.aten.relu.default, [torch.randn(2, 3)], {"dim": 1})
    assert "relu.default" in msg and "(T([2, 3], f32)" in msg and "dim" in msg and "Test error" in msg


def test_cpu_bench_runs_ten_warmups_plus_n():
    n = 0

    def fn():
        nonlocal n
        n += 1

    t = ev.cpu_bench(fn, num_runs=10)
    assert n == 20 and t > 0


def test_eval_one_op_and_stream_screen():
    tests = [Case([torch.tensor([-1.0, 0.0, 1.0])], {}) for _ in range(3)]
    c, p, cr, pr = ev.eval_one_op(torch.relu, torch.relu, tests, tests[:2])
    assert c == 1.0 and float(p) > 0 and len(cr) == 3 and len(pr) == 2 and all(r.successfully_ran for r in pr)

    def makes_stream(x):
        s = torch.cuda.Stream()  # noqa: F841
        return x

    c, p, cr, pr = ev.eval_one_op(torch.relu, makes_stream, tests, tests[:1])
    assert c == 0 and p == 1.0 and cr[0].error_msg == "Skipped: uses CUDA stream" and pr[0].speedup == 0


def test_wrong_impl_counts_as_speedup_one():
    tests = [Case([torch.tensor([1.0, 2.0])], {})]
    score, results = ev.eval_performance(torch.relu, lambda x: x + 42, tests)
    assert float(score) == pytest.approx(1.0) and not results[0].successfully_ran and "not close" in results[0].error_msg


def test_smoke_suite_through_aten_backend():
    backend = AtenBackend()
    for optest in SmokeTestSuite:
        assert optest.op in backend
        c, p, cr, pr = ev.eval_one_op(optest.op, backend[optest.op], optest.correctness_tests, optest.performance_tests)
        assert c == 1.0 and float(p) > 0.1


def test_test_thunks_rerun_on_every_access():
    t = Test(lambda: torch.randn(4), k=lambda: 3)
    assert not torch.equal(t.args[0], t.args[0]) and t.kwargs == {"k": 3}


# ------------------------------------------------------------------ literal vectors the reference pins
def test_reference_literal_vectors_on_aten_backend():
    be = AtenBackend()
    relu, add = torch.ops.aten.relu.default, torch.ops.aten.add.Tensor
    assert torch.equal(be[relu](torch.tensor([-1.0, 0.0, 1.0])), torch.tensor([0.0, 0.0, 1.0]))  # test_monkey_patch.py:99-100
    assert torch.equal(be[add](torch.tensor([-1.0, 0.0, 1.0]), torch.tensor([1.0, 1.0, 1.0])), torch.tensor([0.0, 1.0, 2.0]))  # :135
    import oracle

    assert torch.equal(oracle.relu(torch.tensor([-1.0, 0.0, 1.0])), torch.tensor([0.0, 0.0, 1.0]))
    assert torch.equal(oracle.relu(torch.tensor([-2.0, -1.0, 0.0, 1.0, 2.0])), torch.tensor([0.0, 0.0, 0.0, 1.0, 2.0]))  # test_directory_backend.py:40-45
    assert torch.equal(oracle.add(torch.tensor([1.0, 2.0, 3.0]), torch.tensor([4.0, 5.0, 6.0])), torch.tensor([5.0, 7.0, 9.0]))  # :52-58
    assert torch.equal(oracle.mul(torch.tensor([1.0, 2.0, 3.0]), torch.tensor([4.0, 5.0, 6.0])), torch.tensor([4.0, 10.0, 18.0]))  # :65-71


# ------------------------------------------------------------------ directory backend
def test_b200_backend_loads_all_sixteen_overloads_and_their_variants():
    from backendbench_b200.backward import BACKWARD_TABLE
    from backendbench_b200.variants import VARIANT_TABLE

    be = B200Backend()
    everything = {**OP_TABLE, **VARIANT_TABLE, **BACKWARD_TABLE}
    assert be.name == "b200" and len(OP_TABLE) == 16 and len(be.compiled_kernels) == len(everything) == 41
    assert set(be.compiled_kernels) == {get_operator(spec) for spec in everything}
    assert get_operator("add_.Tensor") is torch.ops.aten.add_.Tensor and get_operator("sum.IntList_out") is torch.ops.aten.sum.IntList_out
    for spec in everything:
        folder = utils.op_name_to_folder_name(spec)
        assert os.path.isfile(os.path.join(KERNELS_DIR, folder, f"{folder}_implementation_v1.py"))
    assert torch.ops.aten.add.Scalar not in be  # only the named overload is registered
    with pytest.raises(KeyError):
        be[torch.ops.aten.abs.default]
    assert isinstance(make_backend("aten"), AtenBackend) and make_backend("b200").name == "b200"


def test_directory_backend_takes_first_sorted_file_and_skips_broken(tmp_path):
    d = tmp_path / "relu__default"
    d.mkdir()
    (d / "relu__default_implementation_v2.py").write_text("def relu__default_kernel_impl(x):\n    return 'v2'\n")
    (d / "relu__default_implementation_v1.py").write_text("def relu__default_kernel_impl(x):\n    return 'v1'\n")
    (d / "notes.py").write_text("raise RuntimeError('not an implementation file')\n")
    e = tmp_path / "abs__default"
    e.mkdir()
    (e / "abs__default_implementation_v1.py").write_text("def wrong_name(x):\n    return x\n")
    (tmp_path / "add___Tensor").mkdir()
    (tmp_path / "add___Tensor" / "add___Tensor_implementation_v1.py").write_text("def add___Tensor_kernel_impl(a, b):\n    return 'inplace'\n")
    be = DirectoryBackend(str(tmp_path))
    assert be[torch.ops.aten.relu.default](None) == "v1"
    assert torch.ops.aten.abs.default not in be
    assert be[torch.ops.aten.add_.Tensor](None, None) == "inplace"
    assert DirectoryBackend(str(tmp_path / "missing")).compiled_kernels == {}


def test_no_cpu_fallback_kernels_fail_loudly_on_cpu_tensors():
    be = B200Backend()
    with pytest.raises(UnsupportedByB200, match="no CPU path"):
        be[torch.ops.aten.relu.default](torch.randn(4))
    with pytest.raises(UnsupportedByB200):
        be[torch.ops.aten.mm.default](torch.randn(4, 4), torch.randn(4, 4))


def test_enable_disable_on_cpu_key_with_watermark(tmp_path, capsys):
    """Registration mechanics on the CPU dispatch key with a constant-returning kernel
    (the reference's watermark idea, scripts/create_watermarked_operators.py:24-29)."""
    d = tmp_path / "relu__default"
    d.mkdir()
    (d / "relu__default_implementation_v1.py").write_text("import torch\n\ndef relu__default_kernel_impl(x):\n    return torch.full_like(x, 42.0)\n")
    x = torch.tensor([-1.0, 0.0, 1.0])
    with bb.BackendBench.enable(kernel_dir=str(tmp_path), dispatch_key="CPU"):
        assert torch.equal(torch.relu(x), torch.full_like(x, 42.0))
        assert torch.equal(torch.ops.aten.add.Tensor(x, x), x + x)  # other ops untouched
    assert torch.equal(torch.relu(x), torch.tensor([0.0, 0.0, 1.0]))  # registrations gone
    bb.enable(kernel_dir=str(tmp_path), dispatch_key="CPU")
    assert torch.equal(torch.relu(x), torch.full_like(x, 42.0))
    bb.disable()
    assert torch.equal(torch.relu(x), torch.tensor([0.0, 0.0, 1.0]))
    bb.enable(kernel_dir=str(tmp_path / "nope"))  # missing directory: warning, no exception
