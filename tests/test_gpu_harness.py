"""The evaluation path on the GPU: fused device-side allclose/error pass, CUDA-event
timing, the directory-backend drop-in through eval_one_op, the runtime override through
the aten dispatcher, and the process-per-GPU sweep with descriptor tasks."""

import math

import pytest
import torch

import backendbench_b200 as bb
from backendbench_b200 import eval as ev
from backendbench_b200 import ops, utils
from backendbench_b200.backends import KERNELS_DIR, AtenBackend, B200Backend, DirectoryBackend
from backendbench_b200.cases import sweep_cases
from backendbench_b200.multiprocessing_eval import BackendRef, MultiprocessingEvaluator, SpecTest
from backendbench_b200.opregistry import get_operator
from backendbench_b200.suite import make_smoke_suite

pytestmark = pytest.mark.gpu
DEV = "cuda"


class Case:
    def __init__(self, args, kwargs=None):
        self.args, self.kwargs = args, kwargs or {}


def test_device_compare_matches_host_formula():
    g = torch.Generator(device=DEV).manual_seed(0)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        a = torch.randn(1_000_003, generator=g, device=DEV).to(dt)
        b = (a.float() + torch.randn(1_000_003, generator=g, device=DEV) * 0.004).to(dt)
        ok, mabs, mrel = ev.compare(a, b)
        habs, hrel = utils.compute_errors(a, b)
        want = bool(torch.isclose(a.double(), b.double(), rtol=1e-2, atol=1e-2, equal_nan=True).all())
        assert ok is want and mabs == pytest.approx(habs, rel=1e-6) and mrel == pytest.approx(hrel, rel=1e-5)
        b2 = b.clone()
        b2[12345] += 1.0
        assert ev.compare(a, b2)[0] is False and ev.allclose(a, b2) is False
    a = torch.tensor([1.0, math.nan, math.inf, -math.inf, 0.0], device=DEV)
    assert ev.compare(a, a.clone())[0] is True and math.isnan(ev.compare(a, a.clone())[1])
    assert ev.compare(a, torch.tensor([1.0, 2.0, math.inf, -math.inf, 0.0], device=DEV))[0] is False
    assert ev.compare(torch.tensor([math.inf], device=DEV), torch.tensor([-math.inf], device=DEV))[0] is False
    for dt in (torch.bfloat16, torch.float16):  # 16-bit vectors that are bit-identical leave the kernel early
        h = torch.randn(100_003, generator=g, device=DEV).to(dt)
        assert ev.compare(h, h.clone()) == (True, 0.0, 0.0)
        one = h.clone()
        one[50_001] = one[50_001] + 1.0  # a single element inside an otherwise identical tensor
        ok, mabs, _ = ev.compare(h, one)
        assert ok is False and mabs == pytest.approx(float((h.float() - one.float()).abs().max()), rel=1e-6)
        for special in (math.inf, -math.inf, math.nan):  # identical, but inf - inf and NaN make the error NaN, as on the host
            sp = h.clone()
            sp[8 * 1234 + 3] = special
            ok, mabs, mrel = ev.compare(sp, sp.clone())
            assert ok is True and math.isnan(mabs)
            habs, _ = utils.compute_errors(sp, sp.clone())
            assert math.isnan(habs)
        z = torch.zeros(64, device=DEV, dtype=dt)
        assert ev.compare(z, -z) == (True, 0.0, 0.0)  # +0 and -0 differ in bits, not in value
    i = torch.arange(100000, device=DEV)
    assert ev.compare(i, i.clone()) == (True, 0.0, 0.0)
    j = i.clone()
    j[777] += 3  # inside the harness band (1e-2 + 1e-2 * 780), which assert_close applies to integers too
    assert ev.compare(i, j)[0] is True and ev.compare(i, j, 0.0, 0.0)[0] is False and ev.compare(i, j)[1] == 3.0
    j[777] += 30
    assert ev.compare(i, j)[0] is False and ev.compare(i, j)[1] == 33.0
    assert ev.compare((a, i), (a.clone(), i.clone()))[0] is True  # tuples accumulate into one record
    assert ev.allclose(a, a.double()) is False and ev.allclose(a, a[:3]) is False  # dtype / shape
    assert ev.compare(i.view(400, 250).t(), i.view(400, 250).t().clone())[0] is True  # strided inputs


def test_cuda_bench_and_l2_flush():
    x = torch.randn(4096, 4096, device=DEV)
    relu = B200Backend()[torch.ops.aten.relu.default]
    ms = ev.cuda_bench(lambda: relu(x), reps=10)
    assert 0.005 < ms < 5.0  # 128 MiB of traffic: tens of microseconds on a B200
    times = ev.cuda_bench(lambda: relu(x), reps=5, return_all=True)
    assert len(times) == 5 and times == sorted(times)


def test_directory_backend_drop_in_through_eval_one_op():
    backend = DirectoryBackend(KERNELS_DIR)
    for optest in make_smoke_suite(DEV):
        assert optest.op in backend
        c, p, cres, pres = ev.eval_one_op(optest.op, backend[optest.op], optest.correctness_tests, optest.performance_tests)
        assert c == 1.0 and float(p) > 0.1 and pres[0].successfully_ran and pres[0].benchmark_time_ms > 0
    op = torch.ops.aten.add.Tensor
    tests = [Case([torch.randn(64, 64, device=DEV), torch.randn(64, device=DEV)], {"alpha": 2})]
    c, p, cres, pres = ev.eval_one_op(op, backend[op], tests, tests, tolerances="dtype")
    assert c == 1.0 and cres[0].max_abs_error < 1e-5 and cres[0].args == "((T([64, 64], f32), T([64], f32),), {'alpha': 2})"
    c, _, cres, _ = ev.eval_one_op(op, lambda a, b, alpha=1: a + b, tests, [])  # a wrong kernel is caught
    assert c == 0.0 and cres[0].max_abs_error > 0.1


def test_runtime_override_through_the_dispatcher(monkeypatch):
    """enable() registers the kernels for the CUDA key; unchanged model code then runs on
    them (counted here by wrapping the host functions), and disable() restores aten."""
    calls = {}

    def counting(name):
        fn = getattr(ops, name)

        def wrapped(*a, **k):
            calls[name] = calls.get(name, 0) + 1
            return fn(*a, **k)

        return wrapped

    for name in ("relu", "add_Tensor", "mul_Tensor", "addmm_default", "mm_default", "_softmax_default", "native_layer_norm_default", "embedding_default"):
        monkeypatch.setattr(ops, name, counting(name))
    torch.manual_seed(0)
    emb = torch.nn.Embedding(100, 64).to(DEV)
    lin = torch.nn.Linear(64, 32).to(DEV)
    ln = torch.nn.LayerNorm(32).to(DEV)
    idx = torch.randint(0, 100, (16,), device=DEV)

    def model():
        h = torch.relu(lin(emb(idx)))
        return torch.softmax(ln(h) * 2.0 + h, dim=-1)

    with torch.no_grad():
        want = model()
        with bb.BackendBench.enable(kernel_dir=KERNELS_DIR):
            got = model()
        assert calls.get("relu") == 1 and calls.get("addmm_default") == 1 and calls.get("embedding_default") == 1
        assert calls.get("native_layer_norm_default") == 1 and calls.get("_softmax_default") == 1 and calls.get("add_Tensor", 0) >= 1
        assert ev.compare(want, got, 1e-5, 1e-4)[0]
        n = dict(calls)
        model()
        assert calls == n  # registrations are gone after the block
        bb.enable(kernel_dir=KERNELS_DIR)
        try:
            assert ev.compare(want, model(), 1e-5, 1e-4)[0] and calls["relu"] == n["relu"] + 1
            x = torch.tensor([-1.0, 0.0, 1.0], device=DEV)
            assert torch.equal(torch.relu(x).cpu(), torch.tensor([0.0, 0.0, 1.0]))  # test_monkey_patch.py:99-100
            assert torch.equal((x + torch.ones_like(x)).cpu(), torch.tensor([0.0, 1.0, 2.0]))  # :135
        finally:
            bb.disable()
    ops.check_device_status()


def test_one_worker_sweep_with_descriptor_tasks():
    cases = [c for c in sweep_cases(96, seed=2, max_log2=18)][:40]
    with MultiprocessingEvaluator(1, backend=BackendRef("b200")) as evaluator:
        for c in cases:
            evaluator.submit_task(c.op, BackendRef("b200"), [SpecTest(c, "cuda")], [SpecTest(c, "cuda")] if c.case_id % 8 == 0 else [], "dtype")
        evaluator.start_evaluation()
        results = evaluator.get_results()
    assert len(results) == len(cases)
    failed = [(cases[r.task_id].label(), r.error or r.correctness_results[0].error_msg[:300], r.correctness_results[0].max_abs_error) for r in results if r.correctness_score != 1.0]
    # scatter_add is compared with aten CUDA here, whose atomics sum in another order: allow its fp differences only
    failed = [f for f in failed if not f[0].startswith("scatter_add")]
    assert not failed, failed
    assert any(r.performance_results for r in results)


def test_two_workers_share_one_queue_of_per_case_tasks():
    """Worker i on GPU i, one shared queue, per-case tasks longest first
    (BackendBench/multiprocessing_eval.py:226-395 has only ever run with one worker)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    from backendbench_b200.sharding import lpt_order

    cases = lpt_order([c for c in sweep_cases(96, seed=3, max_log2=20)][:48])
    ref = BackendRef("b200")
    with MultiprocessingEvaluator(2, backend=ref) as evaluator:
        for c in cases:
            evaluator.submit_task(c.op, ref, [SpecTest(c, "cuda")], [], "dtype")
        evaluator.start_evaluation()
        results = evaluator.get_results()
        tl = evaluator.timeline()
    assert len(results) == len(cases) and tl["lost_tasks"] == [] and tl["restarts"] == 0
    assert {r.worker_id for r in results} == {0, 1} and sum(tl["per_worker_tasks"].values()) == len(cases)
    assert tl["all_workers_ready_s"] is not None and tl["wall_s"] >= tl["first_result_s"] > 0
    failed = [cases[r.task_id].label() for r in results if r.correctness_score != 1.0 and not cases[r.task_id].op.startswith("scatter_add")]
    assert not failed, failed


def test_integer_results_get_the_harness_tolerance_band():
    """assert_close applies atol + rtol * |expected| to integers as well: 5000 and 5001 are
    close under the harness's 1e-2 and differ under zero tolerances."""
    a = torch.tensor([5000, 7, -3, 1 << 60], device=DEV)
    b = torch.tensor([5001, 7, -3, 1 << 60], device=DEV)
    assert ev.compare(a, b)[0] is True and ev.compare(a, b, 0.0, 0.0)[0] is False
    assert ev.compare(a.cpu(), b.cpu())[0] is True  # same verdict as the host path
    c = torch.tensor([5000, 9, -3, 1 << 60], device=DEV)
    assert ev.compare(a, c)[0] is False  # |7 - 9| > 1e-2 + 1e-2 * 9
    big = torch.tensor([(1 << 60) + 1], device=DEV)
    assert ev.compare(torch.tensor([1 << 60], device=DEV), big, 0.0, 0.0)[0] is False  # exact means exact beyond 2^53 too


def test_out_of_range_index_fails_its_own_test_only():
    """A kernel that zero-filled rows for a bad index reports it through the status word; the
    evaluation reads the word per test, so exactly that test fails, with the reason."""
    emb = torch.ops.aten.embedding.default
    impl = B200Backend()[emb]
    table = torch.randn(32, 8, device=DEV)

    class Lying:  # the reference side gets valid indices, the implementation a bad one
        def __init__(self, bad):
            self.bad = bad

        def __call__(self, w, idx, *a, **k):
            return impl(w, torch.tensor([1, 99, 3], device=DEV) if self.bad else idx, *a, **k)

    good = Case([table, torch.tensor([1, 2, 3], device=DEV)])
    r_bad = ev.eval_correctness_test(emb, Lying(True), good)
    r_ok = ev.eval_correctness_test(emb, Lying(False), good)
    assert r_bad.is_correct is False and "IndexError" in r_bad.error_type and "index out of range" in r_bad.error_msg
    assert r_ok.is_correct is True and r_ok.error_msg == ""
    ops.check_device_status()  # the word was cleared by the failing test


def test_trace_replay_through_the_cli_on_the_gpu(tmp_path):
    """TorchBench-format ingestion end to end (BackendBench/suite/torchbench.py:45-105): a local
    trace in the documented grammar becomes device tests and runs through `--suite torchbench
    --backend b200`. Made-up shapes; the public dataset is not reproduced."""
    from click.testing import CliRunner

    from backendbench_b200.scripts.main import cli
    from backendbench_b200.trace_suite import TraceTestSuite

    trace = tmp_path / "trace.txt"
    trace.write_text(
        "Operator: aten.relu.default\n"
        "cnt: 3, ((T([64, 128], f16),), {})\n"
        "cnt: 1, ((T([4, 16], f32),), {})\n"
        "Operator: aten.add.Tensor\n"
        "cnt: 7, ((T([8, 32], f32), T([32], f32)), {})\n"
        "cnt: 2, ((T([8, 32], bf16), T([8, 32], bf16)), {'alpha': 2})\n"
        "Operator: aten.mm.default\n"
        "cnt: 1, ((T([16, 24], f32), T([24, 8], f32, [1, 24])), {})\n"
        "Operator: aten._softmax.default\n"
        "cnt: 4, ((T([32, 1000], f16), -1, False), {})\n"
    )
    suite = TraceTestSuite("torchbench", str(trace), None, None)
    backend = B200Backend()
    for optest in suite:
        assert optest.op in backend
        score, _, cres, _ = ev.eval_one_op(optest.op, backend[optest.op], optest.correctness_tests, [], "dtype")
        assert score == 1.0, (optest.op, [c.error_msg[:200] for c in cres if not c.is_correct])
        assert all(c.args.startswith("((T(") for c in cres)
    out = tmp_path / "report"
    r = CliRunner().invoke(cli, ["--suite", "torchbench", "--alternative-torchbench-data-path", str(trace), "--backend", "b200", "--log-dir", str(out)])
    assert r.exit_code == 0, r.output
    assert "correctness score (mean pass rate over all operators): 1.00" in r.output
    assert (out / "full_results.json").exists() and (out / "operator_summary.csv").exists()
