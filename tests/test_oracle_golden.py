"""The CPU oracle against the golden vectors made by the reference harness over aten CPU
(tests/golden/make_golden.py): bit-exact for integer / indexing results and scatter_add,
within the stated tolerance for floating point."""

import math

import pytest
import torch

import oracle
from backendbench_b200.eval import compare
from conftest import EXACT_OPS, bits_equal, first_dtype, tolerance_for_case


def _as_tuple(x):
    return tuple(x) if isinstance(x, (tuple, list)) else (x,)


def test_golden_covers_every_operator_the_oracle_restates(golden_cases):
    assert {c["op"] for c in golden_cases} == set(oracle.ORACLE)
    assert len(golden_cases) >= 80


def test_oracle_matches_golden(golden_cases):
    failures = []
    for c in golden_cases:
        got = oracle.run(c["op"], c["args"], c["kwargs"])
        ref = c["ref"]
        if c["op"] == "native_layer_norm.default":
            # aten CPU keeps mean/rstd in the input dtype; the oracle (like the CUDA path) in fp32
            got = (got[0], got[1].to(ref[1].dtype), got[2].to(ref[2].dtype))
        atol, rtol = tolerance_for_case(c["op"], first_dtype(ref))
        for r, g in zip(_as_tuple(ref), _as_tuple(got)):
            if r is None or g is None:  # an output masked out (native_layer_norm_backward's output_mask)
                assert r is None and g is None, c["tag"]
                continue
            assert r.shape == g.shape and r.dtype == g.dtype, (c["tag"], r.shape, g.shape, r.dtype, g.dtype)
            if c["op"] in EXACT_OPS:
                if not bits_equal(r, g):
                    failures.append((c["tag"], "bits differ"))
            else:
                ok, a, b = compare(r, g, atol, rtol)
                if not ok:
                    failures.append((c["tag"], a, b))
    assert not failures, failures


def test_oracle_scatter_add_order_is_sequential():
    """Many collisions on few destinations: the result depends on the summation order, and
    the oracle must reproduce the ascending-source-row order bit for bit."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4, 3, generator=g)
    idx = torch.randint(0, 4, (200, 3), generator=g)
    src = torch.randn(200, 3, generator=g) * 1e3
    want = x.clone()
    for i in range(200):
        for j in range(3):
            want[idx[i, j], j] += src[i, j]
    assert torch.equal(oracle.scatter_add(x, 0, idx, src), want)
    assert torch.equal(oracle.scatter_add(x, 0, idx, src), torch.ops.aten.scatter_add(x, 0, idx, src))


def test_oracle_compare_matches_harness_known_answers(harness_golden):
    mism, mabs, mrel = oracle.compare(torch.tensor([2.0, 4.0, 6.0, 8.0]), torch.tensor([2.2, 4.4, 6.6, 8.8]))
    want_abs, want_rel = (float(v) for v in harness_golden["compute_errors"]["ten_percent"])
    assert mism == 4 and mabs == pytest.approx(want_abs, rel=1e-6) and mrel == pytest.approx(want_rel, rel=1e-6)
    mism, mabs, mrel = oracle.compare(torch.tensor([1.0, math.nan]), torch.tensor([1.0, math.nan]))
    assert mism == 0 and math.isnan(mabs) and math.isnan(mrel)
    assert oracle.compare(torch.tensor([0.0]), torch.tensor([0.009]))[0] == 0
    assert oracle.compare(torch.tensor([0.0]), torch.tensor([0.011]))[0] == 1
    assert oracle.compare(torch.tensor([math.inf]), torch.tensor([3e38]))[0] == 1


def test_oracle_rounding_helpers_match_torch():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(4096, generator=g) * 100
    x[:4] = torch.tensor([math.nan, math.inf, -math.inf, 0.0])
    for dt in (torch.bfloat16, torch.float16):
        got = oracle.narrow(x.numpy(), dt)
        want = x.to(dt)
        assert torch.equal(got.view(torch.int16)[1:], want.view(torch.int16)[1:])  # NaN payloads may differ
        assert torch.isnan(got[0])
        assert torch.equal(torch.from_numpy(oracle.widen(want))[1:], want.float()[1:])
