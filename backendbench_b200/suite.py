"""Case containers the evaluation path consumes (BackendBench/suite/base.py:8-36).

A `Test` holds argument THUNKS: `.args` / `.kwargs` re-run them on every access, so a
case never keeps tensors alive between uses. Anything with `.args` and `.kwargs`
attributes works as a test (the evaluator is duck-typed, test/test_eval.py:103-108).
"""

from __future__ import annotations

import torch

from .opregistry import get_operator


class Test:
    __test__ = False  # a case container, not a pytest class

    def __init__(self, *args, **kwargs):
        self._args = args
        self._kwargs = kwargs

    @property
    def args(self):
        return [thunk() for thunk in self._args]

    @property
    def kwargs(self):
        return {k: thunk() for k, thunk in self._kwargs.items()}


class OpTest:
    def __init__(self, op, correctness_tests, performance_tests):
        self.op = op
        self.correctness_tests = correctness_tests
        self.performance_tests = performance_tests


class TestSuite:
    __test__ = False

    def __init__(self, name, optests):
        self.name = name
        self.optests = optests

    def __iter__(self):
        yield from self.optests


def randn(*args, **kwargs):
    return lambda: torch.randn(*args, **kwargs)


def make_smoke_suite(device="cpu") -> TestSuite:
    """One relu OpTest: a 2-element correctness case and a 1024x1024 performance case
    (BackendBench/suite/smoke.py:18-35, which pins device="cpu")."""
    relu = get_operator(torch.ops.aten.relu.default)
    return TestSuite("smoke", [OpTest(relu, [Test(randn(2, device=device))], [Test(randn(2**10, 2**10, device=device))])])


SmokeTestSuite = make_smoke_suite("cpu")
