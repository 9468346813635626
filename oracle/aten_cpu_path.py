"""The reference's own CPU path for one correctness case -- TEST/BENCH INFRASTRUCTURE.

What BackendBench does for a case when the backend is its identity `AtenBackend`
(BackendBench/backends/aten.py:10-18) and the tensors live on the CPU:
`eval_correctness_test` (BackendBench/eval.py:93-126) computes `ref = op(*args)`, then
`res = impl(*args)` with impl = the op itself, then `allclose` (eval.py:68-90:
`torch.testing.assert_close(ref, res, equal_nan=True, atol=1e-2, rtol=1e-2)`, lists
pairwise) and `compute_errors` (BackendBench/utils.py:185-242). The arithmetic is
PyTorch ATen on the host cores -- the third-party library the reference calls -- with
all the threads torch uses by default. bench.py times this as the CPU baseline and as
its `--impl reference` arm; it is never part of the product path.
"""

from __future__ import annotations

import torch


def _assert_close_tree(a, b, atol=1e-2, rtol=1e-2) -> bool:
    stack = [(a, b)]
    try:
        while stack:
            x, y = stack.pop()
            if isinstance(x, torch.Tensor):
                torch.testing.assert_close(x, y, equal_nan=True, atol=atol, rtol=rtol)
            elif isinstance(x, (list, tuple)):
                assert len(x) == len(y)
                stack.extend(reversed(list(zip(x, y))))
            else:
                assert x == y
        return True
    except Exception:
        return False


def _errors(ref, res, eps=1e-10):
    if isinstance(ref, torch.Tensor):
        if ref.numel() == 0:
            return 0.0, 0.0
        r, s = ref.float(), res.float()
        d = (r - s).abs()
        return d.max().item(), (d / (r.abs() + eps)).max().item()
    pairs = [_errors(r, s) for r, s in zip(ref, res) if isinstance(r, torch.Tensor)]
    return max(p[0] for p in pairs), max(p[1] for p in pairs)


def eval_case_cpu(op, args, kwargs) -> bool:
    """One reference correctness evaluation on CPU tensors; True when the case passes."""
    ref = op(*args, **kwargs)
    res = op(*args, **kwargs)  # AtenBackend: the implementation is the operator itself
    ok = _assert_close_tree(ref, res)
    _errors(ref, res)
    return ok


def host_threads() -> int:
    return torch.get_num_threads()
