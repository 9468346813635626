"""Backward neighbours of the row operators (`_softmax_backward_data`,
`_log_softmax_backward_data`; BackendBench/backends/flag_gems.py:196,233) against aten CUDA on
the same device tensors and against the CPU oracle, at full size and on the ragged /
non-last-dim / mixed-dtype geometries the fallback kernel serves."""

import pytest
import torch

import oracle
from backendbench_b200 import ops
from backendbench_b200.backends import B200Backend
from backendbench_b200.cases import named_case, scaled_down
from backendbench_b200.eval import compare
from backendbench_b200.opregistry import get_operator

pytestmark = pytest.mark.gpu
DEV = "cuda"
SOFT = "_softmax_backward_data.default"
LOGSOFT = "_log_softmax_backward_data.default"


@pytest.fixture(scope="module")
def backend():
    return B200Backend()


def _tol(dtype):
    return (1e-2, 1e-2) if dtype in (torch.bfloat16, torch.float16) else (1e-5, 1e-5)


@pytest.mark.parametrize("name", ["softmax_backward_bf16_8192x4096", "log_softmax_backward_bf16_8192x4096", "softmax_backward_f32_65536x1024", "log_softmax_backward_f32_65536x1024"])
def test_full_size_matches_aten_cuda_and_oracle_rows(backend, name):
    c = named_case(name)
    op = get_operator(c.op)
    args, kwargs = c.build(DEV)
    got = backend[op](*args, **kwargs)
    want = op(*args, **kwargs)
    atol, rtol = _tol(got.dtype)
    ok, ea, er = compare(want, got, atol, rtol)
    assert ok and got.dtype == want.dtype and got.shape == want.shape, (ea, er)
    head = [a[:64].cpu() if isinstance(a, torch.Tensor) else a for a in args]
    ok, ea, er = compare(oracle.run(c.op, head, {}).to(DEV), got[:64], atol, rtol)
    assert ok, (ea, er)
    # rows of a softmax gradient sum to zero: sum_j (g_j - s) y_j = s - s
    if c.op == SOFT:
        assert float(got.float().sum(-1).abs().max()) < (2e-2 if got.dtype != torch.float32 else 1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_ragged_non_last_dim_and_strided_inputs(backend, dtype):
    g = torch.Generator(device=DEV).manual_seed(6)
    atol, rtol = _tol(dtype)
    for shape, dim in [((300, 67), -1), ((5, 1000, 9), 1), ((40, 7, 33), 0), ((1, 8192), 1), ((3, 0, 4), 2), ((2049,), 0)]:
        x = torch.randn(shape, device=DEV, generator=g)
        grad = torch.randn(shape, device=DEV, generator=g).to(dtype)
        for spec, fwd in ((SOFT, torch.softmax), (LOGSOFT, torch.log_softmax)):
            y = fwd(x, dim).to(dtype)
            op = get_operator(spec)
            ok, ea, er = compare(op(grad, y, dim, dtype), backend[op](grad, y, dim, dtype), atol, rtol)
            assert ok, (spec, shape, dim, ea, er)
    x = torch.randn(64, 96, device=DEV, generator=g)
    grad_t = torch.randn(96, 64, device=DEV, generator=g).to(dtype).t()  # a transposed incoming gradient
    y = torch.softmax(x, -1).to(dtype)
    op = get_operator(SOFT)
    ok, ea, er = compare(op(grad_t, y, -1, dtype), backend[op](grad_t, y, -1, dtype), atol, rtol)
    assert ok, (ea, er)
    ops.check_device_status()


def test_float_gradients_for_a_half_input(backend):
    """The half_to_float form: fp32 grad_output / output, 16-bit grad_input."""
    g = torch.Generator(device=DEV).manual_seed(7)
    for shape in [(128, 4096), (77, 130)]:
        x = torch.randn(shape, device=DEV, generator=g)
        grad = torch.randn(shape, device=DEV, generator=g)
        for spec, fwd in ((SOFT, torch.softmax), (LOGSOFT, torch.log_softmax)):
            op = get_operator(spec)
            for dt in (torch.float16, torch.bfloat16):
                # aten CUDA takes this form for an f16 input only; the bf16 result is checked against the fp32 one, rounded
                want = op(grad, fwd(x, -1), -1, dt) if dt == torch.float16 else op(grad, fwd(x, -1), -1, torch.float32).to(dt)
                got = backend[op](grad, fwd(x, -1), -1, dt)
                ok, ea, er = compare(want, got, 1e-2, 1e-2)
                assert ok and got.dtype == dt, (spec, shape, dt, ea, er)


LNB = "native_layer_norm_backward.default"


def _check_tuple(want, got, atol, rtol, tag):
    assert len(want) == len(got), tag
    for i, (w_, g_) in enumerate(zip(want, got)):
        if w_ is None or g_ is None:
            assert w_ is None and g_ is None, (tag, i)
            continue
        assert w_.shape == g_.shape and w_.dtype == g_.dtype, (tag, i, w_.shape, g_.shape, w_.dtype, g_.dtype)
        ok, ea, er = compare(w_, g_, atol, rtol)
        assert ok, (tag, i, ea, er)


@pytest.mark.parametrize("name", ["layer_norm_backward_bf16_8192x4096", "layer_norm_backward_f32_65536x1024"])
def test_full_size_layer_norm_backward(backend, name):
    c = named_case(name)
    op = get_operator(c.op)
    args, kwargs = c.build(DEV)
    got = backend[op](*args, **kwargs)
    want = op(*args, **kwargs)
    # dx to the dtype's tolerance; dw / db are sums over thousands of rows: compare at the size of those sums
    atol, rtol = _tol(got[0].dtype)
    _check_tuple(want[:1], got[:1], atol, rtol, name)
    scale = float(want[1].float().abs().max())
    _check_tuple(want[1:], got[1:], max(atol, 2e-3 * scale), 1e-2 if got[0].dtype != torch.float32 else 1e-3, name)
    head = [a[:64].cpu() if isinstance(a, torch.Tensor) and a.dim() == 2 and a.shape[0] == args[0].shape[0] else (a.cpu() if isinstance(a, torch.Tensor) else a) for a in args]
    head[-1] = [True, False, False]
    _check_tuple(oracle.run(c.op, head, {})[:1], (got[0][:64].cpu(),), atol, rtol, name + "/oracle")
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_layer_norm_backward_geometries_and_masks(backend, dtype):
    g = torch.Generator(device=DEV).manual_seed(9)
    atol, rtol = (3e-2, 2e-2) if dtype != torch.float32 else (1e-4, 1e-4)
    op = get_operator(LNB)
    for shape, nd in [((300, 67), 1), ((5, 40, 1000), 1), ((6, 8, 5), 2), ((64, 8200), 1), ((3, 16384), 1), ((1, 96), 1), ((2000, 17), 1)]:
        x = torch.randn(shape, device=DEV, generator=g).to(dtype)
        dy = torch.randn(shape, device=DEV, generator=g).to(dtype)
        ns = list(shape[-nd:])
        w, b = torch.randn(ns, device=DEV, generator=g).to(dtype), torch.randn(ns, device=DEV, generator=g).to(dtype)
        _, mean, rstd = torch.ops.aten.native_layer_norm.default(x, ns, w, b, 1e-5)
        for weight, bias, mask in [(w, b, [True, True, True]), (w, None, [True, True, False]), (None, None, [True, False, False]), (w, b, [False, True, True]), (w, b, [True, False, False])]:
            want = op(dy, x, ns, mean, rstd, weight, bias, mask)
            got = backend[op](dy, x, ns, mean, rstd, weight, bias, mask)
            rows = x.numel() // max(1, int(torch.tensor(ns).prod()))
            _check_tuple(want[:1], got[:1], atol, rtol, (shape, mask))
            _check_tuple(want[1:], got[1:], atol * max(1.0, rows**0.5), rtol, (shape, mask))
    # fp32 parameters with 16-bit activations (autocast-style)
    if dtype != torch.float32:
        x = torch.randn(128, 512, device=DEV, generator=g).to(dtype)
        dy = torch.randn(128, 512, device=DEV, generator=g).to(dtype)
        w32 = torch.randn(512, device=DEV, generator=g)
        xf = x.float()
        mean, rstd = xf.mean(-1, keepdim=True), torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + 1e-5)
        got = backend[op](dy, x, [512], mean, rstd, w32, w32, [True, True, True])
        xhat = (xf - mean) * rstd
        gy = dy.float() * w32
        dx = rstd * (gy - gy.mean(-1, keepdim=True) - xhat * (gy * xhat).mean(-1, keepdim=True))
        _check_tuple((dx.to(dtype), (dy.float() * xhat).sum(0), dy.float().sum(0)), got, 3e-2, 2e-2, "fp32 params")
    ops.check_device_status()


EMB = "embedding_dense_backward.default"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_embedding_backward_matches_oracle_bit_for_bit_and_aten_closely(backend, dtype):
    """Rows are added in ascending position in fp32 and rounded once: the CPU oracle does the
    same, so results agree bit for bit (and run to run); aten CUDA agrees to tolerance."""
    g = torch.Generator().manual_seed(10)
    op = get_operator(EMB)
    impl = backend[op]
    for n_shape, V, D, hot in [((500,), 97, 64, None), ((40, 50), 300, 257, None), ((5000,), 50, 96, 3), ((70000,), 8, 40, 2), ((3,), 1000, 8, None), ((0,), 10, 16, None)]:
        idx = torch.randint(0, V, n_shape, generator=g)
        if hot is not None:  # most positions on a few rows: the many-contributions path
            idx[torch.rand(n_shape, generator=g) < 0.9] = hot
        grad = torch.randn(n_shape + (D,), generator=g).to(dtype)
        pad = 1 if V > 1 else -1
        got = impl(grad.to(DEV), idx.to(DEV), V, pad, False)
        want = oracle.embedding_backward(grad, idx, V, pad, False)
        from conftest import bits_equal

        assert got.shape == (V, D) and got.dtype == dtype and bits_equal(want, got.cpu()), (n_shape, V, D)
        assert bits_equal(got, impl(grad.to(DEV), idx.to(DEV).int(), V, pad, False))  # int32 indices, and reproducible
        ref = op(grad.to(DEV), idx.to(DEV), V, pad, False)
        contributions = max(1, idx.numel() // V if hot is None else idx.numel())
        ok, ea, er = compare(ref, got, (2e-2 if dtype != torch.float32 else 1e-5) * contributions**0.5, 2e-2 if dtype != torch.float32 else 1e-4)
        assert ok, (n_shape, V, D, ea, er)
    ops.check_device_status()
    idx = torch.tensor([1, 5, 99, 2], device=DEV)
    impl(torch.randn(4, 8, device=DEV).to(dtype), idx, 10, -1, False)
    with pytest.raises(IndexError):
        ops.check_device_status()


def test_full_size_embedding_backward(backend):
    c = named_case("embedding_backward_bf16_128256x4096_16384")
    op = get_operator(c.op)
    args, kwargs = c.build(DEV)
    got, want = backend[op](*args, **kwargs), op(*args, **kwargs)
    ok, ea, er = compare(want, got, 2e-2, 2e-2)
    assert ok and got.shape == want.shape and got.dtype == want.dtype, (ea, er)
    touched = torch.zeros(128256, dtype=torch.bool, device=DEV)
    touched[args[1]] = True
    assert float(got[~touched].abs().max()) == 0.0  # rows nobody indexed are exactly zero


def test_autograd_through_registered_overrides():
    """With the kernels registered through torch.library, a softmax forward + backward of an
    ordinary autograd graph runs on them and matches aten."""
    import backendbench_b200 as bb

    x = torch.randn(200, 512, device=DEV, requires_grad=True)
    w = torch.randn(200, 512, device=DEV)
    (torch.softmax(x, -1) * w).sum().backward()
    want = x.grad.clone()
    x.grad = None
    bb.enable()
    try:
        (torch.softmax(x, -1) * w).sum().backward()
    finally:
        bb.disable()
    torch.testing.assert_close(x.grad, want, rtol=1e-5, atol=1e-6)
    # layer norm forward + backward, parameters included
    ln = torch.nn.LayerNorm(512).to(DEV)
    x.grad = None
    (ln(x) * w).sum().backward()
    want = [x.grad.clone(), ln.weight.grad.clone(), ln.bias.grad.clone()]
    x.grad = ln.weight.grad = ln.bias.grad = None
    bb.enable()
    try:
        (ln(x) * w).sum().backward()
    finally:
        bb.disable()
    for got_t, want_t in zip([x.grad, ln.weight.grad, ln.bias.grad], want):
        torch.testing.assert_close(got_t, want_t, rtol=1e-4, atol=1e-4)
    # embedding forward + backward
    emb = torch.nn.Embedding(1000, 64).to(DEV)
    tok = torch.randint(0, 1000, (32, 50), device=DEV)
    up = torch.randn(32, 50, 64, device=DEV)
    (emb(tok) * up).sum().backward()
    want_w = emb.weight.grad.clone()
    emb.weight.grad = None
    bb.enable()
    try:
        (emb(tok) * up).sum().backward()
    finally:
        bb.disable()
    torch.testing.assert_close(emb.weight.grad, want_w, rtol=1e-5, atol=1e-5)
