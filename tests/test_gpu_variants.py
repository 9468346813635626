"""`.out` and in-place overloads (BackendBench/scripts/op_map.py:7-1148 lists them beside each
functional operator): same kernels, result placed in the tensor the overload names --
written directly for contiguous in-place elementwise calls, through the strided-to-strided
copy kernel otherwise. Checked against aten on the same device tensors."""

import pytest
import torch

from backendbench_b200 import ops
from backendbench_b200.backends import B200Backend
from backendbench_b200.opregistry import get_operator
from backendbench_b200.variants import VARIANT_TABLE
from conftest import bits_equal

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def backend():
    return B200Backend()


def _impl(backend, spec):
    return backend[get_operator(spec)]


def test_every_variant_is_served_by_the_backend(backend):
    for spec in VARIANT_TABLE:
        assert get_operator(spec) in backend, spec


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_in_place_elementwise(backend, dtype):
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(300, 257, device=DEV, generator=g).to(dtype)
    y = torch.randn(257, device=DEV, generator=g).to(dtype)
    for spec, aten_fn, extra in [("relu_.default", torch.Tensor.relu_, ()), ("add_.Tensor", torch.Tensor.add_, (y,)), ("mul_.Tensor", torch.Tensor.mul_, (y,))]:
        mine, ref = x.clone(), x.clone()
        ptr = mine.data_ptr()
        ret = _impl(backend, spec)(mine, *extra)
        assert ret is mine and mine.data_ptr() == ptr and bits_equal(aten_fn(ref, *extra), mine), spec
    # a non-contiguous `self`: a transposed view and a strided slice are updated through their own strides
    base_m, base_r = x.clone(), x.clone()
    _impl(backend, "relu_.default")(base_m.t())
    base_r.t().relu_()
    assert bits_equal(base_r, base_m)
    base_m, base_r = x.clone(), x.clone()
    _impl(backend, "add_.Tensor")(base_m[::2, 1::3], y[1::3], alpha=2)
    base_r[::2, 1::3].add_(y[1::3], alpha=2)
    assert bits_equal(base_r, base_m)
    # operands that alias `self`
    sq_m, sq_r = x[:257].clone(), x[:257].clone()
    _impl(backend, "add_.Tensor")(sq_m, sq_m)
    sq_r.add_(sq_r)
    assert bits_equal(sq_r, sq_m)
    sq_m, sq_r = x[:257].clone(), x[:257].clone()
    _impl(backend, "mul_.Tensor")(sq_m, sq_m.t())  # same storage, different layout: must not be updated while it is read
    sq_r.mul_(sq_r.t().clone())
    assert bits_equal(sq_r, sq_m)
    with pytest.raises(RuntimeError):
        _impl(backend, "add_.Tensor")(y.clone(), x)  # the broadcast result does not fit `self`
    ops.check_device_status()


def test_out_overloads_fill_resize_and_respect_strides(backend):
    g = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn(64, 200, device=DEV, generator=g)
    y = torch.randn(64, 200, device=DEV, generator=g)
    idx = torch.randint(0, 64, (64, 200), device=DEV, generator=g)
    sel = torch.randint(0, 200, (33,), device=DEV, generator=g)
    w, b = torch.randn(200, device=DEV, generator=g), torch.randn(200, device=DEV, generator=g)
    m1, m2 = torch.randn(64, 96, device=DEV, generator=g), torch.randn(96, 200, device=DEV, generator=g)
    b1, b2 = torch.randn(3, 64, 96, device=DEV, generator=g), torch.randn(3, 96, 200, device=DEV, generator=g)
    table = torch.randn(500, 32, device=DEV, generator=g)
    jobs = [
        ("relu.out", torch.relu, (x,), {}, True),
        ("add.out", torch.add, (x, y), {"alpha": 3}, True),
        ("mul.out", torch.mul, (x, y), {}, True),
        ("where.self_out", torch.where, (x > 0, x, y), {}, True),
        ("_softmax.out", torch.ops.aten._softmax.default, (x, 1, False), {}, False),
        ("_log_softmax.out", torch.ops.aten._log_softmax.default, (x, 1, False), {}, False),
        ("sum.IntList_out", torch.sum, (x, [1]), {}, False),
        ("argmax.out", torch.argmax, (x, 1), {}, True),
        ("embedding.out", torch.ops.aten.embedding.default, (table, sel), {}, True),
        ("index_select.out", torch.index_select, (x, 1, sel), {}, True),
        ("gather.out", torch.gather, (x, 0, idx), {}, True),
        ("mm.out", torch.mm, (m1, m2), {}, False),
        ("bmm.out", torch.bmm, (b1, b2), {}, False),
        ("addmm.out", torch.addmm, (x, m1, m2), {"beta": 0.5, "alpha": 2}, False),
    ]
    for spec, aten_fn, args, kwargs, exact in jobs:
        want = aten_fn(*args, **kwargs)
        for kind in ("fits", "wrong_shape", "strided"):
            if kind == "fits":
                out = torch.empty_like(want)
            elif kind == "wrong_shape":
                out = torch.empty(0, dtype=want.dtype, device=DEV)
            else:
                out = torch.empty(tuple(want.shape[:-1]) + (want.shape[-1] * 2 + 1,), dtype=want.dtype, device=DEV)[..., 1::2] if want.dim() else torch.empty((), dtype=want.dtype, device=DEV)
            ret = _impl(backend, spec)(*args, **kwargs, out=out)
            assert ret is out and out.shape == want.shape, (spec, kind)
            if exact:
                assert bits_equal(want, out), (spec, kind)
            else:
                torch.testing.assert_close(out, want, rtol=1e-4, atol=1e-4)
    with pytest.raises(RuntimeError):
        _impl(backend, "relu.out")(x, out=torch.empty_like(x, dtype=torch.float16))
    ops.check_device_status()


def test_layer_norm_out_scatter_add_and_addmm_in_place(backend):
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn(128, 96, device=DEV, generator=g)
    w, b = torch.randn(96, device=DEV, generator=g), torch.randn(96, device=DEV, generator=g)
    want = torch.ops.aten.native_layer_norm.default(x, [96], w, b, 1e-5)
    outs = [torch.empty_like(t) for t in want]
    got = _impl(backend, "native_layer_norm.out")(x, [96], w, b, 1e-5, out0=outs[0], out1=outs[1], out2=outs[2])
    for o, r, t in zip(outs, got, want):
        assert r is o
        torch.testing.assert_close(o, t, rtol=1e-4, atol=1e-4)
    idx = torch.randint(0, 128, (300, 96), device=DEV, generator=g)
    src = torch.randn(300, 96, device=DEV, generator=g)
    mine = x.clone()
    ret = _impl(backend, "scatter_add_.default")(mine, 0, idx, src)
    assert ret is mine and bits_equal(x.cpu().scatter_add(0, idx.cpu(), src.cpu()), mine)  # aten CPU order, bit for bit
    out = torch.empty(5, device=DEV)
    ret = _impl(backend, "scatter_add.out")(x, 0, idx, src, out=out)
    assert ret is out and bits_equal(mine, out)
    m1, m2 = torch.randn(128, 40, device=DEV, generator=g), torch.randn(40, 96, device=DEV, generator=g)
    acc = x.clone()
    ret = _impl(backend, "addmm_.default")(acc, m1, m2, beta=2, alpha=0.5)
    assert ret is acc
    torch.testing.assert_close(acc, torch.addmm(x, m1, m2, beta=2, alpha=0.5), rtol=1e-4, atol=1e-4)
    ops.check_device_status()


def test_registered_overrides_serve_in_place_and_out_calls():
    """With the kernels registered through torch.library (BackendBench.enable's mechanism),
    ordinary PyTorch spellings reach the variants."""
    import backendbench_b200 as bb

    x = torch.randn(100, 40, device=DEV)
    y = torch.randn(100, 40, device=DEV)
    want_relu, want_add = torch.relu(x), x + y
    bb.enable()
    try:
        a = x.clone()
        a.relu_()
        out = torch.empty_like(x)
        torch.add(x, y, out=out)
    finally:
        bb.disable()
    assert bits_equal(want_relu, a) and bits_equal(want_add, out)


def test_mixed_precision_targets_follow_aten(backend):
    """add_/mul_ and add.out / mul.out / sum.out accept any target type the result type can be
    cast to (aten rounds the full-precision result once into the target); the other overloads
    insist on the exact type, with aten's message."""
    g = torch.Generator(device=DEV).manual_seed(11)
    xb = torch.randn(129, 65, device=DEV, generator=g).to(torch.bfloat16)
    yf = torch.randn(129, 65, device=DEV, generator=g)
    for spec, aten_fn in (("add_.Tensor", torch.Tensor.add_), ("mul_.Tensor", torch.Tensor.mul_)):
        mine, ref = xb.clone(), xb.clone()
        ret = _impl(backend, spec)(mine, yf)
        assert ret is mine and mine.dtype == torch.bfloat16 and bits_equal(aten_fn(ref, yf), mine), spec
    mine, ref = xb.clone(), xb.clone()
    _impl(backend, "add_.Tensor")(mine, yf, alpha=0.5)
    assert bits_equal(ref.add_(yf, alpha=0.5), mine)
    out_m, out_r = torch.empty(129, 65, device=DEV, dtype=torch.bfloat16), torch.empty(129, 65, device=DEV, dtype=torch.bfloat16)
    _impl(backend, "add.out")(yf, yf * 3, out=out_m)
    torch.add(yf, yf * 3, out=out_r)
    assert bits_equal(out_r, out_m)
    _impl(backend, "mul.out")(yf, xb, out=out_m)
    torch.mul(yf, xb, out=out_r)
    assert bits_equal(out_r, out_m)
    s_m, s_r = torch.empty(129, device=DEV, dtype=torch.bfloat16), torch.empty(129, device=DEV, dtype=torch.bfloat16)
    _impl(backend, "sum.IntList_out")(yf, [-1], out=s_m)
    torch.sum(yf, [-1], out=s_r)
    # aten rounds the INPUTS to the out type before it adds (65 values of magnitude ~1, each off by
    # up to 2^-9 relative); this backend adds the fp32 inputs and rounds the sum once
    assert torch.allclose(s_m.float(), s_r.float(), rtol=1e-2, atol=0.1) and torch.allclose(s_m.float(), yf.double().sum(-1).float(), rtol=1e-2, atol=1e-2)
    with pytest.raises(RuntimeError, match="can't be cast to the desired output type Long"):
        _impl(backend, "add.out")(yf, yf, out=torch.empty(129, 65, device=DEV, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="Expected out tensor to have dtype"):
        _impl(backend, "mm.out")(yf, yf.t().contiguous(), out=torch.empty(129, 129, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="Expected out tensor to have dtype"):
        _impl(backend, "relu.out")(yf, out=torch.empty(129, 65, device=DEV, dtype=torch.bfloat16))
