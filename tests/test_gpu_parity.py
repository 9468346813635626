"""Parity of the CUDA kernels (through the C-ABI-backed operators) with the golden vectors
made by the reference harness over aten CPU, with the CPU oracle on seeded sweep cases,
and -- at the full named sizes -- through aten on the same device tensors plus
size-independent properties. Bit-exact for integer / indexing results and scatter_add;
floating point within the tolerance written in `conftest.tolerance_for_case`."""

import math

import pytest
import torch

import oracle
from backendbench_b200 import _abi, ops
from backendbench_b200.backends import B200Backend
from backendbench_b200.cases import named_case, named_cases, scaled_down, sweep_cases
from backendbench_b200.eval import compare
from backendbench_b200.opregistry import get_operator
from conftest import EXACT_OPS, bits_equal, first_dtype, tolerance_for_case

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def backend():
    assert torch.cuda.is_available()
    assert _abi.lib().b200_abi_version() == _abi.ABI_VERSION  # the native library is the thing under test
    return B200Backend()


def _to_dev(x):
    if isinstance(x, torch.Tensor):
        return x.to(DEV)
    if isinstance(x, (list, tuple)):
        return type(x)(_to_dev(y) for y in x)
    return x


def _tup(x):
    return tuple(x) if isinstance(x, (tuple, list)) else (x,)


def _check(op_name, ref, got, tag):
    """`ref` on CPU (golden / oracle), `got` from the GPU."""
    ref, got = _tup(ref), tuple(g.cpu() if g is not None else None for g in _tup(got))
    assert len(ref) == len(got), tag
    atol, rtol = tolerance_for_case(op_name, first_dtype(ref))
    for i, (r, g) in enumerate(zip(ref, got)):
        if r is None or g is None:  # an output masked out (native_layer_norm_backward's output_mask)
            assert r is None and g is None, tag
            continue
        if op_name == "native_layer_norm.default" and i > 0:
            r, g = r.float(), g.float()  # statistics: CPU keeps the input dtype, CUDA fp32
            if r.dtype != torch.float32 or atol < 1e-2:
                pass
            a, rt = (1e-2, 1e-2) if first_dtype(ref) != torch.float32 else (atol, rtol)
            ok, ea, er = compare(r, g, a, rt)
            assert ok, (tag, "stat", i, ea, er)
            continue
        assert r.shape == g.shape and r.dtype == g.dtype, (tag, r.shape, g.shape, r.dtype, g.dtype)
        if op_name in EXACT_OPS:
            assert bits_equal(r, g), (tag, "bits differ")
        else:
            ok, ea, er = compare(r, g, atol, rtol)
            assert ok, (tag, ea, er)


def test_gpu_matches_golden_vectors(backend, golden_cases):
    for c in golden_cases:
        impl = backend[get_operator(c["op"])]
        got = impl(*_to_dev(c["args"]), **_to_dev(c["kwargs"]))
        ops.check_device_status()
        _check(c["op"], c["ref"], got, c["tag"])


def test_gpu_matches_oracle_on_seeded_sweep_cases(backend):
    """Every sweep case small enough for the single-threaded oracle (edge cases included:
    zero-size dims, broadcast dims, transposed strides, NaN/Inf injection)."""
    cases = [c for c in sweep_cases(512, seed=0) if c.algorithmic_bytes() < 6e6 and c.flops() < 6e8]
    assert len(cases) > 250 and {c.edge for c in cases} >= {"", "zero", "bcast", "transposed", "naninf"}
    for c in cases:
        args, kwargs = c.build(DEV, gen_device="cpu")
        got = backend[get_operator(c.op)](*args, **kwargs)
        want = oracle.run(c.op, args, kwargs)
        _check(c.op, want, got, c.label())
    ops.check_device_status()


def test_gpu_matches_oracle_second_seed_and_other_paths(backend):
    cases = [c for c in sweep_cases(384, seed=1) if c.algorithmic_bytes() < 3e6 and c.flops() < 3e8]
    for c in cases:
        args, kwargs = c.build(DEV, gen_device="cpu")
        got = backend[get_operator(c.op)](*args, **kwargs)
        _check(c.op, oracle.run(c.op, args, kwargs), got, c.label())
    ops.check_device_status()


@pytest.mark.parametrize("name", [c.name for c in named_cases()])
def test_named_configs_scaled_to_oracle_size(backend, name):
    c = scaled_down(named_case(name), 16)
    args, kwargs = c.build(DEV, gen_device="cpu")
    got = backend[get_operator(c.op)](*args, **kwargs)
    ops.check_device_status()
    _check(c.op, oracle.run(c.op, args, kwargs), got, c.label())


# ------------------------------------------------------------------ full named sizes
def _full(name, backend):
    c = named_case(name)
    args, kwargs = c.build(DEV)
    op = get_operator(c.op)
    return c, op, backend[op], args, kwargs


@pytest.mark.parametrize("name", ["relu_f32_4096x4096", "add_f32_4096x4096", "mul_f32_4096x4096", "where_f32_4096x4096"])
def test_full_size_elementwise_bit_exact_vs_aten(backend, name):
    c, op, impl, args, kwargs = _full(name, backend)
    got, ref = impl(*args, **kwargs), op(*args, **kwargs)
    assert bits_equal(ref, got)  # one fp32 operation per element: no rounding freedom
    if name.startswith("relu"):
        assert bits_equal(impl(got), got) and float(got.min()) >= 0  # idempotent, non-negative
    if name.startswith("where"):
        cond, x, y = args
        other = impl(~cond, x, y)
        assert bits_equal(torch.where(cond, got, other), x) and bits_equal(torch.where(cond, other, got), y)


@pytest.mark.parametrize("tag", ["bf16_8192x4096", "f32_65536x1024"])
def test_full_size_softmax_family(backend, tag):
    c, op, impl, args, kwargs = _full(f"softmax_{tag}", backend)
    got, ref = impl(*args, **kwargs), op(*args, **kwargs)
    atol, rtol = tolerance_for_case(c.op, got.dtype)
    assert compare(ref, got, atol, rtol)[0]
    rows = got.float().sum(-1)
    assert torch.allclose(rows, torch.ones_like(rows), atol=2e-2 if got.dtype != torch.float32 else 1e-5)
    assert float(got.min()) >= 0
    softmax_impl = impl
    c, op, impl, args, kwargs = _full(f"log_softmax_{tag}", backend)
    lg, lref = impl(*args, **kwargs), op(*args, **kwargs)
    assert compare(lref, lg, atol, rtol)[0]
    assert compare(got.float(), lg.float().exp(), 2e-2 if got.dtype != torch.float32 else 1e-5, 1e-2)[0]  # exp(log_softmax) == softmax
    # shift invariance softmax(x + c) == softmax(x); in fp32 the shift perturbs x by < 1e-6
    if got.dtype == torch.float32:
        xs = args[0] + 8.0
        ok, ea, er = compare(got, softmax_impl(xs, -1, False), 1e-5, 1e-3)
        assert ok, (ea, er)


@pytest.mark.parametrize("tag", ["bf16_8192x4096", "f32_65536x1024"])
def test_full_size_sum_and_layer_norm(backend, tag):
    c, op, impl, args, kwargs = _full(f"sum_{tag}", backend)
    got, ref = impl(*args, **kwargs), op(*args, **kwargs)
    atol, rtol = tolerance_for_case(c.op, got.dtype)
    assert compare(ref, got, max(atol, 1e-3), rtol)[0]
    # against fp64 on the device, and linearity sum(2x) == 2 sum(x) (exact: scaling by 2 commutes with rounding)
    exact = args[0].double().sum(-1)
    assert compare(exact.to(got.dtype), got, 2.5e-1 if got.dtype != torch.float32 else 1e-3, rtol)[0]
    assert bits_equal(impl((args[0] * 2), [-1]), got * 2)
    c, op, impl, args, kwargs = _full(f"layer_norm_{tag}", backend)
    (y, mean, rstd), (ry, rmean, rrstd) = impl(*args, **kwargs), op(*args, **kwargs)
    assert mean.dtype == rmean.dtype and mean.shape == rmean.shape  # aten CUDA's statistics dtype and shape
    assert compare(ry, y, *tolerance_for_case(c.op, y.dtype))[0]
    assert compare(rmean, mean, 1e-4, 1e-4)[0] and compare(rrstd, rstd, 1e-4, 1e-4)[0]
    x = args[0].float()
    assert compare(x.mean(-1, keepdim=True), mean, 1e-4, 1e-4)[0]
    # with unit weight and zero bias every row has mean 0 and variance 1
    y1, _, _ = impl(args[0], args[1], None, None, 1e-5)
    yf = y1.float()
    tol = 2e-2 if y1.dtype != torch.float32 else 1e-4
    assert float(yf.mean(-1).abs().max()) < tol and float((yf.var(-1, unbiased=False) - 1).abs().max()) < 5 * tol


def test_full_size_embedding_and_index_select_bit_exact(backend):
    c, op, impl, args, kwargs = _full("embedding_bf16_128256x4096_16384", backend)
    got = impl(*args, **kwargs)
    assert bits_equal(op(*args, **kwargs), got)
    table, idx = args
    # the oracle on the same bits (CPU copy), on a slice of the lookups
    assert bits_equal(oracle.embedding(table.cpu(), idx[:512].cpu()), got[:512])
    # round trip: looking up a permutation and then its inverse restores the rows
    perm = torch.randperm(4096, device=DEV)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(4096, device=DEV)
    sub = table[:4096]
    assert bits_equal(impl(impl(sub, perm), inv), sub)
    c, op, impl, args, kwargs = _full("index_select_bf16_128256x4096_16384", backend)
    assert bits_equal(op(*args, **kwargs), impl(*args, **kwargs))
    ops.check_device_status()


def test_full_size_gather_bit_exact(backend):
    c, op, impl, args, kwargs = _full("gather_f32_4096x4096", backend)
    got = impl(*args, **kwargs)
    assert bits_equal(op(*args, **kwargs), got)
    x, dim, idx = args
    assert bits_equal(oracle.gather(x.cpu(), 0, idx[:64].cpu()), got[:64])
    ident = torch.arange(4096, device=DEV).unsqueeze(1).expand(4096, 4096).contiguous()
    assert bits_equal(impl(x, 0, ident), x)  # identity index: gather is the identity
    assert bits_equal(op(x, 1, idx), impl(x, 1, idx))  # the other dimension
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_elementwise_on_transposed_views_goes_through_tiles(backend, dtype):
    """Operands whose unit stride runs along the second-to-last dim: 2-D and batched, ragged
    tile edges, one or both operands transposed, a broadcast partner, and the strided copy."""
    g = torch.Generator().manual_seed(41)
    add, mul, relu = backend[torch.ops.aten.add.Tensor], backend[torch.ops.aten.mul.Tensor], backend[torch.ops.aten.relu.default]
    for shape in [(1000, 70), (33, 1025), (5, 130, 47)]:
        tshape = shape[:-2] + (shape[-1], shape[-2])
        a = torch.randn(tshape, generator=g).to(dtype).to(DEV).transpose(-1, -2)
        b = torch.randn(tshape, generator=g).to(dtype).to(DEV).transpose(-1, -2)
        c = torch.randn(shape, generator=g).to(dtype).to(DEV)
        row = torch.randn(shape[-1], generator=g).to(dtype).to(DEV)
        assert not a.is_contiguous()
        for got, want in [(add(a, b), a + b), (add(a, c, alpha=2), torch.add(a, c, alpha=2)), (mul(c, b), c * b), (mul(a, row), a * row), (relu(a), torch.relu(a)),
                          (ops._contig(a), a.contiguous())]:
            assert bits_equal(want, got), shape
    ints = torch.randint(-5, 5, (300, 41), generator=g, dtype=torch.int64).to(DEV).t()
    assert bits_equal(ints.contiguous(), ops._contig(ints))


def test_index_select_along_the_last_dim_through_shared_memory(backend):
    impl = backend[torch.ops.aten.index_select.default]
    g = torch.Generator().manual_seed(8)
    for shape, dtype, n_idx in [((1000, 300), torch.float32, 1190), ((513, 77), torch.bfloat16, 40), ((400, 64), torch.int64, 64), ((3, 700, 1024), torch.float16, 16), ((2000, 33), torch.uint8, 100)]:
        x = (torch.randn(shape, generator=g) * 100).to(dtype).to(DEV)
        idx = torch.randint(0, shape[-1], (n_idx,), generator=g).to(DEV)
        assert bits_equal(torch.index_select(x, -1, idx), impl(x, x.dim() - 1, idx))
        assert bits_equal(torch.index_select(x, -1, idx.int()), impl(x, x.dim() - 1, idx.int()))
    ops.check_device_status()
    x = torch.randn(600, 128, device=DEV)
    idx = torch.randint(0, 128, (64,), device=DEV)
    idx[5] = 128
    got = impl(x, 1, idx)
    with pytest.raises(IndexError):
        ops.check_device_status()
    want = torch.index_select(x, 1, idx.clamp(0, 127))
    want[:, 5] = 0
    assert bits_equal(want, got)


def test_gather_rows_of_self_held_in_shared_memory(backend):
    """dim-0 gather whose source strip fits in shared memory: ragged row counts, row splits,
    a source with a row pitch, and an out-of-range index that must be reported, not read."""
    impl = backend[torch.ops.aten.gather.default]
    g = torch.Generator(device="cpu").manual_seed(7)
    for self_rows, rows, cols in [(1000, 777, 1280), (4096, 2051, 1192), (513, 4099, 2368)]:
        wide = torch.randn(self_rows, cols + 8, generator=g).to(DEV)
        for x in (wide[:, :cols].contiguous(), wide[:, 4 : cols + 4]):  # dense, and pitched with an offset
            idx = torch.randint(0, self_rows, (rows, cols), generator=g).to(DEV)
            assert bits_equal(torch.gather(x, 0, idx), impl(x, 0, idx))
            ops.check_device_status()
    x = torch.randn(600, 1280, device=DEV)
    idx = torch.randint(0, 600, (700, 1280), device=DEV)
    idx[5, 9] = 600
    idx[699, 1279] = -1
    got = impl(x, 0, idx)
    with pytest.raises(IndexError):
        ops.check_device_status()
    ok = idx.clamp(0, 599)
    want = torch.gather(x, 0, ok)
    want[5, 9] = 0
    want[699, 1279] = 0
    assert bits_equal(want, got)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_argmax_rows_where_whole_vectors_are_skipped(backend, dtype):
    """The row kernel screens 16-byte vectors (largest element and a NaN guard) before it looks
    at elements: ties must still go to the first index, NaN to the first NaN, and vectors
    holding both infinities (whose guard sum is NaN) must take the exact path."""
    impl = backend[torch.ops.aten.argmax.default]
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 4096, generator=g).to(dtype)
    x[0] = 1.5                                   # all equal: index 0
    x[1] = float("-inf")                         # all -inf: index 0
    x[2, 100] = float("inf"); x[2, 101] = float("-inf"); x[2, 3000] = float("inf")   # first +inf wins
    x[3, 7] = 9.0; x[3, 2049] = float("nan"); x[3, 4000] = float("nan")              # first NaN wins over a larger value before it
    x[4, 4095] = 50.0                            # the very last element
    x[5, :2048] = 2.0; x[5, 2048:] = 2.0; x[5, 1234] = 2.0                            # a plateau
    x[6] = torch.arange(4096, 0, -1).to(dtype)   # descending: nothing after index 0 is ever taken
    x[7] = torch.arange(4096).to(dtype)          # ascending: every vector replaces the best
    want = torch.argmax(x, dim=-1)
    got = impl(x.to(DEV), -1)
    assert torch.equal(want, got.cpu())
    long_rows = torch.randn(3, 70000, generator=g).to(dtype)  # split rows
    long_rows[1, 69999] = float("nan")
    assert torch.equal(torch.argmax(long_rows, dim=-1), impl(long_rows.to(DEV), -1).cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_gather_along_the_last_dim(backend, dtype):
    """2-D gather along the last dim: 16 bytes of adjacent outputs per thread; fewer index rows
    than source rows, a pitched source, an index width that is not a multiple of the vector
    (falls to the element kernel), an out-of-range index."""
    impl = backend[torch.ops.aten.gather.default]
    g = torch.Generator(device="cpu").manual_seed(17)
    for self_rows, self_cols, rows, cols in [(300, 1024, 200, 1024), (64, 5000, 64, 256), (17, 33, 17, 4096), (500, 100, 500, 1003)]:
        wide = torch.randn(self_rows, self_cols + 8, generator=g).to(dtype).to(DEV)
        for x in (wide[:, :self_cols].contiguous(), wide[:, 3 : self_cols + 3]):
            idx = torch.randint(0, self_cols, (rows, cols), generator=g).to(DEV)
            assert bits_equal(torch.gather(x, 1, idx), impl(x, 1, idx))
            ops.check_device_status()
    x = torch.randn(40, 96, device=DEV).to(dtype)
    idx = torch.randint(0, 96, (40, 64), device=DEV)
    idx[3, 7] = 96
    idx[39, 63] = -5
    got = impl(x, 1, idx)
    with pytest.raises(IndexError):
        ops.check_device_status()
    want = torch.gather(x, 1, idx.clamp(0, 95))
    want[3, 7] = 0
    want[39, 63] = 0
    assert bits_equal(want, got)


def test_full_size_scatter_add_bit_exact_vs_aten_cpu_order(backend):
    c, op, impl, args, kwargs = _full("scatter_add_f32_4096x4096", backend)
    x, dim, idx, src = args
    got = impl(x, dim, idx, src)
    want = oracle.scatter_add(x.cpu(), 0, idx.cpu(), src.cpu())  # sequential CPU order, a second or so in C
    assert bits_equal(want, got)
    # identity rows: every destination gets exactly one contribution -> self + src, exactly
    ident = torch.arange(4096, device=DEV).unsqueeze(1).expand(4096, 4096).contiguous()
    assert bits_equal(impl(x, 0, ident, src), x + src)
    # all rows onto row 0: a 4096-term ordered sum per column
    zeros = torch.zeros(4096, 4096, dtype=torch.int64, device=DEV)
    got0 = impl(x, 0, zeros, src)
    want0 = oracle.scatter_add(x.cpu(), 0, zeros.cpu(), src.cpu())
    assert bits_equal(want0, got0)
    # dim 1 goes through the generic ordered path
    got1 = impl(x[:512], 1, idx[:512], src[:512])
    assert bits_equal(oracle.scatter_add(x[:512].cpu(), 1, idx[:512].cpu(), src[:512].cpu()), got1)
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_scatter_add_eight_column_strips_bit_exact(backend, dtype):
    """Destinations of at most 4096 rows with many columns take the eight-column strip
    kernel: ragged source-row counts, few destinations (every step collides and is ranked),
    an index narrower than self, a batch dimension, a strided source, a bad index."""
    impl = backend[torch.ops.aten.scatter_add.default]
    g = torch.Generator().manual_seed(33)

    def rn(*shape):
        return torch.randn(*shape, generator=g).to(dtype)

    def ri(high, *shape):
        return torch.randint(0, high, shape, generator=g)

    cases = [
        (rn(300, 1024), 0, ri(300, 1000, 1024), rn(1000, 1024)),
        (rn(4096, 640), 0, ri(4096, 2051, 640), rn(2051, 640)),
        (rn(7, 1184), 0, ri(7, 700, 1184), rn(700, 1184)),  # 7 destinations: ~2 rows of every 16 collide
        (rn(1, 1184), 0, ri(1, 300, 1184), rn(300, 1184)),  # one destination: a fully ordered sum
        (rn(2, 500, 768), 1, ri(500, 2, 777, 760), rn(2, 777, 768)[:, :, :760]),  # batch, narrower index, strided src
        (rn(1000, 1280), 0, ri(1000, 512, 1280), rn(600, 1288)[:512, 8:]),
    ]
    for x, dim, idx, src in cases:
        got = impl(x.to(DEV), dim, idx.to(DEV), src.to(DEV))
        assert bits_equal(oracle.scatter_add(x, dim, idx, src), got), (tuple(x.shape), dim, tuple(idx.shape))
    ops.check_device_status()
    x, idx, src = rn(300, 1024), ri(300, 1000, 1024), rn(1000, 1024)
    idx[17, 5] = 300
    idx[999, 1023] = -2
    got = impl(x.to(DEV), 0, idx.to(DEV), src.to(DEV))
    with pytest.raises(IndexError):
        ops.check_device_status()
    src[17, 5] = 0  # a skipped contribution is a contribution of nothing
    src[999, 1023] = 0
    assert bits_equal(oracle.scatter_add(x, 0, idx.clamp(0, 299), src), got)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_scatter_add_grouped_by_destination_path_bit_exact(backend, dtype):
    """Tall / narrow / ragged / strided geometries (too little column or row parallelism for
    the shared-memory kernels) are grouped by destination and replayed in source order; a
    few destinations with thousands of contributions take the cooperative replay."""
    impl = backend[torch.ops.aten.scatter_add.default]
    g = torch.Generator().manual_seed(21)

    def rn(*shape):
        return torch.randn(*shape, generator=g).to(dtype)

    def ri(high, *shape):
        return torch.randint(0, high, shape, generator=g)

    cases = [
        (rn(20000, 8), 0, ri(20000, 20000, 8), rn(20000, 8)),
        (rn(30000, 24), 0, ri(30000, 15000, 24), rn(15000, 24)),
        (rn(70000, 9), 0, ri(70000, 70000, 9), rn(70000, 9)),
        (rn(64, 16), 0, ri(3, 9000, 16), rn(9000, 16)),  # ~3000 contributions per destination
        (rn(16, 100000), 1, ri(100000, 16, 100000), rn(16, 100000)),
        (rn(4, 3000, 10), 1, ri(3000, 4, 9000, 10), rn(4, 9000, 10)),
        (rn(5000, 40), 0, ri(5000, 4000, 33), rn(6000, 48)[:, :40]),  # index narrower than self, strided src
    ]
    for x, dim, idx, src in cases:
        got = impl(x.to(DEV), dim, idx.to(DEV), src.to(DEV))
        assert bits_equal(oracle.scatter_add(x, dim, idx, src), got), (tuple(x.shape), dim, tuple(idx.shape))
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_scatter_add_with_an_empty_index_copies_self(backend, dtype):
    """No contributions at all (an index with a zero extent): the result is self, for every
    dtype and geometry, and no scratch is asked for."""
    impl = backend[torch.ops.aten.scatter_add.default]
    g = torch.Generator().manual_seed(5)
    for shape, dim, ishape in [((605, 128), 0, (0, 128)), ((184566, 16), 1, (0, 16)), ((61, 32), 0, (0, 32)), ((7, 9, 11), 1, (7, 0, 11)), ((4096, 1024), 0, (0, 1024))]:
        x = torch.randn(*shape, generator=g).to(dtype).to(DEV)
        idx = torch.zeros(ishape, dtype=torch.int64, device=DEV)
        src = torch.zeros(ishape, dtype=dtype, device=DEV)
        got = impl(x, dim, idx, src)
        assert got.data_ptr() != x.data_ptr() and bits_equal(x, got), (shape, dim, ishape)
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_scatter_add_few_long_rows_bit_exact(backend, dtype):
    """Scatter along the last dim with a handful of long rows: several warps share a row, each
    with a range of its destinations, every one reading all of the row's sources in order."""
    impl = backend[torch.ops.aten.scatter_add.default]
    g = torch.Generator().manual_seed(41)

    def rn(*shape):
        return torch.randn(*shape, generator=g).to(dtype)

    def ri(high, *shape):
        return torch.randint(0, high, shape, generator=g)

    cases = [
        (rn(34, 2051), 1, ri(2051, 17, 2051), rn(17, 2051)),
        (rn(3, 5000), 1, ri(5000, 3, 4000), rn(3, 4000)),
        (rn(1, 300), 1, ri(300, 1, 1000), rn(1, 1000)),          # ~3 contributions per destination
        (rn(5, 129), 1, ri(2, 5, 700), rn(5, 700)),              # two hot destinations: every step is ranked
        (rn(2, 3, 1000), 2, ri(1000, 2, 3, 999), rn(2, 3, 1001)[:, :, :999]),
        (rn(40, 6000), 1, ri(6000, 40, 257), rn(40, 257)),
    ]
    for x, dim, idx, src in cases:
        got = impl(x.to(DEV), dim, idx.to(DEV), src.to(DEV))
        assert bits_equal(oracle.scatter_add(x, dim, idx, src), got), (tuple(x.shape), dim, tuple(idx.shape))
    ops.check_device_status()
    x, idx, src = rn(6, 700), ri(700, 6, 900), rn(6, 900)
    idx[2, 5] = 700
    idx[5, 899] = -1
    got = impl(x.to(DEV), 1, idx.to(DEV), src.to(DEV))
    with pytest.raises(IndexError):
        ops.check_device_status()
    src[2, 5] = 0
    src[5, 899] = 0
    assert bits_equal(oracle.scatter_add(x, 1, idx.clamp(0, 699), src), got)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_many_short_rows_and_long_non_last_dims(backend, dtype):
    """Millions-of-tiny-rows geometries take the thread-per-row kernels; a long reduction over
    a non-last dim with few columns takes the transposed route / split reductions."""
    g = torch.Generator().manual_seed(31)
    x = torch.randn(6000, 17, generator=g).to(dtype)
    x[5, 3] = float("nan")
    x[7, :] = float("-inf")
    w, b = torch.randn(17, generator=g).to(dtype), torch.randn(17, generator=g).to(dtype)
    tall = torch.randn(3000, 24, generator=g).to(dtype)
    jobs = [
        ("_softmax.default", [x, -1, False]), ("_log_softmax.default", [x, -1, False]), ("sum.dim_IntList", [x[:, :7].contiguous(), [-1]]),
        ("argmax.default", [x, -1]), ("native_layer_norm.default", [x[8:], [17], w, b, 1e-5]), ("native_layer_norm.default", [x[8:, :5].contiguous(), [5], None, None, 1e-5]),
        ("_softmax.default", [tall, 0, False]), ("_log_softmax.default", [tall, 0, False]), ("sum.dim_IntList", [tall, [0]]), ("argmax.default", [tall, 0]),
        ("_softmax.default", [tall.view(3000, 4, 6), 0, False]), ("sum.dim_IntList", [torch.randn(9000, 40, generator=g).to(dtype), [0], True]),
    ]
    for op_name, args in jobs:
        got = backend[get_operator(op_name)](*_to_dev(args))
        _check(op_name, oracle.run(op_name, args, {}), got, (op_name, tuple(args[0].shape)))
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_reductions_over_rows_of_a_narrow_matrix(backend, dtype):
    """sum / argmax over dim 0 of [rows, 2 .. 32 columns] (the bias-gradient shape): the lanes of
    a warp tile rows x columns; ties go to the first row, a NaN wins, batches reduce apart."""
    g = torch.Generator().manual_seed(36)
    jobs = []
    for cols in (2, 7, 16, 17, 32):
        x = torch.randn(5003, cols, generator=g).to(dtype)
        x[100, 0] = x[4000, 0] = 50.0  # a tie: the earlier row
        x[77, cols - 1] = float("nan")
        jobs += [("sum.dim_IntList", [x[:, : cols - 1].contiguous() if cols > 2 else x[:, :1].contiguous(), [0]]), ("sum.dim_IntList", [x.nan_to_num(0.0), [0], True]),
                 ("argmax.default", [x, 0]), ("argmax.default", [x.nan_to_num(0.0), 0, True])]
    xb = torch.randn(6, 700, 12, generator=g).to(dtype)
    jobs += [("sum.dim_IntList", [xb, [1]]), ("argmax.default", [xb, 1])]
    for op_name, args in jobs:
        got = backend[get_operator(op_name)](*_to_dev(args))
        _check(op_name, oracle.run(op_name, args, {}), got, (op_name, tuple(args[0].shape)))
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_add_mul_with_a_bias_vector_or_a_value_per_row(backend, dtype):
    """x + bias[C], x * scale[R, 1], either operand first, 2-d and 3-d, row lengths on and off the
    16-byte grid, a row-pitched matrix view, alpha: bit-identical to aten on the same tensors
    (one fp32 operation and one rounding per element)."""
    g = torch.Generator(device=DEV).manual_seed(35)
    add, mul = backend[get_operator("add.Tensor")], backend[get_operator("mul.Tensor")]
    for R, C in ((1109, 8195), (300, 4096), (70000, 12), (5, 1), (1, 777)):
        x = torch.randn(R, C, generator=g, device=DEV).to(dtype)
        bias, col = torch.randn(C, generator=g, device=DEV).to(dtype), torch.randn(R, 1, generator=g, device=DEV).to(dtype)
        wide = torch.randn(R, C + 8, generator=g, device=DEV).to(dtype)[:, :C]  # rows with a pitch
        for a, b in ((x, bias), (bias, x), (x, col), (col, x), (wide, bias), (wide, col), (col, bias), (x, wide)):
            assert bits_equal(torch.add(a, b), add(a, b)), (R, C, a.shape, b.shape)
            assert bits_equal(torch.mul(a, b), mul(a, b)), (R, C, a.shape, b.shape)
        assert bits_equal(torch.add(x, bias, alpha=0.5), add(x, bias, alpha=0.5))
    x3 = torch.randn(7, 33, 256, generator=g, device=DEV).to(dtype)
    b3 = torch.randn(256, generator=g, device=DEV).to(dtype)
    assert bits_equal(torch.add(x3, b3), add(x3, b3)) and bits_equal(torch.mul(b3, x3), mul(b3, x3))
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_short_rows_every_length_staged_and_direct(backend, dtype):
    """Thread-per-row kernels over row lengths on both sides of each register-slot count (8,
    16, 24, 32), with strides that are and are not multiples of 8 bytes (direct / staged
    through shared memory), a last CTA holding 3 rows, and a base pointer off the 16-byte grid."""
    g = torch.Generator().manual_seed(33)
    jobs = []
    for cols in (1, 3, 5, 8, 9, 10, 15, 16, 17, 21, 24, 25, 30, 31, 32):
        x = torch.randn(4099 + 1, cols, generator=g).to(dtype)
        x[9, cols // 2] = float("nan")
        x[11, :] = float("-inf")
        w, b = torch.randn(cols, generator=g).to(dtype), torch.randn(cols, generator=g).to(dtype)
        xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
        for lo, hi in ((1, 4100), (0, 4099)):  # a view keeps its offset on the device: base off / on the 16-byte grid
            v, vd = x[lo:hi], xd[lo:hi]
            jobs += [("_softmax.default", [v, -1, False], [vd, -1, False]), ("_log_softmax.default", [v, -1, False], [vd, -1, False]), ("sum.dim_IntList", [v, [-1]], [vd, [-1]]),
                     ("argmax.default", [v, -1], [vd, -1]), ("native_layer_norm.default", [v[12:], [cols], w, b, 1e-5], [vd[12:], [cols], wd, bd, 1e-5])]
        if dtype != torch.float32:
            jobs.append(("_softmax.default", [x[:4099], -1, True], [xd[:4099], -1, True]))  # half_to_float: fp32 output
    for op_name, args, dev_args in jobs:
        got = backend[get_operator(op_name)](*dev_args)
        _check(op_name, oracle.run(op_name, args, {}), got, (op_name, tuple(args[0].shape), args[0].storage_offset()))
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_long_and_misaligned_rows_take_the_vector_streaming_softmax(backend, dtype):
    """Rows too long for a CTA's registers (a vocabulary of 50257 or 131072 entries) and long
    rows that start off the 16-byte grid: two passes of 16-byte accesses over the aligned
    span around each row. Special rows: a NaN, all -inf, one +inf, -inf everywhere but one."""
    g = torch.Generator().manual_seed(34)
    for rows, cols in ((9, 1025), (7, 4099), (6, 33000), (5, 50257), (5, 131072), (6, 70001)):
        x = (torch.randn(rows + 1, cols, generator=g) * 3).to(dtype)
        x[1, cols // 3] = float("nan")
        x[2, :] = float("-inf")
        x[3, cols - 1] = float("inf")
        x[4, :] = float("-inf")
        x[4, 0] = 1.5
        xd = x.to(DEV)
        for lo in (0, 1):  # with odd `cols`, the view from row 1 starts off the 16-byte grid
            v, vd = x[lo:lo + rows], xd[lo:lo + rows]
            for op_name in ("_softmax.default", "_log_softmax.default"):
                got = backend[get_operator(op_name)](vd, -1, False)
                _check(op_name, oracle.run(op_name, [v, -1, False], {}), got, (op_name, rows, cols, lo))
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_ragged_mid_size_rows_one_warp_each(backend, dtype):
    """Rows of 33 ... 1024 elements off the 16-byte grid (odd lengths, or an odd base offset)
    take the warp-per-row kernels; a row with NaN and an all -inf row behave as in aten."""
    g = torch.Generator().manual_seed(32)
    jobs = []
    for cols in (33, 67, 100, 257, 513, 1000):
        x = torch.randn(300, cols, generator=g).to(dtype)
        x[5, 3] = float("nan")
        x[7, :] = float("-inf")
        w, b = torch.randn(cols, generator=g).to(dtype), torch.randn(cols, generator=g).to(dtype)
        jobs += [("_softmax.default", [x, -1, False]), ("_log_softmax.default", [x, -1, False]), ("native_layer_norm.default", [x[8:], [cols], w, b, 1e-5]),
                 ("native_layer_norm.default", [x[8:], [cols], None, None, 1e-5])]
    for op_name, args in jobs:
        got = backend[get_operator(op_name)](*_to_dev(args))
        _check(op_name, oracle.run(op_name, args, {}), got, (op_name, tuple(args[0].shape)))
    ops.check_device_status()


def test_full_size_argmax_bit_exact(backend):
    c, op, impl, args, kwargs = _full("argmax_f32_8192x32000", backend)
    got = impl(*args, **kwargs)
    assert got.dtype == torch.int64 and bits_equal(op(*args, **kwargs), got)
    x = args[0]
    assert bits_equal(x.gather(1, got.unsqueeze(1)).squeeze(1), x.max(-1).values)  # the value there is the row maximum
    x2 = x[:64].clone()
    x2[:, 1000] = float("nan")
    x2[:, 2000] = float("nan")
    assert bool((impl(x2, -1) == 1000).all())  # NaN counts as the maximum, the first one wins
    x3 = x[:64].clone()
    x3[:, 777] = 100.0
    x3[:, 31999] = 100.0
    assert bool((impl(x3, -1) == 777).all())  # ties -> first index
    assert int(impl(x)) == int(op(x))  # flattened (split across CTAs, finished from scratch memory)


def _gemm_rows_fp64(a, b, rows):
    return a[rows].double().cpu() @ b.double().cpu()


def test_full_size_mm_addmm_bmm(backend):
    c, op, impl, args, kwargs = _full("mm_bf16_8192x4096x11008", backend)
    a, b = args
    got, ref = impl(a, b), op(a, b)
    assert compare(ref, got, 1e-2, 1e-2)[0]
    rows = torch.tensor([0, 1, 127, 128, 4095, 8191], device=DEV)
    exact = _gemm_rows_fp64(a, b, rows)
    assert compare(exact.to(torch.bfloat16), got[rows].cpu(), 4e-3, 1e-2)[0]  # |C| ~ 1/64: bf16 rounding + fp32 accumulation
    # linearity in the first operand, scaling by a power of two is exact
    assert bits_equal(impl(a * 2, b), got * 2)
    c, op, impl, args, kwargs = _full("addmm_bf16_8192x4096x11008", backend)
    bias, a, b = args
    g2, r2 = impl(bias, a, b), op(bias, a, b)
    assert compare(r2, g2, 1e-2, 1e-2)[0]
    assert compare((exact + bias.double().cpu()).to(torch.bfloat16), g2[rows].cpu(), 2e-2, 1e-2)[0]
    c, op, impl, args, kwargs = _full("bmm_bf16_32x2048x128x2048", backend)
    g3, r3 = impl(*args), op(*args)
    assert compare(r3, g3, 1e-2, 1e-2)[0]
    e3 = (args[0][5].double() @ args[1][5].double()).to(torch.bfloat16)
    assert compare(e3, g3[5], 1e-2, 1e-2)[0]


def test_index_out_of_range_is_reported_not_faulted(backend):
    """A bad index never touches memory out of bounds: the row is zero-filled, a status bit
    is set, and the next status check raises IndexError; the context stays usable."""
    table = torch.randn(16, 8, device=DEV)
    idx = torch.tensor([1, 99, 3, -1], device=DEV)
    out = backend[torch.ops.aten.embedding.default](table, idx)
    with pytest.raises(IndexError):
        ops.check_device_status()
    assert bits_equal(out[0], table[1]) and bits_equal(out[2], table[3]) and float(out[1].abs().sum()) == 0.0 and float(out[3].abs().sum()) == 0.0
    ops.check_device_status()  # cleared; and the device still works:
    assert bits_equal(backend[torch.ops.aten.relu.default](table), torch.relu(table))


def test_unsupported_requests_fail_loudly(backend):
    with pytest.raises(NotImplementedError):
        backend[torch.ops.aten.relu.default](torch.arange(4, device=DEV))  # integer relu: not implemented, no fallback
    with pytest.raises(NotImplementedError):
        backend[torch.ops.aten.mm.default](torch.randn(4, 4, device=DEV, dtype=torch.float64), torch.randn(4, 4, device=DEV, dtype=torch.float64))
    with pytest.raises(RuntimeError):
        backend[torch.ops.aten.mm.default](torch.randn(4, 5, device=DEV), torch.randn(4, 5, device=DEV))


def test_strip_gather_on_a_second_device_in_one_process(backend):
    """The strip kernel asks for 128 KB of dynamic shared memory, an opt-in that belongs to
    the device: the same process must be able to run it on cuda:0 and then on cuda:1."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    gather = backend[torch.ops.aten.gather.default]
    for dev in ("cuda:0", "cuda:1"):
        with torch.cuda.device(dev):
            g = torch.Generator(device=dev).manual_seed(5)
            src = torch.randn(2048, 2048, device=dev, generator=g)
            idx = torch.randint(0, 2048, (2048, 2048), device=dev, generator=g)
            got = gather(src, 0, idx)
            assert bits_equal(got, torch.gather(src, 0, idx)), dev
            ops.check_device_status(torch.device(dev))
