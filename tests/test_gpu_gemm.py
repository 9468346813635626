"""mm / addmm / bmm on the tcgen05 tensor-core path: every operand layout the kernel takes
without copying (A row- or column-major, B as [K,N] or as a transposed [N,K] view), ragged
tile edges, batches, the fused bias / alpha / beta epilogue -- against an fp64 product of the
same bf16 / f16 inputs. The device status word must stay clean (no bounded wait gave up)."""

import pytest
import torch

from backendbench_b200 import _abi, ops
from backendbench_b200.eval import compare

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(params=[1, 0], ids=["small-path-on", "small-path-off"])
def small_path(request):
    """Small 16-bit products normally take the mma.sync kernel; with the path switched off the
    same shapes exercise the tcgen05 / CUDA-core kernels (ragged tiles, every layout)."""
    prev = _abi.lib().b200_gemm_small_path(request.param)
    try:
        yield request.param
    finally:
        _abi.lib().b200_gemm_small_path(prev)


def _uses_tc(a, b, batch, M, N, K, sa, sb):
    return bool(_abi.lib().b200_gemm_uses_tensor_cores(batch, M, N, K, sa[0], sa[1], sa[2], sb[0], sb[1], sb[2], _abi.BF16 if a.dtype == torch.bfloat16 else _abi.F16, a.data_ptr(), b.data_ptr(), a.data_ptr()))


def _rand(shape, dtype, g, std):
    return (torch.randn(shape, generator=g, device=DEV) * std).to(dtype)


def _check(got, exact, dtype):
    # fp32 accumulation + one rounding to a 16-bit type: relative 2^-8 (bf16) / 2^-11 (f16) of the value, plus accumulation noise
    ok, ea, er = compare(exact.to(dtype), got, 2e-2 if dtype == torch.bfloat16 else 4e-3, 1e-2)
    assert ok, (ea, er)


SHAPES = [(128, 256, 64), (128, 256, 256), (256, 512, 128), (130, 264, 72), (33, 48, 64), (1, 256, 512), (257, 8, 4096), (512, 1000, 136), (384, 768, 2048)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_mm_all_layouts(dtype, a_t, b_t, small_path):
    g = torch.Generator(device=DEV).manual_seed(5)
    for M, N, K in SHAPES:
        Mp, Kp, Np = (M + 7) // 8 * 8, (K + 7) // 8 * 8, (N + 7) // 8 * 8
        a = _rand((Kp, Mp), dtype, g, K**-0.5).t()[:M, :K] if a_t else _rand((Mp, Kp), dtype, g, K**-0.5)[:M, :K]
        b = _rand((Np, Kp), dtype, g, 1.0).t()[:K, :N] if b_t else _rand((Kp, Np), dtype, g, 1.0)[:K, :N]
        assert _uses_tc(a, b, 1, M, N, K, (0, a.stride(0), a.stride(1)), (0, b.stride(0), b.stride(1))), (M, N, K, a.stride(), b.stride())
        got = ops.mm_default(a, b)
        ops.check_device_status()
        assert got.shape == (M, N) and got.dtype == dtype and got.is_contiguous()
        _check(got, a.double() @ b.double(), dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_addmm_epilogue_variants(dtype, small_path):
    g = torch.Generator(device=DEV).manual_seed(6)
    M, N, K = 300, 520, 192
    a, b = _rand((M, K), dtype, g, K**-0.5), _rand((K, N), dtype, g, 1.0)
    exact = a.double() @ b.double()
    for bias_shape in [(N,), (M, N), (1, N), (M, 1), ()]:
        bias = _rand(bias_shape, dtype, g, 1.0)
        _check(ops.addmm_default(bias, a, b), exact + bias.double(), dtype)
        _check(ops.addmm_default(bias, a, b, beta=0.5, alpha=2), 2 * exact + 0.5 * bias.double(), dtype)
    nan_bias = torch.full((N,), float("nan"), dtype=dtype, device=DEV)
    _check(ops.addmm_default(nan_bias, a, b, beta=0), exact, dtype)  # beta = 0 ignores the bias
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_bmm_batches_and_strided_views(dtype, small_path):
    g = torch.Generator(device=DEV).manual_seed(7)
    for B, M, K, N in [(3, 128, 64, 256), (5, 200, 72, 136), (32, 256, 128, 320), (2, 64, 1024, 64)]:
        a, b = _rand((B, M, K), dtype, g, K**-0.5), _rand((B, K, N), dtype, g, 1.0)
        _check(ops.bmm_default(a, b), a.double() @ b.double(), dtype)
        bt = _rand((B, N, K), dtype, g, 1.0).transpose(1, 2)  # K-major B, as attention scores use it
        _check(ops.bmm_default(a, bt), a.double() @ bt.double(), dtype)
        at = _rand((B, K, M), dtype, g, K**-0.5).transpose(1, 2)
        _check(ops.bmm_default(at, b), at.double() @ b.double(), dtype)
    ops.check_device_status()


def test_layouts_the_tensor_core_path_declines_still_work():
    """K stride off the 16-byte grid, fp32 operands, unaligned bases: the CUDA-core kernel."""
    g = torch.Generator(device=DEV).manual_seed(8)
    a, b = _rand((64, 100), torch.bfloat16, g, 0.1), _rand((100, 50), torch.bfloat16, g, 1.0)
    assert not _uses_tc(a, b, 1, 64, 50, 100, (0, 100, 1), (0, 50, 1))
    _check(ops.mm_default(a, b), a.double() @ b.double(), torch.bfloat16)
    a32, b32 = torch.randn(96, 200, device=DEV, generator=g), torch.randn(200, 72, device=DEV, generator=g)
    ok, ea, er = compare((a32.double() @ b32.double()).float(), ops.mm_default(a32, b32), 1e-4, 1e-4)
    assert ok, (ea, er)
    av = _rand((65, 129), torch.float16, g, 0.1)[1:, 1:]  # base pointer 2 bytes off alignment
    bv = _rand((128, 64), torch.float16, g, 1.0)
    _check(ops.mm_default(av, bv), av.double() @ bv.double(), torch.float16)
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_large_misaligned_operands_are_repitched_onto_tensor_cores(dtype):
    """Row pitches / bases off the 16-byte grid (K = 2049, N = 127, sliced views): large
    products get their operands re-pitched by the library's copy kernel and still match."""
    g = torch.Generator(device=DEV).manual_seed(9)
    a, b = _rand((1024, 2049), dtype, g, 2049**-0.5), _rand((2049, 127), dtype, g, 1.0)
    _check(ops.mm_default(a, b), a.double() @ b.double(), dtype)
    at = _rand((2049, 1030), dtype, g, 2049**-0.5).t()[1:, :]  # M-major A with an odd base offset
    _check(ops.mm_default(at, b), at.double() @ b.double(), dtype)
    bias = _rand((127,), dtype, g, 1.0)
    _check(ops.addmm_default(bias, a, b, beta=2, alpha=0.5), 0.5 * (a.double() @ b.double()) + 2 * bias.double(), dtype)
    x, y = _rand((4, 300, 1001), dtype, g, 1001**-0.5), _rand((4, 260, 1001), dtype, g, 1.0).transpose(1, 2)  # K-major B, K = 1001
    _check(ops.bmm_default(x, y), x.double() @ y.double(), dtype)
    ops.check_device_status()


def _check32(got, a, b, extra=None, alpha=1.0, beta=1.0):
    """fp32 result against the fp64 product. The tensor core truncates each of its K/16
    additions into the accumulator (half a unit in the last place of the running sum on
    average, always toward zero), so the allowed error is K/16 such units of a running sum
    as large as the result or four standard deviations of it."""
    K = a.shape[-1]
    exact = alpha * (a.double() @ b.double())
    spread = abs(alpha) * ((a.double() ** 2) @ (b.double() ** 2)).sqrt()
    if extra is not None:
        exact = exact + beta * extra.double()
    err = (got.double() - exact).abs()
    bound = 2.0**-24 * (K / 16 + 4) * (exact.abs() + 4 * spread) + 1e-30
    assert got.dtype == torch.float32 and bool((err <= bound).all()), float((err / bound).max())


@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_large_fp32_products_take_split_bf16_planes_on_tensor_cores(a_t, b_t):
    """fp32 mm / addmm / bmm above the size threshold: operands split into three bf16 planes,
    six plane products accumulated in fp32 by the tcgen05 kernel. Every operand layout, ragged
    M / N / K (K padded to 64 inside the planes), bias with alpha / beta, batches."""
    g = torch.Generator(device=DEV).manual_seed(12)
    for M, N, K in [(512, 512, 512), (446, 2048, 1024), (130, 1000, 1111), (1000, 36, 4099), (33, 8192, 300)]:
        assert M * N * K >= ops.F32_SPLIT_MIN_MACS
        a = torch.randn((K, M) if a_t else (M, K), generator=g, device=DEV)
        b = torch.randn((N, K) if b_t else (K, N), generator=g, device=DEV)
        a = a.t() if a_t else a
        b = b.t() if b_t else b
        _check32(ops.mm_default(a, b), a, b)
        bias = torch.randn(N, generator=g, device=DEV)
        _check32(ops.addmm_default(bias, a, b, beta=0.5, alpha=-1.5), a, b, bias.expand(M, N), -1.5, 0.5)
    B, M, N, K = 4, 200, 264, 640
    a = torch.randn((B, K, M) if a_t else (B, M, K), generator=g, device=DEV)
    b = torch.randn((B, N, K) if b_t else (B, K, N), generator=g, device=DEV)
    a = a.transpose(1, 2) if a_t else a
    b = b.transpose(1, 2) if b_t else b
    _check32(ops.bmm_default(a, b), a, b)
    ops.check_device_status()


def test_split_fp32_product_keeps_special_values_and_wide_ranges():
    g = torch.Generator(device=DEV).manual_seed(13)
    a = torch.randn(512, 512, generator=g, device=DEV) * torch.logspace(-20, 20, 512, device=DEV)  # columns spanning 40 decades
    b = torch.randn(512, 512, generator=g, device=DEV) * torch.logspace(20, -20, 512, device=DEV).unsqueeze(1)
    _check32(ops.mm_default(a, b), a, b)
    a = torch.randn(512, 512, generator=g, device=DEV)
    b = torch.randn(512, 512, generator=g, device=DEV)
    a[3, 7] = float("inf")
    a[5, 9] = float("nan")
    a[8, 1] = 3.4e38  # rounds to infinity as bf16: must stay finite
    b[1] *= 1e-3      # ... and its products stay below the fp32 maximum
    got, want = ops.mm_default(a, b), a @ b
    assert bool(torch.isnan(got[5]).all()) and bool(torch.isinf(got[3]).all()) and bool((got[3] == want[3]).all())
    assert bool(torch.isfinite(got[8]).all()) and bool(((got[8] - want[8]).abs() <= 1e-5 * want[8].abs()).all())
    b[:, 11] = float("-inf")  # a whole output column: -inf * a, NaN where a is 0 or NaN
    a[40, :] = 0.0
    got, want = ops.mm_default(a, b), a @ b
    assert bool((torch.isnan(got[:, 11]) == torch.isnan(want[:, 11])).all()) and bool((got[:, 11][~torch.isnan(want[:, 11])] == want[:, 11][~torch.isnan(want[:, 11])]).all())
    rest = [i for i in range(512) if i not in (3, 5, 8)]
    cols = [j for j in range(512) if j != 11]
    _check32(got[rest][:, cols], a[rest], b[:, cols])
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_odd_output_widths_on_the_tensor_core_path(dtype):
    """N off the 8-element grid: B is re-pitched, C rows start at odd addresses, and the
    epilogue writes them row by row from its staging buffer (every column tail length, a
    ragged last row block, batches, bias and scaling)."""
    g = torch.Generator(device=DEV).manual_seed(15)
    for M, N, K in [(300, 513, 192), (1000, 127, 1024), (129, 65, 2048), (4100, 255, 64), (257, 1, 4096), (640, 71, 512)]:
        a, b = _rand((M, K), dtype, g, K**-0.5), _rand((K, N), dtype, g, 1.0)
        exact = a.double() @ b.double()
        _check(ops.mm_default(a, b), exact, dtype)
        bias = _rand((N,), dtype, g, 1.0)
        _check(ops.addmm_default(bias, a, b, beta=0.5, alpha=2), 2 * exact + 0.5 * bias.double(), dtype)
    a3, b3 = _rand((5, 700, 256), dtype, g, 1 / 16), _rand((5, 256, 127), dtype, g, 1.0)
    _check(ops.bmm_default(a3, b3), a3.double() @ b3.double(), dtype)
    ops.check_device_status()


def test_many_rows_few_columns_take_the_row_per_thread_kernel():
    """fp32 (and 16-bit below the re-pitch threshold) products with at most 16 output columns
    and some hundred thousand rows: both accumulator counts (8, 16), K tails that are not whole
    16-byte vectors, K longer than one chunk of B, batches, bias and scaling, specials; and
    the same shapes just outside the kernel's range (19 and 32 columns, few rows)."""
    g = torch.Generator(device=DEV).manual_seed(16)
    for M, K, N in [(80000, 256, 8), (76000, 300, 13), (100000, 64, 1), (16384, 1024, 19), (9473, 2060, 32), (12000, 600, 13)]:
        a32, b32, bias = torch.randn(M, K, generator=g, device=DEV), torch.randn(K, N, generator=g, device=DEV), torch.randn(1, N, generator=g, device=DEV)
        _check32(ops.mm_default(a32, b32), a32, b32)
        _check32(ops.addmm_default(bias, a32, b32, beta=2, alpha=0.5), a32, b32, extra=bias.expand(M, N), alpha=0.5, beta=2.0)
    wide = torch.randn(90000, 132, generator=g, device=DEV)
    a32, b32 = wide[:, :130], torch.randn(130, 5, generator=g, device=DEV)  # rows 16-byte aligned, K = 130 leaves a tail of 2
    _check32(ops.mm_default(a32, b32), a32, b32)
    a3, b3 = torch.randn(16, 8192, 96, generator=g, device=DEV), torch.randn(16, 96, 5, generator=g, device=DEV)
    a3[3, 100, 7] = float("inf")
    b3[9, 50, 2] = float("nan")
    got, ref = ops.bmm_default(a3, b3), torch.bmm(a3, b3)
    assert torch.equal(torch.isnan(got), torch.isnan(ref)) and torch.equal(torch.isinf(got), torch.isinf(ref))
    fin = torch.isfinite(ref)
    assert torch.allclose(got[fin], ref[fin], atol=1e-4, rtol=1e-4)
    for dt in (torch.bfloat16, torch.float16):
        h, w = _rand((90000, 64), dt, g, 1 / 8), _rand((64, 6), dt, g, 1.0)
        _check(ops.mm_default(h, w), h.double() @ w.double(), dt)
    ops.check_device_status()


def test_long_contractions_with_small_outputs_leave_the_single_cta_path():
    """K in the thousands with a handful of outputs: 16-bit operands are re-pitched onto the
    tensor cores whatever their alignment, fp32 operands share K among the CTAs of a cluster
    (every cluster size from 2 to 8, a K that leaves the last CTAs of the cluster empty)."""
    g = torch.Generator(device=DEV).manual_seed(14)
    a, b, bias = _rand((32, 4096), torch.bfloat16, g, 4096**-0.5), _rand((4096, 31), torch.bfloat16, g, 1.0), _rand((32, 1), torch.bfloat16, g, 1.0)
    _check(ops.addmm_default(bias, a, b), a.double() @ b.double() + bias.double(), torch.bfloat16)
    a32, b32 = torch.randn(16, 8192, generator=g, device=DEV), torch.randn(8192, 40, generator=g, device=DEV)
    _check32(ops.mm_default(a32, b32), a32, b32)
    a32, b32 = torch.randn(1, 4096, generator=g, device=DEV), torch.randn(4096, 1024, generator=g, device=DEV)
    _check32(ops.mm_default(a32, b32), a32, b32)
    for M, K, N in [(2, 130, 256), (55, 200, 70), (100, 257, 33), (33, 330, 130), (7, 400, 9), (140, 450, 20), (64, 513, 64), (3, 2048, 17), (165, 4096, 32), (44, 2072, 1024)]:
        a32, b32, bias = torch.randn(M, K, generator=g, device=DEV), torch.randn(K, N, generator=g, device=DEV), torch.randn(M, 1, generator=g, device=DEV)
        _check32(ops.mm_default(a32, b32), a32, b32)
        _check32(ops.mm_default(a32.t().contiguous().t(), b32.t().contiguous().t()), a32, b32)  # both operands in the other memory order
        _check32(ops.addmm_default(bias, a32, b32, beta=2, alpha=0.5), a32, b32, extra=bias.expand(M, N), alpha=0.5, beta=2.0)
    a3, b3 = torch.randn(5, 21, 1024, generator=g, device=DEV), torch.randn(5, 1024, 40, generator=g, device=DEV)
    a3[2, 3, 100] = float("inf")
    b3[4, 7, 5] = float("nan")
    got, ref = ops.bmm_default(a3, b3), torch.bmm(a3, b3)
    assert torch.equal(torch.isnan(got), torch.isnan(ref)) and torch.equal(torch.isinf(got), torch.isinf(ref))
    fin = torch.isfinite(ref)
    assert torch.allclose(got[fin], ref[fin], atol=1e-3, rtol=1e-4)
    for dt in (torch.float16, torch.bfloat16):  # 16-bit operands off the 16-byte grid, K below the re-pitch threshold
        h, w = _rand((9, 1000), dt, g, 1000**-0.5), _rand((1000, 7), dt, g, 1.0)
        _check(ops.mm_default(h, w), h.double() @ w.double(), dt)
    ops.check_device_status()


def test_a_wait_that_cannot_complete_ends_in_a_status_not_a_hang():
    """The failure-detection form this kernel has: every mbarrier wait carries a time limit.
    The probe entry withholds one K slab (so the MMA warp's wait for it can never complete)
    with a 1 ms limit; the kernel must come back by itself, report B200_DEV_WAIT_TIMEOUT in
    the status word, and leave the context and the tensor memory usable for the next product."""
    import time

    g = torch.Generator(device=DEV).manual_seed(9)
    a = _rand((512, 1024), torch.bfloat16, g, 1024**-0.5)
    b = _rand((1024, 768), torch.bfloat16, g, 1.0)
    c = torch.empty(512, 768, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = _abi.lib().b200_gemm_wait_probe(a.data_ptr(), b.data_ptr(), c.data_ptr(), 512, 768, 1024, _abi.BF16, 1000, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert int(status.item()) & _abi.DEV_WAIT_TIMEOUT
    assert took < 1.0, took  # a handful of 1 ms limits, not the 2 s of an ordinary call
    # limits outside 50 us .. 0.1 s are refused, as are operands that would not reach the kernel
    assert _abi.lib().b200_gemm_wait_probe(a.data_ptr(), b.data_ptr(), c.data_ptr(), 512, 768, 1024, _abi.BF16, 5_000_000, status.data_ptr(), 0) < 0
    assert _abi.lib().b200_gemm_wait_probe(a.data_ptr(), b.data_ptr(), c.data_ptr(), 512, 768, 1024, _abi.F32, 1000, status.data_ptr(), 0) < 0
    # the same context, the same tensor memory: an ordinary product right behind it is correct
    got = ops.mm_default(a, b)
    ops.check_device_status()
    _check(got, a.double() @ b.double(), torch.bfloat16)


PAIR_SHAPES = [(256, 256, 320), (300, 520, 640), (1000, 1000, 1000), (129, 130, 4096), (2048, 384, 512), (513, 257, 328)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
def test_cta_pair_tiles_every_layout_and_ragged_edge(dtype, a_t, b_t):
    """Products of more than 128 rows and columns with more than four K slabs run on CTA pairs
    (256 x 256 tiles, tcgen05 cta_group::2): rows that end in the first or in the second CTA of
    the last pair, columns that end in either half of B, K off the 64 grid, all four operand
    layouts -- against the fp64 product, and bit for bit against the single-CTA kernel's rule
    (fp32 accumulation, one rounding) through the tolerance of `_check`."""
    g = torch.Generator(device=DEV).manual_seed(21)
    for M, N, K in PAIR_SHAPES:
        Mp, Kp, Np = (M + 7) // 8 * 8, (K + 7) // 8 * 8, (N + 7) // 8 * 8
        a = _rand((Kp, Mp), dtype, g, K**-0.5).t()[:M, :K] if a_t else _rand((Mp, Kp), dtype, g, K**-0.5)[:M, :K]
        b = _rand((Np, Kp), dtype, g, 1.0).t()[:K, :N] if b_t else _rand((Kp, Np), dtype, g, 1.0)[:K, :N]
        got = ops.mm_default(a, b)
        ops.check_device_status()
        assert got.shape == (M, N) and got.dtype == dtype
        _check(got, a.double() @ b.double(), dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_cta_pair_epilogue_and_batches(dtype):
    g = torch.Generator(device=DEV).manual_seed(22)
    M, N, K = 300, 520, 704
    a, b = _rand((M, K), dtype, g, K**-0.5), _rand((K, N), dtype, g, 1.0)
    exact = a.double() @ b.double()
    for bias_shape in [(N,), (M, N), (1, N), (M, 1), ()]:
        bias = _rand(bias_shape, dtype, g, 1.0)
        _check(ops.addmm_default(bias, a, b), exact + bias.double(), dtype)  # alpha = beta = 1: the single-add epilogue
        _check(ops.addmm_default(bias, a, b, beta=0.5, alpha=2), 2 * exact + 0.5 * bias.double(), dtype)
    for B, M, K, N in [(3, 256, 384, 256), (5, 200, 520, 136), (2, 640, 1024, 300)]:
        x, y = _rand((B, M, K), dtype, g, K**-0.5), _rand((B, K, N), dtype, g, 1.0)
        _check(ops.bmm_default(x, y), x.double() @ y.double(), dtype)
        yt = _rand((B, N, K), dtype, g, 1.0).transpose(1, 2)
        _check(ops.bmm_default(x, yt), x.double() @ yt.double(), dtype)
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_long_contraction_with_few_tiles_is_split_along_k(dtype):
    """A handful of output tiles and K >= 1024: the contraction runs as up to 32 ranges side by
    side and the fp32 partial products are added in a fixed order. Same answer as the unsplit
    product to rounding, bit-identical from run to run, every operand layout, bias and scales
    applied once, and shapes the split declines (K not divisible) fall through."""
    g = torch.Generator(device=DEV).manual_seed(15)
    dt = _abi.BF16 if dtype == torch.bfloat16 else _abi.F16
    for M, N, K, split in [(5, 512, 4096, True), (45, 2048, 4096, True), (12, 512, 2048, True), (44, 32, 4096, True), (130, 264, 1096, False), (1, 7, 4104, True), (300, 200, 8200, True)]:
        a, b = _rand((M, K), dtype, g, K**-0.5), _rand((K, N), dtype, g, 1.0)
        c = torch.empty(M, N, dtype=dtype, device=DEV)
        need = _abi.lib().b200_gemm_splitk_scratch_bytes(a.data_ptr(), b.data_ptr(), c.data_ptr(), 1, M, N, K, 0, K, 1, 0, N, 1, dt)
        if N % 8 == 0:  # B [K, N] with rows off the 16-byte grid never reaches the tensor cores
            assert (need > 0) == split, (M, N, K, need)
        exact = a.double() @ b.double()
        got = ops.mm_default(a, b)
        _check(got, exact, dtype)
        assert torch.equal(got, ops.mm_default(a, b))
        bias = _rand((N,), dtype, g, 1.0)
        _check(ops.addmm_default(bias, a, b, beta=0.5, alpha=2), 2 * exact + 0.5 * bias.double(), dtype)
        at = _rand((K, (M + 7) // 8 * 8), dtype, g, K**-0.5).t()[:M]  # M-major A
        bt = _rand(((N + 7) // 8 * 8, K), dtype, g, 1.0).t()[:, :N]   # K-major B
        _check(ops.mm_default(at, bt), at.double() @ bt.double(), dtype)
    ops.check_device_status()


def test_fp32_products_with_a_narrow_result():
    """C of at most 16 columns under a long row-major fp32 A: a warp per row of A (16-byte
    pieces of the row per lane, B in shared memory, the lanes' partial sums folded by a halving
    exchange). Ragged K, every N up to 16, batches, bias and scales, rows that do not fill the
    last CTA; against an fp64 product."""
    g = torch.Generator(device=DEV).manual_seed(23)
    for B, M, K, N in [(1, 2000, 280, 8), (1, 1500, 128, 16), (1, 5001, 1000, 3), (3, 700, 260, 9), (1, 16384, 256, 8), (2, 1999, 2052, 16), (1, 1300, 132, 1)]:
        a = torch.randn(B, M, K, generator=g, device=DEV) * K**-0.5
        b = torch.randn(B, K, N, generator=g, device=DEV)
        exact = a.double() @ b.double()
        got = ops.bmm_default(a, b)
        assert got.shape == (B, M, N) and got.dtype == torch.float32
        ok, ea, er = compare(exact.float(), got, 1e-4, 1e-4)
        assert ok, (B, M, K, N, ea, er)
        assert torch.equal(got, ops.bmm_default(a, b))  # fixed order of additions
        bias = torch.randn(M, N, generator=g, device=DEV)
        got = ops.addmm_default(bias, a[0], b[0], beta=0.5, alpha=2)
        ok, ea, er = compare((2 * exact[0] + 0.5 * bias.double()).float(), got, 1e-4, 1e-4)
        assert ok, (M, K, N, ea, er)
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_small_products_on_the_mma_kernel(dtype):
    """Few 64 x 64 tiles and a short contraction: the four-warp mma.sync kernel when both
    operands are on the 16-byte grid (all four layout pairs, ragged M / N / K, batches, bias and
    scales); offset bases, odd pitches and operands with no unit stride go to the other kernels."""
    g = torch.Generator(device=DEV).manual_seed(29)
    dt = _abi.BF16 if dtype == torch.bfloat16 else _abi.F16

    def prefers(a, b, B, M, N, K):
        sa = (a.stride(0) if B > 1 else 0, a.stride(-2), a.stride(-1))
        sb = (b.stride(0) if B > 1 else 0, b.stride(-2), b.stride(-1))
        return _abi.lib().b200_gemm_prefers_small(a.data_ptr(), b.data_ptr(), B, M, N, K, sa[0], sa[1], sa[2], sb[0], sb[1], sb[2], dt)

    for B, M, N, K in [(1, 41, 64, 256), (64, 2, 64, 64), (1, 367, 264, 40), (1, 227, 72, 256), (1, 36, 24, 32), (32, 15, 8, 256), (2, 4, 72, 64), (1, 1, 8, 200), (3, 136, 72, 104), (1, 64, 64, 8),
                       (1, 5, 8, 248), (8, 6, 16, 40), (1, 17, 9 * 8, 136), (2, 49, 40, 72)]:
        for a_t in (False, True):
            for b_t in (False, True):
                Mp = (M + 7) // 8 * 8
                a = _rand((B, K, Mp), dtype, g, K**-0.5).transpose(1, 2)[:, :M] if a_t else _rand((B, M, K), dtype, g, K**-0.5)
                b = _rand((B, N, K), dtype, g, 1.0).transpose(1, 2) if b_t else _rand((B, K, N), dtype, g, 1.0)
                assert prefers(a, b, B, M, N, K) == 1, (B, M, N, K, a.stride(), b.stride())
                got = ops.bmm_default(a, b)
                assert got.shape == (B, M, N) and got.dtype == dtype and got.is_contiguous()
                _check(got, a.double() @ b.double(), dtype)
        a2, b2 = _rand((M, K), dtype, g, K**-0.5), _rand((K, N), dtype, g, 1.0)
        for bias_shape in [(N,), (M, N), (M, 1), ()]:
            bias = _rand(bias_shape, dtype, g, 1.0)
            _check(ops.addmm_default(bias, a2, b2, beta=0.5, alpha=2), 2 * (a2.double() @ b2.double()) + 0.5 * bias.double(), dtype)
        nan_bias = torch.full((N,), float("nan"), dtype=dtype, device=DEV)
        _check(ops.addmm_default(nan_bias, a2, b2, beta=0), a2.double() @ b2.double(), dtype)
        # off the grid: an offset base, an odd pitch, no unit stride -- other kernels, same answer
        shifted = _rand((M, K + 8), dtype, g, K**-0.5)[:, 3 : K + 3]
        every_other = _rand((M, 2 * K), dtype, g, K**-0.5)[:, ::2]
        for a3 in (shifted, every_other):
            assert prefers(a3, b2, 1, M, N, K) == 0
            _check(ops.mm_default(a3, b2), a3.double() @ b2.double(), dtype)
    ops.check_device_status()
