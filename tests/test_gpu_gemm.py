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
def test_mm_all_layouts(dtype, a_t, b_t):
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
def test_addmm_epilogue_variants(dtype):
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
def test_bmm_batches_and_strided_views(dtype):
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
