"""b200_sum_static: the sum for hosts that cannot allocate device memory.

Some users of the C-ABI have no allocator to give scratch from -- a C/C++ (or cgo / JNI)
serving loop whose GPU memory belongs to another pool, or a latency path where a
cudaMalloc would stall the device. For them the library keeps the partial sums of a
split reduction in a fixed 1 MiB array of its own. This test calls that entry point
straight through the C-ABI and checks it against the regular `b200_sum` (caller-provided
scratch) bit for bit -- both run the same kernels with the same split plan -- on two
calls in a row with different data (the shared array keeps the first call's partials; the
second result must not see them), on a geometry that needs no scratch, and checks that a
geometry beyond the fixed maximum is refused without launching anything. The file sorts
last so that a run stopping at the first failure has already run every other test.
"""

import pytest
import torch

from backendbench_b200 import _abi

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {torch.float32: _abi.F32, torch.bfloat16: _abi.BF16, torch.float16: _abi.F16}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _sum_regular(x, outer, dim, inner, out_dtype):
    lib = _abi.lib()
    out = torch.empty(outer * inner, dtype=out_dtype, device=DEV)
    need = lib.b200_reduce_scratch_bytes(outer, dim, inner)
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    _abi.check(lib.b200_sum(x.data_ptr(), out.data_ptr(), outer, dim, inner, DT[x.dtype], DT[out_dtype], scratch.data_ptr() if need else None, need, _stream()), "b200_sum")
    return out, need


def _sum_static(x, outer, dim, inner, out_dtype):
    lib = _abi.lib()
    out = torch.empty(outer * inner, dtype=out_dtype, device=DEV)
    _abi.check(lib.b200_sum_static(x.data_ptr(), out.data_ptr(), outer, dim, inner, DT[x.dtype], DT[out_dtype], _stream()), "b200_sum_static")
    return out


@pytest.mark.parametrize("outer,dim,inner,dtype", [(1, 1 << 22, 1, torch.float32), (3, 100_000, 7, torch.bfloat16), (2, 70_001, 1, torch.float16)])
def test_static_scratch_sum_matches_regular_sum_twice_in_a_row(outer, dim, inner, dtype):
    g = torch.Generator(device=DEV).manual_seed(11)
    for call in range(2):  # second call: new data over the first call's leftover partials
        x = (torch.randn(outer * dim * inner, generator=g, device=DEV) * (1 + 9 * call)).to(dtype)
        want, need = _sum_regular(x, outer, dim, inner, dtype)
        assert 0 < need <= _abi.STATIC_SCRATCH_BYTES  # these geometries do split across CTAs
        got = _sum_static(x, outer, dim, inner, dtype)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16 if dtype != torch.float32 else torch.int32), want.view(torch.int16 if dtype != torch.float32 else torch.int32))
        exact = x.double().view(outer, dim, inner).sum(1).reshape(-1)
        tol = 1e-2 if dtype != torch.float32 else 1e-4
        assert torch.allclose(got.double(), exact, rtol=tol, atol=tol * max(1.0, float(exact.abs().max())))


def test_static_scratch_sum_without_split_and_refusal():
    lib = _abi.lib()
    x = torch.randn(4096 * 512, device=DEV)
    want, need = _sum_regular(x, 4096, 512, 1, torch.float32)
    assert need == 0
    assert torch.equal(_sum_static(x, 4096, 512, 1, torch.float32), want)
    # partials of this geometry need more than the fixed array: refused, nothing launched
    outer, dim, inner = 1, 16384, 40_000
    assert lib.b200_reduce_scratch_bytes(outer, dim, inner) > _abi.STATIC_SCRATCH_BYTES
    big = torch.zeros(outer * dim * inner, dtype=torch.bfloat16, device=DEV)
    out = torch.full((inner,), 7.0, dtype=torch.bfloat16, device=DEV)
    rc = lib.b200_sum_static(big.data_ptr(), out.data_ptr(), outer, dim, inner, _abi.BF16, _abi.BF16, _stream())
    assert rc == -4 and b"scratch" in lib.b200_strerror(rc)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())  # untouched
