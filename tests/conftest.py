import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_cases():
    return torch.load(os.path.join(GOLDEN, "aten_ops_golden.pt"), weights_only=False)["cases"]


@pytest.fixture(scope="session")
def harness_golden():
    with open(os.path.join(GOLDEN, "harness_golden.json")) as fh:
        return json.load(fh)


@pytest.fixture(scope="session", autouse=True)
def _built():
    """The shared library and the oracle are built once per session (seconds, CPU only)."""
    from backendbench_b200.build import build

    build()
    import oracle

    oracle.build()


EXACT_OPS = ("embedding.default", "index_select.default", "gather.default", "scatter_add.default", "argmax.default", "where.self")


def tolerance_for_case(op: str, dtype) -> tuple:
    """(atol, rtol) the parity tests use: 0 for the bit-exact operators, the harness's
    1e-2 for bf16/f16 results, 1e-5 for fp32 elementwise, 1e-4 for fp32 reductions,
    normalisations and contractions (accumulation order differs)."""
    if op in EXACT_OPS:
        return 0.0, 0.0
    if op == "native_layer_norm_backward.default" and dtype in (torch.bfloat16, torch.float16):
        # aten CPU, which made the golden vectors, adds the parameter gradients up in the
        # 16-bit type: its running sums (magnitude ~16 over 37 rows) are rounded to 0.125, so
        # an element that cancels to ~0 carries that much error; fp32 accumulation does not
        return 0.25, 1e-2
    if op == "embedding_dense_backward.default" and dtype in (torch.bfloat16, torch.float16):
        # same story: aten CPU rounds to the 16-bit type after every added row (sums of ~5
        # rows reach magnitude 4-8, where a bf16 step is 0.03-0.06)
        return 0.07, 1e-2
    if dtype in (torch.bfloat16, torch.float16):
        return 1e-2, 1e-2
    if op.split(".")[0] in ("relu", "add", "mul"):
        return 1e-5, 1e-5
    return 1e-4, 1e-4


def first_dtype(x):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x.dtype
    for y in x:
        d = first_dtype(y)
        if d is not None:
            return d
    return None


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Same shape, dtype and bit pattern (signed zeros and infinities included). NaNs must
    sit in the same places; their payload bits are not compared (arithmetic that produces
    a NaN, e.g. inf + -inf in scatter_add, may pick any quiet-NaN encoding)."""
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    if a.numel() == 0:
        return True
    a = a.detach().cpu().contiguous().reshape(-1)
    b = b.detach().cpu().contiguous().reshape(-1)
    if a.dtype == torch.bool:
        return torch.equal(a, b)
    if a.dtype.is_floating_point:
        na, nb = torch.isnan(a), torch.isnan(b)
        if not torch.equal(na, nb):
            return False
        a, b = a.masked_fill(na, 0), b.masked_fill(nb, 0)
    return torch.equal(a.view(torch.uint8), b.view(torch.uint8))


class GuardBands:
    """Allocator for `ops._allocator`: every output / scratch tensor of the host wrappers sits
    between two 512-byte bands of a sentinel byte inside one uint8 buffer, and the payload
    itself starts out as the sentinel too. `verify()` synchronises and asserts that no kernel
    wrote a band -- the stand-in for a memory checker on a pool where none can be run.
    The upper band starts at the byte after the tensor's last element, so a one-element
    overrun is caught; the payload keeps the 512-byte alignment of a fresh allocation."""

    BAND = 512
    SENTINEL = 0xA5
    MAX_LIVE_BYTES = 8 << 30

    def __init__(self):
        self.live = []  # (buffer, payload bytes, shape, dtype)
        self.live_bytes = 0
        self.allocations = 0
        self.checked = 0

    def __call__(self, shape, dtype, device):
        if isinstance(shape, int):
            shape = (shape,)
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if self.live_bytes + nbytes > self.MAX_LIVE_BYTES:
            self.verify()
        buf = torch.full((nbytes + 2 * self.BAND,), self.SENTINEL, dtype=torch.uint8, device=device)
        self.live.append((buf, nbytes, shape, dtype))
        self.live_bytes += nbytes
        self.allocations += 1
        return buf[self.BAND : self.BAND + nbytes].view(dtype).view(shape)

    def verify(self):
        torch.cuda.synchronize()
        for buf, nbytes, shape, dtype in self.live:
            lo = bool((buf[: self.BAND] == self.SENTINEL).all().item())
            hi = bool((buf[self.BAND + nbytes :] == self.SENTINEL).all().item())
            assert lo and hi, f"a kernel wrote outside its {dtype} output of shape {list(shape)}: band below intact={lo}, band above intact={hi}"
            self.checked += 1
        self.live.clear()
        self.live_bytes = 0


GUARDED_MODULES = ("test_gpu_parity", "test_gpu_gemm", "test_gpu_backward", "test_gpu_variants")


@pytest.fixture(autouse=True)
def guard_bands(request):
    """In the kernel parity modules every tensor the host wrappers allocate is guard-banded,
    and the bands are checked when the test ends (and whenever 8 GB of them are live)."""
    if request.module.__name__.split(".")[-1] not in GUARDED_MODULES or not torch.cuda.is_available():
        yield None
        return
    from backendbench_b200 import ops

    guard = GuardBands()
    ops._scratch_cache.clear()  # scratch buffers of earlier tests have no bands
    ops._allocator = guard
    try:
        yield guard
        guard.verify()
        assert guard.allocations == 0 or guard.checked > 0
    finally:
        ops._allocator = None
        ops._scratch_cache.clear()
