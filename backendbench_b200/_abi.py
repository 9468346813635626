"""ctypes binding of ``libb200ops.so`` (declared in ``include/b200ops.h``).

The library is the only compute path of this package: there is no CPU or PyTorch
fallback. ``lib()`` raises ``B200LibraryMissing`` when the shared object has not been
built (``python -m backendbench_b200.build``), and every wrapper turns a non-zero
return code into ``B200Error`` -- operators fail loudly instead of silently falling
back to aten.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_int, c_int64, c_uint32, c_void_p

CSRC_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
# B200OPS_LIB names another build of the same library (same ABI version), e.g. one compiled
# with other tuning constants, without touching the in-tree one
LIB_PATH = os.environ.get("B200OPS_LIB") or os.path.join(CSRC_DIR, "libb200ops.so")

ABI_VERSION = 1
MAX_DIMS = 8

# b200_dtype codes
F32, BF16, F16, I32, I64, BOOL, U8, I8, I16, F64 = range(10)

# bits of a device status word
DEV_INDEX_OOB = 1
DEV_WAIT_TIMEOUT = 2

STATIC_SCRATCH_BYTES = 1 << 20  # B200_STATIC_SCRATCH_BYTES


class B200LibraryMissing(RuntimeError):
    """libb200ops.so is not built or cannot be loaded."""


class B200Error(RuntimeError):
    """A C-ABI call returned a negative status code."""


I64P = POINTER(c_int64)

# name -> (restype, argtypes); mirrors include/b200ops.h one to one
SIGNATURES = {
    "b200_abi_version": (c_int, []),
    "b200_strerror": (c_char_p, [c_int]),
    "b200_last_cuda_error": (c_char_p, []),
    "b200_launch_count": (ctypes.c_longlong, []),
    "b200_relu": (c_int, [c_void_p, c_void_p, c_int, I64P, I64P, c_int, c_void_p]),
    "b200_add": (c_int, [c_void_p, c_void_p, c_void_p, c_int, I64P, I64P, I64P, c_int, c_int, c_int, c_double, c_void_p]),
    "b200_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int, I64P, I64P, I64P, c_int, c_int, c_int, c_void_p]),
    "b200_add_scalar": (c_int, [c_void_p, c_void_p, c_int, I64P, I64P, c_int, c_int, c_double, c_void_p]),
    "b200_mul_scalar": (c_int, [c_void_p, c_void_p, c_int, I64P, I64P, c_int, c_int, c_double, c_void_p]),
    "b200_where": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, I64P, I64P, I64P, I64P, c_int, c_int, c_int, c_void_p]),
    "b200_copy_strided": (c_int, [c_void_p, c_void_p, c_int, I64P, I64P, c_int, c_int, c_void_p]),
    "b200_copy_pitched": (c_int, [c_void_p, c_void_p] + [c_int64] * 8 + [c_int, c_void_p]),
    "b200_copy_into": (c_int, [c_void_p, c_void_p, c_int, I64P, I64P, I64P, c_int, c_void_p]),
    "b200_softmax": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_softmax_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p]),
    "b200_reduce_scratch_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "b200_sum": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p]),
    "b200_sum_static": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]),
    "b200_layer_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_double, c_int, c_int, c_int, c_void_p]),
    "b200_layer_norm_backward_scratch_bytes": (c_int64, [c_int64, c_int64]),
    "b200_layer_norm_backward": (c_int, [c_void_p] * 8 + [c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_int64, c_void_p]),
    "b200_argmax": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_int64, c_void_p]),
    "b200_gather_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "b200_index_select": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "b200_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_int, I64P, I64P, I64P, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "b200_scatter_add_scratch_bytes": (c_int64, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, I64P, I64P, I64P, I64P, c_int, c_int]),
    "b200_scatter_add": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, I64P, I64P, I64P, I64P, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "b200_embedding_backward_scratch_bytes": (c_int64, [c_int64, c_int64]),
    "b200_embedding_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "b200_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p] + [c_int64] * 12 + [c_double, c_double, c_int, c_void_p, c_void_p]),
    "b200_gemm_uses_tensor_cores": (c_int, [c_int64] * 10 + [c_int, c_void_p, c_void_p, c_void_p]),
    "b200_gemm_wait_probe": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int64, c_void_p, c_void_p]),
    "b200_gemm_prefers_small": (c_int, [c_void_p, c_void_p] + [c_int64] * 10 + [c_int]),
    "b200_gemm_small_path": (c_int, [c_int]),
    "b200_gemm_splitk_scratch_bytes": (c_int64, [c_void_p, c_void_p, c_void_p] + [c_int64] * 10 + [c_int]),
    "b200_gemm_splitk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p] + [c_int64] * 12 + [c_double, c_double, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "b200_gemm_f32_scratch_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int64]),
    "b200_gemm_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p] + [c_int64] * 12 + [c_double, c_double, c_void_p, c_int64, c_void_p, c_void_p]),
    "b200_allclose": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_double, c_double, c_void_p, c_int, c_void_p]),
    "b200_l2_flush": (c_int, [c_void_p, c_int64, c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Load (once) and return the shared library with typed signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise B200LibraryMissing(
            f"{LIB_PATH} is missing: build it with `python -m backendbench_b200.build` "
            "(needs nvcc; sm_100a only). There is no CPU fallback."
        )
    try:
        handle = ctypes.CDLL(LIB_PATH)
    except OSError as e:  # pragma: no cover - depends on the box
        raise B200LibraryMissing(f"cannot load {LIB_PATH}: {e}") from e
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    got = handle.b200_abi_version()
    if got != ABI_VERSION:
        raise B200LibraryMissing(f"{LIB_PATH} has ABI version {got}, this package needs {ABI_VERSION}")
    _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    """Raise B200Error for a negative return code of entry point `what`."""
    if rc == 0:
        return
    handle = lib()
    msg = handle.b200_strerror(rc).decode()
    if rc == -3:
        msg += ": " + handle.b200_last_cuda_error().decode()
    raise B200Error(f"{what} failed with code {rc}: {msg}")


def i64_array(values):
    """A C int64 array from a Python sequence (at least one slot so the pointer is valid)."""
    n = len(values)
    return (c_int64 * max(n, 1))(*values)
