"""The C-ABI library loads on a machine without a GPU and exports exactly what
include/b200ops.h declares (no compute calls here)."""

import ctypes
import os
import re

from backendbench_b200 import _abi
from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "b200ops.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_reports_version():
    lib = _abi.lib()
    assert lib.b200_abi_version() == _abi.ABI_VERSION == 1
    assert lib.b200_strerror(0) == b"ok"
    assert b"dtype" in lib.b200_strerror(-2)


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert len(names) >= 23
    handle = ctypes.CDLL(_abi.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/b200ops.h but not exported"
    assert set(names) == set(_abi.SIGNATURES), set(names) ^ set(_abi.SIGNATURES)


def test_argument_validation_needs_no_gpu():
    lib = _abi.lib()
    shape = _abi.i64_array([4])
    # unsupported dtype and bad rank are rejected before anything touches the device
    assert lib.b200_relu(None, None, 1, shape, shape, _abi.I64, None) == -2
    assert lib.b200_relu(None, None, 99, shape, shape, _abi.F32, None) == -1
    assert lib.b200_softmax(None, None, -1, 4, 1, _abi.F32, _abi.F32, 0, None) == -1
    assert lib.b200_reduce_scratch_bytes(1, 1 << 26, 1) > 0
    assert lib.b200_reduce_scratch_bytes(8192, 4096, 1) == 0
    assert lib.b200_gemm(None, None, None, None, 1, 0, 5, 5, 0, 5, 1, 0, 5, 1, 0, 0, 1.0, 0.0, _abi.F32, None, None) == 0
