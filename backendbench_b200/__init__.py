"""backendbench_b200: a B200-native ATen operator backend behind BackendBench's own
override API, plus the evaluation path around it.

`enable()` / `disable()` / `BackendBench.enable(...)` register the kernels of a
directory backend with `torch.library.Library("aten", "IMPL", key)` exactly as
BackendBench/__init__.py:29-158 does, so model code runs on them unchanged.
"""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Optional, Union

import torch

from .backends import KERNELS_DIR, AtenBackend, B200Backend, Backend, DirectoryBackend

logger = logging.getLogger(__name__)

__version__ = "0.1.0"
__all__ = ["enable", "disable", "BackendBench", "Backend", "AtenBackend", "DirectoryBackend", "B200Backend", "KERNELS_DIR"]

_lib = None  # the Library object holding the process-wide registrations


def _monkey_patch_operators(lib, op_custom_impl, namespace="aten", dispatch_key="CUDA"):
    """Register every (OpOverload -> callable) pair on `lib` for `dispatch_key`."""
    assert dispatch_key in ["CPU", "CUDA"], "Only CPU and CUDA dispatch keys are supported"
    patched = 0
    for op, impl in op_custom_impl.items():
        try:
            schema = op._schema
            full_name = f"{schema.name}.{schema.overload_name}" if schema.overload_name else schema.name
            lib.impl(full_name, impl, dispatch_key)
            patched += 1
        except Exception as e:  # some operators cannot be overridden
            logger.warning(f"Could not register {op}: {e}")
    print(f"Successfully registered {patched} custom operators" if patched else "No custom operators registered")


def enable(kernel_dir: Optional[Union[str, Path]] = None, namespace: str = "aten", dispatch_key: str = "CUDA", lib=None) -> None:
    """Override aten operators with the kernels found under `kernel_dir`
    (default: the sm_100a kernels shipped with this package)."""
    global _lib
    print("Enabling DirectoryBackend")
    kernel_dir = Path(kernel_dir) if kernel_dir is not None else Path(KERNELS_DIR)
    if not kernel_dir.exists():
        logger.warning(f"Kernel directory {kernel_dir} does not exist.")
        return
    try:
        backend = DirectoryBackend(str(kernel_dir))
        if lib is None:
            if _lib is None:
                _lib = torch.library.Library(namespace, "IMPL", dispatch_key)
            lib = _lib
        _monkey_patch_operators(lib, backend.compiled_kernels, namespace, dispatch_key)
    except Exception as e:
        logger.warning(f"Failed to enable DirectoryBackend: {e}")


def disable() -> None:
    """Drop the process-wide registrations; aten's own kernels are back in place."""
    global _lib
    if _lib is None:
        logger.warning("DirectoryBackend is not currently enabled")
        return
    _lib = None
    print("DirectoryBackend disabled")


class _BackendBenchContext:
    """`with BackendBench.enable(...)`: registrations live exactly as long as the block."""

    def __init__(self, kernel_dir=None, namespace="aten", dispatch_key="CUDA"):
        self.kernel_dir = kernel_dir
        self.namespace = namespace
        self.dispatch_key = dispatch_key
        self.lib = torch.library.Library(namespace, "IMPL", dispatch_key)

    def __enter__(self):
        enable(self.kernel_dir, self.namespace, self.dispatch_key, self.lib)
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.lib = None


class BackendBench:
    @classmethod
    def enable(cls, kernel_dir=None, namespace="aten", dispatch_key="CUDA"):
        return _BackendBenchContext(kernel_dir, namespace, dispatch_key)
