"""Backend plugin protocol: a backend maps an aten OpOverload to a callable.

`name`, `op in backend`, `backend[op]` -- the protocol the harness uses at
BackendBench/scripts/main.py:247-254. `AtenBackend` (backends/aten.py:10-18) is the
identity/oracle backend, `DirectoryBackend` (backends/directory.py:18-110) loads one
`<folder>_kernel_impl` per operator folder, and `B200Backend` is a DirectoryBackend
pointed at the kernels this package ships.
"""

from __future__ import annotations

import importlib.util
import logging
import os
from typing import Callable, Dict

from .utils import folder_name_to_op_name, get_pytorch_op

logger = logging.getLogger(__name__)

KERNELS_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernels")


class Backend:
    def __init__(self, name):
        self.name = name


class AtenBackend(Backend):
    """Every operator implemented by itself: the reference/oracle backend."""

    def __init__(self) -> None:
        super().__init__("aten")

    def __getitem__(self, key):
        return key

    def __contains__(self, key):
        return True


class DirectoryBackend(Backend):
    """Loads `<ops_dir>/<folder>/<folder>_implementation*.py` (first in sorted order) and
    registers its `<folder>_kernel_impl` for exactly the overload the folder names."""

    def __init__(self, ops_dir="generated_kernels"):
        super().__init__("directory")
        self.ops_dir = ops_dir
        self.compiled_kernels: Dict[object, Callable] = {}
        self._load_kernels()

    def _load_kernels(self):
        if not os.path.exists(self.ops_dir):
            logger.warning(f"ops directory {self.ops_dir} does not exist")
            return
        for folder in sorted(os.listdir(self.ops_dir)):
            op_dir = os.path.join(self.ops_dir, folder)
            if not os.path.isdir(op_dir):
                continue
            candidates = sorted(f for f in os.listdir(op_dir) if f.endswith(".py") and f.startswith(f"{folder}_implementation"))
            if not candidates:
                logger.debug(f"No implementation files found in {op_dir}")
                continue
            op_name = folder_name_to_op_name(folder)
            try:
                fn = self._load_kernel_from_file(os.path.join(op_dir, candidates[0]), folder)
                op = get_pytorch_op(op_name)
                if op is not None:
                    self.compiled_kernels[op] = fn
                    logger.info(f"Loaded {op_name} from {candidates[0]}")
            except Exception as e:  # a broken kernel file must not take the backend down
                logger.error(f"Error loading {op_name} from {candidates[0]}: {e}")
        logger.info(f"DirectoryBackend loaded {len(self.compiled_kernels)} kernels from {self.ops_dir}/")

    def _load_kernel_from_file(self, file_path: str, folder_name: str) -> Callable:
        spec = importlib.util.spec_from_file_location(f"op_{folder_name}", file_path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        fn = getattr(module, f"{folder_name}_kernel_impl", None)
        if fn is None:
            raise ValueError(f"No function named {folder_name}_kernel_impl found in {file_path}")
        return fn

    def __getitem__(self, key):
        try:
            return self.compiled_kernels[key]
        except KeyError:
            raise KeyError(f"Operator {key} not implemented in DirectoryBackend - add implementation to {self.ops_dir}/") from None

    def __contains__(self, key):
        return key in self.compiled_kernels


class B200Backend(DirectoryBackend):
    """The sixteen sm_100a operators shipped in `backendbench_b200/kernels/`."""

    def __init__(self):
        super().__init__(KERNELS_DIR)
        self.name = "b200"


def make_backend(name: str, ops_directory: str = None) -> Backend:
    """Backend by CLI name: "aten", "directory" (needs ops_directory) or "b200"."""
    if name == "aten":
        return AtenBackend()
    if name == "b200":
        return B200Backend()
    if name == "directory":
        return DirectoryBackend(ops_directory or "generated_kernels")
    raise ValueError(f"unknown backend {name!r} (choices: aten, directory, b200)")
