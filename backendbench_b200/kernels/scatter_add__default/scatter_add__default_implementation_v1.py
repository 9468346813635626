"""aten.scatter_add.default on B200: ordered (aten-CPU-order) scatter-add along dim.

Loaded by a BackendBench DirectoryBackend (BackendBench/backends/directory.py:47-100):
the folder name is the overload with "." spelt "__", the exported callable is
`<folder>_kernel_impl`. The arithmetic runs in libb200ops.so through the C-ABI; this
file forwards the aten arguments to the `b200::scatter_add` operator, whose CUDA kernel is the host
wrapper of that C-ABI call.
"""

import os
import sys

try:
    from backendbench_b200 import custom_ops as _custom_ops
except ImportError:  # loaded by path from outside the repository root
    sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))
    from backendbench_b200 import custom_ops as _custom_ops


_b200_scatter_add = _custom_ops.entry("scatter_add")  # torch.ops.b200.scatter_add


def scatter_add__default_kernel_impl(*args, **kwargs):
    return _b200_scatter_add(*args, **kwargs)
