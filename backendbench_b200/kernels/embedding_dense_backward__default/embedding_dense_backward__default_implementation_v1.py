"""aten.embedding_dense_backward.default on B200: backward of aten.embedding.default.

Loaded by a BackendBench DirectoryBackend (BackendBench/backends/directory.py:47-100):
the folder name is the overload with "." spelt "__", the exported callable is
`<folder>_kernel_impl`. The arithmetic runs in libb200ops.so through the C-ABI; this
file only forwards the aten arguments to the host wrapper.
"""

import os
import sys

try:
    from backendbench_b200 import backward as _backward
except ImportError:  # loaded by path from outside the repository root
    sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))
    from backendbench_b200 import backward as _backward


def embedding_dense_backward__default_kernel_impl(*args, **kwargs):
    return _backward.embedding_dense_backward_default(*args, **kwargs)
