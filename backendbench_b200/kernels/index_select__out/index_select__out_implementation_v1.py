"""aten.index_select.out on B200: the `out=` overload of aten.index_select.default, same kernels.

Loaded by a BackendBench DirectoryBackend (BackendBench/backends/directory.py:47-100):
the folder name is the overload with "." spelt "__", the exported callable is
`<folder>_kernel_impl`. The arithmetic runs in libb200ops.so through the C-ABI; this
file only forwards the aten arguments to the host wrapper, which places the result in the
tensor the overload names (BackendBench/scripts/op_map.py:7-1148 lists these spellings).
"""

import os
import sys

try:
    from backendbench_b200 import variants as _variants
except ImportError:  # loaded by path from outside the repository root
    sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))
    from backendbench_b200 import variants as _variants


def index_select__out_kernel_impl(*args, **kwargs):
    return _variants.index_select_out(*args, **kwargs)
