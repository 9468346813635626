"""aten._log_softmax_backward_data.default on B200: backward of aten._log_softmax.default.

Loaded by a BackendBench DirectoryBackend (BackendBench/backends/directory.py:47-100):
the folder name is the overload with "." spelt "__", the exported callable is
`<folder>_kernel_impl`. The arithmetic runs in libb200ops.so through the C-ABI; this
file forwards the aten arguments to the `b200::log_softmax_backward` operator, whose CUDA kernel is the host
wrapper of that C-ABI call.
"""

import os
import sys

try:
    from backendbench_b200 import custom_ops as _custom_ops
except ImportError:  # loaded by path from outside the repository root
    sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))
    from backendbench_b200 import custom_ops as _custom_ops


_b200_log_softmax_backward = _custom_ops.entry("log_softmax_backward")  # torch.ops.b200.log_softmax_backward


def _log_softmax_backward_data__default_kernel_impl(*args, **kwargs):
    return _b200_log_softmax_backward(*args, **kwargs)
