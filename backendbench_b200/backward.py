"""Backward neighbours of the row operators.

BackendBench/backends/flag_gems.py:196,233 lists `_softmax_backward_data` and
`_log_softmax_backward_data` beside the forward operators, and the reference's
training demo (README.md:40-42) needs them for a model to stay on one backend through a
backward pass. Same boundary as the forward operators: host wrapper here, kernels behind
the C-ABI (`b200_softmax_backward`), no aten arithmetic.
"""

from __future__ import annotations

import torch

from . import ops
from ._abi import check, lib


def _softmax_backward(grad_output: torch.Tensor, output: torch.Tensor, dim: int, input_dtype: torch.dtype, log: bool) -> torch.Tensor:
    ops._require_cuda(grad_output, output)
    if grad_output.shape != output.shape:
        raise RuntimeError(f"grad_output and output must have the same shape, got {list(grad_output.shape)} and {list(output.shape)}")
    if grad_output.dtype != output.dtype:
        raise RuntimeError(f"expected grad_output and output to have the same dtype, got {grad_output.dtype} and {output.dtype}")
    if grad_output.dtype not in ops._FLOATS or input_dtype not in ops._FLOATS:
        raise ops.UnsupportedByB200(f"softmax backward: dtypes {grad_output.dtype} -> {input_dtype}")
    dim = ops._norm_dim(dim, grad_output.dim())
    out = torch.empty(grad_output.shape, dtype=input_dtype, device=grad_output.device)
    if out.numel():
        outer, d, inner = ops._split_at(list(grad_output.shape) or [1], dim)
        g, y = ops._contig(grad_output), ops._contig(output)
        check(
            lib().b200_softmax_backward(g.data_ptr(), y.data_ptr(), out.data_ptr(), outer, d, inner, ops._dt(g.dtype), ops._dt(input_dtype), 1 if log else 0, ops._stream_handle()),
            "b200_softmax_backward",
        )
    return out


def _softmax_backward_data_default(grad_output, output, dim, input_dtype) -> torch.Tensor:
    """aten._softmax_backward_data.default -- (grad - sum(grad * output, dim)) * output."""
    return _softmax_backward(grad_output, output, dim, input_dtype, False)


def _log_softmax_backward_data_default(grad_output, output, dim, input_dtype) -> torch.Tensor:
    """aten._log_softmax_backward_data.default -- grad - exp(output) * sum(grad, dim)."""
    return _softmax_backward(grad_output, output, dim, input_dtype, True)


# op spec name -> host function, the same form as ops.OP_TABLE
BACKWARD_TABLE = {
    "_softmax_backward_data.default": _softmax_backward_data_default,
    "_log_softmax_backward_data.default": _log_softmax_backward_data_default,
}
