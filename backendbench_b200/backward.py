"""Backward neighbours of the row operators.

BackendBench/backends/flag_gems.py:113,140,196,233 lists `embedding_dense_backward`, `native_layer_norm_backward`,
`_softmax_backward_data` and `_log_softmax_backward_data` beside the forward operators, and the reference's
training demo (README.md:40-42) needs them for a model to stay on one backend through a
backward pass. Same boundary as the forward operators: host wrapper here, kernels behind
the C-ABI (`b200_softmax_backward`, `b200_layer_norm_backward`, `b200_embedding_backward`), no aten
arithmetic.
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
    out = ops._new(grad_output.shape, input_dtype, grad_output.device)
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


def native_layer_norm_backward_default(grad_out, input, normalized_shape, mean, rstd, weight, bias, output_mask):
    """aten.native_layer_norm_backward.default -> (grad_input, grad_weight, grad_bias), each None
    where `output_mask` is False. With xhat = (x - mean) * rstd and gy = grad_out * weight:
    grad_input = rstd * (gy - mean(gy) - xhat * mean(gy * xhat)) over the normalized dims,
    grad_weight = sum over rows of grad_out * xhat, grad_bias = sum over rows of grad_out."""
    ops._require_cuda(grad_out, input, mean, rstd)
    if input.dtype not in ops._FLOATS or grad_out.dtype != input.dtype:
        raise ops.UnsupportedByB200(f"native_layer_norm_backward: dtypes {grad_out.dtype} / {input.dtype}")
    normalized_shape = [int(s) for s in normalized_shape]
    nd = len(normalized_shape)
    if nd == 0 or list(input.shape[-nd:]) != normalized_shape or grad_out.shape != input.shape:
        raise RuntimeError(f"native_layer_norm_backward: input {list(input.shape)} / grad {list(grad_out.shape)} do not end with normalized_shape {normalized_shape}")
    want_dx, want_dw, want_db = (bool(m) for m in output_mask)
    if weight is not None and (weight.dtype not in ops._FLOATS or list(weight.shape) != normalized_shape):
        raise RuntimeError("native_layer_norm_backward: weight must be a floating tensor of normalized_shape")
    if (want_dw or want_db) and weight is None and bias is None:
        raise ops.UnsupportedByB200("native_layer_norm_backward: parameter gradients requested without parameters")
    cols = ops._prod(normalized_shape)
    rows = input.numel() // cols if cols else 0
    param = weight if weight is not None else bias
    wb_dtype = param.dtype if param is not None else input.dtype
    dx = ops._new(input.shape, input.dtype, input.device) if want_dx else None
    dw = ops._new(normalized_shape, wb_dtype, input.device) if want_dw else None
    db = ops._new(normalized_shape, wb_dtype, input.device) if want_db else None
    if cols and (rows or want_dw or want_db):
        dy, x = ops._contig(grad_out), ops._contig(input)
        mu, rs = ops._contig(mean), ops._contig(rstd)
        if mu.numel() != rows or rs.numel() != rows or mu.dtype != rs.dtype or mu.dtype not in ops._FLOATS:
            raise RuntimeError("native_layer_norm_backward: mean / rstd must hold one floating value per normalized row")
        w = ops._contig(weight) if weight is not None else None
        need = int(lib().b200_layer_norm_backward_scratch_bytes(rows, cols)) if (want_dw or want_db) else 0
        scratch = ops._scratch(input.device, need) if need else None
        check(
            lib().b200_layer_norm_backward(
                dy.data_ptr(), x.data_ptr(), mu.data_ptr(), rs.data_ptr(), w.data_ptr() if w is not None else None, dx.data_ptr() if dx is not None else None,
                dw.data_ptr() if dw is not None else None, db.data_ptr() if db is not None else None, rows, cols, ops._dt(x.dtype), ops._dt(wb_dtype), ops._dt(mu.dtype),
                scratch.data_ptr() if scratch is not None else None, need, ops._stream_handle(),
            ),
            "b200_layer_norm_backward",
        )
    return dx, dw, db


def embedding_dense_backward_default(grad_output, indices, num_weights, padding_idx=-1, scale_grad_by_freq=False) -> torch.Tensor:
    """aten.embedding_dense_backward.default -> [num_weights, D]: row v is the sum of the rows of
    grad_output whose index is v (v != padding_idx), added in ascending position in fp32."""
    ops._require_cuda(grad_output, indices)
    if scale_grad_by_freq:
        raise ops.UnsupportedByB200("embedding_dense_backward: scale_grad_by_freq")
    if grad_output.dtype not in ops._FLOATS:
        raise ops.UnsupportedByB200(f"embedding_dense_backward: dtype {grad_output.dtype}")
    if indices.dtype not in (torch.int64, torch.int32):
        raise RuntimeError(f"Expected tensor for argument 'indices' to have scalar type Long or Int, but got {indices.dtype}")
    if grad_output.dim() < 1 or list(grad_output.shape[:-1]) != list(indices.shape):
        raise RuntimeError(f"embedding_dense_backward: grad_output {list(grad_output.shape)} is not indices {list(indices.shape)} + [D]")
    num_weights = int(num_weights)
    row_len = int(grad_output.shape[-1])
    out = ops._new((num_weights, row_len), grad_output.dtype, grad_output.device)
    if out.numel():
        g, idx = ops._contig(grad_output), ops._contig(indices)
        n = idx.numel()
        need = int(lib().b200_embedding_backward_scratch_bytes(n, num_weights))
        scratch = ops._scratch(out.device, need)
        check(
            lib().b200_embedding_backward(
                g.data_ptr(), idx.data_ptr(), out.data_ptr(), n, num_weights, row_len, int(padding_idx), ops._dt(g.dtype), ops._dt(idx.dtype), scratch.data_ptr(), need,
                ops._status(out.device).data_ptr(), ops._stream_handle(),
            ),
            "b200_embedding_backward",
        )
    return out


# op spec name -> host function, the same form as ops.OP_TABLE
BACKWARD_TABLE = {
    "_softmax_backward_data.default": _softmax_backward_data_default,
    "_log_softmax_backward_data.default": _log_softmax_backward_data_default,
    "native_layer_norm_backward.default": native_layer_norm_backward_default,
    "embedding_dense_backward.default": embedding_dense_backward_default,
}
