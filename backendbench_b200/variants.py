"""`.out` and in-place overloads of the sixteen operators, on the same kernels.

BackendBench/scripts/op_map.py:7-1148 lists, next to every functional aten operator, its
`out=` and in-place spellings; a model that calls `x.relu_()` or `torch.mm(a, b, out=c)`
stays on this backend only if those overloads are overridden too
(docs/correctness.md:155-181). Each variant here runs the functional host wrapper of
`ops.py` and places the result where the overload says:

* in-place on a tensor the kernel can write directly (elementwise operators whose `self`
  is contiguous and already has the result's shape and dtype): the kernel writes `self`;
* everything else: the result is produced in a fresh buffer and copied into the target by
  the library's strided-to-strided copy kernel (`b200_copy_into`), after the target has
  been resized the way aten resizes an `out=` tensor of the wrong shape.

Nothing here falls back to aten arithmetic.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops
from ._abi import check, i64_array, lib

_stream_handle = ops._stream_handle


def _copy_into(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """dst[...] = src for equal shapes and dtypes, any strides on either side."""
    if dst.numel() == 0:
        return dst
    shape = list(src.shape) or [1]
    sx = list(src.stride()) or [1]
    so = list(dst.stride()) or [1]
    shape, (sx, so) = ops._coalesce(shape, [sx, so])
    check(lib().b200_copy_into(src.data_ptr(), dst.data_ptr(), len(shape), i64_array(shape), i64_array(sx), i64_array(so), src.element_size(), _stream_handle()), "b200_copy_into")
    return dst


_TYPE_NAMES = {torch.float32: "Float", torch.bfloat16: "BFloat16", torch.float16: "Half", torch.float64: "Double", torch.int64: "Long", torch.int32: "Int", torch.int16: "Short", torch.int8: "Char", torch.uint8: "Byte", torch.bool: "Bool"}


def _as_dtype(result: torch.Tensor, dtype: torch.dtype, what: str) -> torch.Tensor:
    """`result` in the target's dtype, the way aten treats a result whose type differs from
    the `out=` / in-place target: allowed when `torch.can_cast(result type, target type)`
    (then the full-precision result is rounded ONCE into the target type -- `bf16.add_(f32)`
    adds in fp32 and rounds to bf16), an error with aten's message otherwise. The conversion
    runs in the library's converting copy kernel (floating types)."""
    if result.dtype == dtype:
        return result
    if not torch.can_cast(result.dtype, dtype):
        raise RuntimeError(f"result type {_TYPE_NAMES.get(result.dtype, result.dtype)} can't be cast to the desired output type {_TYPE_NAMES.get(dtype, dtype)}")
    if result.dtype not in ops._FLOATS or dtype not in ops._FLOATS:
        raise ops.UnsupportedByB200(f"{what}: converting a {result.dtype} result into a {dtype} target")
    out = ops._new(result.shape, dtype, result.device)
    if out.numel():
        nd, shp, (st,) = ops._iter_layout(result.shape, [result])
        check(lib().b200_copy_strided(result.data_ptr(), out.data_ptr(), nd, shp, st, ops._dt(result.dtype), ops._dt(dtype), _stream_handle()), "b200_copy_strided")
    return out


def _deliver(result: torch.Tensor, out: torch.Tensor, what: str, cast: bool = False) -> torch.Tensor:
    """aten's `out=` contract: a wrong shape is resized, then the tensor is filled. The out
    tensor's dtype must equal the result's, except for the TensorIterator operators
    (`cast=True`: add, mul, sum), which accept any type the result type can be cast to."""
    if out is result:
        return out
    if not out.is_cuda:
        raise ops.UnsupportedByB200(f"{what}: out tensor on {out.device}")
    if cast:
        result = _as_dtype(result, out.dtype, what)
    elif out.dtype != result.dtype:
        raise RuntimeError(f"Expected out tensor to have dtype {result.dtype}, but got {out.dtype} instead")
    if out.shape != result.shape:
        out.resize_(result.shape)  # storage management only; aten warns when the old shape was non-empty
    return _copy_into(out, result)


def _in_place(self: torch.Tensor, result: torch.Tensor, what: str, cast: bool = False) -> torch.Tensor:
    """aten's in-place contract: the result must already have `self`'s shape (no resize); its
    type must be `self`'s, or (`cast=True`: add_, mul_) one that can be cast to it."""
    if result.shape != self.shape:
        raise RuntimeError(f"output with shape {list(self.shape)} doesn't match the broadcast shape {list(result.shape)}")
    if result is self:
        return self
    if cast:
        result = _as_dtype(result, self.dtype, what)
    elif result.dtype != self.dtype:
        raise RuntimeError(f"result type {_TYPE_NAMES.get(result.dtype, result.dtype)} can't be cast to the desired output type {_TYPE_NAMES.get(self.dtype, self.dtype)}")
    return _copy_into(self, result)


def _direct_target(self: torch.Tensor, others, shape, dtype) -> Optional[torch.Tensor]:
    """`self` when an elementwise kernel may write it while reading it: contiguous, final
    shape and dtype, and no OTHER operand overlapping it with a different layout."""
    if not (self.is_cuda and self.is_contiguous() and tuple(self.shape) == tuple(shape) and self.dtype == dtype):
        return None
    base = self.untyped_storage().data_ptr()
    for t in others:
        if isinstance(t, torch.Tensor) and t.is_cuda and t.untyped_storage().data_ptr() == base:
            if not (t.data_ptr() == self.data_ptr() and t.shape == self.shape and t.stride() == self.stride()):
                return None
    return self


# --------------------------------------------------------------------- elementwise
def relu_(self: torch.Tensor) -> torch.Tensor:
    """aten.relu_.default"""
    target = _direct_target(self, (), self.shape, self.dtype)
    return _in_place(self, ops.relu(self, _into=target), "relu_")


def relu_out(self: torch.Tensor, *, out: torch.Tensor) -> torch.Tensor:
    """aten.relu.out"""
    return _deliver(ops.relu(self), out, "relu.out")


def _result_shape_dtype(a, b):
    dtype = torch.result_type(a, b)
    shape = a.shape if not isinstance(b, torch.Tensor) or b.dim() == 0 or a.shape == b.shape else ops._broadcast_shape(a.shape, b.shape)
    return tuple(shape), dtype


def add__Tensor(self: torch.Tensor, other, *, alpha=1) -> torch.Tensor:
    """aten.add_.Tensor"""
    shape, dtype = _result_shape_dtype(self, other)
    target = _direct_target(self, (other,), shape, dtype)
    return _in_place(self, ops._binary("add", self, other, float(alpha), _into=target), "add_", cast=True)


def mul__Tensor(self: torch.Tensor, other) -> torch.Tensor:
    """aten.mul_.Tensor"""
    shape, dtype = _result_shape_dtype(self, other)
    target = _direct_target(self, (other,), shape, dtype)
    return _in_place(self, ops._binary("mul", self, other, 1.0, _into=target), "mul_", cast=True)


def add_out(self, other, *, alpha=1, out: torch.Tensor) -> torch.Tensor:
    """aten.add.out"""
    return _deliver(ops.add_Tensor(self, other, alpha=alpha), out, "add.out", cast=True)


def mul_out(self, other, *, out: torch.Tensor) -> torch.Tensor:
    """aten.mul.out"""
    return _deliver(ops.mul_Tensor(self, other), out, "mul.out", cast=True)


def where_self_out(condition, self, other, *, out: torch.Tensor) -> torch.Tensor:
    """aten.where.self_out"""
    return _deliver(ops.where_self(condition, self, other), out, "where.self_out")


# --------------------------------------------------------------------- row operators
def _softmax_out(self, dim, half_to_float, *, out: torch.Tensor) -> torch.Tensor:
    """aten._softmax.out"""
    return _deliver(ops._softmax_default(self, dim, half_to_float), out, "_softmax.out")


def _log_softmax_out(self, dim, half_to_float, *, out: torch.Tensor) -> torch.Tensor:
    """aten._log_softmax.out"""
    return _deliver(ops._log_softmax_default(self, dim, half_to_float), out, "_log_softmax.out")


def sum_IntList_out(self, dim=None, keepdim=False, *, dtype=None, out: torch.Tensor) -> torch.Tensor:
    """aten.sum.IntList_out"""
    return _deliver(ops.sum_dim_IntList(self, dim, keepdim, dtype=dtype), out, "sum.IntList_out", cast=True)


def native_layer_norm_out(input, normalized_shape, weight, bias, eps, *, out0: torch.Tensor, out1: torch.Tensor, out2: torch.Tensor):
    """aten.native_layer_norm.out"""
    y, mean, rstd = ops.native_layer_norm_default(input, normalized_shape, weight, bias, eps)
    return _deliver(y, out0, "native_layer_norm.out"), _deliver(mean, out1, "native_layer_norm.out"), _deliver(rstd, out2, "native_layer_norm.out")


def argmax_out(self, dim=None, keepdim=False, *, out: torch.Tensor) -> torch.Tensor:
    """aten.argmax.out"""
    return _deliver(ops.argmax_default(self, dim, keepdim), out, "argmax.out")


# --------------------------------------------------------------------- indexing
def embedding_out(weight, indices, padding_idx=-1, scale_grad_by_freq=False, sparse=False, *, out: torch.Tensor) -> torch.Tensor:
    """aten.embedding.out"""
    return _deliver(ops.embedding_default(weight, indices, padding_idx, scale_grad_by_freq, sparse), out, "embedding.out")


def index_select_out(self, dim, index, *, out: torch.Tensor) -> torch.Tensor:
    """aten.index_select.out"""
    return _deliver(ops.index_select_default(self, dim, index), out, "index_select.out")


def gather_out(self, dim, index, *, sparse_grad=False, out: torch.Tensor) -> torch.Tensor:
    """aten.gather.out"""
    return _deliver(ops.gather_default(self, dim, index, sparse_grad=sparse_grad), out, "gather.out")


def scatter_add_(self: torch.Tensor, dim, index, src) -> torch.Tensor:
    """aten.scatter_add_.default"""
    return _in_place(self, ops.scatter_add_default(self, dim, index, src), "scatter_add_")


def scatter_add_out(self, dim, index, src, *, out: torch.Tensor) -> torch.Tensor:
    """aten.scatter_add.out"""
    return _deliver(ops.scatter_add_default(self, dim, index, src), out, "scatter_add.out")


# --------------------------------------------------------------------- contraction
def mm_out(self, mat2, *, out: torch.Tensor) -> torch.Tensor:
    """aten.mm.out"""
    return _deliver(ops.mm_default(self, mat2), out, "mm.out")


def bmm_out(self, mat2, *, out: torch.Tensor) -> torch.Tensor:
    """aten.bmm.out"""
    return _deliver(ops.bmm_default(self, mat2), out, "bmm.out")


def addmm_out(self, mat1, mat2, *, beta=1, alpha=1, out: torch.Tensor) -> torch.Tensor:
    """aten.addmm.out"""
    return _deliver(ops.addmm_default(self, mat1, mat2, beta=beta, alpha=alpha), out, "addmm.out")


def addmm_(self: torch.Tensor, mat1, mat2, *, beta=1, alpha=1) -> torch.Tensor:
    """aten.addmm_.default"""
    return _in_place(self, ops.addmm_default(self, mat1, mat2, beta=beta, alpha=alpha), "addmm_")


# op spec name -> host function, the same form as ops.OP_TABLE
VARIANT_TABLE = {
    "relu_.default": relu_,
    "relu.out": relu_out,
    "add_.Tensor": add__Tensor,
    "add.out": add_out,
    "mul_.Tensor": mul__Tensor,
    "mul.out": mul_out,
    "where.self_out": where_self_out,
    "_softmax.out": _softmax_out,
    "_log_softmax.out": _log_softmax_out,
    "sum.IntList_out": sum_IntList_out,
    "native_layer_norm.out": native_layer_norm_out,
    "argmax.out": argmax_out,
    "embedding.out": embedding_out,
    "index_select.out": index_select_out,
    "gather.out": gather_out,
    "scatter_add_.default": scatter_add_,
    "scatter_add.out": scatter_add_out,
    "mm.out": mm_out,
    "bmm.out": bmm_out,
    "addmm.out": addmm_out,
    "addmm_.default": addmm_,
}
