"""Host side of the sixteen overridden ATen operators.

Each function takes exactly the arguments of its aten overload (the way
``impl(*args, **kwargs)`` is called at BackendBench/eval.py:102 and through the
dispatcher at BackendBench/__init__.py:91), returns what aten returns (same structure,
shape, dtype and device -- ``assert_close`` at BackendBench/eval.py:76 checks all of
them) and does the arithmetic only through the C-ABI of ``libb200ops.so``. PyTorch is
used for three things: allocating the output (``torch.empty``), reading shapes /
strides / data pointers, and naming the current CUDA stream. Inputs are never mutated.

Nothing here calls the aten operator it implements, so registering these functions
for the CUDA dispatch key cannot recurse.
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

from . import _abi
from ._abi import check, i64_array, lib

_DT = {
    torch.float32: _abi.F32,
    torch.bfloat16: _abi.BF16,
    torch.float16: _abi.F16,
    torch.int32: _abi.I32,
    torch.int64: _abi.I64,
    torch.bool: _abi.BOOL,
    torch.uint8: _abi.U8,
    torch.int8: _abi.I8,
    torch.int16: _abi.I16,
    torch.float64: _abi.F64,
}
_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


class UnsupportedByB200(NotImplementedError):
    """The request is outside what the CUDA kernels implement (there is no fallback)."""


def _dt(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise UnsupportedByB200(f"dtype {dtype} is not supported by the B200 backend") from None


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise UnsupportedByB200(
                "the B200 backend only runs on CUDA tensors (got a tensor on " + str(t.device) + "); there is no CPU path"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"Expected all tensors to be on the same device, got {dev} and {t.device}")
    return dev


# Every output and scratch buffer of the host wrappers is allocated here. `_allocator` is a
# hook for the guard-band tests (a callable (shape, dtype, device) -> tensor that places the
# tensor between sentinel bands); None means PyTorch's caching allocator.
_allocator = None


def _new(shape, dtype, device) -> torch.Tensor:
    if _allocator is not None:
        return _allocator(shape, dtype, device)
    return torch.empty(shape, dtype=dtype, device=device)


try:  # the raw handle of the current stream without building a torch.cuda.Stream object (about 2 us less per call)
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:  # pragma: no cover - older / newer torch without the private accessor
    _raw_stream = None


def _stream_handle() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


# --------------------------------------------------------------------- device status
_status_words = {}


def _status(device: torch.device) -> torch.Tensor:
    """The 4-byte device word index kernels OR their error bits into (one per device)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = w
    return w


def check_device_status(device: Optional[torch.device] = None) -> None:
    """Synchronise, read the status word and raise if an index kernel flagged an error.

    The kernels never fault on a bad index: they zero the affected output, set a bit
    and carry on, and the error surfaces here (aten CPU raises IndexError eagerly; aten
    CUDA trips a device-side assert that poisons the context -- this keeps it usable).
    """
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(key)
    if w is None:
        return
    bits = int(w.item())
    if bits:
        w.zero_()
        if bits & _abi.DEV_INDEX_OOB:
            raise IndexError("index out of range in a B200 indexing kernel (embedding/index_select/gather/scatter_add)")
        raise RuntimeError(f"B200 kernel reported device status {bits:#x} (bounded wait timed out)")


# --------------------------------------------------------------------- layout helpers
def _expanded_strides(t: torch.Tensor, shape: Sequence[int]) -> List[int]:
    """Strides of `t` broadcast to `shape` (stride 0 on broadcast dims), without a view op."""
    nd = len(shape)
    off = nd - t.dim()
    ts, tst = t.shape, t.stride()
    out = [0] * nd
    for d in range(t.dim()):
        out[off + d] = 0 if (ts[d] == 1 and shape[off + d] != 1) else tst[d]
    return out


def _broadcast_shape(*shapes) -> List[int]:
    nd = max(len(s) for s in shapes)
    out = [1] * nd
    for s in shapes:
        off = nd - len(s)
        for d, n in enumerate(s):
            cur = out[off + d]
            if cur == 1:
                out[off + d] = n
            elif n != 1 and n != cur:
                raise RuntimeError(
                    f"The size of tensor a ({cur}) must match the size of tensor b ({n}) at non-singleton dimension {off + d}"
                )
    return out


def _coalesce(shape: List[int], strides: List[List[int]]) -> Tuple[List[int], List[List[int]]]:
    """Drop size-1 dims and merge neighbours that are jointly contiguous in every operand."""
    dims = [d for d in range(len(shape)) if shape[d] != 1]
    if not dims:
        return [1], [[0] for _ in strides]
    new_shape = [shape[dims[0]]]
    new_strides = [[s[dims[0]]] for s in strides]
    for d in dims[1:]:
        n = shape[d]
        if all(ns[-1] == s[d] * n for ns, s in zip(new_strides, strides)):
            new_shape[-1] *= n
            for ns, s in zip(new_strides, strides):
                ns[-1] = s[d]
        else:
            new_shape.append(n)
            for ns, s in zip(new_strides, strides):
                ns.append(s[d])
    return new_shape, new_strides


def _contiguous_strides(shape: Sequence[int]) -> List[int]:
    st, acc = [0] * len(shape), 1
    for d in range(len(shape) - 1, -1, -1):
        st[d] = acc
        acc *= max(shape[d], 1)
    return st


_array_memo = {}


def _memo_array(values: tuple):
    """`i64_array(values)`, remembered: the kernels only read these arrays, and a sweep asks
    for the same few shapes and strides over and over."""
    arr = _array_memo.get(values)
    if arr is None:
        if len(_array_memo) > 8192:
            _array_memo.clear()
        arr = _array_memo[values] = i64_array(values)
    return arr


def _iter_layout(out_shape: Sequence[int], operands: Sequence[torch.Tensor]):
    """(ndim, shape array, [stride arrays]) for a contiguous output of `out_shape`."""
    if all(t.shape == out_shape and t.is_contiguous() for t in operands):
        # the common case: everything contiguous and of the output's shape is one flat run
        n = 1
        for d in out_shape:
            n *= d
        one = _memo_array((1,))
        return 1, _memo_array((n,)), [one] * len(operands)
    shape = list(out_shape)
    strides = [_expanded_strides(t, shape) for t in operands]
    strides.append(_contiguous_strides(shape))  # the output constrains merging too
    shape, strides = _coalesce(shape, strides)
    if len(shape) > _abi.MAX_DIMS:
        raise UnsupportedByB200(f"more than {_abi.MAX_DIMS} non-mergeable dimensions")
    return len(shape), _memo_array(tuple(shape)), [_memo_array(tuple(st)) for st in strides[:-1]]


def _contig(t: torch.Tensor) -> torch.Tensor:
    """`t` itself when contiguous, else a contiguous copy made by the strided-copy kernel."""
    if t.is_contiguous():
        return t
    out = _new(t.shape, t.dtype, t.device)
    if out.numel():
        nd, shp, (st,) = _iter_layout(t.shape, [t])
        check(lib().b200_copy_strided(t.data_ptr(), out.data_ptr(), nd, shp, st, _dt(t.dtype), _dt(t.dtype), _stream_handle()), "b200_copy_strided")
    return out


def _prod(xs) -> int:
    p = 1
    for x in xs:
        p *= int(x)
    return p


def _is_wrapped_scalar(x) -> bool:
    return isinstance(x, (int, float, bool)) or (isinstance(x, torch.Tensor) and x.dim() == 0 and not x.is_cuda)


def _scalar_value(x) -> float:
    return float(x.item()) if isinstance(x, torch.Tensor) else float(x)


# --------------------------------------------------------------------- elementwise
def relu(self: torch.Tensor, *, _into: Optional[torch.Tensor] = None) -> torch.Tensor:
    """aten.relu.default -- max(x, 0) with NaN propagated (x <= 0 ? 0 : x). `_into`: a
    contiguous tensor of the result's shape and dtype to write instead of a fresh one (the
    in-place overloads pass `self`)."""
    _require_cuda(self)
    if self.dtype not in _FLOATS:
        raise UnsupportedByB200(f"relu: dtype {self.dtype}")
    out = _into if _into is not None else _new(self.shape, self.dtype, self.device)
    if out.numel():
        nd, shp, (sx,) = _iter_layout(self.shape, [self])
        check(lib().b200_relu(self.data_ptr(), out.data_ptr(), nd, shp, sx, _dt(self.dtype), _stream_handle()), "b200_relu")
    return out


def _binary(name: str, a, b, alpha: float, _into: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not isinstance(a, torch.Tensor) or (a.dim() == 0 and not a.is_cuda and isinstance(b, torch.Tensor) and b.is_cuda):
        if _into is not None:
            raise UnsupportedByB200(f"{name}: in-place on a wrapped number")
        if name == "mul":
            return _binary(name, b, a, alpha)  # commutative
        if not isinstance(b, torch.Tensor):
            raise UnsupportedByB200("add of two non-tensors")
        # scalar + tensor: a + alpha*b == (alpha*b) + a; only exact-scalar alpha==1 is cheap to swap
        if alpha != 1:
            raise UnsupportedByB200("add.Tensor with a wrapped-number `self` and alpha != 1")
        return _binary(name, b, a, 1.0)
    res_dtype = torch.result_type(a, b)
    if res_dtype not in _FLOATS or a.dtype not in _FLOATS:
        raise UnsupportedByB200(f"{name}: result dtype {res_dtype} (inputs {a.dtype}, {getattr(b, 'dtype', type(b))})")
    _require_cuda(a)
    st = _stream_handle()
    if _is_wrapped_scalar(b):
        out = _into if _into is not None else _new(a.shape, res_dtype, a.device)
        if out.numel():
            nd, shp, (sa,) = _iter_layout(a.shape, [a])
            val = _scalar_value(b)
            if name == "add":
                check(lib().b200_add_scalar(a.data_ptr(), out.data_ptr(), nd, shp, sa, _dt(a.dtype), _dt(res_dtype), alpha * val, st), "b200_add_scalar")
            else:
                check(lib().b200_mul_scalar(a.data_ptr(), out.data_ptr(), nd, shp, sa, _dt(a.dtype), _dt(res_dtype), val, st), "b200_mul_scalar")
        return out
    if b.dtype not in _FLOATS:
        raise UnsupportedByB200(f"{name}: operand dtype {b.dtype}")
    _require_cuda(a, b)
    if a.shape == b.shape:
        shape = a.shape
    else:
        shape = _broadcast_shape(a.shape, b.shape)
    out = _into if _into is not None else _new(shape, res_dtype, a.device)
    if out.numel():
        nd, shp, (sa, sb) = _iter_layout(shape, [a, b])
        if name == "add":
            check(lib().b200_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), nd, shp, sa, sb, _dt(a.dtype), _dt(b.dtype), _dt(res_dtype), float(alpha), st), "b200_add")
        else:
            check(lib().b200_mul(a.data_ptr(), b.data_ptr(), out.data_ptr(), nd, shp, sa, sb, _dt(a.dtype), _dt(b.dtype), _dt(res_dtype), st), "b200_mul")
    return out


def add_Tensor(self, other, *, alpha=1) -> torch.Tensor:
    """aten.add.Tensor -- self + alpha*other with broadcasting and type promotion."""
    return _binary("add", self, other, float(alpha))


def mul_Tensor(self, other) -> torch.Tensor:
    """aten.mul.Tensor -- self * other with broadcasting and type promotion."""
    return _binary("mul", self, other, 1.0)


def where_self(condition: torch.Tensor, self, other) -> torch.Tensor:
    """aten.where.self -- condition ? self : other (bit-exact select, promoted dtype)."""
    dev = _require_cuda(condition)
    if condition.dtype not in (torch.bool, torch.uint8):
        raise RuntimeError(f"where expected condition to be a boolean tensor, but got a tensor with dtype {condition.dtype}")
    res_dtype = torch.result_type(self, other)

    def as_dev(t):
        if isinstance(t, torch.Tensor) and t.is_cuda:
            return t
        # wrapped number (0-dim CPU tensor or Python scalar): materialise one device element
        return torch.full((), _scalar_value(t), dtype=res_dtype, device=dev)

    x, y = as_dev(self), as_dev(other)
    _require_cuda(condition, x, y)
    shape = _broadcast_shape(condition.shape, x.shape, y.shape)
    out = _new(shape, res_dtype, dev)
    if out.numel():
        if x.dtype != y.dtype and not (x.dtype in _FLOATS and y.dtype in _FLOATS):
            raise UnsupportedByB200(f"where: mixed dtypes {x.dtype}/{y.dtype}")
        nd, shp, (sc, sx, sy) = _iter_layout(shape, [condition, x, y])
        check(
            lib().b200_where(condition.data_ptr(), x.data_ptr(), y.data_ptr(), out.data_ptr(), nd, shp, sc, sx, sy, _dt(x.dtype), _dt(y.dtype), _dt(res_dtype), _stream_handle()),
            "b200_where",
        )
    return out


# --------------------------------------------------------------------- row kernels
def _split_at(shape, dim):
    return _prod(shape[:dim]), int(shape[dim]) if len(shape) else 1, _prod(shape[dim + 1 :])


def _norm_dim(dim: int, ndim: int) -> int:
    lim = max(ndim, 1)
    if dim < -lim or dim >= lim:
        raise IndexError(f"Dimension out of range (expected to be in range of [{-lim}, {lim - 1}], but got {dim})")
    return dim % lim


def _softmax_impl(self: torch.Tensor, dim: int, half_to_float: bool, log: bool) -> torch.Tensor:
    _require_cuda(self)
    if self.dtype not in _FLOATS:
        raise UnsupportedByB200(f"softmax: dtype {self.dtype}")
    if half_to_float and self.dtype == torch.float32:
        raise RuntimeError("conversion is supported for Half type only")
    dim = _norm_dim(dim, self.dim())
    out_dtype = torch.float32 if half_to_float else self.dtype
    out = _new(self.shape, out_dtype, self.device)
    if out.numel():
        outer, d, inner = _split_at(list(self.shape) or [1], dim)
        if inner > 1 and d >= 128 and outer * ((inner + 127) // 128) < 592:
            # a long reduction over a non-last dim with few columns: too few threads for the
            # column kernel. Move the dim last with the strided-copy kernel, run the row
            # kernel, and copy the result back through the inverse permutation.
            xt = _contig(self.movedim(dim, -1))
            tmp = _new(xt.shape, out_dtype, self.device)
            check(lib().b200_softmax(xt.data_ptr(), tmp.data_ptr(), xt.numel() // d, d, 1, _dt(xt.dtype), _dt(out_dtype), 1 if log else 0, _stream_handle()), "b200_softmax")
            back = tmp.movedim(-1, dim)  # a view with out's shape
            nd, shp, (st,) = _iter_layout(out.shape, [back])
            check(lib().b200_copy_strided(back.data_ptr(), out.data_ptr(), nd, shp, st, _dt(out_dtype), _dt(out_dtype), _stream_handle()), "b200_copy_strided")
            return out
        x = _contig(self)
        check(lib().b200_softmax(x.data_ptr(), out.data_ptr(), outer, d, inner, _dt(x.dtype), _dt(out_dtype), 1 if log else 0, _stream_handle()), "b200_softmax")
    return out


def _softmax_default(self, dim, half_to_float) -> torch.Tensor:
    """aten._softmax.default -- exp(x - max) / sum along dim, fp32 internally."""
    return _softmax_impl(self, dim, bool(half_to_float), False)


def _log_softmax_default(self, dim, half_to_float) -> torch.Tensor:
    """aten._log_softmax.default -- x - max - log(sum(exp(x - max))) along dim."""
    return _softmax_impl(self, dim, bool(half_to_float), True)


_scratch_cache = {}


_SCRATCH_MAX_STREAMS = 64


def _scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """A scratch buffer of at least `nbytes` for the current stream of `device` (grown
    geometrically, reused; per stream, so that operators queued on different streams never
    share one)."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = _new(max(nbytes, 1 << 20), torch.uint8, device)
        _scratch_cache.pop(key, None)
        _scratch_cache[key] = buf
        while len(_scratch_cache) > _SCRATCH_MAX_STREAMS:  # streams come and go: keep the most recently sized buffers only
            _scratch_cache.pop(next(iter(_scratch_cache)))
    return buf


def _reduce_layout(self: torch.Tensor, dims: List[int]):
    """Contiguous tensor + (outer, dim, inner) such that the reduction runs over `dim`."""
    nd = self.dim()
    dims = sorted(set(dims))
    if dims == list(range(dims[0], dims[0] + len(dims))):
        x = _contig(self)
        shp = list(x.shape)
        return x, _prod(shp[: dims[0]]), _prod(shp[dims[0] : dims[-1] + 1]), _prod(shp[dims[-1] + 1 :])
    kept = [d for d in range(nd) if d not in dims]
    x = _contig(self.permute(kept + dims))  # permute is a view; the copy is our kernel
    return x, _prod(self.shape[d] for d in kept), _prod(self.shape[d] for d in dims), 1


def sum_dim_IntList(self: torch.Tensor, dim=None, keepdim: bool = False, *, dtype=None) -> torch.Tensor:
    """aten.sum.dim_IntList -- fp32 accumulation, result rounded once to the output dtype."""
    _require_cuda(self)
    out_dtype = dtype if dtype is not None else self.dtype
    if self.dtype not in _FLOATS or out_dtype not in _FLOATS:
        raise UnsupportedByB200(f"sum: dtypes {self.dtype} -> {out_dtype}")
    nd = self.dim()
    if dim is None or (isinstance(dim, (list, tuple)) and len(dim) == 0):
        dims = list(range(nd))
    else:
        dims = [dim] if isinstance(dim, int) else list(dim)
        dims = [_norm_dim(int(d), nd) for d in dims]
        if len(set(dims)) != len(dims):
            raise RuntimeError("dim appears multiple times in the list of dims")
    if nd == 0:
        dims = []
    out_shape = [(1 if d in dims else s) for d, s in enumerate(self.shape)] if keepdim else [s for d, s in enumerate(self.shape) if d not in dims]
    out = _new(out_shape, out_dtype, self.device)
    if out.numel() == 0:
        return out
    if not dims:  # 0-dim input: the sum of one element
        x, outer, d, inner = _contig(self), 1, 1, 1
    else:
        x, outer, d, inner = _reduce_layout(self, dims)
    L = lib()
    need = L.b200_reduce_scratch_bytes(outer, d, inner)
    scratch = _scratch(self.device, need) if need else None
    check(
        L.b200_sum(x.data_ptr(), out.data_ptr(), outer, d, inner, _dt(x.dtype), _dt(out_dtype), scratch.data_ptr() if need else None, need, _stream_handle()),
        "b200_sum",
    )
    return out


# dtype of mean/rstd returned by aten's CUDA layer norm: the accumulate type (fp32) for
# every floating input, not the input dtype (that is the CPU kernel's convention).
LAYER_NORM_STAT_DTYPE_CUDA = torch.float32


def native_layer_norm_default(input: torch.Tensor, normalized_shape, weight=None, bias=None, eps: float = 1e-5):
    """aten.native_layer_norm.default -> (out, mean, rstd); statistics in fp32."""
    _require_cuda(input, weight, bias)
    if input.dtype not in _FLOATS:
        raise UnsupportedByB200(f"native_layer_norm: dtype {input.dtype}")
    ns = [int(s) for s in normalized_shape]
    k = len(ns)
    if k == 0 or list(input.shape[input.dim() - k :]) != ns:
        raise RuntimeError(f"Given normalized_shape={ns}, expected input with shape [*, {', '.join(map(str, ns))}], but got input of size {list(input.shape)}")
    for name, t in (("weight", weight), ("bias", bias)):
        if t is not None and list(t.shape) != ns:
            raise RuntimeError(f"Expected {name} to be of same shape as normalized_shape, but got {name} of shape {list(t.shape)} and normalized_shape = {ns}")
    wb_dtype = weight.dtype if weight is not None else (bias.dtype if bias is not None else input.dtype)
    if weight is not None and bias is not None and weight.dtype != bias.dtype:
        raise UnsupportedByB200("native_layer_norm: weight and bias dtypes differ")
    lead = list(input.shape[: input.dim() - k])
    rows, cols = _prod(lead), _prod(ns)
    stat_shape = lead + [1] * k
    out = _new(input.shape, input.dtype, input.device)
    mean = _new(stat_shape, LAYER_NORM_STAT_DTYPE_CUDA, input.device)
    rstd = _new(stat_shape, LAYER_NORM_STAT_DTYPE_CUDA, input.device)
    if rows:
        x = _contig(input)
        w = _contig(weight) if weight is not None else None
        b = _contig(bias) if bias is not None else None
        check(
            lib().b200_layer_norm(
                x.data_ptr(), w.data_ptr() if w is not None else None, b.data_ptr() if b is not None else None,
                out.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, cols, float(eps),
                _dt(x.dtype), _dt(wb_dtype), _dt(mean.dtype), _stream_handle(),
            ),
            "b200_layer_norm",
        )
    return out, mean, rstd


def argmax_default(self: torch.Tensor, dim=None, keepdim: bool = False) -> torch.Tensor:
    """aten.argmax.default -- int64 index of the first maximum (NaN is the maximum)."""
    _require_cuda(self)
    if self.dtype not in _FLOATS:
        raise UnsupportedByB200(f"argmax: dtype {self.dtype}")
    nd = self.dim()
    if dim is None:
        if self.numel() == 0:
            raise IndexError("argmax(): Expected reduction dim to be specified for input.numel() == 0. Specify the reduction dim with the 'dim' argument.")
        x = _contig(self)
        outer, d, inner = 1, x.numel(), 1
        out_shape = [1] * nd if keepdim else []
    else:
        dim = _norm_dim(int(dim), nd)
        shape = list(self.shape) or [1]
        if shape[dim] == 0:
            raise IndexError(f"argmax(): Expected reduction dim {dim} to have non-zero size.")
        x = _contig(self)
        outer, d, inner = _split_at(shape, dim)
        out_shape = [(1 if i == dim else s) for i, s in enumerate(self.shape)] if keepdim else [s for i, s in enumerate(self.shape) if i != dim]
    out = _new(out_shape, torch.int64, self.device)
    if out.numel():
        L = lib()
        need = L.b200_reduce_scratch_bytes(outer, d, inner)
        scratch = _scratch(self.device, need) if need else None
        check(L.b200_argmax(x.data_ptr(), out.data_ptr(), outer, d, inner, _dt(x.dtype), scratch.data_ptr() if need else None, need, _stream_handle()), "b200_argmax")
    return out


# --------------------------------------------------------------------- indexing
def _index_dtype(index: torch.Tensor, what: str) -> int:
    if index.dtype == torch.int64:
        return _abi.I64
    if index.dtype == torch.int32:
        return _abi.I32
    raise RuntimeError(f"{what}: Expected tensor for argument 'indices' to have one of the following scalar types: Long, Int; but got {index.dtype} instead")


def embedding_default(weight: torch.Tensor, indices: torch.Tensor, padding_idx: int = -1, scale_grad_by_freq: bool = False, sparse: bool = False) -> torch.Tensor:
    """aten.embedding.default -- out[..., :] = weight[indices[...], :] (bit copy)."""
    _require_cuda(weight, indices)
    if weight.dim() < 1:
        raise RuntimeError("'weight' must be at least 1-D")
    idt = _index_dtype(indices, "embedding")
    out = _new(list(indices.shape) + list(weight.shape[1:]), weight.dtype, weight.device)
    if out.numel():
        w, idx = _contig(weight), _contig(indices)
        row_bytes = _prod(w.shape[1:]) * w.element_size()
        check(
            lib().b200_gather_rows(w.data_ptr(), idx.data_ptr(), out.data_ptr(), w.shape[0], row_bytes, idx.numel(), idt, _status(w.device).data_ptr(), _stream_handle()),
            "b200_gather_rows",
        )
    return out


def index_select_default(self: torch.Tensor, dim: int, index: torch.Tensor) -> torch.Tensor:
    """aten.index_select.default -- gather whole slices along `dim` (bit copy)."""
    _require_cuda(self, index)
    if index.dim() > 1:
        raise IndexError("index_select(): Index is supposed to be a vector")
    idt = _index_dtype(index, "index_select")
    dim = _norm_dim(int(dim), self.dim())
    shape = list(self.shape) or [1]
    n_idx = index.numel()
    out_shape = list(self.shape)
    if self.dim():
        out_shape[dim] = n_idx
    elif n_idx != 1:
        raise IndexError("index_select(): Index to scalar can have only 1 value")
    out = _new(out_shape, self.dtype, self.device)
    if out.numel():
        x, idx = _contig(self), _contig(index)
        outer, d, inner = _split_at(shape, dim)
        check(
            lib().b200_index_select(x.data_ptr(), idx.data_ptr(), out.data_ptr(), outer, d, inner, n_idx, x.element_size(), idt, _status(x.device).data_ptr(), _stream_handle()),
            "b200_index_select",
        )
    return out


def _check_gather_shapes(self, dim, index, src=None, what="gather"):
    if index.dtype != torch.int64:
        raise RuntimeError(f"{what}(): Expected dtype int64 for index")
    sd, idd = max(self.dim(), 1), max(index.dim(), 1)
    if sd != idd:
        raise RuntimeError("Index tensor must have the same number of dimensions as input tensor")
    if src is not None and max(src.dim(), 1) != idd:
        raise RuntimeError("Index tensor must have the same number of dimensions as src tensor")
    ss = list(self.shape) or [1]
    ix = list(index.shape) or [1]
    for d in range(sd):
        if d != dim and ix[d] > ss[d]:
            raise RuntimeError(f"Size does not match at dimension {d} expected index {ix} to be smaller than self {ss} apart from dimension {dim}")
    if src is not None:
        sr = list(src.shape) or [1]
        for d in range(sd):
            if ix[d] > sr[d]:
                raise RuntimeError(f"Size does not match at dimension {d} expected index {ix} to be smaller than src {sr}")


def gather_default(self: torch.Tensor, dim: int, index: torch.Tensor, *, sparse_grad: bool = False) -> torch.Tensor:
    """aten.gather.default -- out[p] = self[p with p[dim] = index[p]] (bit copy)."""
    _require_cuda(self, index)
    dim = _norm_dim(int(dim), self.dim())
    out = _new(index.shape, self.dtype, self.device)
    if index.numel() == 0:
        return out
    _check_gather_shapes(self, dim, index)
    nd = max(index.dim(), 1)
    if nd > _abi.MAX_DIMS:
        raise UnsupportedByB200("gather: too many dimensions")
    ishape = list(index.shape) or [1]
    istr = list(index.stride()) or [1]
    sstr = list(self.stride()) or [1]
    sshape = list(self.shape) or [1]
    check(
        lib().b200_gather(
            self.data_ptr(), index.data_ptr(), out.data_ptr(), nd, i64_array(ishape), i64_array(sstr), i64_array(istr),
            sshape[dim], dim, self.element_size(), _status(self.device).data_ptr(), _stream_handle(),
        ),
        "b200_gather",
    )
    return out


def scatter_add_default(self: torch.Tensor, dim: int, index: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """aten.scatter_add.default -- out = self; out[p with p[dim]=index[p]] += src[p],
    contributions applied in ascending p[dim] (the aten CPU order, bit-exact)."""
    _require_cuda(self, index, src)
    if self.dtype not in _FLOATS:
        raise UnsupportedByB200(f"scatter_add: dtype {self.dtype}")
    if src.dtype != self.dtype:
        raise RuntimeError("scatter(): Expected self.dtype to be equal to src.dtype")
    dim = _norm_dim(int(dim), self.dim())
    out = _new(self.shape, self.dtype, self.device)
    if out.numel() == 0:
        return out
    if index.numel():
        _check_gather_shapes(self, dim, index, src, "scatter_add")
    x = _contig(self)
    nd = max(self.dim(), 1)
    if nd > _abi.MAX_DIMS:
        raise UnsupportedByB200("scatter_add: too many dimensions")
    sshape = list(x.shape) or [1]
    if index.numel():
        ishape = list(index.shape) or [1]
        istr = list(index.stride()) or [1]
        rstr = list(src.stride()) or [1]
    else:
        ishape, istr, rstr = [0] * nd, [0] * nd, [0] * nd
    L = lib()
    a_self, a_idx, a_src = i64_array(sshape), i64_array(ishape), i64_array(istr)
    a_rstr = i64_array(rstr)
    idx_ptr = index.data_ptr() if index.numel() else None
    src_ptr = src.data_ptr() if index.numel() else None
    need = L.b200_scatter_add_scratch_bytes(x.data_ptr(), idx_ptr, src_ptr, out.data_ptr(), nd, a_self, a_idx, a_src, a_rstr, dim, _dt(x.dtype))
    scratch = _scratch(x.device, need) if need else None
    check(
        L.b200_scatter_add(
            x.data_ptr(), idx_ptr, src_ptr, out.data_ptr(), nd, a_self, a_idx, a_src, a_rstr, dim, _dt(x.dtype),
            scratch.data_ptr() if need else None, need, _status(x.device).data_ptr(), _stream_handle(),
        ),
        "b200_scatter_add",
    )
    return out


# --------------------------------------------------------------------- contraction
F32_SPLIT_MIN_MACS = 1 << 26  # batch*M*N*K from which an fp32 product takes the split tensor-core path
SPLITK_MIN_K = 1536  # a 16-bit product is offered to the K-split only from this depth ...
SPLITK_MAX_OUTPUTS = 37 * 128 * 256  # ... and up to this many outputs (the library has the last word)

def _tma_ready(t: torch.Tensor, s_b: int, s_mn: int, s_k: int, batch: int) -> bool:
    """An operand [batch, mn, k] the tensor-core kernel can load as is: one unit stride, the
    other (and the batch stride) a multiple of 8 elements, base 16-byte aligned."""
    if t.data_ptr() % 16 or (batch > 1 and (s_b % 8 or s_b <= 0)):
        return False
    return (s_k == 1 and s_mn % 8 == 0 and s_mn > 0) or (s_mn == 1 and s_k % 8 == 0 and s_k > 0)


def _repitch(t: torch.Tensor, batch: int, rows: int, cols: int, s_b: int, s_r: int, s_c: int):
    """Copy a [batch, rows, cols] view into a fresh buffer whose row pitch is a multiple of 8
    elements (pad columns stay uninitialised: the tensor map's extents exclude them)."""
    pitch = (cols + 7) // 8 * 8
    buf = _new((batch, rows, pitch), t.dtype, t.device)
    check(lib().b200_copy_pitched(t.data_ptr(), buf.data_ptr(), batch, rows, cols, s_b, s_r, s_c, rows * pitch, pitch, t.element_size(), _stream_handle()), "b200_copy_pitched")
    return buf, (rows * pitch, pitch)


def _gemm(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor], batch: int, M: int, N: int, K: int, sa, sb, alpha: float, beta: float, out_shape) -> torch.Tensor:
    if a.dtype != b.dtype:
        raise RuntimeError(f"expected m1 and m2 to have the same dtype, but got: {a.dtype} != {b.dtype}")
    if a.dtype not in _FLOATS:
        raise UnsupportedByB200(f"matmul: dtype {a.dtype}")
    out = _new(out_shape, a.dtype, a.device)
    if out.numel() == 0:
        return out
    # 16-bit operands whose layout the tensor-core path cannot load (row pitch or base off the
    # 16-byte grid, e.g. K = 2049) are re-pitched once when the product is large enough for
    # the tensor cores to pay for the extra copy; otherwise the CUDA-core kernel takes them
    # (a long contraction with a small output is re-pitched too: the CUDA-core kernel would
    # walk all of K in one or two CTAs)
    # (small products whose operands are on the 16-byte grid go to the mma.sync kernel as they are)
    if a.dtype != torch.float32 and (M * N * K * batch >= (1 << 24) or K >= 1024) and K >= 16 and not lib().b200_gemm_prefers_small(a.data_ptr(), b.data_ptr(), batch, M, N, K, sa[0], sa[1], sa[2], sb[0], sb[1], sb[2], _dt(a.dtype)):
        if not _tma_ready(a, sa[0], sa[1], sa[2], batch):
            if sa[1] != 1 or sa[2] == 1:  # keep A K-major unless it is M-major
                a, (pb, pr) = _repitch(a, batch, M, K, sa[0], sa[1], sa[2])
                sa = (pb, pr, 1)
            else:
                a, (pb, pr) = _repitch(a, batch, K, M, sa[0], sa[2], sa[1])
                sa = (pb, 1, pr)
        if not _tma_ready(b, sb[0], sb[2], sb[1], batch):
            if sb[1] != 1 or sb[2] == 1:  # keep B N-major ([K, N] rows) unless it is K-major
                b, (pb, pr) = _repitch(b, batch, K, N, sb[0], sb[1], sb[2])
                sb = (pb, pr, 1)
            else:
                b, (pb, pr) = _repitch(b, batch, N, K, sb[0], sb[2], sb[1])
                sb = (pb, 1, pr)
    sbm = sbn = 0
    bias_ptr = None
    if bias is not None:
        if bias.dtype != a.dtype:
            raise RuntimeError(f"self and mat2 must have the same dtype, but got {bias.dtype} and {a.dtype}")
        bs = _expanded_strides(bias, [M, N])
        _broadcast_shape(bias.shape, [M, N])  # raises on a non-broadcastable bias
        if bias.dim() > 2:
            raise RuntimeError("addmm: self must be broadcastable to a matrix")
        sbm, sbn = bs
        bias_ptr = bias.data_ptr()
    # Large fp32 products run on the tensor cores too: the operands are split into three bf16
    # planes each in scratch memory and six plane products are accumulated in fp32, which
    # keeps fp32 accuracy (see include/b200ops.h). Small ones stay on the CUDA-core kernel,
    # which shares a long contraction with few outputs among the CTAs of a cluster.
    # A product of only a handful of tensor-core tiles (M below two tiles, few column tiles)
    # leaves the split path one CTA per tile walking six plane pairs of all of K; the
    # CUDA-core kernel with K shared among a cluster is faster there.
    macs = batch * M * N * K
    tc_tiles = batch * ((M + 127) // 128) * ((N + 255) // 256)
    # (a C of 64 rows or columns or fewer fills half a tensor-core tile at best: the CUDA-core
    # kernel won every such shape measured, e.g. 16384 x 2060 x 32 in 0.117 ms against 0.150 ms)
    if a.dtype == torch.float32 and macs >= F32_SPLIT_MIN_MACS and K >= 32 and M > 64 and N > 64 and (tc_tiles >= 8 or macs >= (1 << 30)):
        need = int(lib().b200_gemm_f32_scratch_bytes(batch, M, N, K))
        if need > 0:
            scratch = _scratch(a.device, need)
            check(
                lib().b200_gemm_f32(
                    a.data_ptr(), b.data_ptr(), bias_ptr, out.data_ptr(), batch, M, N, K, sa[0], sa[1], sa[2], sb[0], sb[1], sb[2], sbm, sbn,
                    float(alpha), float(beta), scratch.data_ptr(), need, _status(a.device).data_ptr(), _stream_handle(),
                ),
                "b200_gemm_f32",
            )
            return out
    # A 16-bit product with a long contraction and only a few output tiles: the library cuts K
    # into ranges that run side by side and adds the fp32 partial products in a fixed order
    # (scratch: one fp32 copy of C per range)
    if a.dtype != torch.float32 and batch == 1 and K >= SPLITK_MIN_K and M * N <= SPLITK_MAX_OUTPUTS:
        need = int(lib().b200_gemm_splitk_scratch_bytes(a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, M, N, K, sa[0], sa[1], sa[2], sb[0], sb[1], sb[2], _dt(a.dtype)))
        if need > 0:
            scratch = _scratch(a.device, need)
            check(
                lib().b200_gemm_splitk(
                    a.data_ptr(), b.data_ptr(), bias_ptr, out.data_ptr(), batch, M, N, K, sa[0], sa[1], sa[2], sb[0], sb[1], sb[2], sbm, sbn,
                    float(alpha), float(beta), _dt(a.dtype), scratch.data_ptr(), need, _status(a.device).data_ptr(), _stream_handle(),
                ),
                "b200_gemm_splitk",
            )
            return out
    check(
        lib().b200_gemm(
            a.data_ptr(), b.data_ptr(), bias_ptr, out.data_ptr(), batch, M, N, K, sa[0], sa[1], sa[2], sb[0], sb[1], sb[2], sbm, sbn,
            float(alpha), float(beta), _dt(a.dtype), _status(a.device).data_ptr(), _stream_handle(),
        ),
        "b200_gemm",
    )
    return out


def mm_default(self: torch.Tensor, mat2: torch.Tensor) -> torch.Tensor:
    """aten.mm.default -- [M,K] @ [K,N], fp32 accumulation, one rounding."""
    _require_cuda(self, mat2)
    if self.dim() != 2 or mat2.dim() != 2:
        raise RuntimeError("self must be a matrix" if self.dim() != 2 else "mat2 must be a matrix")
    M, K = self.shape
    K2, N = mat2.shape
    if K != K2:
        raise RuntimeError(f"mat1 and mat2 shapes cannot be multiplied ({M}x{K} and {K2}x{N})")
    return _gemm(self, mat2, None, 1, M, N, K, (0, self.stride(0), self.stride(1)), (0, mat2.stride(0), mat2.stride(1)), 1.0, 0.0, [M, N])


def addmm_default(self: torch.Tensor, mat1: torch.Tensor, mat2: torch.Tensor, *, beta=1, alpha=1) -> torch.Tensor:
    """aten.addmm.default -- beta*self + alpha*(mat1 @ mat2), self broadcast to [M,N]."""
    _require_cuda(self, mat1, mat2)
    if mat1.dim() != 2 or mat2.dim() != 2:
        raise RuntimeError("mat1 and mat2 must be matrices")
    M, K = mat1.shape
    K2, N = mat2.shape
    if K != K2:
        raise RuntimeError(f"mat1 and mat2 shapes cannot be multiplied ({M}x{K} and {K2}x{N})")
    return _gemm(mat1, mat2, self, 1, M, N, K, (0, mat1.stride(0), mat1.stride(1)), (0, mat2.stride(0), mat2.stride(1)), float(alpha), float(beta), [M, N])


def bmm_default(self: torch.Tensor, mat2: torch.Tensor) -> torch.Tensor:
    """aten.bmm.default -- batched [B,M,K] @ [B,K,N]."""
    _require_cuda(self, mat2)
    if self.dim() != 3 or mat2.dim() != 3:
        raise RuntimeError("batch1 and batch2 must be 3D tensors")
    B, M, K = self.shape
    B2, K2, N = mat2.shape
    if B != B2 or K != K2:
        raise RuntimeError(f"Expected size for first two dimensions of batch2 tensor to be: [{B}, {K}] but got: [{B2}, {K2}].")
    return _gemm(self, mat2, None, B, M, N, K, tuple(self.stride()), tuple(mat2.stride()), 1.0, 0.0, [B, M, N])


# op spec name (as BackendBench/opregistry.py spells it) -> host function
OP_TABLE = {
    "relu.default": relu,
    "add.Tensor": add_Tensor,
    "mul.Tensor": mul_Tensor,
    "where.self": where_self,
    "_softmax.default": _softmax_default,
    "_log_softmax.default": _log_softmax_default,
    "sum.dim_IntList": sum_dim_IntList,
    "native_layer_norm.default": native_layer_norm_default,
    "argmax.default": argmax_default,
    "embedding.default": embedding_default,
    "index_select.default": index_select_default,
    "gather.default": gather_default,
    "scatter_add.default": scatter_add_default,
    "mm.default": mm_default,
    "addmm.default": addmm_default,
    "bmm.default": bmm_default,
}
