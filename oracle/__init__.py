"""CPU oracle for the CUDA kernels -- TEST INFRASTRUCTURE, not product code.

Only tests/, `__graft_entry__.smoke()` and bench.py's CPU-baseline leg may import this
package; the product (`backendbench_b200`) never does. It wraps `liboracle.so`
(oracle_ops.c, a plain-C restatement of the sixteen aten overloads the reference
evaluates at BackendBench/eval.py:100) and exposes one entry point per overload that
takes and returns CPU torch tensors with aten's argument conventions. torch is used as a
container only: all arithmetic happens in the C functions.

Pinned by tests/golden/ (vectors from the reference harness over aten CPU).
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int64, c_uint8, c_uint16, c_void_p

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile oracle_ops.c with gcc (a second or two)."""
    src = os.path.join(_HERE, "oracle_ops.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.oracle_index_select.restype = c_int64
        _lib.oracle_gather.restype = c_int64
        _lib.oracle_scatter_add.restype = c_int64
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(c_void_p)


def _i64(xs):
    return (c_int64 * max(len(xs), 1))(*[int(x) for x in xs])


# ------------------------------------------------------------------ dtype plumbing
def widen(t: torch.Tensor) -> np.ndarray:
    """Contiguous fp32 numpy copy of a float tensor (bf16/f16 widen exactly)."""
    t = t.detach().cpu().contiguous()
    L = lib()
    if t.dtype == torch.float32:
        return t.numpy().copy()
    raw = t.view(torch.int16).numpy().view(np.uint16)
    out = np.empty(raw.shape, dtype=np.float32)
    fn = L.oracle_widen_bf16 if t.dtype == torch.bfloat16 else L.oracle_widen_f16
    fn(_ptr(raw), _ptr(out), c_int64(raw.size))
    return out


def narrow(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """fp32 numpy -> tensor of `dtype`, one round-to-nearest-even."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if dtype == torch.float32:
        return torch.from_numpy(a.copy())
    out = np.empty(a.shape, dtype=np.uint16)
    fn = lib().oracle_round_bf16 if dtype == torch.bfloat16 else lib().oracle_round_f16
    fn(_ptr(a), _ptr(out), c_int64(a.size))
    return torch.from_numpy(out.view(np.int16)).view(dtype)


def _bytes_view(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    return t.view(torch.uint8).numpy() if t.dim() else t.reshape(1).view(torch.uint8).numpy()


def _from_bytes(a: np.ndarray, shape, dtype) -> torch.Tensor:
    if a.size == 0:
        return torch.empty(list(shape), dtype=dtype)
    return torch.from_numpy(a.copy()).view(dtype).reshape(shape)


def _norm(dim, nd):
    return dim % max(nd, 1)


def _prod(xs):
    p = 1
    for x in xs:
        p *= int(x)
    return p


# ------------------------------------------------------------------ operators
def relu(x):
    a = widen(x)
    out = np.empty_like(a)
    lib().oracle_relu(_ptr(a), _ptr(out), c_int64(a.size))
    return narrow(out, x.dtype).reshape(x.shape)


def _binary(fn_name, x, y, alpha=None):
    res_dtype = torch.result_type(x, y)
    if not isinstance(y, torch.Tensor):
        y = torch.tensor(y, dtype=res_dtype)
    shape = torch.broadcast_shapes(x.shape, y.shape)
    a = np.ascontiguousarray(np.broadcast_to(widen(x), shape))
    b = np.ascontiguousarray(np.broadcast_to(widen(y), shape))
    out = np.empty(shape, dtype=np.float32)
    if fn_name == "add":
        lib().oracle_add(_ptr(a), _ptr(b), _ptr(out), c_int64(out.size), c_float(alpha))
    else:
        lib().oracle_mul(_ptr(a), _ptr(b), _ptr(out), c_int64(out.size))
    return narrow(out, res_dtype).reshape(shape)


def add(x, y, *, alpha=1):
    return _binary("add", x, y, float(alpha))


def mul(x, y):
    return _binary("mul", x, y)


def where(cond, x, y):
    res_dtype = torch.result_type(x, y)
    shape = torch.broadcast_shapes(cond.shape, x.shape, y.shape)
    if x.dtype != res_dtype:
        x = narrow(widen(x), res_dtype).reshape(x.shape)
    if y.dtype != res_dtype:
        y = narrow(widen(y), res_dtype).reshape(y.shape)
    es = x.element_size()
    c = np.ascontiguousarray(np.broadcast_to(cond.detach().cpu().to(torch.uint8).numpy(), shape))
    xb = np.ascontiguousarray(np.broadcast_to(_bytes_view(x).reshape(tuple(x.shape) + (es,)), tuple(shape) + (es,)))
    yb = np.ascontiguousarray(np.broadcast_to(_bytes_view(y).reshape(tuple(y.shape) + (es,)), tuple(shape) + (es,)))
    out = np.empty_like(xb)
    lib().oracle_where(_ptr(c), _ptr(xb), _ptr(yb), _ptr(out), c_int64(c.size), c_int(es))
    return _from_bytes(out.reshape(-1), shape, res_dtype)


def _split(shape, dim):
    shape = list(shape) or [1]
    return _prod(shape[:dim]), shape[dim], _prod(shape[dim + 1 :])


def softmax(x, dim, half_to_float=False, log=False):
    dim = _norm(dim, x.dim())
    a = widen(x)
    out = np.empty_like(a)
    o, d, i = _split(x.shape, dim)
    if a.size:
        lib().oracle_softmax(_ptr(a), _ptr(out), c_int64(o), c_int64(d), c_int64(i), c_int(1 if log else 0))
    return narrow(out, torch.float32 if half_to_float else x.dtype).reshape(x.shape)


def log_softmax(x, dim, half_to_float=False):
    return softmax(x, dim, half_to_float, log=True)


def softmax_backward(grad, output, dim, input_dtype, log=False):
    dim = _norm(dim, grad.dim())
    g, y = widen(grad), widen(output)
    out = np.empty_like(g)
    o, d, i = _split(grad.shape, dim)
    if g.size:
        lib().oracle_softmax_backward(_ptr(g), _ptr(y), _ptr(out), c_int64(o), c_int64(d), c_int64(i), c_int(1 if log else 0))
    return narrow(out, input_dtype).reshape(grad.shape)


def log_softmax_backward(grad, output, dim, input_dtype):
    return softmax_backward(grad, output, dim, input_dtype, log=True)


def sum_dims(x, dim=None, keepdim=False, *, dtype=None):
    nd = x.dim()
    dims = list(range(nd)) if dim is None or (isinstance(dim, (list, tuple)) and not dim) else [_norm(d, nd) for d in ([dim] if isinstance(dim, int) else dim)]
    if nd == 0:
        dims = []
    kept = [d for d in range(nd) if d not in dims]
    a = np.ascontiguousarray(np.transpose(widen(x), kept + dims)) if nd else widen(x).reshape(1)
    outer, red = _prod(x.shape[d] for d in kept), _prod(x.shape[d] for d in dims)
    out = np.zeros(max(outer, 1) if outer else 0, dtype=np.float32)
    if outer:
        lib().oracle_sum(_ptr(a), _ptr(out), c_int64(outer), c_int64(red), c_int64(1))
    shape = [(1 if d in dims else s) for d, s in enumerate(x.shape)] if keepdim else [x.shape[d] for d in kept]
    return narrow(out, dtype or x.dtype).reshape(shape)


def layer_norm(x, normalized_shape, weight=None, bias=None, eps=1e-5, stat_dtype=torch.float32):
    k = len(normalized_shape)
    lead = list(x.shape[: x.dim() - k])
    rows, cols = _prod(lead), _prod(normalized_shape)
    a = widen(x)
    w = widen(weight) if weight is not None else None
    b = widen(bias) if bias is not None else None
    y = np.empty_like(a)
    mean = np.empty(rows, dtype=np.float32)
    rstd = np.empty(rows, dtype=np.float32)
    if rows:
        lib().oracle_layer_norm(_ptr(a), _ptr(w) if w is not None else None, _ptr(b) if b is not None else None, _ptr(y), _ptr(mean), _ptr(rstd), c_int64(rows), c_int64(cols), c_double(eps))
    stat_shape = lead + [1] * k
    return narrow(y, x.dtype).reshape(x.shape), narrow(mean, stat_dtype).reshape(stat_shape), narrow(rstd, stat_dtype).reshape(stat_shape)


def embedding_backward(grad_output, indices, num_weights, padding_idx=-1, scale_grad_by_freq=False):
    if scale_grad_by_freq:
        raise NotImplementedError("scale_grad_by_freq")
    row_len = grad_output.shape[-1] if grad_output.dim() else 1
    g = widen(grad_output).reshape(-1, row_len) if grad_output.numel() else np.zeros((0, row_len), dtype=np.float32)
    idx = np.ascontiguousarray(indices.reshape(-1).to(torch.int64).numpy())
    out = np.zeros((num_weights, row_len), dtype=np.float32)
    if out.size:
        lib().oracle_embedding_backward.restype = c_int64
        bad = lib().oracle_embedding_backward(_ptr(np.ascontiguousarray(g)), _ptr(idx), _ptr(out), c_int64(idx.size), c_int64(num_weights), c_int64(row_len), c_int64(padding_idx))
        if bad:
            raise IndexError("index out of range in embedding_dense_backward")
    return narrow(out, grad_output.dtype)


def layer_norm_backward(grad_out, input, normalized_shape, mean, rstd, weight, bias, output_mask):
    cols = _prod(normalized_shape)
    rows = input.numel() // max(cols, 1)
    dy, x = widen(grad_out), widen(input)
    mu, rs = widen(mean).reshape(-1), widen(rstd).reshape(-1)
    w = widen(weight) if weight is not None else None
    dx = np.empty_like(x) if output_mask[0] else None
    dw = np.empty(cols, dtype=np.float32) if output_mask[1] else None
    db = np.empty(cols, dtype=np.float32) if output_mask[2] else None
    if cols:
        lib().oracle_layer_norm_backward(_ptr(dy), _ptr(x), _ptr(mu), _ptr(rs), _ptr(w) if w is not None else None, _ptr(dx) if dx is not None else None,
                                         _ptr(dw) if dw is not None else None, _ptr(db) if db is not None else None, c_int64(rows), c_int64(cols))
    wb_dtype = weight.dtype if weight is not None else input.dtype
    return (narrow(dx, input.dtype).reshape(input.shape) if dx is not None else None,
            narrow(dw, wb_dtype).reshape(list(normalized_shape)) if dw is not None else None,
            narrow(db, wb_dtype).reshape(list(normalized_shape)) if db is not None else None)


def argmax(x, dim=None, keepdim=False):
    a = widen(x)
    if dim is None:
        o, d, i = 1, a.size, 1
        shape = [1] * x.dim() if keepdim else []
    else:
        dim = _norm(dim, x.dim())
        o, d, i = _split(x.shape, dim)
        shape = [(1 if k == dim else s) for k, s in enumerate(x.shape)] if keepdim else [s for k, s in enumerate(x.shape) if k != dim]
    out = np.empty(o * i, dtype=np.int64)
    if out.size:
        lib().oracle_argmax(_ptr(a), _ptr(out), c_int64(o), c_int64(d), c_int64(i))
    return torch.from_numpy(out).reshape(shape)


def index_select(x, dim, index):
    dim = _norm(dim, x.dim())
    o, d, i = _split(x.shape, dim)
    es = x.element_size()
    xb = _bytes_view(x)
    idx = index.detach().cpu().to(torch.int64).contiguous().numpy().reshape(-1)
    out = np.empty(o * idx.size * i * es, dtype=np.uint8)
    bad = 0
    if out.size:
        bad = lib().oracle_index_select(_ptr(xb), _ptr(idx), _ptr(out), c_int64(o), c_int64(d), c_int64(i * es), c_int64(idx.size))
    if bad:
        raise IndexError("index out of range in self")
    shape = list(x.shape)
    shape[dim] = idx.size
    return _from_bytes(out, shape, x.dtype)


def embedding(weight, indices, padding_idx=-1, scale_grad_by_freq=False, sparse=False):
    flat = index_select(weight, 0, indices.reshape(-1))
    return flat.reshape(list(indices.shape) + list(weight.shape[1:]))


def gather(x, dim, index, *, sparse_grad=False):
    dim = _norm(dim, x.dim())
    x = x.detach().cpu().contiguous()
    es = x.element_size()
    idx = index.detach().cpu().contiguous().numpy()
    out = np.empty(idx.size * es, dtype=np.uint8)
    nd = max(x.dim(), 1)
    bad = 0
    if idx.size:
        bad = lib().oracle_gather(_ptr(_bytes_view(x)), _ptr(idx), _ptr(out), c_int(nd), _i64(list(index.shape) or [1]), _i64(list(x.stride()) or [1]), c_int64((list(x.shape) or [1])[dim]), c_int(dim), c_int(es))
    if bad:
        raise RuntimeError("index out of bounds")
    return _from_bytes(out, index.shape, x.dtype)


def scatter_add(x, dim, index, src):
    dim = _norm(dim, x.dim())
    out = widen(x)
    idx = index.detach().cpu().contiguous().numpy()
    s = widen(src)
    nd = max(x.dim(), 1)
    bad = 0
    if idx.size:
        bad = lib().oracle_scatter_add(_ptr(out), _ptr(idx), _ptr(s), c_int(nd), _i64(list(x.shape) or [1]), _i64(list(index.shape) or [1]), _i64(list(src.shape) or [1]), c_int(dim))
    if bad:
        raise RuntimeError("index out of bounds")
    return narrow(out, x.dtype).reshape(x.shape)


def _gemm(a, b, bias, batch, M, N, K, alpha, beta):
    A, B = widen(a), widen(b)
    C = np.empty(batch * M * N, dtype=np.float32)
    sbm = sbn = 0
    bb = None
    if bias is not None:
        bb = np.ascontiguousarray(np.broadcast_to(widen(bias), (M, N)))
        sbm, sbn = N, 1
    if C.size:
        lib().oracle_gemm(_ptr(A), _ptr(B), _ptr(bb) if bb is not None else None, _ptr(C), c_int64(batch), c_int64(M), c_int64(N), c_int64(K), c_int64(sbm), c_int64(sbn), c_double(alpha), c_double(beta))
    return narrow(C, a.dtype)


def mm(a, b):
    return _gemm(a, b, None, 1, a.shape[0], b.shape[1], a.shape[1], 1.0, 0.0).reshape(a.shape[0], b.shape[1])


def addmm(bias, a, b, *, beta=1, alpha=1):
    return _gemm(a, b, bias, 1, a.shape[0], b.shape[1], a.shape[1], float(alpha), float(beta)).reshape(a.shape[0], b.shape[1])


def bmm(a, b):
    return _gemm(a, b, None, a.shape[0], a.shape[1], b.shape[2], a.shape[2], 1.0, 0.0).reshape(a.shape[0], a.shape[1], b.shape[2])


def compare(ref, res, rtol=1e-2, atol=1e-2):
    """(mismatches, max_abs, max_rel) of two same-shape tensors: the harness's closeness
    rule and error metrics (BackendBench/eval.py:68-90, utils.py:185-242)."""
    a, b = widen(ref.float()), widen(res.float())
    out = (c_double * 3)()
    lib().oracle_compare(_ptr(a), _ptr(b), c_int64(a.size), c_double(rtol), c_double(atol), out)
    return int(out[0]), float(out[1]), float(out[2])


# spec name -> oracle function with the aten overload's calling convention
ORACLE = {
    "relu.default": relu,
    "add.Tensor": add,
    "mul.Tensor": mul,
    "where.self": where,
    "_softmax.default": softmax,
    "_log_softmax.default": log_softmax,
    "_softmax_backward_data.default": softmax_backward,
    "_log_softmax_backward_data.default": log_softmax_backward,
    "sum.dim_IntList": sum_dims,
    "native_layer_norm.default": layer_norm,
    "native_layer_norm_backward.default": layer_norm_backward,
    "embedding_dense_backward.default": embedding_backward,
    "argmax.default": argmax,
    "embedding.default": embedding,
    "index_select.default": index_select,
    "gather.default": gather,
    "scatter_add.default": scatter_add,
    "mm.default": mm,
    "addmm.default": addmm,
    "bmm.default": bmm,
}


def run(op_name: str, args, kwargs=None):
    """Evaluate the oracle for a spec name on CPU copies of (args, kwargs)."""
    cpu = [a.detach().cpu() if isinstance(a, torch.Tensor) else a for a in args]
    kw = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in (kwargs or {}).items()}
    return ORACLE[op_name](*cpu, **kw)
