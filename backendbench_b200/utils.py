"""Name mapping, case (de)serialisation and error metrics of the evaluation path.

Mirrors the part of BackendBench/utils.py the hot path uses: operator <-> folder names
(utils.py:252-345), the `T([shape], dtype[, stride])` case grammar (utils.py:100-182),
`compute_errors` (utils.py:185-242) and the stream-creation screen `uses_cuda_stream`
(utils.py:50-97). The LLM file helpers of that module are not part of this path.
"""

from __future__ import annotations

import ast
import gc
import inspect
import logging
import math
import re
import textwrap

import torch

logger = logging.getLogger(__name__)

OP_NAME_ESCAPE_SEQUENCE = "__"

dtype_abbrs = {
    torch.bfloat16: "bf16",
    torch.float64: "f64",
    torch.float32: "f32",
    torch.float16: "f16",
    torch.complex32: "c32",
    torch.complex64: "c64",
    torch.complex128: "c128",
    torch.int8: "i8",
    torch.int16: "i16",
    torch.int32: "i32",
    torch.int64: "i64",
    torch.bool: "b8",
    torch.uint8: "u8",
}
dtype_abbrs_parsing = {abbr: dt for dt, abbr in dtype_abbrs.items()}
_FLOATING = (torch.float16, torch.bfloat16, torch.float32, torch.float64)

# ------------------------------------------------------------------ operator names


def op_name_to_folder_name(op_name: str) -> str:
    """"add.Tensor" -> "add__Tensor": dots are not valid in Python identifiers."""
    return op_name.replace(".", OP_NAME_ESCAPE_SEQUENCE)


def folder_name_to_op_name(folder_name: str) -> str:
    """Inverse of op_name_to_folder_name. Escape sequences are matched from the RIGHT so
    the in-place spelling "add___Tensor" becomes "add_.Tensor", not "add._Tensor"."""
    rev = folder_name[::-1].replace(OP_NAME_ESCAPE_SEQUENCE[::-1], ".")
    return rev[::-1]


def is_overload_folder_name(folder_name: str) -> bool:
    return OP_NAME_ESCAPE_SEQUENCE in folder_name


def extract_operator_name(op_str: str) -> str:
    """"aten.add.Tensor" -> "add.Tensor"; names without the prefix pass through."""
    return op_str.split("aten.")[-1] if "aten." in op_str else op_str


def get_pytorch_op(op_name: str):
    """"add.Tensor" | "relu.default" | "relu" -> the OpOverload under torch.ops.aten, or None."""
    base, _, overload = op_name.partition(".")
    try:
        return getattr(getattr(torch.ops.aten, base), overload or "default")
    except AttributeError:
        logger.warning(f"Could not find PyTorch operation for {op_name}")
        return None


# ------------------------------------------------------------------ case grammar


def _deserialize_tensor(size, dtype, stride=None, device="cuda"):
    """T(size, dtype[, stride]): floating tensors are U[0,1), integers torch's default range."""
    from torch.testing import make_tensor

    extra = {"low": 0, "high": 1} if dtype in _FLOATING else {}
    if device == "cuda" and not torch.cuda.is_available():
        device = "cpu"
    if stride is None:
        return make_tensor(size, dtype=dtype, device=device, **extra)
    extent = 1 + sum((n - 1) * s for n, s in zip(size, stride))
    return make_tensor(extent, dtype=dtype, device=device, **extra).as_strided(size, stride)


def _serialize_value(value) -> str:
    if isinstance(value, torch.Tensor):
        head = f"T({list(value.shape)}, {dtype_abbrs[value.dtype]}"
        return head + (")" if value.is_contiguous() else f", {list(value.stride())})")
    if isinstance(value, list):
        return "[" + ", ".join(_serialize_value(v) for v in value) + "]"
    return repr(value)


def serialize_args(args, kwargs) -> str:
    """`((arg, ...,), {'key': val, ...})` with tensors spelt T([shape], dtype[, stride])."""
    if args is None or kwargs is None:
        return "None"
    pos = ", ".join(_serialize_value(a) for a in args)
    kw = ", ".join(f"'{k}': {_serialize_value(v)}" for k, v in kwargs.items())
    return f"({'(' + pos + ',)' if pos else '()'}, {{{kw}}})"


def deserialize_args(inps: str):
    """Parse a serialised case back into (args, kwargs) with freshly generated tensors."""
    text = inps.strip().strip("'")
    for abbr in dtype_abbrs_parsing:
        text = text.replace(f"'{abbr}'", abbr)
    text = re.sub(r'["\']torch\.device\((.*?)\)["\']', r"torch.device(\1)", text)
    env = {"T": _deserialize_tensor, "th": torch, "torch": torch, "inf": math.inf, **dtype_abbrs_parsing}
    return eval(text.strip().strip("'").strip('"'), env)


# ------------------------------------------------------------------ error metrics


def compute_errors(ref, res, eps=1e-10):
    """(max abs error, max rel error) of `res` against `ref`; (None, None) when undefined.

    rel = |ref - res| / (|ref| + eps) after conversion to fp32; tuples/lists report the
    maximum over their tensor members. Host formula -- the CUDA evaluation path gets the
    same two numbers from the fused device pass in `backendbench_b200.eval`.
    """
    if isinstance(ref, torch.Tensor) and isinstance(res, torch.Tensor):
        if ref.shape != res.shape or (ref.is_sparse and res.is_sparse):
            return None, None
        if ref.numel() == 0 and res.numel() == 0:
            return 0.0, 0.0
        r, s = ref.float(), res.float()
        diff = (r - s).abs()
        return diff.max().item(), (diff / (r.abs() + eps)).max().item()
    if isinstance(ref, (list, tuple)) and isinstance(res, (list, tuple)):
        if len(ref) != len(res):
            return None, None
        if not any(isinstance(x, torch.Tensor) for x in ref) or not any(isinstance(x, torch.Tensor) for x in res):
            return None, None
        pairs = [compute_errors(r, s, eps) for r, s in zip(ref, res)]
        pairs = [p for p in pairs if p[0] is not None and p[1] is not None]
        if not pairs:
            return None, None
        return max(p[0] for p in pairs), max(p[1] for p in pairs)
    return None, None


# ------------------------------------------------------------------ stream screen

_STREAM_PATTERNS = [
    r"torch\.cuda\.Stream\(",
    r"cupy\.cuda\.Stream\(",
    r"cuda\.Stream\(",
    r"pycuda.*Stream\(",
    r"\bStream\(",
    r"make_stream\(",
    r"create_stream\(",
]


def uses_cuda_stream(func) -> bool:
    """True when the source of `func` creates CUDA streams (such kernels are not evaluated:
    timing on the current stream would not see their work)."""
    try:
        source = inspect.getsource(func)
        tree = ast.parse(textwrap.dedent(source))
    except (TypeError, OSError, IndentationError, SyntaxError):
        return False  # builtins / OpOverloads have no source, hence create no streams
    if any(re.search(p, source, re.IGNORECASE) for p in _STREAM_PATTERNS):
        return True
    for node in ast.walk(tree):
        if isinstance(node, ast.Call):
            f = node.func
            if getattr(f, "attr", None) == "Stream" or getattr(f, "id", None) == "Stream":
                return True
    return False


def cleanup_memory_and_gpu():
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
