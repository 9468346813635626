"""`torch.ops.b200.<op>`: the kernels of libb200ops.so as PyTorch operators of their own.

BackendBench overrides an aten operator by registering a Python callable for a dispatch key
(BackendBench/__init__.py:81-91: `lib.impl(name, fn, "CUDA")`). A bare Python callable has no
schema of its own, cannot be traced by shape (FakeTensor / `torch.export` / `torch.compile`
see an opaque function) and cannot be called as `torch.ops.<ns>.<op>`. This module gives every
host wrapper of `ops.py` / `backward.py` exactly that: a schema in the `b200` namespace with
the aten overload's argument list, the C-ABI-backed wrapper as its CUDA kernel, and a fake
(shape / dtype / stride only) kernel, so the plugin files can hand the harness an operator
instead of a function. The plugin implementations call these operators.

There is still no CPU path: the CPU kernel registered here is the same wrapper, which raises
`UnsupportedByB200` for host tensors. The operators carry no autograd formula; under the
aten override the autograd key is aten's own (the override sits below it), and the backward
operators of this package are registered as operators of their own.
"""

from __future__ import annotations

import torch

from . import backward as _bw
from . import ops as _ops

_aten = torch.ops.aten

# name in the b200 namespace -> (schema after the name, (module, attribute) of the host wrapper,
# aten overload it mirrors)
OPERATORS = {
    "relu": ("(Tensor self) -> Tensor", (_ops, "relu"), _aten.relu.default),
    "add": ("(Tensor self, Tensor other, *, Scalar alpha=1) -> Tensor", (_ops, "add_Tensor"), _aten.add.Tensor),
    "mul": ("(Tensor self, Tensor other) -> Tensor", (_ops, "mul_Tensor"), _aten.mul.Tensor),
    "where": ("(Tensor condition, Tensor self, Tensor other) -> Tensor", (_ops, "where_self"), _aten.where.self),
    "softmax": ("(Tensor self, int dim, bool half_to_float) -> Tensor", (_ops, "_softmax_default"), _aten._softmax.default),
    "log_softmax": ("(Tensor self, int dim, bool half_to_float) -> Tensor", (_ops, "_log_softmax_default"), _aten._log_softmax.default),
    "sum": ("(Tensor self, int[1]? dim, bool keepdim=False, *, ScalarType? dtype=None) -> Tensor", (_ops, "sum_dim_IntList"), _aten.sum.dim_IntList),
    "layer_norm": ("(Tensor input, SymInt[] normalized_shape, Tensor? weight, Tensor? bias, float eps) -> (Tensor, Tensor, Tensor)", (_ops, "native_layer_norm_default"), _aten.native_layer_norm.default),
    "argmax": ("(Tensor self, int? dim=None, bool keepdim=False) -> Tensor", (_ops, "argmax_default"), _aten.argmax.default),
    "embedding": ("(Tensor weight, Tensor indices, SymInt padding_idx=-1, bool scale_grad_by_freq=False, bool sparse=False) -> Tensor", (_ops, "embedding_default"), _aten.embedding.default),
    "index_select": ("(Tensor self, int dim, Tensor index) -> Tensor", (_ops, "index_select_default"), _aten.index_select.default),
    "gather": ("(Tensor self, int dim, Tensor index, *, bool sparse_grad=False) -> Tensor", (_ops, "gather_default"), _aten.gather.default),
    "scatter_add": ("(Tensor self, int dim, Tensor index, Tensor src) -> Tensor", (_ops, "scatter_add_default"), _aten.scatter_add.default),
    "mm": ("(Tensor self, Tensor mat2) -> Tensor", (_ops, "mm_default"), _aten.mm.default),
    "addmm": ("(Tensor self, Tensor mat1, Tensor mat2, *, Scalar beta=1, Scalar alpha=1) -> Tensor", (_ops, "addmm_default"), _aten.addmm.default),
    "bmm": ("(Tensor self, Tensor mat2) -> Tensor", (_ops, "bmm_default"), _aten.bmm.default),
    # backward neighbours
    "softmax_backward": ("(Tensor grad_output, Tensor output, int dim, ScalarType input_dtype) -> Tensor", (_bw, "_softmax_backward_data_default"), _aten._softmax_backward_data.default),
    "log_softmax_backward": ("(Tensor grad_output, Tensor output, int dim, ScalarType input_dtype) -> Tensor", (_bw, "_log_softmax_backward_data_default"), _aten._log_softmax_backward_data.default),
    "layer_norm_backward": ("(Tensor grad_out, Tensor input, SymInt[] normalized_shape, Tensor mean, Tensor rstd, Tensor? weight, Tensor? bias, bool[3] output_mask) -> (Tensor?, Tensor?, Tensor?)", (_bw, "native_layer_norm_backward_default"), _aten.native_layer_norm_backward.default),
    "embedding_backward": ("(Tensor grad_output, Tensor indices, SymInt num_weights, SymInt padding_idx, bool scale_grad_by_freq) -> Tensor", (_bw, "embedding_dense_backward_default"), _aten.embedding_dense_backward.default),
}

# aten spec name ("add.Tensor") -> name in the b200 namespace
ATEN_TO_B200 = {str(a).split("aten.", 1)[-1]: name for name, (_, _, a) in OPERATORS.items()}

_library = torch.library.Library("b200", "DEF")  # lives as long as the module


def _fake_from(aten_op):
    def fake(*args, **kwargs):
        # under FakeTensorMode the aten overload runs its meta kernel: the result has the
        # shape, dtype, strides and device aten would give, which is what the real kernel returns
        return aten_op(*args, **kwargs)

    return fake


def _kernel_for(module, attr):
    def kernel(*args, **kwargs):
        # looked up per call, so whoever wraps or replaces the host wrapper (a call counter
        # in a test, a profiler shim) is seen by the operator too
        return getattr(module, attr)(*args, **kwargs)

    kernel.__name__ = attr
    return kernel


def host_wrapper(name: str):
    module, attr = OPERATORS[name][1]
    return getattr(module, attr)


for _name, (_schema, (_module, _attr), _aten_op) in OPERATORS.items():
    _library.define(_name + _schema)
    _library.impl(_name, _kernel_for(_module, _attr), "CUDA")
    _library.impl(_name, _kernel_for(_module, _attr), "CPU")  # raises UnsupportedByB200: there is no host path
    torch.library.register_fake(f"b200::{_name}", _fake_from(_aten_op), lib=_library)


def operator(name: str):
    """The `b200::<name>` overload object (`torch.ops.b200.<name>.default`)."""
    return getattr(torch.ops.b200, name).default


def for_aten(spec_name: str):
    """The b200 operator that mirrors aten overload `spec_name` (e.g. "add.Tensor")."""
    return operator(ATEN_TO_B200[spec_name])


def entry(name: str):
    """The callable a plugin file exports for `b200::<name>`: the operator itself, except that
    a Python number in a Tensor slot (aten wraps such numbers before it dispatches; somebody
    calling the plugin directly may not have) goes to the host wrapper, which takes numbers
    as they are."""
    op = operator(name)
    fn = _kernel_for(*OPERATORS[name][1])
    slots = [i for i, a in enumerate(op._schema.arguments) if not a.kwarg_only and str(a.type) == "Tensor"]

    def run(*args, **kwargs):
        for i in slots:
            if i < len(args) and not isinstance(args[i], torch.Tensor):
                return fn(*args, **kwargs)
        return op(*args, **kwargs)

    run.__name__ = f"b200_{name}"
    return run
