"""`torch.ops.b200.*` without a GPU: every operator has the schema of the aten overload it
mirrors, a fake kernel that gives aten's shapes / dtypes for CUDA fake tensors, and no host
path (BackendBench/__init__.py:81-91 registers bare callables; these are operators)."""

import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

from backendbench_b200 import custom_ops
from backendbench_b200.backends import B200Backend
from backendbench_b200.ops import UnsupportedByB200


def _args_of(schema):
    return [(a.name, str(a.type), a.kwarg_only) for a in schema.arguments]


def test_every_operator_mirrors_its_aten_schema():
    assert len(custom_ops.OPERATORS) == 20
    for name, (_, _, aten_op) in custom_ops.OPERATORS.items():
        mine = custom_ops.operator(name)._schema
        assert mine.name == f"b200::{name}"
        assert _args_of(mine) == _args_of(aten_op._schema), name  # same names, types and keyword-only split
        if name == "layer_norm_backward":  # aten says Tensor and hands back undefined tensors for masked-out gradients; here they are None, and the schema says so
            assert [str(r.type) for r in mine.returns] == ["Optional[Tensor]"] * 3
        else:
            assert [str(r.type) for r in mine.returns] == [str(r.type) for r in aten_op._schema.returns], name
    assert custom_ops.for_aten("add.Tensor") is torch.ops.b200.add.default


def test_fake_kernels_give_atens_shapes_for_cuda_fake_tensors():
    with FakeTensorMode():
        x = torch.empty(8, 16, device="cuda", dtype=torch.bfloat16)
        w = torch.empty(100, 16, device="cuda")
        i = torch.empty(5, dtype=torch.int64, device="cuda")
        idx = torch.empty(8, 16, dtype=torch.int64, device="cuda")
        assert torch.ops.b200.relu(x).shape == (8, 16) and torch.ops.b200.relu(x).device.type == "cuda"
        out, mean, rstd = torch.ops.b200.layer_norm(x, [16], None, None, 1e-5)
        assert out.dtype == torch.bfloat16 and mean.shape == (8, 1) and rstd.dtype == torch.float32
        assert torch.ops.b200.sum(x, [-1]).shape == (8,) and torch.ops.b200.sum(x, [0], True).shape == (1, 16)
        assert torch.ops.b200.argmax(x, -1).dtype == torch.int64 and torch.ops.b200.argmax(x).shape == ()
        assert torch.ops.b200.add(x, x.float(), alpha=2).dtype == torch.float32
        assert torch.ops.b200.embedding(w, i).shape == (5, 16) and torch.ops.b200.index_select(w, 0, i).shape == (5, 16)
        assert torch.ops.b200.gather(x, 0, idx).shape == (8, 16) and torch.ops.b200.scatter_add(x, 0, idx, x).shape == (8, 16)
        assert torch.ops.b200.mm(x, x.t()).shape == (8, 8) and torch.ops.b200.addmm(x[:, :8], x, x.t()).shape == (8, 8)
        assert torch.ops.b200.bmm(x[None], x.t()[None]).shape == (1, 8, 8)
        assert torch.ops.b200.softmax(x, -1, False).dtype == torch.bfloat16
        assert torch.ops.b200.where(x > 0, x, x).shape == (8, 16)
        dx, dw, db = torch.ops.b200.layer_norm_backward(x, x, [16], mean, rstd, None, None, [True, False, False])
        assert dx.shape == (8, 16) and dw is None and db is None


def test_there_is_no_host_path_and_the_plugins_call_the_operators():
    with pytest.raises(UnsupportedByB200, match="no CPU path"):
        torch.ops.b200.relu(torch.randn(4))
    backend = B200Backend()
    impl = backend[torch.ops.aten.mul.Tensor]
    with pytest.raises(UnsupportedByB200):
        impl(torch.randn(4), torch.randn(4))  # tensors: through torch.ops.b200.mul
    with pytest.raises(UnsupportedByB200):
        impl(torch.randn(4), 2.0)  # a Python number in a Tensor slot: straight to the host wrapper, same refusal
