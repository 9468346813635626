"""`torch.ops.b200.<op>`: the C-ABI-backed host wrappers registered as PyTorch operators of
their own (schema, CUDA kernel, fake kernel). Checked bit for bit against the direct ctypes
path, under FakeTensorMode, and under the aten override (BackendBench/__init__.py:81-91),
where an implementation that ended up in the aten operator it replaces would recurse."""

import pytest
import torch

import backendbench_b200 as bb
from backendbench_b200 import _abi, custom_ops, ops
from backendbench_b200.backends import KERNELS_DIR, B200Backend
from backendbench_b200.cases import named_cases, scaled_down
from backendbench_b200.opregistry import get_operator
from conftest import bits_equal

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _tup(x):
    return tuple(x) if isinstance(x, (tuple, list)) else (x,)


def test_relu_operator_equals_the_ctypes_call_bit_for_bit():
    x = torch.randn(1000, 333, device=DEV)
    x[5, 7] = float("nan")
    direct = torch.empty_like(x)
    shape, stride = _abi.i64_array([x.numel()]), _abi.i64_array([1])
    _abi.check(_abi.lib().b200_relu(x.data_ptr(), direct.data_ptr(), 1, shape, stride, _abi.F32, torch.cuda.current_stream().cuda_stream), "b200_relu")
    got = torch.ops.b200.relu(x)
    assert bits_equal(direct, got) and bits_equal(got, torch.relu(x))
    assert str(torch.ops.b200.relu.default._schema) == "b200::relu(Tensor self) -> Tensor"


def test_every_operator_matches_the_host_wrapper_and_its_fake_kernel():
    from torch._subclasses.fake_tensor import FakeTensorMode

    backend = B200Backend()
    seen = set()
    for case in named_cases():
        small = scaled_down(case, 64)
        args, kwargs = small.build(DEV)
        name = custom_ops.ATEN_TO_B200[small.op]
        seen.add(name)
        via_op = getattr(torch.ops.b200, name)(*args, **kwargs)
        via_wrapper = ops.OP_TABLE[small.op](*args, **kwargs)
        via_plugin = backend[get_operator(small.op)](*args, **kwargs)
        for a, b, c in zip(_tup(via_op), _tup(via_wrapper), _tup(via_plugin)):
            assert bits_equal(a, b) and bits_equal(a, c), small.label()
        with FakeTensorMode() as mode:
            fargs = [mode.from_tensor(a) if isinstance(a, torch.Tensor) else a for a in args]
            fake = getattr(torch.ops.b200, name)(*fargs, **kwargs)
        for f, r in zip(_tup(fake), _tup(via_op)):
            assert f.shape == r.shape and f.dtype == r.dtype and f.device == r.device, (small.label(), f.shape, r.shape, f.dtype, r.dtype)
    ops.check_device_status()
    assert seen == {n for n, (_, _, a) in custom_ops.OPERATORS.items() if "backward" not in n}


def test_plugin_takes_a_python_number_where_aten_would_have_wrapped_it():
    backend = B200Backend()
    x = torch.randn(64, 64, device=DEV)
    assert bits_equal(backend[torch.ops.aten.mul.Tensor](x, 2.0), x * 2.0)
    assert bits_equal(backend[torch.ops.aten.add.Tensor](x, 1.5, alpha=2), torch.add(x, 1.5, alpha=2))


def test_no_host_path_and_no_recursion_under_the_override():
    with pytest.raises(NotImplementedError, match="no CPU path"):
        torch.ops.b200.relu(torch.randn(4))
    x = torch.randn(257, 129, device=DEV)
    want = torch.relu(x)
    with bb.BackendBench.enable(kernel_dir=KERNELS_DIR):
        # aten::relu on CUDA now lands in the plugin -> b200::relu -> the C-ABI; if anything on
        # that path called aten::relu again this would never return
        got = torch.relu(x)
        y = torch.nn.functional.softmax(x @ x.t(), dim=-1)
    assert bits_equal(want, got) and y.shape == (257, 257)
    ops.check_device_status()
