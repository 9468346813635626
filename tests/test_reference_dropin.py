"""Drop-in proof against the reference's own loader, run only where the reference checkout
is present (it does not travel to the GPU box): BackendBench's DirectoryBackend loads the
kernels directory of this package unmodified, and the reference's name/serialisation
helpers agree with ours on the spot."""

import os
import sys

import pytest
import torch

REF = os.environ.get("BACKENDBENCH_REFERENCE", "/root/reference")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "BackendBench")), reason="reference checkout not present")


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, REF)
    try:
        import BackendBench
        from BackendBench import eval as ref_eval
        from BackendBench import utils as ref_utils
        from BackendBench.backends import DirectoryBackend

        yield {"pkg": BackendBench, "eval": ref_eval, "utils": ref_utils, "DirectoryBackend": DirectoryBackend}
    finally:
        sys.path.remove(REF)


def test_reference_directory_backend_loads_our_kernels(ref):
    from backendbench_b200.backends import KERNELS_DIR
    from backendbench_b200.ops import OP_TABLE

    from backendbench_b200.variants import VARIANT_TABLE

    be = ref["DirectoryBackend"](KERNELS_DIR)
    assert len(be.compiled_kernels) == 16 + len(VARIANT_TABLE)
    for spec in list(OP_TABLE) + list(VARIANT_TABLE):
        op = ref["utils"].get_pytorch_op(spec)
        assert op in be and callable(be[op])
        assert not ref["utils"].uses_cuda_stream(be[op])  # the reference would refuse to evaluate it otherwise


def test_reference_and_local_helpers_agree(ref):
    from backendbench_b200 import eval as ev
    from backendbench_b200 import utils

    for name in ["add.Tensor", "relu.default", "add_.Tensor", "_log_softmax.default", "sum.dim_IntList"]:
        folder = ref["utils"].op_name_to_folder_name(name)
        assert utils.op_name_to_folder_name(name) == folder
        assert utils.folder_name_to_op_name(folder) == ref["utils"].folder_name_to_op_name(folder) == name
    args = [torch.zeros(3, 4, dtype=torch.float16).t(), [1, 2]]
    assert utils.serialize_args(args, {"k": 1.5}) == ref["utils"].serialize_args(args, {"k": 1.5})
    g = torch.Generator().manual_seed(0)
    a = torch.randn(64, generator=g)
    b = a + torch.randn(64, generator=g) * 0.01
    assert ev.allclose(a, b) == ref["eval"].allclose(a, b)
    ours, theirs = ev.compare(a, b)[1:], ref["utils"].compute_errors(a, b)
    assert ours[0] == pytest.approx(theirs[0]) and ours[1] == pytest.approx(theirs[1])


def test_reference_eval_accepts_our_result_records(ref):
    """The reference's eval_one_op drives an implementation from our directory through its
    own loop on CPU: the kernel refuses CPU tensors loudly, which the harness records as a
    failed case rather than crashing (BackendBench/eval.py:114-125)."""
    from backendbench_b200.backends import KERNELS_DIR

    be = ref["DirectoryBackend"](KERNELS_DIR)
    op = torch.ops.aten.relu.default

    class Case:
        def __init__(self, a):
            self.args, self.kwargs = a, {}

    score, _, cres, _ = ref["eval"].eval_one_op(op, be[op], [Case([torch.randn(4)])], [])
    assert score == 0.0 and "no CPU path" in cres[0].error_msg
