"""Generate the golden fixtures in this folder by running the REFERENCE harness.

    BACKENDBENCH_REFERENCE=<reference checkout> python tests/golden/make_golden.py

(default: a `reference` folder beside the repository)

Needs the reference checkout (meta-pytorch/BackendBench) importable as `BackendBench`;
it is only available where the fixtures are made, which is why the outputs are
committed: `aten_ops_golden.pt` and `harness_golden.json`.

* aten_ops_golden.pt -- for each of the sixteen overloads (and their backward neighbours) a handful of small seeded
  cases (inputs and the output of `AtenBackend()[op](*args, **kwargs)` on CPU, i.e. the
  `ref` of BackendBench/eval.py:100), each one passed through the reference's own
  `eval_correctness_test` with the identity backend to make sure the harness accepts it.
* harness_golden.json -- known answers of the host logic: operator/folder name mapping,
  `serialize_args` strings, `compute_errors` numbers, the `allclose` truth table,
  `perf_at_p`, spec-name extraction and the stream-creation screen.
"""

import json
import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def tensor_cases():
    """[(op spec name, args, kwargs, tag)] -- small, seeded, covering the edge semantics."""
    g = torch.Generator().manual_seed(1234)
    nan, inf = float("nan"), float("inf")

    def rn(*shape, dtype=torch.float32, std=1.0):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    def ri(high, *shape, dtype=torch.int64):
        return torch.randint(0, high, shape, generator=g, dtype=dtype)

    out = []
    bf, hf, f32 = torch.bfloat16, torch.float16, torch.float32
    # ---- elementwise
    special = torch.tensor([-1.0, 0.0, 1.0, -0.0, nan, inf, -inf, 1e-30, -3.5])
    for dt in (f32, bf, hf):
        out.append(("relu.default", [rn(37, 96, dtype=dt)], {}, f"relu_{dt}"))
        out.append(("add.Tensor", [rn(37, 96, dtype=dt), rn(37, 96, dtype=dt)], {}, f"add_{dt}"))
        out.append(("mul.Tensor", [rn(37, 96, dtype=dt), rn(37, 96, dtype=dt)], {}, f"mul_{dt}"))
    out.append(("relu.default", [special.clone()], {}, "relu_special"))
    out.append(("relu.default", [rn(16, 24).t()], {}, "relu_transposed"))
    out.append(("relu.default", [torch.empty(0, 8)], {}, "relu_empty"))
    out.append(("add.Tensor", [rn(5, 1, 7), rn(4, 1)], {"alpha": 2}, "add_bcast_alpha"))
    out.append(("add.Tensor", [rn(33, dtype=bf), rn(33)], {}, "add_promote_bf16_f32"))
    out.append(("add.Tensor", [rn(6, 5), 2.5], {"alpha": -1}, "add_python_scalar"))
    out.append(("add.Tensor", [special.clone(), special.flip(0).clone()], {}, "add_special"))
    out.append(("mul.Tensor", [rn(8, 3, dtype=hf), rn(3, dtype=hf)], {}, "mul_bcast_f16"))
    out.append(("mul.Tensor", [rn(12, 6).t(), rn(6, 12)], {}, "mul_transposed"))
    out.append(("mul.Tensor", [rn(9), 3.0], {}, "mul_python_scalar"))
    out.append(("where.self", [torch.rand(37, 96, generator=g) < 0.5, rn(37, 96), rn(37, 96)], {}, "where_f32"))
    out.append(("where.self", [torch.rand(1, 9, generator=g) < 0.5, rn(4, 9, dtype=bf), rn(4, 1, dtype=bf)], {}, "where_bcast_bf16"))
    out.append(("where.self", [torch.tensor([True, False, True, False]), torch.tensor([nan, nan, -0.0, -0.0]), torch.tensor([1.0, inf, 0.0, 5.0])], {}, "where_special"))
    out.append(("where.self", [torch.rand(6, 5, generator=g) < 0.5, ri(100, 6, 5), ri(100, 6, 5)], {}, "where_int64"))
    out.append(("where.self", [torch.rand(6, 5, generator=g) < 0.5, rn(6, 5, dtype=hf), rn(6, 5)], {}, "where_promote"))
    # ---- reductions / normalisation
    for dt in (f32, bf, hf):
        x = rn(19, 160, dtype=dt)
        out.append(("_softmax.default", [x, -1, False], {}, f"softmax_{dt}"))
        out.append(("_log_softmax.default", [x, -1, False], {}, f"log_softmax_{dt}"))
        out.append(("sum.dim_IntList", [x, [-1]], {}, f"sum_{dt}"))
        out.append(("native_layer_norm.default", [x, [160], rn(160, dtype=dt, std=0.02) + 1, rn(160, dtype=dt, std=0.02), 1e-5], {}, f"layer_norm_{dt}"))
    x3 = rn(4, 7, 10)
    out.append(("_softmax.default", [x3, 1, False], {}, "softmax_dim1"))
    out.append(("_log_softmax.default", [x3, 0, False], {}, "log_softmax_dim0"))
    out.append(("_softmax.default", [rn(5, 33), -1, False], {}, "softmax_ragged"))
    xs = rn(4, 8)
    xs[0, 3] = nan
    xs[1, :] = -inf
    xs[2, 2] = inf
    out.append(("_softmax.default", [xs, -1, False], {}, "softmax_nonfinite"))
    out.append(("_log_softmax.default", [xs.clone(), -1, False], {}, "log_softmax_nonfinite"))
    out.append(("sum.dim_IntList", [x3, [0, 2], True], {}, "sum_dims02_keepdim"))
    out.append(("sum.dim_IntList", [x3, [1]], {}, "sum_dim1"))
    out.append(("sum.dim_IntList", [rn(6, 9, dtype=bf), [-1]], {"dtype": f32}, "sum_dtype_kw"))
    out.append(("sum.dim_IntList", [torch.empty(3, 0), [-1]], {}, "sum_empty_dim"))
    out.append(("sum.dim_IntList", [rn(20000), [0]], {}, "sum_long_vector"))
    out.append(("sum.dim_IntList", [rn(12, 14).t(), [-1]], {}, "sum_transposed"))
    out.append(("native_layer_norm.default", [rn(3, 5, 24), [5, 24], None, None, 1e-6], {}, "layer_norm_2d_noaffine"))
    out.append(("native_layer_norm.default", [rn(7, 33), [33], rn(33), None, 1e-5], {}, "layer_norm_ragged_weight_only"))
    # ---- contraction
    for dt in (f32, bf, hf):
        a, b = rn(33, 64, dtype=dt, std=0.125), rn(64, 48, dtype=dt, std=0.125)
        out.append(("mm.default", [a, b], {}, f"mm_{dt}"))
        out.append(("addmm.default", [rn(48, dtype=dt), a, b], {}, f"addmm_{dt}"))
        out.append(("bmm.default", [rn(3, 20, 32, dtype=dt, std=0.2), rn(3, 32, 24, dtype=dt, std=0.2)], {}, f"bmm_{dt}"))
    out.append(("mm.default", [rn(17, 40).t(), rn(17, 9)], {}, "mm_transposed_a"))
    out.append(("mm.default", [rn(5, 0), rn(0, 7)], {}, "mm_k0"))
    out.append(("addmm.default", [rn(6, 1), rn(6, 10), rn(10, 4)], {"beta": 0.5, "alpha": 2}, "addmm_beta_alpha_colbias"))
    out.append(("addmm.default", [torch.full((4,), nan), rn(3, 5), rn(5, 4)], {"beta": 0}, "addmm_beta0_nan_bias"))
    out.append(("bmm.default", [rn(2, 6, 8), rn(2, 5, 8).transpose(1, 2)], {}, "bmm_transposed_b"))
    # ---- indexing (bit-exact)
    for dt in (f32, bf, hf):
        tab = rn(50, 24, dtype=dt, std=0.02)
        out.append(("embedding.default", [tab, ri(50, 31)], {}, f"embedding_{dt}"))
        out.append(("index_select.default", [tab, 0, ri(50, 31)], {}, f"index_select_{dt}"))
        out.append(("gather.default", [rn(20, 12, dtype=dt), 0, ri(20, 20, 12)], {}, f"gather_{dt}"))
        out.append(("scatter_add.default", [rn(20, 16, dtype=dt), 0, ri(20, 64, 16), rn(64, 16, dtype=dt)], {}, f"scatter_add_{dt}"))
        out.append(("argmax.default", [rn(9, 300, dtype=dt), -1], {}, f"argmax_{dt}"))
    out.append(("embedding.default", [rn(11, 8), ri(11, 3, 4, dtype=torch.int32)], {}, "embedding_int32_2d_idx"))
    out.append(("index_select.default", [rn(4, 9, 5), 1, ri(9, 6)], {}, "index_select_dim1"))
    out.append(("index_select.default", [rn(6, 7), 0, ri(6, 0)], {}, "index_select_empty_idx"))
    out.append(("gather.default", [rn(6, 8), 1, ri(8, 4, 3)], {}, "gather_dim1_smaller_index"))
    out.append(("gather.default", [rn(3, 4, 5), 2, ri(5, 3, 4, 2)], {}, "gather_3d"))
    out.append(("gather.default", [ri(1000, 7, 9), 0, ri(7, 5, 9)], {}, "gather_int64"))
    out.append(("scatter_add.default", [rn(8, 24), 0, ri(8, 256, 24), rn(256, 24)], {}, "scatter_add_many_collisions"))
    out.append(("scatter_add.default", [rn(6, 10), 1, ri(10, 6, 40), rn(6, 40)], {}, "scatter_add_dim1"))
    out.append(("scatter_add.default", [rn(5, 6), 0, ri(5, 3, 4), rn(7, 9)], {}, "scatter_add_small_index_large_src"))
    out.append(("scatter_add.default", [rn(3, 4, 5), 1, ri(4, 3, 9, 5), rn(3, 9, 5)], {}, "scatter_add_3d"))
    ties = torch.tensor([[1.0, 3.0, 3.0, 2.0], [nan, 5.0, nan, 7.0], [-inf, -inf, -inf, -inf], [2.0, inf, inf, nan]])
    out.append(("argmax.default", [ties, -1], {}, "argmax_ties_nan"))
    out.append(("argmax.default", [ties.clone()], {}, "argmax_flat"))
    out.append(("argmax.default", [rn(5, 6, 7), 1, True], {}, "argmax_dim1_keepdim"))
    out.append(("argmax.default", [rn(20000)], {}, "argmax_long_flat"))
    # ---- backward neighbours of the row operators (appended last: earlier cases keep their random draws)
    for dt in (f32, bf, hf):
        x = rn(37, 96, dtype=dt)
        out.append(("_softmax_backward_data.default", [rn(37, 96, dtype=dt), torch.softmax(x.float(), -1).to(dt), -1, dt], {}, f"softmax_backward_{dt}"))
        out.append(("_log_softmax_backward_data.default", [rn(37, 96, dtype=dt), torch.log_softmax(x.float(), -1).to(dt), -1, dt], {}, f"log_softmax_backward_{dt}"))
    x = rn(6, 33, 5)
    out.append(("_softmax_backward_data.default", [rn(6, 33, 5), torch.softmax(x, 1), 1, f32], {}, "softmax_backward_dim1"))
    out.append(("_log_softmax_backward_data.default", [rn(6, 33, 5), torch.log_softmax(x, 0), 0, f32], {}, "log_softmax_backward_dim0"))
    x = rn(9, 67)
    out.append(("_softmax_backward_data.default", [rn(9, 67), torch.softmax(x, -1), -1, f32], {}, "softmax_backward_ragged"))
    out.append(("_log_softmax_backward_data.default", [rn(9, 67), torch.log_softmax(x, -1), -1, f32], {}, "log_softmax_backward_ragged"))
    out.append(("_softmax_backward_data.default", [torch.empty(0, 7), torch.empty(0, 7), 1, f32], {}, "softmax_backward_empty"))
    for dt in (f32, bf, hf):
        x, w, b = rn(37, 96, dtype=dt), rn(96, dtype=dt), rn(96, dtype=dt)
        _, mean, rstd = torch.ops.aten.native_layer_norm.default(x, [96], w, b, 1e-5)
        out.append(("native_layer_norm_backward.default", [rn(37, 96, dtype=dt), x, [96], mean, rstd, w, b, [True, True, True]], {}, f"layer_norm_backward_{dt}"))
    x, w = rn(5, 6, 33), rn(33)
    _, mean, rstd = torch.ops.aten.native_layer_norm.default(x, [33], w, None, 1e-5)
    out.append(("native_layer_norm_backward.default", [rn(5, 6, 33), x, [33], mean, rstd, w, None, [True, True, False]], {}, "layer_norm_backward_ragged_no_bias"))
    x = rn(4, 3, 8, 5)
    _, mean, rstd = torch.ops.aten.native_layer_norm.default(x, [8, 5], None, None, 1e-5)
    out.append(("native_layer_norm_backward.default", [rn(4, 3, 8, 5), x, [8, 5], mean, rstd, None, None, [True, False, False]], {}, "layer_norm_backward_two_dims_no_affine"))
    x, w, b = rn(9, 64), rn(64), rn(64)
    _, mean, rstd = torch.ops.aten.native_layer_norm.default(x, [64], w, b, 1e-5)
    out.append(("native_layer_norm_backward.default", [rn(9, 64), x, [64], mean, rstd, w, b, [False, True, True]], {}, "layer_norm_backward_parameters_only"))
    for dt in (f32, bf, hf):
        out.append(("embedding_dense_backward.default", [rn(50, 24, dtype=dt), ri(11, 50), 11, -1, False], {}, f"embedding_backward_{dt}"))
    out.append(("embedding_dense_backward.default", [rn(4, 9, 10), ri(7, 4, 9, dtype=torch.int32), 7, 3, False], {}, "embedding_backward_2d_int32_padding_idx"))
    out.append(("embedding_dense_backward.default", [rn(300, 6), ri(2, 300), 5, -1, False], {}, "embedding_backward_two_hot_rows"))
    out.append(("embedding_dense_backward.default", [torch.empty(0, 8), ri(4, 0), 4, -1, False], {}, "embedding_backward_no_indices"))
    return out


def main():
    repo_root = os.path.dirname(os.path.dirname(HERE))
    ref_root = os.environ.get("BACKENDBENCH_REFERENCE", os.path.join(os.path.dirname(repo_root), "reference"))
    sys.path.insert(0, ref_root)
    import BackendBench  # noqa: F401  (the reference)
    from BackendBench import eval as ref_eval
    from BackendBench import utils as ref_utils
    from BackendBench.backends import AtenBackend
    from BackendBench.opregistry import _extract_spec_name_from_op, get_operator

    class Case:
        def __init__(self, args, kwargs):
            self.args, self.kwargs = args, kwargs

    backend = AtenBackend()
    golden = []
    for spec, args, kwargs, tag in tensor_cases():
        op = get_operator(spec)
        ref = backend[op](*args, **kwargs)
        res = ref_eval.eval_correctness_test(op, backend[op], Case(args, kwargs))
        assert res.is_correct, (tag, res.error_msg)
        golden.append({"op": spec, "tag": tag, "args": args, "kwargs": kwargs, "ref": ref, "serialized": res.args})
    torch.save({"torch": torch.__version__, "cases": golden}, os.path.join(HERE, "aten_ops_golden.pt"))

    h = {"torch": torch.__version__}
    names = ["add.Tensor", "relu.default", "add_.Tensor", "_log_softmax.default", "sum.dim_IntList", "native_layer_norm.default", "nn.functional.relu", "_native_batch_norm", "aten.add.Tensor"]
    h["op_to_folder"] = {n: ref_utils.op_name_to_folder_name(n) for n in names}
    folders = list(h["op_to_folder"].values()) + ["add___Tensor", "relu___default", "where__self", "my_op_name"]
    h["folder_to_op"] = {f: ref_utils.folder_name_to_op_name(f) for f in folders}
    h["extract_operator_name"] = {s: ref_utils.extract_operator_name(s) for s in ["aten.add.Tensor", "add.Tensor", "torch.ops.aten.relu.default"]}
    ours = ["relu.default", "add.Tensor", "mul.Tensor", "where.self", "_softmax.default", "_log_softmax.default", "sum.dim_IntList", "native_layer_norm.default", "argmax.default",
            "embedding.default", "index_select.default", "gather.default", "scatter_add.default", "mm.default", "addmm.default", "bmm.default"]
    h["spec_names"] = {n: _extract_spec_name_from_op(ref_utils.get_pytorch_op(n)) for n in ours}
    h["op_dunder_name"] = {n: ref_utils.get_pytorch_op(n).__name__ for n in ours}
    g = torch.Generator().manual_seed(7)
    ser_inputs = {
        "plain": ([torch.zeros(2, 3)], {}),
        "kw": ([torch.zeros(2, 3, dtype=torch.bfloat16), 1], {"dim": 1, "keepdim": True}),
        "strided": ([torch.zeros(4, 6).t()], {}),
        "list": ([[torch.zeros(2), torch.zeros(3, dtype=torch.int64)], 2.5], {}),
        "empty": ([], {}),
        "scalars": ([1, 2.0, None, "s"], {"x": [1, 2]}),
    }
    h["serialize_args"] = {k: ref_utils.serialize_args(a, kw) for k, (a, kw) in ser_inputs.items()}
    h["serialize_none"] = ref_utils.serialize_args(None, None)
    pairs = {
        "identical": ([1.0, 2.0, 3.0, 4.0], [1.0, 2.0, 3.0, 4.0]),
        "ten_percent": ([2.0, 4.0, 6.0, 8.0], [2.2, 4.4, 6.6, 8.8]),
        "zero_ref": ([0.0, 1.0], [0.1, 1.1]),
        "with_nan": ([1.0, math.nan], [1.0, math.nan]),
        "with_inf": ([math.inf, 1.0], [math.inf, 1.5]),
    }
    ce = {}
    for k, (a, b) in pairs.items():
        x, y = ref_utils.compute_errors(torch.tensor(a), torch.tensor(b))
        ce[k] = [repr(float(x)), repr(float(y))]
    h["compute_errors"] = ce
    x, y = ref_utils.compute_errors([torch.tensor([1.0, 2.0]), torch.tensor([3.0, 4.0])], [torch.tensor([1.1, 2.2]), torch.tensor([3.3, 4.4])])
    h["compute_errors_list"] = [repr(float(x)), repr(float(y))]
    h["compute_errors_none"] = [ref_utils.compute_errors(1.0, 2.0) == (None, None), ref_utils.compute_errors(torch.ones(3, 4), torch.ones(3, 5)) == (None, None)]
    t = torch.tensor
    table = {
        "equal": (t([1.0, 2.0, 3.0]), t([1.0, 2.0, 3.0])),
        "within": (t([1.0, 2.0, 3.0]), t([1.0, 2.0, 3.01])),
        "outside": (t([1.0, 2.0]), t([1.1, 2.1])),
        "nan_nan": (t([1.0, math.nan]), t([1.0, math.nan])),
        "nan_vs_number": (t([1.0, math.nan]), t([1.0, 2.0])),
        "inf_inf": (t([math.inf, -math.inf]), t([math.inf, -math.inf])),
        "inf_vs_neg_inf": (t([math.inf]), t([-math.inf])),
        "inf_vs_big": (t([math.inf]), t([3e38])),
        "dtype_mismatch": (t([1.0]), t([1.0], dtype=torch.float64)),
        "shape_mismatch": (t([1.0, 2.0]), t([[1.0, 2.0]])),
        "int_equal": (t([1, 2, 3]), t([1, 2, 3])),
        "int_off_by_one": (t([1, 2, 3]), t([1, 2, 4])),
        "bool_diff": (t([True, False]), t([True, True])),
        "nested_ok": ([[t([1.0])], (t([2.0]), t([3.0]))], [[t([1.01])], (t([2.01]), t([3.01]))]),
        "length_mismatch": ([t([1.0]), t([2.0])], [t([1.0])]),
        "scalars_equal": (1, 1),
        "scalars_differ": (1, 2),
        "strings": ("test", "test"),
        "near_zero_atol": (t([0.0]), t([0.009])),
        "near_zero_outside": (t([0.0]), t([0.011])),
        "rtol_on_second_operand": (t([100.0]), t([101.015])),
    }
    h["allclose"] = {k: bool(ref_eval.allclose(a, b)) for k, (a, b) in table.items()}
    h["perf_at_p"] = {
        "basic": float(ref_eval.perf_at_p([1, 1, 0, 1], [2.0, 0.5, 3.0, 1.0], 1.0)),
        "p0": float(ref_eval.perf_at_p([1, 0], [0.2, 5.0], 0.0)),
        "p2": float(ref_eval.perf_at_p([True, True, True], [2.5, 2.0, 1.9], 2.0)),
    }
    snippets = {
        "plain": "def f(x):\n    return x + 1\n",
        "torch_stream": "def f(x):\n    s = torch.cuda.Stream()\n    return x\n",
        "current_stream": "def f(x):\n    s = torch.cuda.current_stream().cuda_stream\n    return x\n",
        "bare_stream": "def f(x):\n    s = Stream(device=0)\n    return x\n",
        "make_stream": "def f(x):\n    s = make_stream()\n    return x\n",
    }
    verdicts = {}
    import importlib.util
    import tempfile

    for k, src in snippets.items():
        with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as fh:
            fh.write("import torch\n" + src)
        spec = importlib.util.spec_from_file_location(f"snip_{k}", fh.name)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        verdicts[k] = bool(ref_utils.uses_cuda_stream(mod.f))
        os.unlink(fh.name)
    h["uses_cuda_stream"] = verdicts
    h["uses_cuda_stream_sources"] = snippets
    with open(os.path.join(HERE, "harness_golden.json"), "w") as fh:
        json.dump(h, fh, indent=1, sort_keys=True)
    print(f"wrote {len(golden)} operator cases and the harness known answers")


if __name__ == "__main__":
    main()
