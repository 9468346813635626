"""Seeded synthetic cases: the four named operator configurations and the 512-case sweep.

A case is a small picklable descriptor (`CaseSpec`); the tensors are generated from its
seed where they are needed -- on the worker's own GPU for the throughput sweep, on the
CPU (then copied) when the aten CPU result is the oracle and both sides must see the
same bits. These generators stand in for the reference's public case sources (OpInfo,
FACTO and the TorchBench trace dataset, BackendBench/suite/*.py, data_loaders.py:26-28),
none of which is available offline; no item of those suites is reproduced.
"""

from __future__ import annotations

import math
import random
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import torch

DTYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
ITEMSIZE = {"f32": 4, "bf16": 2, "f16": 2}

FAMILIES: Dict[str, List[str]] = {
    "elementwise": ["relu.default", "add.Tensor", "mul.Tensor", "where.self"],
    "reduce": ["_softmax.default", "_log_softmax.default", "sum.dim_IntList", "native_layer_norm.default"],
    "gemm": ["mm.default", "addmm.default", "bmm.default"],
    "indexing": ["embedding.default", "index_select.default", "gather.default", "scatter_add.default", "argmax.default"],
}
EDGE_KINDS = ("zero", "bcast", "transposed", "naninf")


@dataclass(frozen=True)
class CaseSpec:
    case_id: int
    op: str  # spec name, e.g. "add.Tensor"
    dtype: str  # "f32" | "bf16" | "f16"
    shape: Tuple[int, ...]  # the operator's primary shape (meaning depends on op, see build)
    seed: int
    extra: Tuple[Tuple[str, object], ...] = ()  # op-specific parameters
    edge: str = ""  # "" or one of EDGE_KINDS
    family: str = ""
    name: str = ""  # set for the named configurations

    def param(self, key, default=None):
        for k, v in self.extra:
            if k == key:
                return v
        return default

    # ---------------------------------------------------------------- tensors
    def build(self, device="cuda", gen_device=None):
        """(args, kwargs) for `torch.ops.aten.<op>`. Random numbers are drawn on
        `gen_device` (default: `device`) and then moved to `device`."""
        gen_device = gen_device or device
        g = torch.Generator(device=gen_device).manual_seed(self.seed)
        dt = DTYPES[self.dtype]

        def normal(shape, std=1.0, mean=0.0):
            t = torch.randn(shape, generator=g, device=gen_device, dtype=torch.float32)
            if std != 1.0:
                t = t * std
            if mean != 0.0:
                t = t + mean
            return t.to(dt)

        def randint(high, shape, dtype=torch.int64):
            return torch.randint(0, max(int(high), 1), shape, generator=g, device=gen_device, dtype=dtype)

        def poison(t, inf_ok=True):
            """1% of the elements become NaN / +Inf / -Inf (NaN only when `inf_ok` is False)."""
            if self.edge != "naninf" or t.numel() == 0:
                return t
            r = torch.rand(t.shape, generator=g, device=gen_device)
            t = t.clone()
            t[r < (0.004 if inf_ok else 0.010)] = float("nan")
            if inf_ok:
                t[(r >= 0.004) & (r < 0.007)] = float("inf")
                t[(r >= 0.007) & (r < 0.010)] = float("-inf")
            return t

        def transposed(shape2d, **kw):
            """A [r, c] view with strides (1, r): the transpose of a contiguous [c, r] tensor."""
            r, c = shape2d
            return normal((c, r), **kw).t()

        op, shp = self.op, tuple(self.shape)
        kwargs = {}
        if op == "relu.default":
            x = transposed(shp) if self.edge == "transposed" and len(shp) == 2 else normal(shp)
            args = [poison(x)]
        elif op in ("add.Tensor", "mul.Tensor"):
            x = transposed(shp) if self.edge == "transposed" and len(shp) == 2 else normal(shp)
            yshape = tuple(self.param("other_shape", shp))
            args = [poison(x), poison(normal(yshape))]
            if op == "add.Tensor" and self.param("alpha") is not None:
                kwargs["alpha"] = self.param("alpha")
        elif op == "where.self":
            cshape = tuple(self.param("cond_shape", shp))
            cond = torch.rand(cshape, generator=g, device=gen_device) < 0.5
            x = transposed(shp) if self.edge == "transposed" and len(shp) == 2 else normal(shp)
            args = [cond, poison(x), poison(normal(shp))]
        elif op in ("_softmax.default", "_log_softmax.default"):
            x = transposed(shp) if self.edge == "transposed" and len(shp) == 2 else normal(shp)
            args = [poison(x), self.param("dim", -1), False]
        elif op in ("_softmax_backward_data.default", "_log_softmax_backward_data.default"):
            # a forward output of the right kind (rows of a softmax / log_softmax) and a random incoming gradient
            dim = self.param("dim", -1)
            y = torch.softmax(normal(shp).float(), dim) if op == "_softmax_backward_data.default" else torch.log_softmax(normal(shp).float(), dim)
            args = [normal(shp), y.to(dt), dim, dt]
        elif op == "embedding_dense_backward.default":
            rows, cols = shp  # the table whose gradient is produced
            n_idx = int(self.param("n_idx", 16384))
            args = [normal((n_idx, cols)), randint(rows, (n_idx,)), rows, -1, False]
        elif op == "native_layer_norm_backward.default":
            cols = shp[-1]
            x = normal(shp)
            w = normal((cols,), std=0.02, mean=1.0)
            b = normal((cols,), std=0.02)
            xf = x.float()
            mean = xf.mean(-1, keepdim=True)  # fp32 statistics, as the CUDA forward returns them
            rstd = torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + 1e-5)
            args = [normal(shp), x, [cols], mean, rstd, w, b, [True, True, True]]
        elif op == "sum.dim_IntList":
            x = transposed(shp) if self.edge == "transposed" and len(shp) == 2 else normal(shp)
            args = [poison(x), list(self.param("dim", (-1,)))]
            if self.param("keepdim"):
                args.append(True)
        elif op == "native_layer_norm.default":
            cols = shp[-1]
            # NaN only: for a row holding +-inf aten's own kernels disagree with each other
            # (mean comes out NaN or inf depending on where the infinity falls in the
            # kernel's internal chunking), so there is no single reference result to match
            x = poison(normal(shp), inf_ok=False)
            w = normal((cols,), std=0.02, mean=1.0)
            b = normal((cols,), std=0.02)
            args = [x, [cols], w, b, 1e-5]
        elif op in ("mm.default", "addmm.default"):
            M, K, N = shp
            std = 1.0 / math.sqrt(max(K, 1))
            a = transposed((M, K), std=std) if self.edge == "transposed" else normal((M, K), std=std)
            bm = normal((K, N), std=std)
            a, bm = poison(a), poison(bm)
            if op == "mm.default":
                args = [a, bm]
            else:
                bias_shape = tuple(self.param("bias_shape", (N,)))
                args = [normal(bias_shape), a, bm]
                if self.param("beta") is not None:
                    kwargs = {"beta": self.param("beta"), "alpha": self.param("alpha", 1)}
        elif op == "bmm.default":
            B, M, K, N = shp
            std = 1.0 / math.sqrt(max(K, 1))
            a = normal((B, M, K), std=std)
            bm = normal((B, N, K), std=std).transpose(1, 2) if self.edge == "transposed" else normal((B, K, N), std=std)
            args = [poison(a), poison(bm)]
        elif op == "embedding.default":
            V, D = shp
            n = self.param("n_idx")
            table = poison(normal((V, D), std=0.02))
            idt = torch.int32 if self.param("idx32") else torch.int64
            idx_shape = tuple(self.param("idx_shape", (n,)))
            args = [table, randint(V, idx_shape, idt)]
        elif op == "index_select.default":
            dim = self.param("dim", 0)
            x = transposed(shp) if self.edge == "transposed" and len(shp) == 2 else normal(shp, std=0.02)
            args = [poison(x), dim, randint(shp[dim], (self.param("n_idx"),))]
        elif op == "gather.default":
            dim = self.param("dim", 0)
            ishape = tuple(self.param("index_shape", shp))
            x = transposed(shp) if self.edge == "transposed" and len(shp) == 2 else normal(shp)
            args = [poison(x), dim, randint(shp[dim], ishape)]
        elif op == "scatter_add.default":
            dim = self.param("dim", 0)
            ishape = tuple(self.param("index_shape", shp))
            args = [poison(normal(shp)), dim, randint(shp[dim], ishape), poison(normal(ishape))]
        elif op == "argmax.default":
            x = transposed(shp) if self.edge == "transposed" and len(shp) == 2 else normal(shp)
            x = poison(x)
            dim = self.param("dim", -1)
            args = [x] if dim is None else [x, dim]
            if self.param("keepdim"):
                args.append(True)
        else:
            raise ValueError(f"unknown op {op}")
        if str(gen_device) != str(device):
            args = [a.to(device) if isinstance(a, torch.Tensor) else a for a in args]
        return args, kwargs

    # ---------------------------------------------------------------- work model
    def algorithmic_bytes(self) -> int:
        """Bytes an ideal kernel moves: each input read once, each output written once."""
        es = ITEMSIZE[self.dtype]
        n = _prod(self.shape)
        op = self.op
        if op == "relu.default":
            return 2 * n * es
        if op in ("add.Tensor", "mul.Tensor"):
            return (2 * n + _prod(self.param("other_shape", self.shape))) * es
        if op == "where.self":
            return 3 * n * es + _prod(self.param("cond_shape", self.shape))
        if op in ("_softmax.default", "_log_softmax.default"):
            return 2 * n * es
        if op in ("_softmax_backward_data.default", "_log_softmax_backward_data.default"):
            return 3 * n * es  # grad and output in, grad_input out
        if op == "native_layer_norm_backward.default":
            rows = n // max(self.shape[-1], 1)
            return 3 * n * es + 3 * self.shape[-1] * es + 2 * rows * 4  # dy, x in, dx out; w in, dw, db out; fp32 mean / rstd in
        if op == "embedding_dense_backward.default":
            n_idx = int(self.param("n_idx", 16384))
            return n * es + n_idx * self.shape[-1] * es + n_idx * 8  # the whole table gradient out, the gathered rows and the indices in
        if op == "sum.dim_IntList":
            dims = [d % len(self.shape) for d in self.param("dim", (-1,))]
            out = _prod(s for i, s in enumerate(self.shape) if i not in dims)
            return (n + out) * es
        if op == "native_layer_norm.default":
            rows = n // max(self.shape[-1], 1)
            return 2 * n * es + 2 * self.shape[-1] * es + 2 * rows * 4
        if op in ("mm.default", "addmm.default"):
            M, K, N = self.shape
            b = (M * K + K * N + M * N) * es
            return b + (_prod(self.param("bias_shape", (N,))) * es if op == "addmm.default" else 0)
        if op == "bmm.default":
            B, M, K, N = self.shape
            return B * (M * K + K * N + M * N) * es
        if op == "embedding.default":
            V, D = self.shape
            ni = _prod(self.param("idx_shape", (self.param("n_idx"),)))
            return 2 * ni * D * es + ni * (4 if self.param("idx32") else 8)
        if op == "index_select.default":
            dim = self.param("dim", 0)
            out = n // max(self.shape[dim], 1) * self.param("n_idx")
            return 2 * out * es + self.param("n_idx") * 8
        if op == "gather.default":
            ni = _prod(self.param("index_shape", self.shape))
            return ni * (8 + 2 * es)
        if op == "scatter_add.default":
            ni = _prod(self.param("index_shape", self.shape))
            return 2 * n * es + ni * (8 + es)
        if op == "argmax.default":
            dim = self.param("dim", -1)
            out = 1 if dim is None else n // max(self.shape[dim], 1)
            return n * es + out * 8
        raise ValueError(op)

    def flops(self) -> int:
        if self.op in ("mm.default", "addmm.default"):
            M, K, N = self.shape
            return 2 * M * N * K
        if self.op == "bmm.default":
            B, M, K, N = self.shape
            return 2 * B * M * N * K
        return 0

    def label(self) -> str:
        return self.name or f"{self.op}[{self.dtype}]{list(self.shape)}{('/' + self.edge) if self.edge else ''}"


def _prod(xs) -> int:
    p = 1
    for x in xs:
        p *= int(x)
    return p


# ---------------------------------------------------------------------- named configs
def named_cases() -> List[CaseSpec]:
    """The per-operator configurations throughput is quoted on (all seed 0)."""
    c: List[CaseSpec] = []

    def add(name, op, dtype, shape, family, **extra):
        c.append(CaseSpec(len(c), op, dtype, tuple(shape), 0, tuple(sorted(extra.items())), "", family, name))

    # elementwise plumbing, fp32 [4096, 4096]
    for op in ("relu.default", "add.Tensor", "mul.Tensor"):
        add(f"{op.split('.')[0]}_f32_4096x4096", op, "f32", (4096, 4096), "elementwise")
    # reductions and normalisation, bf16 [8192, 4096] and fp32 [65536, 1024]
    for dtype, shape in (("bf16", (8192, 4096)), ("f32", (65536, 1024))):
        tag = f"{dtype}_{shape[0]}x{shape[1]}"
        add(f"softmax_{tag}", "_softmax.default", dtype, shape, "reduce", dim=-1)
        add(f"log_softmax_{tag}", "_log_softmax.default", dtype, shape, "reduce", dim=-1)
        add(f"sum_{tag}", "sum.dim_IntList", dtype, shape, "reduce", dim=(-1,))
        add(f"layer_norm_{tag}", "native_layer_norm.default", dtype, shape, "reduce")
    # dense contraction, bf16
    add("mm_bf16_8192x4096x11008", "mm.default", "bf16", (8192, 4096, 11008), "gemm")
    add("addmm_bf16_8192x4096x11008", "addmm.default", "bf16", (8192, 4096, 11008), "gemm", bias_shape=(11008,))
    add("bmm_bf16_32x2048x128x2048", "bmm.default", "bf16", (32, 2048, 128, 2048), "gemm")
    # integer / indexing, bit-exact
    add("embedding_bf16_128256x4096_16384", "embedding.default", "bf16", (128256, 4096), "indexing", n_idx=16384)
    add("index_select_bf16_128256x4096_16384", "index_select.default", "bf16", (128256, 4096), "indexing", n_idx=16384, dim=0)
    add("gather_f32_4096x4096", "gather.default", "f32", (4096, 4096), "indexing", dim=0)
    add("scatter_add_f32_4096x4096", "scatter_add.default", "f32", (4096, 4096), "indexing", dim=0)
    add("argmax_f32_8192x32000", "argmax.default", "f32", (8192, 32000), "indexing", dim=-1)
    add("where_f32_4096x4096", "where.self", "f32", (4096, 4096), "elementwise")
    return c


def neighbour_cases() -> List[CaseSpec]:
    """Configurations next to the named ones: the backward neighbours of the sixteen operators
    at the shapes of their forward operators, and softmax / log_softmax over vocabulary-size
    rows (longer than a CTA's registers hold; 50257 is odd, so every second row starts off
    the 16-byte grid) and over millions of 17-element rows (a thread per row). Not part of
    the per-op bench table."""
    c: List[CaseSpec] = []
    for dtype, shape in (("bf16", (8192, 4096)), ("f32", (65536, 1024))):
        tag = f"{dtype}_{shape[0]}x{shape[1]}"
        for name, op in (("softmax_backward", "_softmax_backward_data.default"), ("log_softmax_backward", "_log_softmax_backward_data.default")):
            c.append(CaseSpec(1000 + len(c), op, dtype, shape, 0, (("dim", -1),), "", "reduce", f"{name}_{tag}"))
        c.append(CaseSpec(1000 + len(c), "native_layer_norm_backward.default", dtype, shape, 0, (), "", "reduce", f"layer_norm_backward_{tag}"))
    c.append(CaseSpec(1000 + len(c), "embedding_dense_backward.default", "bf16", (128256, 4096), 0, (("n_idx", 16384),), "", "indexing", "embedding_backward_bf16_128256x4096_16384"))
    c.append(CaseSpec(1000 + len(c), "_softmax.default", "bf16", (4096, 128256), 0, (("dim", -1),), "", "reduce", "softmax_bf16_4096x128256"))
    c.append(CaseSpec(1000 + len(c), "_log_softmax.default", "bf16", (4096, 50257), 0, (("dim", -1),), "", "reduce", "log_softmax_bf16_4096x50257"))
    c.append(CaseSpec(1000 + len(c), "_softmax.default", "f16", (3126099, 17), 0, (("dim", -1),), "", "reduce", "softmax_f16_3126099x17"))
    # fp32 products off the tensor-core path: a long contraction with few output tiles (K shared
    # among the CTAs of a cluster) and very many rows with 8 output columns (a row per thread)
    c.append(CaseSpec(1000 + len(c), "mm.default", "f32", (44, 4096, 1024), 0, (), "", "gemm", "mm_f32_44x4096x1024"))
    c.append(CaseSpec(1000 + len(c), "bmm.default", "f32", (64, 8192, 256, 8), 0, (), "", "gemm", "bmm_f32_64x8192x256x8"))
    # an elementwise operator over a transposed view (read through 32 x 32 shared-memory tiles)
    c.append(CaseSpec(1000 + len(c), "add.Tensor", "f32", (39934, 1024), 0, (), "transposed", "elementwise", "add_f32_39934x1024_transposed"))
    return c


def named_case(name: str) -> CaseSpec:
    for c in named_cases() + neighbour_cases():
        if c.name == name:
            return c
    raise KeyError(name)


def scaled_down(case: CaseSpec, factor: int) -> CaseSpec:
    """The same operator and layout with the leading (row / M / table) extent divided by
    `factor` -- what parity tests use when the CPU oracle must finish in seconds."""
    shp = list(case.shape)
    extra = dict(case.extra)
    if case.op in ("mm.default", "addmm.default"):
        shp = [max(shp[0] // factor, 128), max(shp[1] // max(factor // 4, 1), 64), max(shp[2] // factor, 128)]
        if "bias_shape" in extra:
            extra["bias_shape"] = (shp[2],)
    elif case.op == "bmm.default":
        shp[0] = max(shp[0] // factor, 1)
    elif case.op in ("embedding.default", "index_select.default"):
        shp[0] = max(shp[0] // factor, 8)
        extra["n_idx"] = max(extra["n_idx"] // factor, 8)
    else:
        shp[0] = max(shp[0] // factor, 1)
    return CaseSpec(case.case_id, case.op, case.dtype, tuple(shp), case.seed, tuple(sorted(extra.items())), case.edge, case.family, case.name + f"/{factor}")


# ---------------------------------------------------------------------- the sweep
def _split2(rng: random.Random, numel: int, lo_log2=2, hi_log2=14) -> Tuple[int, int]:
    """Factor `numel` roughly into (rows, cols) with cols a (sometimes ragged) power of two."""
    e = max(int(math.log2(max(numel, 1))), 0)
    hi = max(min(hi_log2, e - 1), lo_log2)
    cols = 1 << rng.randint(lo_log2, hi)
    if rng.random() < 0.25 and cols > 4:
        cols += rng.choice((-1, 1, 3, -cols // 4))  # ragged widths leave the vector paths
    rows = max(numel // cols, 1)
    return rows, cols


def sweep_cases(n_cases: int = 512, seed: int = 0, max_log2: float = 26.0, edge_fraction: float = 0.15) -> List[CaseSpec]:
    """`n_cases` (op, shape, dtype) cases: family and op uniform, dtype uniform over
    fp32/bf16/fp16, element count log-uniform in 2^8..2^max_log2, `edge_fraction` of them
    edge cases (a zero-size dim, size-1 broadcast dims, transposed strides, 1% NaN/Inf)."""
    rng = random.Random(seed)
    fams = list(FAMILIES)
    out: List[CaseSpec] = []
    for cid in range(n_cases):
        fam = rng.choice(fams)
        op = rng.choice(FAMILIES[fam])
        dtype = rng.choice(list(DTYPES))
        numel = int(2 ** rng.uniform(8.0, max_log2))
        edge = rng.choice(EDGE_KINDS) if rng.random() < edge_fraction else ""
        out.append(_make_sweep_case(rng, cid, fam, op, dtype, numel, edge, seed * 1_000_003 + cid))
    return out


def _make_sweep_case(rng, cid, fam, op, dtype, numel, edge, seed) -> CaseSpec:
    extra: Dict[str, object] = {}
    if fam == "elementwise":
        r, c = _split2(rng, numel)
        shape = (r, c)
        if edge == "zero":
            shape = (0, c)
        if edge == "bcast":
            if op in ("add.Tensor", "mul.Tensor"):
                extra["other_shape"] = rng.choice([(1, c), (r, 1), (1, 1)])
            elif op == "where.self":
                extra["cond_shape"] = rng.choice([(1, c), (r, 1)])
            else:
                edge = "naninf"
        if op == "add.Tensor" and rng.random() < 0.3:
            extra["alpha"] = rng.choice([2, 0.5, -1])
    elif fam == "reduce":
        r, c = _split2(rng, numel, 3, 13)
        shape = (r, c)
        if edge == "bcast":
            shape = (r, 1) if rng.random() < 0.5 else (1, c)
        if edge == "zero":
            shape = (0, c)
        if op == "native_layer_norm.default":
            if edge == "transposed":
                edge = "naninf"
        else:
            dim = rng.choice([-1, -1, -1, 0])
            if op == "sum.dim_IntList":
                extra["dim"] = (dim,)
                extra["keepdim"] = rng.random() < 0.3
            else:
                extra["dim"] = dim
    elif fam == "gemm":
        k = 1 << rng.randint(5, 12)
        if rng.random() < 0.2:
            k += rng.choice((1, 8, 24))  # K off the 64-element tile grid / off alignment
        if op == "bmm.default":
            b = 1 << rng.randint(0, 6)
            m, n = _split2(rng, max(numel // b, 64), 3, 11)
            m, n, k = min(m, 1 << 13), min(n, 1 << 13), min(k, 1 << 10)
            shape = (b, m, k, n)
            if edge == "zero":
                shape = rng.choice([(0, m, k, n), (b, 0, k, n), (b, m, 0, n)])
            if edge == "bcast":
                shape = (b, 1, k, n)
        else:
            m, n = _split2(rng, numel, 3, 12)
            m, n = min(m, 1 << 14), min(n, 1 << 14)
            while m * k > (1 << 26) or k * n > (1 << 26):
                k //= 2
            shape = (m, k, n)
            if edge == "zero":
                shape = rng.choice([(0, k, n), (m, 0, n), (m, k, 0)])
            if edge == "bcast":
                shape = (1, k, n) if rng.random() < 0.5 else (m, k, 1)
            if op == "addmm.default":
                extra["bias_shape"] = rng.choice([(shape[2],), (shape[0], shape[2]), (1, shape[2]), (shape[0], 1)])
                if rng.random() < 0.3:
                    extra["beta"] = rng.choice([0, 0.5, 2])
                    extra["alpha"] = rng.choice([1, 0.5, 2])
    else:  # indexing
        if op in ("embedding.default", "index_select.default"):
            d = 1 << rng.randint(3, 12)
            n_idx = max(numel // d, 1)
            v = 1 << rng.randint(4, 17)
            while v * d > (1 << 27):
                v //= 2
            shape = (v, d)
            extra["n_idx"] = n_idx
            if op == "index_select.default":
                extra["dim"] = 0 if rng.random() < 0.7 else 1
                if extra["dim"] == 1:
                    extra["n_idx"] = max(min(n_idx, 4 * d), 1)
            else:
                extra["idx32"] = rng.random() < 0.25
                if edge == "transposed":
                    edge = "naninf"
            if edge == "zero":
                extra["n_idx"] = 0
            if edge == "bcast":
                extra["n_idx"] = 1
        elif op in ("gather.default", "scatter_add.default"):
            r, c = _split2(rng, min(numel, 1 << 24), 3, 13)
            shape = (r, c)
            extra["dim"] = rng.choice([0, 0, 1])
            if edge == "zero":
                extra["index_shape"] = (0, c)
            elif edge == "bcast":
                extra["index_shape"] = (1, c) if extra["dim"] == 0 else (r, 1)
            elif rng.random() < 0.3:
                extra["index_shape"] = (max(r // 2, 1), c)
            if op == "scatter_add.default" and edge == "transposed":
                edge = "naninf"
        else:  # argmax
            r, c = _split2(rng, numel, 3, 15)
            shape = (r, c)
            extra["dim"] = rng.choice([-1, -1, 0, None])
            extra["keepdim"] = extra["dim"] is not None and rng.random() < 0.3
            if edge == "zero":
                shape, extra["dim"] = (0, c), -1
            if edge == "bcast":
                shape = (r, 1) if extra["dim"] != 0 else (1, c)
    return CaseSpec(cid, op, dtype, tuple(shape), seed, tuple(sorted(extra.items(), key=lambda kv: kv[0])), edge, fam)
