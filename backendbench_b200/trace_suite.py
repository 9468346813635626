"""Cases from serialized operator traces: the TorchBench-format suite.

The reference's largest suite replays argument signatures recorded from real models
(BackendBench/suite/torchbench.py:45-105). Its records come from a text trace

    Operator: aten.add.Tensor
    cnt: 12, ((T([8, 128], f16), T([128], f16)), {})

(grammar: BackendBench/data_loaders.py:43-91 for the lines, utils.py:100-182 for the argument
tuple) or from a parquet table with the columns `op_name`, `args`, `count`,
`included_in_benchmark`, ... (data_loaders.py:101-126). The public dataset itself is fetched
from the network by the reference and is not available offline; this module ingests a LOCAL
`.txt` or `.parquet` file in either form (`--suite torchbench
--alternative-torchbench-data-path FILE`, scripts/main.py:100-104 of the reference) and
produces the same per-operator tests: every distinct signature once, largest inputs first,
`topn` of them, tensors generated on the evaluating device when the test is run.
"""

from __future__ import annotations

import hashlib
import re
from typing import Dict, Iterable, Iterator, List, Optional

import torch

from .utils import deserialize_args

_OPERATOR = re.compile(r"Operator: (.*)")
_COUNTED = re.compile(r"cnt: (\d+), (.*)")
# a trace recorded before the overload was renamed
_RENAMED = {"aten.sum.SymInt": "aten.sum.dim_IntList"}


def parse_trace_lines(lines: Iterable, filter: Optional[List[str]] = None, limit: Optional[int] = None) -> List[Dict]:
    """Records {uuid, op_name, args, count, is_synthetic} in file order. `filter`: keep
    operators whose name contains any of the strings; `limit`: stop after that many
    `Operator:` headers."""
    records, op, seen = [], None, 0
    for line in lines:
        if isinstance(line, bytes):
            line = line.decode("utf-8")
        m = _OPERATOR.match(line)
        if m:
            seen += 1
            if limit and seen > limit:
                break
            op = _RENAMED.get(m.group(1).strip(), m.group(1).strip())
            continue
        m = _COUNTED.match(line)
        if m:
            if op is None:
                raise ValueError("trace: a `cnt:` line before any `Operator:` line")
            count, args = int(m.group(1)), m.group(2).rstrip("\n")
            if filter is None or any(f in op for f in filter):
                records.append({"uuid": hashlib.sha256(args.encode() + op.encode()).hexdigest(), "op_name": op, "args": args, "count": count, "is_synthetic": count == 0})
    return records


def load_ops_from_source(source: str, filter: Optional[List[str]] = None, limit: Optional[int] = None) -> List[Dict]:
    """Records of a local `.txt` trace or `.parquet` table (URLs are refused: no network)."""
    src = str(source)
    if src.startswith("http://") or src.startswith("https://"):
        raise ValueError("remote traces are not fetched; download the file and pass its path")
    if src.endswith(".txt"):
        with open(src, "r") as fh:
            return parse_trace_lines(fh, filter, limit)
    if src.endswith(".parquet"):
        import pyarrow.parquet as pq

        rows = pq.read_table(src).to_pylist()
        if filter:
            rows = [r for r in rows if any(f in r["op_name"] for f in filter)]
        return rows[:limit] if limit else rows
    raise ValueError(f"cannot tell the format of {source!r}: expected a .txt trace or a .parquet table")


def ops_to_benchmark_dict(records: List[Dict]) -> Dict[str, List[str]]:
    """op_name -> distinct argument strings, skipping rows a parquet table marks as excluded."""
    out: Dict[str, List[str]] = {}
    for r in records:
        if not r.get("included_in_benchmark", True):
            continue
        bucket = out.setdefault(r["op_name"], [])
        if r["args"] not in bucket:
            bucket.append(r["args"])
    return out


def resolve_operator(name: str):
    """"aten.add.Tensor" -> torch.ops.aten.add.Tensor, by attribute lookup (nothing is evaluated)."""
    obj = torch.ops
    for part in name.split("."):
        obj = getattr(obj, part)
    return obj


def args_nbytes(args) -> int:
    total = 0
    for a in args:
        if isinstance(a, torch.Tensor):
            total += a.numel() * a.element_size()
        elif isinstance(a, (tuple, list)):
            total += args_nbytes(a)
    return total


class TraceTest:
    """One recorded signature; `args` / `kwargs` are generated when first read, so a test
    can be pickled to a worker as its string."""

    def __init__(self, serialized: str):
        self.serialized = serialized
        self._made = None

    def _make(self):
        if self._made is None:
            self._made = deserialize_args(self.serialized)
        return self._made

    @property
    def args(self):
        return self._make()[0]

    @property
    def kwargs(self):
        return self._make()[1]

    def __getstate__(self):
        return {"serialized": self.serialized, "_made": None}


class TraceOpTest:
    def __init__(self, op_name: str, inputs: List[str], topn: Optional[int]):
        self.op = resolve_operator(op_name)
        self.inputs = inputs
        self.topn = topn

    def _ordered(self) -> List[str]:
        sized = []
        for s in self.inputs:
            args, kwargs = deserialize_args(s)
            sized.append((args_nbytes(args) + args_nbytes(list(kwargs.values())), s))
        ordered = [s for _, s in sorted(sized, reverse=True)]  # largest first; ties by the string, as the reference sorts
        return ordered if self.topn is None else ordered[: self.topn]

    @property
    def correctness_tests(self) -> Iterator[TraceTest]:
        return (TraceTest(s) for s in self._ordered())

    @property
    def performance_tests(self) -> Iterator[TraceTest]:
        return (TraceTest(s) for s in self._ordered())


class TraceTestSuite:
    """Iterates TraceOpTest per operator of the file; operators the installed torch does not
    have are skipped with their name kept in `unresolved`."""

    def __init__(self, name: str, filename: str, filter: Optional[List[str]] = None, topn: Optional[int] = None, limit: Optional[int] = None):
        self.name = name
        self.topn = topn
        self.optests = ops_to_benchmark_dict(load_ops_from_source(filename, filter, limit))
        self.unresolved: List[str] = []

    def __iter__(self) -> Iterator[TraceOpTest]:
        for op_name, inputs in self.optests.items():
            try:
                yield TraceOpTest(op_name, inputs, self.topn)
            except AttributeError:
                self.unresolved.append(op_name)
