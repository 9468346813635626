"""Run one named operator configuration on the current GPU a few times and print its
device time -- the small, self-contained command used for profiler captures.

    python -m backendbench_b200.run_case --case softmax_bf16_8192x4096 [--scale 4] [--reps 3] [--warmup 2]
    python -m backendbench_b200.run_case --label "mm.default[f32][16384, 1024, 19]"   # a case of the 512-case sweep
    python -m backendbench_b200.run_case --list

`--scale F` divides the leading extent by F (same operator, same row length) so that a
full-metrics profiler capture holds a few hundred MB instead of GBs.
"""

from __future__ import annotations

import argparse
import json

import torch

from .backends import B200Backend
from .cases import named_case, named_cases, neighbour_cases, scaled_down
from .eval import cuda_bench
from .opregistry import get_operator


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case")
    ap.add_argument("--label", help="a case of the 512-case sweep, by its label")
    ap.add_argument("--scale", type=int, default=1)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--rotate", action="store_true", help="time back-to-back launches over rotating input sets larger than L2 instead of flushing L2 before every launch")
    ap.add_argument("--graph", action="store_true", help="with --rotate: capture the loop in a CUDA graph and time the replay (device time without the host's launch cost)")
    ap.add_argument("--compare", action="store_true", help="time the fused compare kernel on (aten result, backend result) of the case instead of the operator")
    ap.add_argument("--list", action="store_true")
    args = ap.parse_args()
    if args.label:
        from .cases import sweep_cases

        found = [c for c in sweep_cases(512, 0) if c.label() == args.label]
        if not found:
            raise SystemExit(f"no sweep case labelled {args.label!r}")
        case = found[0]
    elif args.list or not args.case:
        print("\n".join(c.name for c in named_cases() + neighbour_cases()))
        return
    else:
        case = named_case(args.case)
    if args.scale > 1:
        case = scaled_down(case, args.scale)
    op = get_operator(case.op)
    impl = B200Backend()[op]
    if args.compare:
        from .eval import compare_enqueue

        a, kw = case.build("cuda")
        ref, res = op(*a, **kw), impl(*a, **kw)
        rec = torch.zeros(8, dtype=torch.int32, device="cuda")
        ms = cuda_bench(lambda: compare_enqueue(ref, res, 1e-4, 1e-4, rec), warmup=args.warmup, reps=args.reps)
        first = ref[0] if isinstance(ref, (tuple, list)) else ref
        nbytes = 2 * first.numel() * first.element_size()
        print(json.dumps({"case": case.label(), "kernel": "compare", "ms": round(ms, 5), "algorithmic_bytes": nbytes, "gbs": round(nbytes / ms / 1e6, 1)}))
        return
    if args.rotate:
        from dataclasses import replace

        from .eval import cuda_bench_rotating

        nsets = max(2, min(8, -(-2 * (126 << 20) // max(case.algorithmic_bytes(), 1))))
        sets = [replace(case, seed=case.seed + i).build("cuda") for i in range(nsets)]
        ms = cuda_bench_rotating([(lambda a=a, k=k: impl(*a, **k)) for a, k in sets], reps=max(args.reps, 20), graph=args.graph)
    else:
        a, kw = case.build("cuda")
        ms = cuda_bench(lambda: impl(*a, **kw), warmup=args.warmup, reps=args.reps)
    out = {"case": case.label(), "ms": round(ms, 5), "algorithmic_bytes": case.algorithmic_bytes(), "gbs": round(case.algorithmic_bytes() / ms / 1e6, 1)}
    if case.flops():
        out["tflops"] = round(case.flops() / ms / 1e9, 2)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
