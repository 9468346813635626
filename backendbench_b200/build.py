"""Build libb200ops.so in-tree: `python -m backendbench_b200.build [--verbose] [--force]`.

Runs the Makefile in csrc/ (nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo).
nvcc cross-compiles without a GPU; the resulting shared object is what `_abi.lib()` loads.
"""

from __future__ import annotations

import os
import subprocess
import sys

from ._abi import CSRC_DIR, LIB_PATH


def build(verbose: bool = False, force: bool = False, jobs: int = 0) -> str:
    jobs = jobs or min(os.cpu_count() or 4, 16)
    cmd = ["make", "-C", CSRC_DIR, f"-j{jobs}"]
    if force:
        cmd.append("-B")
    if verbose:
        cmd.append("VERBOSE=1")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or proc.returncode != 0:
        sys.stdout.write(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError(f"building {LIB_PATH} failed (exit {proc.returncode})")
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
