"""Build libb200moe.so in-tree with nvcc for sm_100a (no torch headers, no JIT cache).

    python -m justgoal_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200moe.so")
SOURCES = ["b200moe.cu"]
HEADERS = ["common.cuh", "routing.cuh", "permute.cuh", "front.cuh", "ep_p2p.cuh", "gemm.cuh", "gemm_pair.cuh", "quant.cuh", os.path.join("..", "..", "include", "b200moe.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libb200moe.so cannot be built")


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False, out: str = None) -> str:
    """`out`: build to another path (kernel variants for A/B timing, loaded through B200MOE_LIB)."""
    if out is None and not force and not needs_build():
        return LIB
    cmd = [_nvcc(), "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC", "-I", os.path.join(HERE, "..", "include"),
           "-o", out or LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    extra = os.environ.get("B200MOE_NVCC_FLAGS")      # e.g. -DB200MOE_ENABLE_ABLATE for timing experiments
    if extra:
        cmd[1:1] = extra.split()
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError("nvcc failed building libb200moe.so")
    return out or LIB


if __name__ == "__main__":
    _out = sys.argv[sys.argv.index("--out") + 1] if "--out" in sys.argv else None
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, out=_out))
