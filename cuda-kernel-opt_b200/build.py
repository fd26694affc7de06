"""Builds libb200gemm.so (the C-ABI shared library) in-tree with nvcc for sm_100a.

    python cuda-kernel-opt_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU. The library links the CUDA runtime only; the driver's
tensor-map encoder is resolved at run time through cudaGetDriverEntryPoint.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200gemm.so")
SOURCES = ["gemm_sm100.cu", "api.cu", "gemm_noalloc.cu"]
HEADERS = ["gemm_sm100.cuh", "ptx_sm100.cuh", "plan.h", "schedule.h", "synth.h", os.path.join("..", "..", "include", "b200_gemm.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--shared", "-cudart", "shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, defines=(), out: str | None = None) -> str:
    """defines: extra -D flags for diagnostic builds (-DB200_TIMELINE: %globaltimer stamps of set-up and
    role milestones in a 32-slot profile buffer). out: write the library elsewhere (a diagnostic build
    beside the normal one; load it with B200_GEMM_LIB=<path>)."""
    if out is None and not defines and not force and not needs_build():
        return LIB
    target = out or LIB
    cmd = [_nvcc()] + NVCC_FLAGS + list(defines) + (["-Xptxas", "-v"] if verbose else []) + ["-o", target] + [os.path.join(CSRC, s) for s in SOURCES]
    env = dict(os.environ)
    # the image exports CC/CXX pointing at a wrapper compiler; nvcc needs the system g++
    if os.path.exists("/usr/bin/g++"):
        cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libb200gemm.so")
    return target


if __name__ == "__main__":
    _out = sys.argv[sys.argv.index("--out") + 1] if "--out" in sys.argv else None
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, defines=[a for a in sys.argv[1:] if a.startswith("-D")], out=_out))
