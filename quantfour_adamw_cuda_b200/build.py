"""Build recipe of libquantfour_b200.so (plain nvcc, sm_100a only, no torch headers).

    python -m quantfour_adamw_cuda_b200.build [--force] [--verbose]

The library is built in-tree next to this file.  It takes the place of the reference's
setup.py / CUDAExtension build (optim/setup.py:1-23).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libquantfour_b200.so")
SOURCES = ["qf_api.cu"]

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    # every floating-point operation that matters is an explicit *_rn intrinsic; contraction is
    # switched off as well so that nothing else can be fused behind our back
    "-fmad=false", "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    # every file of csrc/ is a dependency: a stale library would pass or fail the tests for the wrong source
    deps = [os.path.join(CSRC, d) for d in sorted(os.listdir(CSRC)) if d.endswith((".cu", ".cuh", ".h"))]
    deps.append(os.path.join(INCLUDE, "quantfour_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", INCLUDE, "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
