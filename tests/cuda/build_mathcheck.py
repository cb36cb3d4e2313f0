"""Build tests/cuda/libqf_mathcheck.so (device-side checks of the fast-path arithmetic; test infrastructure)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SRC = os.path.join(HERE, "math_check.cu")
OUT = os.path.join(HERE, "libqf_mathcheck.so")
CSRC = os.path.join(ROOT, "quantfour_adamw_cuda_b200", "csrc")


def build(force: bool = False) -> str:
    deps = [SRC] + [os.path.join(CSRC, f) for f in ("qf_math.cuh", "qf_kernels.cuh", "qf_device.cuh")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps):
        return OUT
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    subprocess.run([nvcc if os.path.exists(nvcc) else "nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                    "-lineinfo", "-fmad=false", "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared",
                    "-I", os.path.join(ROOT, "include"), "-o", OUT, SRC], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
