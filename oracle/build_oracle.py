"""Build recipe for the C oracle (test infrastructure; never imported by the shipped package).

    python oracle/build_oracle.py

compiles oracle/qf_oracle.c into oracle/libqf_oracle.so with gcc.  -ffp-contract=off keeps
every binary32 operation separately rounded (the fused multiply-adds in the source are explicit
fmaf calls); -fopenmp spreads blocks and rows over the host cores for the timed CPU baseline.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "qf_oracle.c")
OUT = os.path.join(HERE, "libqf_oracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = [
        "gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fopenmp",
        "-ffp-contract=off", "-fno-fast-math", "-fno-math-errno", "-mavx2", "-mfma",
        "-Wall", "-Wextra", "-o", OUT, SRC, "-lm",
    ]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
