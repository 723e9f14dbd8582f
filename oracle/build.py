"""Build recipe for the CPU oracle (test infrastructure, never the product path).

`build()` compiles `dcn_oracle.c` next to this file into `oracle/_build/libdcn_oracle.so`
with gcc.  `-ffp-contract=off` keeps gcc from fusing multiply-adds on its own: the
only fused operations are the explicit `fmaf` calls that mirror the reference
kernels' coordinate arithmetic.  No `-march=native`, because the library is built on
one machine and loaded on another.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "dcn_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libdcn_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = [
        "gcc", "-O2", "-fPIC", "-shared", "-std=c11", "-fopenmp", "-ffp-contract=off",
        "-Wall", "-Wextra", "-o", LIB, SRC, "-lm",
    ]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
