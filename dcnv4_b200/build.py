"""Build the CUDA library in-tree: dcnv4_b200/csrc/*.cu -> dcnv4_b200/_C/libdcnv4_b200.so.

    python -m dcnv4_b200.build [--force] [--verbose]

Only sm_100a code is generated (`-gencode arch=compute_100a,code=sm_100a`); the CUDA runtime
is linked statically so the library has no dependency on the Python environment's CUDA
packages.  nvcc cross-compiles without a GPU, so this also runs on a CPU-only build machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_C")
LIB = os.path.join(OUT_DIR, "libdcnv4_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

SOURCES = ("api.cu", "dcnv4_fwd.cu", "dcnv4_bwd.cu", "dcnv4_bwd_tiled.cu", "dcnv4_fwd_tiled.cu", "dcnv4_fwd_fused.cu", "fda_fwd.cu", "fda_bwd.cu", "aux.cu", "layernorm.cu",
           "linear.cu", "bias_act.cu", "center_scale.cu")
ARCH = ("-gencode", "arch=compute_100a,code=sm_100a")
NVCC_FLAGS = ("-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr")


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the dcnv4_b200 CUDA library cannot be built")
    return exe


def _deps_mtime() -> float:
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "dcnv4_b200.h")]
    return max(os.path.getmtime(f) for f in files)


def is_current() -> bool:
    return os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and is_current():
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = _nvcc()
    extra = ("-Xptxas", "-v") if verbose else ()

    def compile_one(src: str) -> str:
        obj = os.path.join(OUT_DIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *ARCH, *NVCC_FLAGS, *extra, "-I", INCLUDE, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    link = [nvcc, *ARCH, "-shared", "-cudart", "static", "-o", LIB, *objs]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc link failed")
    for obj in objs:          # every source is recompiled on any change: the objects are of no further use
        os.remove(obj)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
