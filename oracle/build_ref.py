"""Build the reference's own CUDA extension, unmodified, for sm_100 -- second parity target and
"kernel to beat".  TEST / BENCHMARK INFRASTRUCTURE ONLY; nothing in the product package uses it.

    python oracle/build_ref.py /path/to/reference      ->  oracle/_ref/dcnv4_ref_ext.so

The three translation units of the reference's extension (DCNv4_op/src/vision.cpp,
DCNv4_op/src/cuda/dcnv4_cuda.cu, DCNv4_op/src/cuda/flash_deform_attn_cuda.cu) are compiled
where they lie with nvcc and the flags of the reference's setup.py (DCNv4_op/setup.py:40-46),
plus `-gencode arch=compute_100,code=sm_100`; its own build system is not run (setup.py refuses
to build without a visible GPU, setup.py:36-48).  Only oracle/_ref/ (git-ignored) is written: the
built module, and a byte-for-byte install of the reference's pure-PyTorch core file (the timed CPU
baseline, see oracle/ref_core.py) -- no reference source enters this repository's history.  The result is a regular PyTorch extension module
exporting dcnv4_forward/backward and flash_deform_attn_forward/backward
(DCNv4_op/src/vision.cpp:14-21); `load()` imports it by path.
"""
from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "dcnv4_ref_ext"
LIB = os.path.join(OUT, NAME + ".so")


def install_python_core(ref_root: str) -> str:
    """Place the reference's pure-PyTorch core file, byte for byte, under oracle/_ref/ (git-ignored)
    so that the CPU baseline of bench.py is the reference's own code on machines without the checkout."""
    import shutil
    try:
        from . import ref_core
    except ImportError:  # run as a script: this directory is sys.path[0]
        import ref_core
    src = os.path.join(ref_root, ref_core.REL_PATH)
    if not os.path.isfile(src):
        raise FileNotFoundError(f"reference core not found at {src}")
    os.makedirs(OUT, exist_ok=True)
    shutil.copyfile(src, ref_core.INSTALLED)
    return ref_core.INSTALLED


def build(ref_root: str, force: bool = False) -> str:
    src = os.path.join(ref_root, "DCNv4_op", "src")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"reference sources not found under {src}")
    install_python_core(ref_root)
    if os.path.exists(LIB) and not force:
        return LIB
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT, exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}", f"-I{src}"]
    common = ["-DWITH_CUDA", f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-std=c++17", "-O3",
              "-Xcompiler", "-fPIC", "-w"]
    nvcc_ref = ["-DCUDA_HAS_FP16=1", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                "-D__CUDA_NO_HALF2_OPERATORS__", "-gencode", "arch=compute_100,code=sm_100"]
    units = [("vision.cpp", os.path.join(src, "vision.cpp")),
             ("dcnv4_cuda.cu", os.path.join(src, "cuda", "dcnv4_cuda.cu")),
             ("flash_deform_attn_cuda.cu", os.path.join(src, "cuda", "flash_deform_attn_cuda.cu"))]

    def one(u):
        name, path = u
        obj = os.path.join(OUT, name + ".o")
        cmd = ["nvcc", "-x", "cu", *common, *nvcc_ref, *inc, "-c", path, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=1800)
        if r.returncode != 0:
            sys.stderr.write(r.stdout[-4000:] + r.stderr[-4000:])
            raise RuntimeError(f"nvcc failed on {name}")
        return obj

    with ThreadPoolExecutor(max_workers=3) as ex:
        objs = list(ex.map(one, units))
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    link = ["nvcc", "-shared", "-o", LIB, *objs, f"-L{libdir}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch", "-ltorch_python", "-Xlinker", f"-rpath={libdir}"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    for o in objs:
        os.remove(o)
    return LIB


def load():
    """Import the built module (needs torch; CUDA is only needed to call it)."""
    if not os.path.exists(LIB):
        raise FileNotFoundError(f"{LIB} not built (run oracle/build_ref.py where the reference is mounted)")
    import torch  # noqa: F401  (loads libtorch before the extension)
    spec = importlib.util.spec_from_file_location(NAME, LIB)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    import ref_core as _rc
    _root = next((a for a in sys.argv[1:] if not a.startswith("--")), None) or _rc.reference_root()
    if _root is None:
        raise SystemExit("usage: build_ref.py /path/to/reference (or set DCNV4_REFERENCE_ROOT)")
    print(build(_root, force="--force" in sys.argv))
