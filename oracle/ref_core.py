"""Loader and adapter of the reference's own pure-PyTorch core, `dcnv3_core_pytorch`
(classification/ops_dcnv3/functions/dcnv3_func.py:172-220), imported UNMODIFIED by file path.

TEST / BENCHMARK INFRASTRUCTURE ONLY (see the package docstring): it pins the C oracle through
the golden vectors (tests/golden/make_golden.py) and it is the timed CPU baseline of bench.py.

Where the file comes from, in this order:
  1. a reference checkout: the directory named by the DCNV4_REFERENCE_ROOT environment
     variable, else a directory called `reference` beside this repository;
  2. `oracle/_ref/dcnv3_func.py`, the byte-for-byte install that `oracle/build_ref.py` places
     there when it runs where the checkout is mounted.  `oracle/_ref/` is git-ignored (like the
     reference CUDA extension built into it), so no reference source enters this repository's
     history; the directory travels with a working copy to machines without the checkout.

The compiled `DCNv3` module and the `pkg_resources` version lookup that the file performs at
import time (dcnv3_func.py:18-19) are stubbed: both serve only the CUDA autograd function in
that file, which is never called here.

DCNv4 without softmax is the DCNv3 core fed with an un-normalised mask, which is how the
reference's own scripts compare the two (DCNv4_op/scripts/test_dcnv4.py:80-84); the adapter
only re-slices the packed offset_mask tensor into the core's separate offset / mask arguments.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types
from typing import Optional

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REL_PATH = os.path.join("classification", "ops_dcnv3", "functions", "dcnv3_func.py")
INSTALLED = os.path.join(HERE, "_ref", "dcnv3_func.py")

_core = None


def reference_root() -> Optional[str]:
    """Directory of a reference checkout, or None."""
    cands = [os.environ.get("DCNV4_REFERENCE_ROOT"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, REL_PATH)):
            return c
    return None


def source_path(ref_root: Optional[str] = None) -> Optional[str]:
    root = ref_root or reference_root()
    if root and os.path.isfile(os.path.join(root, REL_PATH)):
        return os.path.join(root, REL_PATH)
    return INSTALLED if os.path.isfile(INSTALLED) else None


def available() -> bool:
    return source_path() is not None


def load(ref_root: Optional[str] = None):
    """Return the reference's `dcnv3_core_pytorch` function."""
    global _core
    if _core is not None and ref_root is None:
        return _core
    path = source_path(ref_root)
    if path is None:
        raise FileNotFoundError("the reference's dcnv3_func.py is neither mounted nor installed under oracle/_ref")
    sys.modules.setdefault("DCNv3", types.ModuleType("DCNv3"))
    try:
        import pkg_resources  # noqa: F401
    except Exception:  # pragma: no cover
        sys.modules["pkg_resources"] = types.ModuleType("pkg_resources")
    import pkg_resources
    real = getattr(pkg_resources, "get_distribution", None)

    class _Dist:
        version = "1.1"

    def fake(name):
        if name == "DCNv3":
            return _Dist()
        return real(name)

    pkg_resources.get_distribution = fake
    try:
        spec = importlib.util.spec_from_file_location("ref_dcnv3_func", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        if real is not None:
            pkg_resources.get_distribution = real
    core = mod.dcnv3_core_pytorch
    if ref_root is None:
        _core = core
    return core


def split_packed(om: torch.Tensor, G: int, K: int):
    """Packed (N,Ho,Wo,Ppad) offset_mask -> the core's offset (N,Ho,Wo,G*K*2) and mask (N,Ho,Wo,G*K)."""
    N, Ho, Wo, _ = om.shape
    g = om[..., : G * K * 3].reshape(N, Ho, Wo, G, 3 * K)
    return (g[..., : 2 * K].reshape(N, Ho, Wo, G * K * 2),
            g[..., 2 * K:].reshape(N, Ho, Wo, G * K))


def repack_grads(goff, gmask, G, K, Ppad):
    """The core's offset / mask gradients -> the packed grad_offset_mask layout (pad columns zero)."""
    N, Ho, Wo, _ = goff.shape
    out = torch.zeros(N, Ho, Wo, Ppad, dtype=goff.dtype)
    out[..., : G * K * 3] = torch.cat(
        (goff.reshape(N, Ho, Wo, G, 2 * K), gmask.reshape(N, Ho, Wo, G, K)), -1
    ).reshape(N, Ho, Wo, G * K * 3)
    return out


def dcnv4_forward(core, value, offset_mask, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, rc):
    off, msk = split_packed(offset_mask, G, kh * kw - rc)
    return core(value, off, msk, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, rc)


def dcnv4_forward_backward(core, value, offset_mask, grad_out, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, rc):
    """Forward through the reference core and its autograd backward; returns (out, grad_value,
    grad_offset_mask) with the gradients in the packed layout."""
    K = kh * kw - rc
    v = value.detach().clone().requires_grad_(True)
    off, msk = split_packed(offset_mask.detach(), G, K)
    off = off.clone().requires_grad_(True)
    msk = msk.clone().requires_grad_(True)
    out = core(v, off, msk, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, rc)
    gv, goff, gmsk = torch.autograd.grad(out, (v, off, msk), grad_out)
    return out.detach(), gv, repack_grads(goff, gmsk, G, K, offset_mask.shape[-1])
