"""Generate the golden vectors under tests/golden/ from the reference's own code.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's pure-PyTorch core `dcnv3_core_pytorch`
(classification/ops_dcnv3/functions/dcnv3_func.py:172-220) UNMODIFIED by file
path (loader: oracle/ref_core.py), runs it on seeded inputs, differentiates it with
autograd, and stores inputs and results as small `.npz` fixtures.  The test
suite then checks the C oracle and the CUDA kernels against these files; the
reference checkout is not needed at test time.

DCNv4 without softmax is the DCNv3 core fed with an un-normalised mask, which is
how the reference's own DCNv4 scripts compare the two
(DCNv4_op/scripts/test_dcnv4.py:80-84); the adapter below only re-slices the
packed offset_mask tensor into the core's separate offset / mask arguments.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import inputs as oin  # noqa: E402
from oracle import ref_core  # noqa: E402
from oracle.ref_core import repack_grads, split_packed  # noqa: E402


# name -> (N,H,W,G,D, kh,kw,sh,sw,ph,pw,dh,dw, offset_scale, remove_center, offset_std, seed)
CASES = {
    # padded size 16 is a power of two: the core's fp32 linspace grid is exact there
    "pow2_14": (1, 14, 14, 4, 16, 3, 3, 1, 1, 1, 1, 1, 1, 1.0, 0, 1.0, 1),
    "pow2_scale2": (1, 14, 14, 2, 16, 3, 3, 1, 1, 1, 1, 1, 1, 2.0, 0, 1.0, 2),
    "pow2_scale_half": (1, 14, 14, 2, 16, 3, 3, 1, 1, 1, 1, 1, 1, 0.5, 0, 2.0, 3),
    "pow2_far_offsets": (1, 6, 6, 2, 16, 3, 3, 1, 1, 1, 1, 1, 1, 1.0, 0, 6.0, 4),
    "pow2_remove_center": (1, 14, 14, 2, 16, 3, 3, 1, 1, 1, 1, 1, 1, 1.0, 1, 1.0, 5),
    "stride2": (1, 14, 14, 2, 16, 3, 3, 2, 2, 1, 1, 1, 1, 1.0, 0, 1.0, 6),
    "dil2_pad2": (1, 12, 12, 2, 16, 3, 3, 1, 1, 2, 2, 2, 2, 1.0, 0, 1.0, 7),
    "odd_9x11": (2, 9, 11, 3, 32, 3, 3, 1, 1, 1, 1, 1, 1, 1.0, 0, 1.5, 8),
}


def run_case(core, spec, dtype):
    (N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw, scale, rc, ostd, seed) = spec
    K = kh * kw - rc
    t = oin.dcnv4_inputs(N, H, W, G, D, kh=kh, kw=kw, sh=sh, sw=sw, ph=ph, pw=pw, dh=dh, dw=dw,
                         remove_center=rc, seed=seed, offset_std=ostd)
    v = t["value"].to(dtype).requires_grad_(True)
    om = t["offset_mask"].to(dtype)
    off, msk = split_packed(om, G, K)
    off.requires_grad_(True)
    msk.requires_grad_(True)
    out = core(v, off, msk, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, rc)
    go = t["grad_out"].to(dtype)
    gv, goff, gmsk = torch.autograd.grad(out, (v, off, msk), go)
    gom = repack_grads(goff, gmsk, G, K, om.shape[-1])
    return t, out.detach(), gv, gom


def main(ref_root: str):
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    core = ref_core.load(ref_root)

    small = {}
    for name, spec in CASES.items():
        t, out, gv, gom = run_case(core, spec, torch.float64)
        small[f"{name}/spec"] = np.array(spec, dtype=np.float64)
        small[f"{name}/value"] = t["value"].numpy()
        small[f"{name}/offset_mask"] = t["offset_mask"].numpy()
        small[f"{name}/grad_out"] = t["grad_out"].numpy()
        small[f"{name}/out"] = out.numpy()
        small[f"{name}/grad_value"] = gv.numpy()
        small[f"{name}/grad_offset_mask"] = gom.numpy()
        print(name, tuple(out.shape), float(out.abs().max()))
    np.savez_compressed(os.path.join(HERE, "dcnv4_ref_core_small.npz"), **small)

    # Benchmark configuration 0: N=2, 56x56, C=64, G=4x16, 3x3/s1/p1/d1, scale 1.0, seed 0, fp32.
    spec0 = (2, 56, 56, 4, 16, 3, 3, 1, 1, 1, 1, 1, 1, 1.0, 0, 1.0, 0)
    t, out32, _, _ = run_case(core, spec0, torch.float32)
    _, out64, gv64, gom64 = run_case(core, spec0, torch.float64)
    # keep the fixture small: every 9th query of the fp32 output, every 29th of the fp64 results
    q32 = torch.arange(0, 2 * 56 * 56, 9)
    q64 = torch.arange(0, 2 * 56 * 56, 29)
    cfg0 = {
        "spec": np.array(spec0, dtype=np.float64),
        "input_checksums": np.array([t["value"].double().sum().item(),
                                     t["offset_mask"].double().sum().item(),
                                     t["grad_out"].double().sum().item(),
                                     t["value"].double().abs().sum().item()]),
        "q32": q32.numpy(), "q64": q64.numpy(),
        "out_fp32": out32.reshape(-1, 64)[q32].numpy(),
        "out_fp64": out64.reshape(-1, 64)[q64].numpy().astype(np.float64),
        "grad_value_fp64": gv64.reshape(-1, 64)[q64].numpy(),
        "grad_offset_mask_fp64": gom64.reshape(-1, gom64.shape[-1])[q64].numpy(),
    }
    np.savez_compressed(os.path.join(HERE, "dcnv4_ref_core_cfg0.npz"), **cfg0)
    for f in ("dcnv4_ref_core_small.npz", "dcnv4_ref_core_cfg0.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else ref_core.reference_root()
    if root is None:
        raise SystemExit("usage: make_golden.py /path/to/reference (or set DCNV4_REFERENCE_ROOT)")
    main(root)
