"""Golden vectors from the reference's own CUDA extension (run on a GPU box).

    python oracle/build_ref.py /path/to/reference      # where the reference is mounted (no GPU needed)
    python tests/golden/make_golden_ref_cuda.py OUTDIR # on a machine with a CUDA GPU

Runs the UNMODIFIED reference kernels (FlashDeformAttn forward/backward and DCNv4
forward/backward, DCNv4_op/src/cuda/*.cuh via DCNv4_op/src/vision.cpp:14-21) on seeded inputs
and stores inputs (as seeds/specs) and sub-sampled outputs in `ref_cuda_golden.npz`.  Only shapes
whose index arithmetic was checked by reading are used: every FlashDeformAttn location lies
inside the map (the reference backward reads an unwritten shared-memory slot otherwise,
flash_deform_col2im_cuda.cuh:272-316) and the block multiplier divides the query count of one
image (the reference's blocks otherwise straddle images, dcnv4_im2col_cuda.cuh:153-154).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import inputs as oin, ref_cuda  # noqa: E402

# name -> (B, levels, G, D, K, Len_q, seed)
FDA_CASES = {
    "detr_small_k4": (2, ((20, 30), (10, 15), (5, 8), (3, 4)), 8, 32, 4, 704, 0),
    "detr_small_k8": (1, ((20, 30), (10, 15), (5, 8), (3, 4)), 8, 32, 8, 320, 1),
    "two_levels_d16": (2, ((12, 16), (6, 8)), 4, 16, 4, 256, 2),
}
# name -> (N, HW, G, D, seed): 3x3/s1/p1/d1, scale 1.0
DCN_CASES = {"n64_56": (64, 56, 4, 16, 0), "n64_28": (64, 28, 8, 16, 1), "n8_16": (8, 16, 4, 16, 2)}


def main(outdir):
    dev = "cuda"
    out = {}
    for name, (B, levels, G, D, K, Lq, seed) in FDA_CASES.items():
        t = oin.fda_inputs(B, levels, G, D, K, Len_q=Lq, seed=seed, loc_lo=0.02, loc_hi=0.98, device=dev)
        y = ref_cuda.fda_forward(t["value"], t["spatial_shapes"], t["level_start_index"], t["sampling_loc_attn"], K)
        gv, gs = ref_cuda.fda_backward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                       t["sampling_loc_attn"], t["grad_out"], K)
        torch.cuda.synchronize()
        out[f"fda/{name}/spec"] = np.array([B, G, D, K, Lq, seed] + [v for hw in levels for v in hw], dtype=np.int64)
        out[f"fda/{name}/out"] = y.cpu().numpy()[:, ::8]
        out[f"fda/{name}/grad_value"] = gv.cpu().numpy()[:, ::8]
        out[f"fda/{name}/grad_sla"] = gs.cpu().numpy()[:, ::8]
        print(name, tuple(y.shape), float(y.abs().max()))
    for name, (N, HW, G, D, seed) in DCN_CASES.items():
        t = oin.dcnv4_inputs(N, HW, HW, G, D, seed=seed, device=dev)
        a = (3, 3, 1, 1, 1, 1, 1, 1, G, D, 1.0, 0)
        y = ref_cuda.dcnv4_forward(t["value"], t["offset_mask"], *a)
        gv, gom = ref_cuda.dcnv4_backward(t["value"], t["offset_mask"], t["grad_out"], *a)
        torch.cuda.synchronize()
        step = max(1, (N * HW * HW) // 500)
        out[f"dcn/{name}/spec"] = np.array([N, HW, G, D, seed, step], dtype=np.int64)
        out[f"dcn/{name}/out"] = y.reshape(-1, G * D)[::step].cpu().numpy()
        out[f"dcn/{name}/grad_value"] = gv.reshape(-1, G * D)[::step].cpu().numpy()
        out[f"dcn/{name}/grad_offset_mask"] = gom.reshape(-1, gom.shape[-1])[::step].cpu().numpy()
        print(name, tuple(y.shape), float(y.abs().max()))
    os.makedirs(outdir, exist_ok=True)
    path = os.path.join(outdir, "ref_cuda_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
