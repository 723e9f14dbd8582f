"""Element-wise parity at the benchmark's FULL sizes.

The operators are per-image: output and gradients of image b depend on image b's tensors only
(DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:163,199-201, dcnv4_col2im_cuda.cuh:287,
flash_deform_im2col_cuda.cuh:145-146,182).  So the GPU runs the whole batch -- the launch
geometry, tile walk and image straddling of the real benchmark call -- and the CPU oracle checks
a few WHOLE images of it (first, middle, last), every element, forward and both gradients.
"""
import os

import pytest
import torch

from oracle import cref, inputs as oin
from tests.util import BWD_TOL, FWD_TOL, close

pytestmark = pytest.mark.gpu
DEV = "cuda"

STAGES = [(64, 56, 64, 4), (64, 28, 128, 8), (64, 14, 256, 16), (64, 7, 512, 32)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16"])
@pytest.mark.parametrize("shape", STAGES, ids=lambda s: f"{s[0]}x{s[1]}x{s[1]}x{s[2]}")
def test_dcnv4_stage_shapes_batch64_against_oracle(shape, dtype):
    """Benchmark configuration 1: N=64 at each FlashInternImage-T stage shape."""
    from dcnv4_b200 import ops
    N, HW, C, G = shape
    D = C // G
    t = oin.dcnv4_inputs(N, HW, HW, G, D, seed=31 + HW, dtype=dtype, device=DEV)
    a = (3, 3, 1, 1, 1, 1, 1, 1, G, D, 1.0)
    out = ops.dcnv4_forward(t["value"], t["offset_mask"], *a, 256, 0)
    gv, gom = ops.dcnv4_backward(t["value"], t["offset_mask"], *a, 256, t["grad_out"], 0)
    for b in (0, N // 2 - 1, N - 1):
        v, om, go = (t[k][b:b + 1].float().cpu() for k in ("value", "offset_mask", "grad_out"))
        ref_out = cref.dcnv4_forward(v, om, *a, 0)
        ref_gv, ref_gom = cref.dcnv4_backward(v, om, go, *a, 0)
        close(out[b:b + 1], ref_out, FWD_TOL[dtype], f"forward, image {b}")
        close(gv[b:b + 1], ref_gv, BWD_TOL[dtype], f"grad_value, image {b}")
        close(gom[b:b + 1], ref_gom, BWD_TOL[dtype], f"grad_offset_mask, image {b}")
    used = 27 * G
    if gom.shape[-1] > used:
        assert float(gom[..., used:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16"])
@pytest.mark.parametrize("levels", [oin.DETR_LEVELS, oin.DETR_LEVELS_ALT], ids=["len20197", "len19947"])
def test_flash_deform_attn_detr_encoder_shape_against_oracle(levels, dtype):
    """Benchmark configuration 2 (8 images, 8 heads x 32 channels, 4 levels x 4 points), in both
    readings of its level sizes: 100x152.. (20,197 positions) and 100x150.. (19,947 positions)."""
    from dcnv4_b200 import ops
    B, G, D, K = 8, 8, 32, 4
    t = oin.fda_inputs(B, levels, G, D, K, seed=41, dtype=dtype, device=DEV)
    Len = t["value"].shape[1]
    assert Len == sum(h * w for h, w in levels)
    out = ops.flash_deform_attn_forward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                        t["sampling_loc_attn"], 64, K)
    gv, gs = ops.flash_deform_attn_backward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                            t["sampling_loc_attn"], t["grad_out"], 64, K)
    ss, ls = t["spatial_shapes"].cpu(), t["level_start_index"].cpu()
    tol_loc = dict(BWD_TOL[dtype])
    tol_loc["atol"] = tol_loc["atol"] * 152      # location gradients carry the level size as a factor
    for b in (0, B - 1):
        v, sla, go = (t[k][b:b + 1].float().cpu() for k in ("value", "sampling_loc_attn", "grad_out"))
        ref_out = cref.fda_forward(v, ss, ls, sla, K)
        ref_gv, ref_gs = cref.fda_backward(v, ss, ls, sla, go, K)
        close(out[b:b + 1], ref_out, FWD_TOL[dtype], f"forward, image {b}")
        close(gv[b:b + 1], ref_gv, BWD_TOL[dtype], f"grad_value, image {b}")
        close(gs[b:b + 1], ref_gs, tol_loc, f"grad_sampling_loc_attn, image {b}")


# ------------------------------------------------------------ the opt-in tiled kernels

def _tiled(on: bool):
    if on:
        os.environ["DCNV4B200_TILED"] = "1"
    else:
        os.environ.pop("DCNV4B200_TILED", None)


TILED_CASES = {
    # N, H, W, G, offset_scale, offset_std, pad
    "stage1_n3": (3, 56, 56, 4, 1.0, 1.0, 1),
    "stage2_n3": (3, 28, 28, 8, 1.0, 1.0, 1),
    "stage3_n5": (5, 14, 14, 16, 1.0, 1.0, 1),
    "stage4_n7": (7, 7, 7, 32, 1.0, 1.0, 1),
    "L_scale2_g80": (1, 8, 8, 80, 2.0, 1.0, 1),
    "far_offsets": (2, 13, 9, 3, 1.0, 6.0, 1),       # most points leave the staged box
    "ragged_19x23": (2, 19, 23, 2, 1.3, 2.0, 1),
    "one_query": (1, 1, 1, 1, 1.0, 0.3, 1),
    "pad0": (2, 12, 10, 2, 1.0, 1.0, 0),
    "pad2": (2, 12, 10, 2, 1.0, 1.0, 2),
    "tall_33x17": (1, 33, 17, 1, 0.5, 3.0, 1),
    "far_offsets_g4": (2, 13, 9, 4, 1.0, 6.0, 1),
    "ragged_19x23_g8": (2, 19, 23, 8, 1.3, 2.0, 1),
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("name", sorted(TILED_CASES))
def test_tiled_kernels_parity(name, dtype):
    """DCNV4B200_TILED=1 routes 3x3 / stride 1 / 16-channel-group calls through the kernels that stage the
    value tile with TMA box loads: the backward also pre-accumulates grad_value in shared memory, the
    forward (group counts that are multiples of four) gathers every corner from the staged box."""
    from dcnv4_b200 import ops
    N, H, W, G, scale, ostd, pad = TILED_CASES[name]
    t = oin.dcnv4_inputs(N, H, W, G, 16, ph=pad, pw=pad, seed=N * 100 + H, offset_std=ostd, dtype=dtype, device=DEV)
    a = (3, 3, 1, 1, pad, pad, 1, 1, G, 16, scale)
    v, om, go = (t[k].float().cpu() for k in ("value", "offset_mask", "grad_out"))
    ref_out = cref.dcnv4_forward(v, om, *a, 0)
    ref_gv, ref_gom = cref.dcnv4_backward(v, om, go, *a, 0)
    try:
        _tiled(True)
        out = ops.dcnv4_forward(t["value"], t["offset_mask"], *a, 256, 0)
        gv, gom = ops.dcnv4_backward(t["value"], t["offset_mask"], *a, 256, t["grad_out"], 0)
        torch.cuda.synchronize()
    finally:
        _tiled(False)
    close(out, ref_out, FWD_TOL[dtype], "forward")
    close(gv, ref_gv, BWD_TOL[dtype], "grad_value")
    close(gom, ref_gom, BWD_TOL[dtype], "grad_offset_mask")
    used = 27 * G
    if gom.shape[-1] > used:
        assert float(gom[..., used:].abs().max()) == 0.0, "pad columns must be exactly zero"
    # grad_offset_mask has no atomics on its path in either kernel; both evaluate the same fp32
    # expressions up to the order of a few additions
    gv2, gom2 = ops.dcnv4_backward(t["value"], t["offset_mask"], *a, 256, t["grad_out"], 0)
    close(gom, gom2.double(), BWD_TOL[dtype], "tiled vs default grad_offset_mask")
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16"])
def test_tiled_kernels_full_size_stage1(dtype):
    from dcnv4_b200 import ops
    N, HW, G = 64, 56, 4
    t = oin.dcnv4_inputs(N, HW, HW, G, 16, seed=77, dtype=dtype, device=DEV)
    a = (3, 3, 1, 1, 1, 1, 1, 1, G, 16, 1.0)
    try:
        _tiled(True)
        out = ops.dcnv4_forward(t["value"], t["offset_mask"], *a, 256, 0)
        gv, gom = ops.dcnv4_backward(t["value"], t["offset_mask"], *a, 256, t["grad_out"], 0)
        torch.cuda.synchronize()
    finally:
        _tiled(False)
    # identity sampling through the staged box: zero offsets, one-hot centre mask
    om1 = torch.zeros_like(t["offset_mask"])
    om1[..., : G * 27].view(N, HW, HW, G, 27)[..., 18 + 4] = 1.0
    try:
        _tiled(True)
        same = ops.dcnv4_forward(t["value"], om1, *a, 256, 0)
    finally:
        _tiled(False)
    assert torch.equal(same, t["value"]), "identity sampling must reproduce the input bit for bit"
    for b in (0, N - 1):
        v, om, go = (t[k][b:b + 1].float().cpu() for k in ("value", "offset_mask", "grad_out"))
        close(out[b:b + 1], cref.dcnv4_forward(v, om, *a, 0), FWD_TOL[dtype], f"forward, image {b}")
        ref_gv, ref_gom = cref.dcnv4_backward(v, om, go, *a, 0)
        close(gv[b:b + 1], ref_gv, BWD_TOL[dtype], f"grad_value, image {b}")
        close(gom[b:b + 1], ref_gom, BWD_TOL[dtype], f"grad_offset_mask, image {b}")
