"""Seeded random sweeps over the operators' parameter space against the CPU oracle: kernel sizes,
strides, pads, dilations, group counts and widths, remove_center, softmax, offset scales, ragged map
sizes, all three storage types -- the combinations no hand-written case list covers."""
import random

import pytest
import torch

from oracle import cref, inputs as oin
from tests.util import BWD_TOL, FWD_TOL, close

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _dcn_config(rng):
    while True:
        kh, kw = rng.choice([1, 2, 3, 3, 3, 4, 5]), rng.choice([1, 2, 3, 3, 3, 4, 5])
        sh, sw = rng.choice([1, 1, 2, 3]), rng.choice([1, 1, 2, 3])
        dh, dw = rng.choice([1, 1, 2, 3]), rng.choice([1, 1, 2, 3])
        ph, pw = rng.randint(0, 3), rng.randint(0, 3)
        H, W = rng.randint(1, 19), rng.randint(1, 19)
        if (H + 2 * ph - (dh * (kh - 1) + 1)) < 0 or (W + 2 * pw - (dw * (kw - 1) + 1)) < 0:
            continue
        rc = int(kh == kw and kh % 2 == 1 and kh > 1 and rng.random() < 0.3)
        return dict(N=rng.randint(1, 3), H=H, W=W, G=rng.randint(1, 5), D=rng.choice([8, 16, 16, 32, 48, 64]),
                    kh=kh, kw=kw, sh=sh, sw=sw, ph=ph, pw=pw, dh=dh, dw=dw, rc=rc,
                    scale=rng.choice([0.5, 1.0, 1.0, 1.7, 2.0]), ostd=rng.choice([0.5, 1.0, 3.0]),
                    softmax=rng.random() < 0.25)


@pytest.mark.parametrize("seed", range(36))
def test_dcnv4_random_configuration(seed):
    from dcnv4_b200 import ops
    rng = random.Random(1000 + seed)
    c = _dcn_config(rng)
    dtype = DTYPES[seed % 3]
    t = oin.dcnv4_inputs(c["N"], c["H"], c["W"], c["G"], c["D"], kh=c["kh"], kw=c["kw"], sh=c["sh"], sw=c["sw"],
                         ph=c["ph"], pw=c["pw"], dh=c["dh"], dw=c["dw"], remove_center=c["rc"], seed=seed,
                         offset_std=c["ostd"], dtype=dtype, device=DEV)
    a = (c["kh"], c["kw"], c["sh"], c["sw"], c["ph"], c["pw"], c["dh"], c["dw"], c["G"], c["D"], c["scale"])
    out = ops.dcnv4_forward(t["value"], t["offset_mask"], *a, 256, c["rc"], softmax=c["softmax"])
    gv, gom = ops.dcnv4_backward(t["value"], t["offset_mask"], *a, 256, t["grad_out"], c["rc"], softmax=c["softmax"])
    v, om, go = (t[k].float().cpu() for k in ("value", "offset_mask", "grad_out"))
    ref_out = cref.dcnv4_forward(v, om, *a, c["rc"], softmax=c["softmax"])
    ref_gv, ref_gom = cref.dcnv4_backward(v, om, go, *a, c["rc"], softmax=c["softmax"])
    what = f"{c} {dtype}"
    close(out, ref_out, FWD_TOL[dtype], f"forward {what}")
    close(gv, ref_gv, BWD_TOL[dtype], f"grad_value {what}")
    tol = dict(BWD_TOL[dtype])
    tol["atol"] = tol["atol"] * max(1.0, c["scale"])       # offset gradients carry offset_scale as a factor
    close(gom, ref_gom, tol, f"grad_offset_mask {what}")
    used = 3 * c["G"] * (c["kh"] * c["kw"] - c["rc"])
    if gom.shape[-1] > used:
        assert float(gom[..., used:].abs().max()) == 0.0


@pytest.mark.parametrize("seed", range(24))
def test_flash_deform_attn_random_configuration(seed):
    from dcnv4_b200 import ops
    rng = random.Random(2000 + seed)
    L = rng.randint(1, 5)
    levels = tuple((rng.randint(1, 12), rng.randint(1, 12)) for _ in range(L))
    B, G, D, K = rng.randint(1, 3), rng.randint(1, 4), rng.choice([8, 16, 32, 32, 64]), rng.choice([1, 2, 4, 4, 8])
    Len_q = rng.randint(1, 90)
    lo, hi = rng.choice([(0.0, 1.0), (-0.5, 1.5), (0.2, 0.8)])
    dtype = DTYPES[seed % 3]
    t = oin.fda_inputs(B, levels, G, D, K, Len_q=Len_q, seed=seed, loc_lo=lo, loc_hi=hi, dtype=dtype, device=DEV)
    out = ops.flash_deform_attn_forward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                        t["sampling_loc_attn"], 64, K)
    gv, gs = ops.flash_deform_attn_backward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                            t["sampling_loc_attn"], t["grad_out"], 64, K)
    v, sla, go = (t[k].float().cpu() for k in ("value", "sampling_loc_attn", "grad_out"))
    ss, ls = t["spatial_shapes"].cpu(), t["level_start_index"].cpu()
    ref_out = cref.fda_forward(v, ss, ls, sla, K)
    ref_gv, ref_gs = cref.fda_backward(v, ss, ls, sla, go, K)
    what = f"B{B} levels{levels} G{G} D{D} K{K} Lq{Len_q} {dtype}"
    close(out, ref_out, FWD_TOL[dtype], f"forward {what}")
    close(gv, ref_gv, BWD_TOL[dtype], f"grad_value {what}")
    tol = dict(BWD_TOL[dtype])
    tol["atol"] = tol["atol"] * 12                          # location gradients carry the level size as a factor
    close(gs, ref_gs, tol, f"grad_sampling_loc_attn {what}")


def test_no_kernel_reported_trouble_during_the_sweeps():
    from dcnv4_b200 import ops
    assert ops.device_status() == 0
