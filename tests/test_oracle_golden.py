"""Pin the C oracle: against golden vectors produced by the reference's own pure-PyTorch
core (tests/golden/make_golden.py) and against the independent grid_sample formulation."""
import os

import numpy as np
import pytest
import torch

from oracle import cref, inputs as oin, torch_core

GOLD = os.path.join(os.path.dirname(__file__), "golden")
SMALL = np.load(os.path.join(GOLD, "dcnv4_ref_core_small.npz"))
CASES = sorted({k.split("/")[0] for k in SMALL.files})


def _spec(name):
    s = SMALL[f"{name}/spec"]
    ints = [int(x) for x in s[:13]]
    return ints, float(s[13]), int(s[14])


@pytest.mark.parametrize("name", CASES)
def test_c_oracle_matches_reference_core_small(name):
    (N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw), scale, rc = _spec(name)
    v = torch.from_numpy(SMALL[f"{name}/value"])
    om = torch.from_numpy(SMALL[f"{name}/offset_mask"])
    go = torch.from_numpy(SMALL[f"{name}/grad_out"])
    out = cref.dcnv4_forward(v, om, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, rc)
    gv, gom = cref.dcnv4_backward(v, om, go, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, rc)
    ref_out = torch.from_numpy(SMALL[f"{name}/out"])
    ref_gv = torch.from_numpy(SMALL[f"{name}/grad_value"])
    ref_gom = torch.from_numpy(SMALL[f"{name}/grad_offset_mask"])
    # The reference core builds its sampling grid from fp32 linspace values even for fp64
    # inputs; the grid is exact when the padded size is a power of two ("pow2_*" cases),
    # otherwise it carries ~1e-7 relative coordinate noise (a few 1e-5 absolute downstream).
    # The oracle itself rounds coordinates to fp32 like the kernels do (~1e-6 downstream).
    exact = name.startswith("pow2")
    tol = dict(rtol=1e-5, atol=2e-5) if exact else dict(rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(out, ref_out, **tol)
    torch.testing.assert_close(gv, ref_gv, **tol)
    # offset gradients divide by nothing but are sums of O(D) products of O(1) terms
    torch.testing.assert_close(gom, ref_gom, **(dict(rtol=1e-4, atol=2e-4) if exact else dict(rtol=1e-3, atol=1e-3)))
    assert float(gom[..., 3 * G * (kh * kw - rc):].abs().max() if gom.shape[-1] > 3 * G * (kh * kw - rc) else 0.0) == 0.0


def test_c_oracle_matches_reference_core_cfg0():
    z = np.load(os.path.join(GOLD, "dcnv4_ref_core_cfg0.npz"))
    t = oin.dcnv4_inputs(2, 56, 56, 4, 16, seed=0)
    chk = z["input_checksums"]
    assert abs(t["value"].double().sum().item() - chk[0]) < 1e-6, "seeded inputs changed"
    assert abs(t["offset_mask"].double().sum().item() - chk[1]) < 1e-6
    out = cref.dcnv4_forward(t["value"], t["offset_mask"], 3, 3, 1, 1, 1, 1, 1, 1, 4, 16, 1.0, 0)
    gv, gom = cref.dcnv4_backward(t["value"], t["offset_mask"], t["grad_out"],
                                  3, 3, 1, 1, 1, 1, 1, 1, 4, 16, 1.0, 0)
    q32, q64 = torch.from_numpy(z["q32"]), torch.from_numpy(z["q64"])
    ref32 = torch.from_numpy(z["out_fp32"]).double()
    ref64 = torch.from_numpy(z["out_fp64"])
    flat = out.reshape(-1, 64)
    # fp32 run of the reference core: its grid noise is ~3e-5 absolute at this size
    torch.testing.assert_close(flat[q32], ref32, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(flat[q64], ref64, rtol=1e-4, atol=1e-4)
    frac = ((flat[q64] - ref64).abs() > 1e-5 + 1e-4 * ref64.abs()).double().mean().item()
    assert frac < 5e-3, f"violations of rtol 1e-4/atol 1e-5 vs reference core: {frac}"
    torch.testing.assert_close(gv.reshape(-1, 64)[q64], torch.from_numpy(z["grad_value_fp64"]),
                               rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(gom.reshape(-1, gom.shape[-1])[q64],
                               torch.from_numpy(z["grad_offset_mask_fp64"]), rtol=1e-3, atol=2e-3)


DCN_EXTRA = [
    # N,H,W,G,D,kh,kw,sh,sw,ph,pw,dh,dw,scale,rc,softmax,ostd
    (1, 7, 9, 2, 16, 3, 3, 1, 1, 1, 1, 1, 1, 1.0, 0, True, 1.0),
    (1, 7, 9, 2, 16, 3, 3, 1, 1, 1, 1, 1, 1, 0.7, 1, True, 2.0),
    (2, 8, 8, 3, 8, 3, 3, 2, 1, 0, 1, 1, 2, 1.3, 0, False, 3.0),
    (1, 10, 6, 1, 32, 5, 3, 1, 1, 2, 1, 1, 1, 1.0, 0, False, 1.0),
    (1, 5, 5, 2, 16, 1, 1, 1, 1, 0, 0, 1, 1, 1.0, 0, False, 4.0),
]


@pytest.mark.parametrize("case", DCN_EXTRA)
def test_c_oracle_matches_grid_sample_dcnv4(case):
    N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw, scale, rc, softmax, ostd = case
    t = oin.dcnv4_inputs(N, H, W, G, D, kh=kh, kw=kw, sh=sh, sw=sw, ph=ph, pw=pw, dh=dh, dw=dw,
                         remove_center=rc, seed=11, offset_std=ostd)
    args = (kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, rc)
    out = cref.dcnv4_forward(t["value"], t["offset_mask"], *args, softmax=softmax)
    gv, gom = cref.dcnv4_backward(t["value"], t["offset_mask"], t["grad_out"], *args, softmax=softmax)
    o2, gv2, gom2 = torch_core.dcnv4_fwd_bwd(t["value"].double(), t["offset_mask"].double(),
                                             t["grad_out"].double(), *args, softmax=softmax)
    # fp32 coordinates in the oracle vs fp64 in the formulation: ~1e-6 coordinate noise
    torch.testing.assert_close(out, o2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gv, gv2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gom, gom2, rtol=1e-3, atol=1e-3)


FDA_CASES = [
    # B, levels, G, D, K, Len_q, loc range
    (2, ((6, 8), (3, 4)), 2, 16, 4, 37, (0.0, 1.0)),
    (1, ((5, 7), (4, 4), (2, 3)), 3, 8, 8, 19, (-0.3, 1.3)),
    (1, ((9, 5),), 1, 32, 4, 11, (0.0, 1.0)),
    (1, ((4, 4), (3, 3), (2, 2), (2, 1), (1, 1)), 2, 16, 4, 23, (-0.5, 1.5)),
]


@pytest.mark.parametrize("case", FDA_CASES)
def test_c_oracle_matches_grid_sample_fda(case):
    B, levels, G, D, K, Len_q, (lo, hi) = case
    t = oin.fda_inputs(B, levels, G, D, K, Len_q=Len_q, seed=5, loc_lo=lo, loc_hi=hi)
    out, corners = cref.fda_forward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                    t["sampling_loc_attn"], K, want_corners=True)
    gv, gs = cref.fda_backward(t["value"], t["spatial_shapes"], t["level_start_index"],
                               t["sampling_loc_attn"], t["grad_out"], K)
    o2, gv2, gs2 = torch_core.fda_fwd_bwd(t["value"].double(), t["spatial_shapes"],
                                          t["level_start_index"], t["sampling_loc_attn"].double(),
                                          t["grad_out"].double(), K)
    torch.testing.assert_close(out, o2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gv, gv2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gs, gs2, rtol=1e-3, atol=1e-3)
    if lo < 0:
        assert (corners == cref.SKIPPED).any(), "case should exercise the range test"


def test_corner_indices_follow_fp32_floor():
    """Corner selection is floor() of the fp32 coordinate formula
    (DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:203-224, common.h:47-48)."""
    t = oin.dcnv4_inputs(1, 6, 6, 2, 16, seed=3, offset_std=2.0)
    _, corners = cref.dcnv4_forward(t["value"], t["offset_mask"], 3, 3, 1, 1, 1, 1, 1, 1, 2, 16,
                                    1.0, 0, want_corners=True)
    off, _ = torch_core.unpack_offset_mask(t["offset_mask"], 2, 9)
    ys = torch.arange(6, dtype=torch.float32).view(1, 6, 1, 1, 1)
    xs = torch.arange(6, dtype=torch.float32).view(1, 1, 6, 1, 1)
    ti = torch.tensor([i for i in range(3) for _ in range(3)], dtype=torch.float32)
    tj = torch.tensor([j for _ in range(3) for j in range(3)], dtype=torch.float32)
    w = (xs - 1.0) + (ti + off[..., 0])      # base = (1 - 1 + x) - 1*1.0 ; scale 1.0 keeps fma exact
    h = (ys - 1.0) + (tj + off[..., 1])
    ok = (h > -1) & (w > -1) & (h < 6) & (w < 6)
    exp_h = torch.where(ok, torch.floor(h).int(), torch.full_like(h, cref.SKIPPED).int())
    exp_w = torch.where(ok, torch.floor(w).int(), torch.full_like(w, cref.SKIPPED).int())
    assert torch.equal(corners[..., 0], exp_h)
    assert torch.equal(corners[..., 1], exp_w)
