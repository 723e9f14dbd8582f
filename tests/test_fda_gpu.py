"""GPU parity tests of the FlashDeformAttn forward/backward kernels through the C ABI."""
import pytest
import torch

from oracle import cref, inputs as oin
from tests.util import BWD_TOL, FWD_TOL, close, oracle_fda

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.float16, torch.bfloat16]

# name -> (B, levels, G, D, K, Len_q, (loc_lo, loc_hi), seed)
CASES = {
    "detr_small": (2, ((20, 30), (10, 15), (5, 8), (3, 4)), 8, 32, 4, 700, (0.0, 1.0), 0),
    "detr_k8": (1, ((20, 30), (10, 15), (5, 8), (3, 4)), 8, 32, 8, 333, (0.0, 1.0), 1),
    "out_of_range": (2, ((6, 8), (3, 4)), 2, 16, 4, 37, (-0.4, 1.4), 2),
    "one_level": (1, ((9, 5),), 1, 32, 4, 11, (0.0, 1.0), 3),
    "five_levels": (1, ((4, 4), (3, 3), (2, 2), (2, 1), (1, 1)), 2, 16, 4, 23, (-0.5, 1.5), 4),
    "ragged_rows": (1, ((5, 7), (4, 4), (2, 3)), 3, 8, 8, 19, (-0.3, 1.3), 5),   # row bytes not 16-aligned in fp16
    "odd_everything": (3, ((7, 3),), 1, 8, 1, 5, (0.0, 1.0), 6),
    "d64_k2": (1, ((8, 8), (4, 4)), 4, 64, 2, 50, (0.0, 1.0), 7),
    "d48_chunks": (1, ((8, 8), (4, 4)), 2, 48, 4, 21, (0.0, 1.0), 8),
}


def gen(case, dtype):
    B, levels, G, D, K, Len_q, (lo, hi), seed = case
    return oin.fda_inputs(B, levels, G, D, K, Len_q=Len_q, seed=seed, loc_lo=lo, loc_hi=hi,
                          dtype=dtype, device=DEV)


def run_gpu(t, K):
    from dcnv4_b200 import ops
    out = ops.flash_deform_attn_forward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                        t["sampling_loc_attn"], 64, K)
    gv, gs = ops.flash_deform_attn_backward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                            t["sampling_loc_attn"], t["grad_out"], 64, K)
    return out, gv, gs


@pytest.mark.parametrize("dtype", DTYPES, ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_forward_backward_parity(name, dtype):
    case = CASES[name]
    K = case[4]
    t = gen(case, dtype)
    out, gv, gs = run_gpu(t, K)
    ref_out, ref_gv, ref_gs = oracle_fda(t, K)
    close(out, ref_out, FWD_TOL[dtype], "forward")
    close(gv, ref_gv, BWD_TOL[dtype], "grad_value")
    # location gradients are scaled by the level size (up to 30 here): scale the abs term too
    tol = dict(BWD_TOL[dtype])
    tol["atol"] = tol["atol"] * 30
    close(gs, ref_gs, tol, "grad_sampling_loc_attn")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16"])
@pytest.mark.parametrize("name", ["detr_small", "out_of_range", "five_levels", "ragged_rows"])
def test_corner_indices_bit_exact(name, dtype):
    from dcnv4_b200 import ops
    case = CASES[name]
    K = case[4]
    t = gen(case, dtype)
    got = ops.flash_deform_attn_corners(t["spatial_shapes"], t["sampling_loc_attn"], K)
    _, ref = cref.fda_forward(t["value"].float().cpu(), t["spatial_shapes"].cpu(), t["level_start_index"].cpu(),
                              t["sampling_loc_attn"].float().cpu(), K, want_corners=True)
    assert torch.equal(got.cpu(), ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16"])
def test_full_size_properties(dtype):
    """Deformable-DETR encoder shape (8 x 20,197 positions, 8 heads x 32, 4 levels x 4 points):
    (a) all points of a head at one pixel centre with any logits reproduce that pixel's
    value (softmax weights sum to 1); (b) adjoint identity <gy, F(v)> == <grad_v, v>."""
    B, G, D, K = 8, 8, 32, 4
    t = oin.fda_inputs(B, oin.DETR_LEVELS, G, D, K, seed=3, dtype=dtype, device=DEV)
    Len = t["value"].shape[1]
    assert Len == 20197
    L = 4
    sla = t["sampling_loc_attn"].clone()
    # every point -> centre of pixel (y=12, x=9) of level 0 (100x152): (9.5/152, 12.5/100) = (1/16, 1/8),
    # both exactly representable in fp16, so the sample sits exactly on the pixel centre
    sla[..., 0: 2 * L * K: 2] = 1.0 / 16
    sla[..., 1: 2 * L * K: 2] = 1.0 / 8
    # logits: only level 0 matters (others pushed to -inf-ish)
    sla[..., 2 * L * K + K:] = -30000.0 if dtype == torch.float16 else -1e30
    from dcnv4_b200 import ops
    out = ops.flash_deform_attn_forward(t["value"], t["spatial_shapes"], t["level_start_index"], sla, 64, K)
    expect = t["value"][:, 12 * 152 + 9].reshape(B, 1, G * D).expand(B, Len, G * D)
    close(out, expect.double(), dict(rtol=2e-3 if dtype == torch.float16 else 1e-5, atol=1e-5), "pixel-centre sampling")

    if dtype == torch.float32:
        out, gv, gs = run_gpu(t, K)
        lhs = (t["grad_out"].double() * out.double()).sum().item()
        rhs = (gv.double() * t["value"].double()).sum().item()
        scale = (t["grad_out"].double() * out.double()).abs().sum().item()
        assert abs(lhs - rhs) <= 1e-5 * scale
        # logit gradients of a softmax sum to zero per (query, head)
        glog = gs[..., 2 * L * K:].double().sum(-1)
        assert glog.abs().max().item() < 1e-3


def test_autograd_function_and_module():
    import dcnv4_b200
    case = CASES["detr_small"]
    K = case[4]
    t = gen(case, torch.float32)
    v = t["value"].clone().requires_grad_(True)
    s = t["sampling_loc_attn"].clone().requires_grad_(True)
    out = dcnv4_b200.FlashDeformAttnFunction.apply(v, t["spatial_shapes"], t["level_start_index"], s, 64, K)
    out.backward(t["grad_out"])
    ref_out, ref_gv, ref_gs = oracle_fda(t, K)
    close(out, ref_out, FWD_TOL[torch.float32])
    close(v.grad, ref_gv, BWD_TOL[torch.float32])
    close(s.grad, ref_gs, dict(rtol=1e-3, atol=3e-3))

    torch.manual_seed(0)
    mod = dcnv4_b200.FlashDeformAttn(d_model=256, n_levels=4, n_heads=8, n_points=4).to(DEV)
    shapes, starts, Len = oin.level_tensors(case[1])
    shapes, starts = shapes.to(DEV), starts.to(DEV)
    q = torch.randn(2, 50, 256, device=DEV, requires_grad=True)
    ref_pts = torch.rand(2, 50, 4, 2, device=DEV)
    feat = torch.randn(2, Len, 256, device=DEV)
    y = mod(q, ref_pts, feat, shapes, starts)
    assert y.shape == (2, 50, 256)
    y.square().mean().backward()
    assert torch.isfinite(q.grad).all() and mod.sampling_offsets.weight.grad.abs().sum() > 0
    with torch.autocast("cuda", dtype=torch.float16):
        y16 = mod(q, ref_pts, feat, shapes, starts)
    close(y16, y.detach().double(), dict(rtol=3e-2, atol=3e-2))
    with pytest.raises(ValueError):
        mod(q, torch.rand(2, 50, 4, 3, device=DEV), feat, shapes, starts)


def test_argument_errors():
    from dcnv4_b200 import ops
    case = CASES["detr_small"]
    t = gen(case, torch.float32)
    with pytest.raises(RuntimeError, match="contiguous"):
        ops.flash_deform_attn_forward(t["value"].transpose(2, 3), t["spatial_shapes"], t["level_start_index"],
                                      t["sampling_loc_attn"], 64, 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.flash_deform_attn_forward(t["value"], t["spatial_shapes"].cpu(), t["level_start_index"],
                                      t["sampling_loc_attn"], 64, 4)
    with pytest.raises(RuntimeError, match="sampling_loc_attn must be"):
        ops.flash_deform_attn_forward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                      t["sampling_loc_attn"], 64, 8)
    with pytest.raises(ValueError, match="supported parameter space"):
        nine = torch.ones(9, 2, dtype=torch.int64, device=DEV)
        ops.flash_deform_attn_forward(torch.zeros(1, 9, 1, 8, device=DEV), nine, torch.arange(9, device=DEV),
                                      torch.zeros(1, 1, 1, 27, device=DEV), 64, 1)


def test_level_outside_the_value_tensor_is_ignored_and_reported():
    """A level whose start + H*W exceeds Len_in (stale shapes, a caller-side bug) must not be read or
    written: the kernels treat it as empty -- its samples contribute nothing, softmax weights as if
    they were there -- and record status 2.  The reference trusts these device tensors unchecked."""
    from dcnv4_b200 import ops
    K = 4
    t = oin.fda_inputs(2, ((6, 8), (3, 4)), 2, 16, K, Len_q=37, seed=9, dtype=torch.float32, device=DEV)
    assert ops.device_status() == 0
    bad_shapes = t["spatial_shapes"].clone()
    bad_shapes[1] = torch.tensor([30, 40])            # 1200 positions claimed, 12 exist
    out = ops.flash_deform_attn_forward(t["value"], bad_shapes, t["level_start_index"], t["sampling_loc_attn"], 64, K)
    gv, gs = ops.flash_deform_attn_backward(t["value"], bad_shapes, t["level_start_index"], t["sampling_loc_attn"],
                                            t["grad_out"], 64, K)
    assert ops.device_status() == 2
    assert ops.device_status() == 0                   # read-and-clear
    # same thing said legally: the true shapes, level 1's points moved far outside the map
    sla = t["sampling_loc_attn"].clone()
    sla[..., 2 * K: 4 * K] = -5.0
    ref_out = cref.fda_forward(t["value"].cpu(), t["spatial_shapes"].cpu(), t["level_start_index"].cpu(), sla.cpu(), K)
    ref_gv, ref_gs = cref.fda_backward(t["value"].cpu(), t["spatial_shapes"].cpu(), t["level_start_index"].cpu(),
                                       sla.cpu(), t["grad_out"].cpu(), K)
    close(out, ref_out, FWD_TOL[torch.float32], "forward")
    close(gv, ref_gv, BWD_TOL[torch.float32], "grad_value")
    assert float(gv[:, 48:].abs().max()) == 0.0       # nothing was added to the rows of the bad level
    tol = dict(BWD_TOL[torch.float32]); tol["atol"] *= 8
    close(gs, ref_gs, tol, "grad_sampling_loc_attn")
    # a negative start is caught the same way
    bad_starts = t["level_start_index"].clone()
    bad_starts[0] = -3
    ops.flash_deform_attn_forward(t["value"], t["spatial_shapes"], bad_starts, t["sampling_loc_attn"], 64, K)
    assert ops.device_status() == 2


def test_module_equals_its_parts_around_the_oracle_with_fp16_rounded_locations():
    """FlashDeformAttn in fp32 = value_proj / sampling_offsets / attention_weights Linears, sampling
    locations rounded to fp16 as the reference module does (DCNv4_op/DCNv4/modules/flash_deform_attn.py:
    132-133), the operator, output_proj.  Without that rounding the result differs by more than the tolerance,
    which the last assertion shows."""
    import dcnv4_b200
    torch.manual_seed(5)
    levels = ((20, 30), (10, 15), (5, 8), (3, 4))
    mod = dcnv4_b200.FlashDeformAttn(d_model=256, n_levels=4, n_heads=8, n_points=4).to(DEV)
    with torch.no_grad():
        mod.sampling_offsets.weight.normal_(0, 0.05)
        mod.attention_weights.weight.normal_(0, 0.05)
    shapes, starts, Len = oin.level_tensors(levels)
    shapes, starts = shapes.to(DEV), starts.to(DEV)
    q = torch.randn(2, 40, 256, device=DEV)
    ref_pts = torch.rand(2, 40, 4, 2, device=DEV)
    feat = torch.randn(2, Len, 256, device=DEV)
    with torch.no_grad():
        y = mod(q, ref_pts, feat, shapes, starts)
        value = mod.value_proj(feat).view(2, Len, 8, 32)
        off = mod.sampling_offsets(q).view(2, 40, 8, 4, 4, 2)
        logits = mod.attention_weights(q).view(2, 40, 8, 16)
        norm = torch.stack([shapes[..., 1], shapes[..., 0]], -1)
        loc = (ref_pts[:, :, None, :, None, :] + off / norm[None, None, None, :, None, :]).flatten(-3)

        def through_oracle(locations):
            sla = torch.cat([locations, logits], -1)
            core = cref.fda_forward(value.cpu(), shapes.cpu(), starts.cpu(), sla.cpu(), 4)
            return mod.output_proj(core.to(DEV).float())

        ref = through_oracle(loc.half().float())
        unrounded = through_oracle(loc)
    close(y, ref, dict(rtol=1e-3, atol=1e-4), "module vs parts with fp16-rounded locations")
    assert float((unrounded - ref).abs().max()) > 1e-3
