"""GPU parity tests of the DCNv4 forward/backward kernels, called through the C ABI
(dcnv4_b200.ops -> libdcnv4_b200.so) and compared with the CPU oracle on the same inputs."""
import os

import numpy as np
import pytest
import torch

from oracle import cref, inputs as oin
from tests.util import BWD_TOL, FWD_TOL, close, dcn_args, oracle_dcn

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def mk(N, H, W, G, D, kh=3, kw=3, sh=1, sw=1, ph=1, pw=1, dh=1, dw=1, scale=1.0, rc=0, ostd=1.0, seed=0):
    return dict(N=N, H=H, W=W, G=G, D=D, kh=kh, kw=kw, sh=sh, sw=sw, ph=ph, pw=pw, dh=dh, dw=dw,
                scale=scale, rc=rc, ostd=ostd, seed=seed)


def gen(spec, dtype):
    return oin.dcnv4_inputs(spec["N"], spec["H"], spec["W"], spec["G"], spec["D"], kh=spec["kh"], kw=spec["kw"],
                            sh=spec["sh"], sw=spec["sw"], ph=spec["ph"], pw=spec["pw"], dh=spec["dh"],
                            dw=spec["dw"], remove_center=spec["rc"], seed=spec["seed"],
                            offset_std=spec["ostd"], dtype=dtype, device=DEV)


def run_gpu(t, spec, softmax=False):
    from dcnv4_b200 import ops
    a = dcn_args(spec)
    out = ops.dcnv4_forward(t["value"], t["offset_mask"], *a[:-1], 256, a[-1], softmax=softmax)
    gv, gom = ops.dcnv4_backward(t["value"], t["offset_mask"], *a[:-1], 256, t["grad_out"], a[-1],
                                 softmax=softmax)
    return out, gv, gom


CASES = {
    "cfg0": mk(2, 56, 56, 4, 16, seed=0),
    "stage1_n3": mk(3, 56, 56, 4, 16, seed=1),
    "stage2_n3": mk(3, 28, 28, 8, 16, seed=2),
    "stage3_n5": mk(5, 14, 14, 16, 16, seed=3),       # tiles straddle images (196 queries/image)
    "stage4_n7": mk(7, 7, 7, 32, 16, seed=4),          # 49 queries/image
    "L_stage4": mk(1, 8, 8, 80, 16, scale=2.0, seed=5),  # G=80: beyond the reference's block limit
    "far_offsets": mk(2, 9, 11, 3, 32, ostd=6.0, seed=6),
    "scale_half": mk(1, 14, 14, 2, 16, scale=0.5, ostd=2.0, seed=7),
    "scale_odd": mk(1, 14, 14, 2, 16, scale=1.3, seed=8),
    "remove_center": mk(2, 14, 14, 4, 16, rc=1, seed=9),
    "stride2": mk(2, 15, 14, 2, 16, sh=2, sw=2, seed=10),
    "dil2_pad2": mk(1, 12, 12, 2, 16, ph=2, pw=2, dh=2, dw=2, seed=11),
    "k5x3": mk(1, 10, 6, 1, 32, kh=5, kw=3, ph=2, pw=1, seed=12),
    "k1": mk(1, 5, 5, 2, 16, kh=1, kw=1, ph=0, pw=0, ostd=3.0, seed=13),
    "d64": mk(1, 12, 12, 2, 64, seed=14),
    "d48_chunks": mk(1, 9, 9, 2, 48, seed=15),           # D/vec not a power of two -> multi-chunk threads
    "d8": mk(2, 6, 6, 3, 8, seed=16),
    "one_query": mk(1, 1, 1, 1, 16, ostd=0.3, seed=17),
}


@pytest.mark.parametrize("dtype", DTYPES, ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_forward_backward_parity(name, dtype):
    spec = CASES[name]
    t = gen(spec, dtype)
    out, gv, gom = run_gpu(t, spec)
    ref_out, ref_gv, ref_gom = oracle_dcn(t, spec)
    close(out, ref_out, FWD_TOL[dtype], "forward")
    close(gv, ref_gv, BWD_TOL[dtype], "grad_value")
    close(gom, ref_gom, BWD_TOL[dtype], "grad_offset_mask")
    used = 3 * spec["G"] * (spec["kh"] * spec["kw"] - spec["rc"])
    if gom.shape[-1] > used:
        assert float(gom[..., used:].abs().max()) == 0.0, "pad columns must be exactly zero"


@pytest.mark.parametrize("name", ["cfg0", "remove_center", "k5x3", "scale_odd"])
def test_softmax_variant(name):
    spec = CASES[name]
    t = gen(spec, torch.float32)
    out, gv, gom = run_gpu(t, spec, softmax=True)
    ref_out, ref_gv, ref_gom = oracle_dcn(t, spec, softmax=True)
    close(out, ref_out, FWD_TOL[torch.float32], "forward")
    close(gv, ref_gv, BWD_TOL[torch.float32], "grad_value")
    close(gom, ref_gom, BWD_TOL[torch.float32], "grad_offset_mask")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16"])
@pytest.mark.parametrize("name", ["cfg0", "far_offsets", "scale_odd", "remove_center", "stride2", "dil2_pad2"])
def test_corner_indices_bit_exact(name, dtype):
    from dcnv4_b200 import ops
    spec = CASES[name]
    t = gen(spec, dtype)
    a = dcn_args(spec)
    got = ops.dcnv4_corners(t["offset_mask"], spec["H"], spec["W"], *a[:8], spec["G"], spec["scale"], spec["rc"])
    _, ref = cref.dcnv4_forward(t["value"].float().cpu(), t["offset_mask"].float().cpu(), *a, want_corners=True)
    assert torch.equal(got.cpu(), ref), "corner selection differs from floor() of the fp32 coordinate formula"


def test_golden_reference_core_cfg0():
    """GPU forward/backward against values produced by the reference's own pure-PyTorch core."""
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "dcnv4_ref_core_cfg0.npz"))
    spec = CASES["cfg0"]
    t = gen(spec, torch.float32)
    out, gv, gom = run_gpu(t, spec)
    q32, q64 = torch.from_numpy(z["q32"]), torch.from_numpy(z["q64"])
    flat = out.reshape(-1, 64).cpu().double()
    ref32 = torch.from_numpy(z["out_fp32"]).double()
    ref64 = torch.from_numpy(z["out_fp64"])
    # the reference core's fp32 sampling grid carries ~3e-5 absolute noise at this size
    torch.testing.assert_close(flat[q32], ref32, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(flat[q64], ref64, rtol=1e-4, atol=1e-4)
    frac = ((flat[q64] - ref64).abs() > 1e-5 + 1e-4 * ref64.abs()).double().mean().item()
    assert frac < 5e-3
    torch.testing.assert_close(gv.reshape(-1, 64).cpu().double()[q64], torch.from_numpy(z["grad_value_fp64"]),
                               rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(gom.reshape(-1, gom.shape[-1]).cpu().double()[q64],
                               torch.from_numpy(z["grad_offset_mask_fp64"]), rtol=1e-3, atol=2e-3)


def test_golden_reference_core_small():
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "dcnv4_ref_core_small.npz"))
    from dcnv4_b200 import ops
    for name in sorted({k.split("/")[0] for k in z.files}):
        s = z[f"{name}/spec"]
        N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw = (int(x) for x in s[:13])
        scale, rc = float(s[13]), int(s[14])
        v = torch.from_numpy(z[f"{name}/value"]).to(DEV)
        om = torch.from_numpy(z[f"{name}/offset_mask"]).to(DEV)
        go = torch.from_numpy(z[f"{name}/grad_out"]).to(DEV)
        out = ops.dcnv4_forward(v, om, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, 256, rc)
        gv, gom = ops.dcnv4_backward(v, om, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, 256, go, rc)
        tol = dict(rtol=1e-4, atol=1e-4)
        close(out, torch.from_numpy(z[f"{name}/out"]), tol, f"{name} forward")
        close(gv, torch.from_numpy(z[f"{name}/grad_value"]), dict(rtol=1e-3, atol=1e-3), f"{name} grad_value")
        close(gom, torch.from_numpy(z[f"{name}/grad_offset_mask"]), dict(rtol=1e-3, atol=1e-3), f"{name} gom")


# ---------------------------------------------------------------- full-size properties

FULL = [(64, 56, 64, 4), (64, 28, 128, 8), (64, 14, 256, 16), (64, 7, 512, 32)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16], ids=["fp32", "fp16"])
@pytest.mark.parametrize("shape", FULL, ids=lambda s: f"{s[0]}x{s[1]}x{s[2]}")
def test_full_size_identity_and_linearity(shape, dtype):
    """Size-independent properties at the benchmark's full stage shapes:
    zero offsets + one-hot centre mask reproduces the input exactly; scaling the mask by a
    power of two scales the output exactly."""
    from dcnv4_b200 import ops
    N, HW, C, G = shape
    D = C // G
    spec = mk(N, HW, HW, G, D, seed=21)
    t = gen(spec, dtype)
    K, P = 9, t["offset_mask"].shape[-1]
    om = torch.zeros_like(t["offset_mask"])
    view = om[..., : G * 27].view(N, HW, HW, G, 27)
    view[..., 18 + 4] = 1.0                                   # centre tap (i=1, j=1) -> k = 4
    a = dcn_args(spec)
    out = ops.dcnv4_forward(t["value"], om, *a[:-1], 256, a[-1])
    assert torch.equal(out, t["value"]), "identity sampling must reproduce the input bit for bit"

    out1 = ops.dcnv4_forward(t["value"], t["offset_mask"], *a[:-1], 256, a[-1])
    om2 = t["offset_mask"].clone()
    om2[..., : G * 27].view(N, HW, HW, G, 27)[..., 18:] *= 2.0
    out2 = ops.dcnv4_forward(t["value"], om2, *a[:-1], 256, a[-1])
    if dtype == torch.float32:
        assert torch.equal(out2, out1 * 2), "output must be exactly linear in the mask"
    else:  # results in fp16's subnormal range round on a fixed 2^-24 grid, so doubling is not exact there
        normal = out1.abs() >= 2.0 ** -13
        assert torch.equal(out2[normal], (out1 * 2)[normal])
        assert (out2.float() - 2 * out1.float()).abs().max().item() <= 2.0 ** -23


@pytest.mark.parametrize("shape", FULL, ids=lambda s: f"{s[0]}x{s[1]}x{s[2]}")
def test_full_size_adjoint_identities(shape):
    """<grad_out, F(value)> == <grad_value, value> (F is linear in value) and
    <grad_out, F> == <grad_mask, mask> (F is linear in the mask), at full size in fp32."""
    N, HW, C, G = shape
    spec = mk(N, HW, HW, G, C // G, seed=22)
    t = gen(spec, torch.float32)
    out, gv, gom = run_gpu(t, spec)
    lhs = (t["grad_out"].double() * out.double()).sum().item()
    rhs_v = (gv.double() * t["value"].double()).sum().item()
    gm = gom[..., : G * 27].reshape(N, HW, HW, G, 27)[..., 18:].double()
    m = t["offset_mask"][..., : G * 27].reshape(N, HW, HW, G, 27)[..., 18:].double()
    rhs_m = (gm * m).sum().item()
    scale = (t["grad_out"].double() * out.double()).abs().sum().item()
    assert abs(lhs - rhs_v) <= 1e-5 * scale
    assert abs(lhs - rhs_m) <= 1e-5 * scale


def test_backward_repeatable_offset_mask_grad():
    """grad_offset_mask has no atomics in its path: two runs give identical bits."""
    spec = CASES["stage1_n3"]
    t = gen(spec, torch.float16)
    _, gv1, gom1 = run_gpu(t, spec)
    _, gv2, gom2 = run_gpu(t, spec)
    assert torch.equal(gom1, gom2)
    close(gv1, gv2.double(), BWD_TOL[torch.float16], "grad_value run-to-run")


def test_no_kernel_gave_up_waiting():
    from dcnv4_b200 import ops
    assert ops.device_status() == 0


# ---------------------------------------------------------------- API behaviour

def test_autograd_function_and_module():
    import dcnv4_b200
    spec = CASES["cfg0"]
    t = gen(spec, torch.float32)
    v = t["value"].clone().requires_grad_(True)
    om = t["offset_mask"].clone().requires_grad_(True)
    out = dcnv4_b200.DCNv4Function.apply(v, om, 3, 3, 1, 1, 1, 1, 1, 1, 4, 16, 1.0, 256, 0)
    out.backward(t["grad_out"])
    ref_out, ref_gv, ref_gom = oracle_dcn(t, spec)
    close(out, ref_out, FWD_TOL[torch.float32])
    close(v.grad, ref_gv, BWD_TOL[torch.float32])
    close(om.grad, ref_gom, BWD_TOL[torch.float32])

    torch.manual_seed(0)
    mod = dcnv4_b200.DCNv4(channels=64, group=4).to(DEV)
    assert mod.offset_mask.out_features == 112
    with torch.no_grad():  # non-trivial offsets (the reference zero-initialises this layer)
        mod.offset_mask.weight.normal_(0, 0.1)
        mod.offset_mask.bias.uniform_(0, 1)
    x = torch.randn(2, 56 * 56, 64, device=DEV, requires_grad=True)
    y = mod(x)
    assert y.shape == x.shape
    y.square().mean().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    assert mod.offset_mask.weight.grad.abs().sum() > 0
    # the module equals projections around the oracle
    with torch.no_grad():
        xv = mod.value_proj(x).reshape(2, 56, 56, 64)
        omv = mod.offset_mask(x).reshape(2, 56, 56, 112)
        core = cref.dcnv4_forward(xv.cpu(), omv.cpu(), 3, 3, 1, 1, 1, 1, 1, 1, 4, 16, 1.0, 0)
        ref = mod.output_proj(core.to(DEV).float().reshape(2, 3136, 64))
    close(y, ref, dict(rtol=1e-3, atol=1e-4))
    # autocast: the op runs in the dtype the projections produce
    with torch.autocast("cuda", dtype=torch.float16):
        y16 = mod(x)
    assert y16.dtype == torch.float16
    close(y16, ref, dict(rtol=2e-2, atol=2e-2))


def test_module_variants_match_composition():
    """The S/B/L-style module configuration (depthwise conv before the offset/mask Linear, centre-feature
    scale, remove_center, offset_scale 2) equals its parts composed around the oracle:
    value_proj / dw-conv + offset_mask Linear -> operator -> sigmoid blend -> output_proj
    (DCNv4_op/DCNv4/modules/dcnv4.py:116-152)."""
    import torch.nn.functional as F

    import dcnv4_b200
    torch.manual_seed(1)
    mod = dcnv4_b200.DCNv4(channels=64, group=4, dw_kernel_size=3, center_feature_scale=True,
                           remove_center=True, output_bias=False, offset_scale=2.0).to(DEV)
    assert mod.offset_mask.out_features == 96 and mod.output_proj.bias is None
    with torch.no_grad():
        mod.offset_mask.weight.normal_(0, 0.1)
        mod.offset_mask.bias.uniform_(0, 1)
        mod.center_feature_scale_proj_weight.normal_(0, 0.1)
        mod.center_feature_scale_proj_bias.normal_(0, 0.5)
    H, W = 12, 10
    x = torch.randn(2, H * W, 64, device=DEV)
    with torch.no_grad():
        y = mod(x, shape=(H, W))
        assert y.shape == x.shape
        xv = mod.value_proj(x).reshape(2, H, W, 64)
        dw = mod.offset_mask_dw(x.view(2, H, W, 64).permute(0, 3, 1, 2)).permute(0, 2, 3, 1).reshape(2, H * W, 64)
        omv = mod.offset_mask(dw).reshape(2, H, W, 96)
        core = cref.dcnv4_forward(xv.cpu(), omv.cpu(), 3, 3, 1, 1, 1, 1, 1, 1, 4, 16, 2.0, 1).to(DEV).float()
        scale = F.linear(core, mod.center_feature_scale_proj_weight, mod.center_feature_scale_proj_bias).sigmoid()
        scale = scale[..., None].repeat(1, 1, 1, 1, 16).flatten(-2)
        blended = core * (1 - scale) + xv * scale
        ref = mod.output_proj(blended.reshape(2, H * W, 64))
    close(y, ref, dict(rtol=1e-3, atol=1e-4), "module with dw conv, centre-feature scale, remove_center")
    # the blend must matter in this test (scale is not ~0 or ~1 everywhere)
    assert 0.2 < float(scale.mean()) < 0.8 and float((blended - core).abs().max()) > 0.1
    sd = mod.state_dict()
    for k in ("offset_mask.weight", "offset_mask_dw.weight", "value_proj.weight", "output_proj.weight",
              "center_feature_scale_proj_weight", "center_feature_scale_proj_bias"):
        assert k in sd
    # and its gradients flow through every part
    xg = x.clone().requires_grad_(True)
    mod(xg, shape=(H, W)).square().mean().backward()
    for prm in (mod.offset_mask_dw.weight, mod.offset_mask.weight, mod.value_proj.weight,
                mod.center_feature_scale_proj_weight):
        assert prm.grad is not None and float(prm.grad.abs().sum()) > 0


def test_argument_errors():
    from dcnv4_b200 import ops
    spec = CASES["cfg0"]
    t = gen(spec, torch.float32)
    a = dcn_args(spec)
    with pytest.raises(RuntimeError, match="contiguous"):
        ops.dcnv4_forward(t["value"].transpose(1, 2), t["offset_mask"], *a[:-1], 256, a[-1])
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.dcnv4_forward(t["value"].cpu(), t["offset_mask"], *a[:-1], 256, a[-1])
    with pytest.raises(RuntimeError, match="wont match"):
        ops.dcnv4_forward(t["value"], t["offset_mask"], 3, 3, 1, 1, 1, 1, 1, 1, 4, 32, 1.0, 256, 0)
    with pytest.raises(RuntimeError, match="im2col_step"):
        ops.dcnv4_forward(t["value"].repeat(3, 1, 1, 1)[:3], t["offset_mask"].repeat(3, 1, 1, 1)[:3],
                          *a[:-1], 2, a[-1])
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ops.dcnv4_forward(t["value"], t["offset_mask"][..., :108].contiguous(), *a[:-1], 256, a[-1])
    with pytest.raises(RuntimeError, match="multiple of 8"):   # too narrow for 3*K*G
        ops.dcnv4_forward(t["value"], t["offset_mask"][..., :104].contiguous(), *a[:-1], 256, a[-1])
    with pytest.raises(ValueError, match="group_channels"):
        v = torch.randn(1, 4, 4, 6, device=DEV)
        om = torch.zeros(1, 4, 4, 56, device=DEV)
        ops.dcnv4_forward(v, om, 3, 3, 1, 1, 1, 1, 1, 1, 2, 3, 1.0, 256, 0)


@pytest.mark.parametrize("dtype", DTYPES, ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("rows,G,D", [(1, 1, 16), (777, 4, 16), (130, 5, 16), (33, 20, 32), (9, 64, 16), (5, 80, 16)])
def test_center_scale_blend_kernel_matches_the_reference_formulation(rows, G, D, dtype):
    """x*(1-s) + x_proj*s with s = sigmoid(Linear(x)) repeated over each group's channels
    (DCNv4_op/DCNv4/modules/dcnv4.py:18-26,142-147), computed in fp32 from the stored values."""
    import torch.nn.functional as F

    from dcnv4_b200 import ops
    C = G * D
    if dtype == torch.float32 and C > 1024:
        pytest.skip("fp32 rows above 1024 channels are outside the kernel's range")
    torch.manual_seed(rows + C)
    x = torch.randn(rows, C, device=DEV).to(dtype)
    xp = torch.randn(rows, C, device=DEV).to(dtype)
    for pdt in {torch.float32, dtype}:
        w = (torch.randn(G, C, device=DEV) / C ** 0.5).to(pdt)
        b = torch.randn(G, device=DEV).to(pdt)
        assert ops.center_scale_blend_supported(x, w, D)
        got = ops.center_scale_blend_forward(x, xp, w, b)
        s = F.linear(x.float(), w.float(), b.float()).sigmoid()[..., None].repeat(1, 1, D).flatten(-2)
        ref = x.float() * (1 - s) + xp.float() * s
        tol = {torch.float32: dict(rtol=1e-5, atol=1e-5), torch.float16: dict(rtol=2e-3, atol=2e-3),
               torch.bfloat16: dict(rtol=1.6e-2, atol=1.6e-2)}[dtype]
        torch.testing.assert_close(got.float(), ref, **tol)
    assert not ops.center_scale_blend_supported(x[:, : C - 8].contiguous(), w, D)
