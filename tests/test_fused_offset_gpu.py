"""DCNv4 forward that computes its own offset/mask rows on the tensor cores, against the two-step
sequence it replaces (the module's `offset_mask` Linear, then the sampling kernel;
DCNv4_op/DCNv4/modules/dcnv4.py:121-140) and against the CPU oracle.

The fused kernel rounds the Linear's result to the storage type before it samples, exactly as the
separate Linear stores it, and samples with the same arithmetic as the stand-alone kernel: the two
paths may differ only where the two products accumulate in a different order.  Tolerance: the
forward tolerance of the 16-bit types (fp16 rtol 1e-2 / atol 1e-3, bf16 rtol 2e-2 / atol 1e-2)."""
import pytest
import torch

from tests.util import FWD_TOL, close

pytestmark = pytest.mark.gpu
DEV = "cuda"

# (N, H, W, G, K): the four FlashInternImage-T stage shapes at a small batch, a batch whose last
# 128-query tile is ragged and straddles images, K not a multiple of 64, a single query, the widest K,
# and group counts that are not a multiple of the four groups of a task (FlashInternImage-S/B/L: 5, 7, 10).
SHAPES = [(2, 56, 56, 4, 64), (3, 28, 28, 8, 128), (5, 14, 14, 16, 256), (3, 7, 7, 32, 512), (3, 5, 9, 8, 72),
          (1, 1, 1, 4, 64), (2, 9, 7, 12, 192), (1, 12, 11, 4, 1024), (2, 13, 13, 5, 80), (2, 10, 14, 7, 112),
          (1, 14, 14, 10, 160), (1, 6, 6, 1, 16), (1, 8, 8, 3, 48)]


def _inputs(N, H, W, G, K, dtype, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    P = (27 * G + 7) // 8 * 8
    value = torch.randn(N, H, W, 16 * G, generator=g).to(dtype).to(DEV)
    x = torch.randn(N, H * W, K, generator=g).to(dtype).to(DEV)
    w = (torch.randn(P, K, generator=g) / K ** 0.5).to(dtype).to(DEV)
    b = (0.5 * torch.randn(P, generator=g)).to(dtype).to(DEV)
    return value, x, w, b


def _two_step(value, x, w, b, G, scale):
    from dcnv4_b200 import ops
    N, H, W, _ = value.shape
    om = ops.linear_forward(x.reshape(N * H * W, -1), w, b).reshape(N, H, W, -1)
    return ops.dcnv4_forward(value, om, 3, 3, 1, 1, 1, 1, 1, 1, G, 16, scale, 256, 0), om


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("N,H,W,G,K", SHAPES)
def test_fused_matches_linear_then_sampling(N, H, W, G, K, dtype):
    from dcnv4_b200 import ops
    value, x, w, b = _inputs(N, H, W, G, K, dtype, seed=N * 1000 + H * 10 + G)
    assert ops.fused_offset_supported(value, x, w, b, G, 16)
    for bias, scale in ((b, 1.0), (None, 2.0), (b, 0.5)):
        out = ops.dcnv4_fused_offset_forward(value, x, w, bias, G, 16, scale)
        ref, _ = _two_step(value, x, w, bias, G, scale)
        assert out.shape == value.shape and out.dtype == dtype
        close(out, ref, FWD_TOL[dtype], f"fused vs two-step, scale {scale}")
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("N,H,W,G,K", [(2, 14, 14, 4, 64), (1, 9, 12, 8, 128), (1, 7, 7, 16, 256)])
def test_fused_matches_oracle(N, H, W, G, K, dtype):
    """Oracle on the offset/mask rows the separate Linear stores (the fused kernel's rows are the
    same products rounded the same way)."""
    from dcnv4_b200 import ops
    from oracle import cref
    value, x, w, b = _inputs(N, H, W, G, K, dtype, seed=77 + G)
    out = ops.dcnv4_fused_offset_forward(value, x, w, b, G, 16, 1.0)
    _, om = _two_step(value, x, w, b, G, 1.0)
    want = cref.dcnv4_forward(value.float().cpu(), om.float().cpu(), 3, 3, 1, 1, 1, 1, 1, 1, G, 16, 1.0, 0)
    close(out, want, FWD_TOL[dtype], "fused vs oracle")


def test_fused_rejects_what_it_does_not_cover():
    from dcnv4_b200 import ops
    value, x, w, b = _inputs(1, 4, 4, 4, 64, torch.float16, seed=1)
    # 32 channels per group, fp32 tensors
    assert not ops.fused_offset_supported(value, x, w, b, 2, 32)
    assert not ops.fused_offset_supported(value.float(), x.float(), w.float(), b.float(), 4, 16)
    with pytest.raises(ValueError):  # unsupported parameter values, as for the other operators
        ops.dcnv4_fused_offset_forward(value, x, w, None, 2, 32, 1.0)
    # too few weight rows for 27 columns per group
    with pytest.raises(RuntimeError):
        ops.dcnv4_fused_offset_forward(value, x, w[:104].contiguous(), None, 4, 16, 1.0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_module_with_fused_offsets_matches_module_without(dtype):
    from dcnv4_b200 import ops
    from dcnv4_b200.modules import DCNv4
    torch.manual_seed(5)
    m = DCNv4(channels=128, group=8, offset_scale=1.0, dw_kernel_size=None, output_bias=True).to(DEV)
    with torch.no_grad():
        m.offset_mask.weight.normal_(0, 0.1)
        m.offset_mask.bias.normal_(0, 0.3)
    m = m.to(dtype).eval()
    x = torch.randn(3, 14 * 14, 128, device=DEV).to(dtype)
    saved = ops.FUSED_OFFSET_MASK
    calls = []
    fused_op = ops.dcnv4_fused_offset_forward
    try:
        ops.dcnv4_fused_offset_forward = lambda *a, **k: (calls.append(1), fused_op(*a, **k))[1]
        with torch.no_grad():
            ops.FUSED_OFFSET_MASK = True
            y_fused = m(x)
            assert calls, "a 128-channel layer at inference takes the fused kernel"
            ops.FUSED_OFFSET_MASK = False
            y_plain = m(x)
            assert len(calls) == 1
    finally:
        ops.FUSED_OFFSET_MASK = saved
        ops.dcnv4_fused_offset_forward = fused_op
    close(y_fused, y_plain, FWD_TOL[dtype], "module, fused offsets vs separate Linear")
    assert ops.device_status() == 0


@pytest.mark.parametrize("shape", [(64, 56, 64, 4), (64, 28, 128, 8), (64, 14, 256, 16), (64, 7, 512, 32)],
                         ids=lambda s: f"{s[0]}x{s[1]}x{s[1]}x{s[2]}")
def test_fused_at_benchmark_stage_shapes_against_oracle(shape):
    """The whole batch of 64 through the fused kernel (its task walk, ring and accumulator hand-over at
    full size); the oracle checks three whole images on the offset/mask rows of the separate Linear, and
    the complete output must equal the two-step path bit for bit."""
    from dcnv4_b200 import ops
    from oracle import cref
    N, HW, C, G = shape
    value, x, w, b = _inputs(N, HW, HW, G, C, torch.float16, seed=900 + HW)
    out = ops.dcnv4_fused_offset_forward(value, x, w, b, G, 16, 1.0)
    ref, om = _two_step(value, x, w, b, G, 1.0)
    assert torch.equal(out, ref), "fused and two-step outputs differ"
    for i in (0, N // 2 - 1, N - 1):
        want = cref.dcnv4_forward(value[i:i + 1].float().cpu(), om[i:i + 1].float().cpu(), 3, 3, 1, 1, 1, 1, 1, 1,
                                  G, 16, 1.0, 0)
        close(out[i:i + 1], want, FWD_TOL[torch.float16], f"image {i}")
    assert ops.device_status() == 0


def test_module_variant_with_depthwise_conv_and_centre_scale_takes_the_fused_kernel():
    """FlashInternImage-S/B/L style layer (depth-wise convolution in front of the offset/mask Linear,
    centre-feature-scale blend behind the operator, a group count that is not a multiple of four)."""
    from dcnv4_b200 import ops
    from dcnv4_b200.modules import DCNv4
    torch.manual_seed(6)
    m = DCNv4(channels=160, group=10, offset_scale=2.0, dw_kernel_size=3, center_feature_scale=True,
              output_bias=True).to(DEV)
    with torch.no_grad():
        m.offset_mask.weight.normal_(0, 0.1)
        m.offset_mask.bias.normal_(0, 0.3)
        m.center_feature_scale_proj_weight.normal_(0, 0.2)
    m = m.half().eval()
    x = torch.randn(2, 14 * 14, 160, device=DEV).half()
    saved = ops.FUSED_OFFSET_MASK
    calls = []
    fused_op = ops.dcnv4_fused_offset_forward
    try:
        ops.dcnv4_fused_offset_forward = lambda *a, **k: (calls.append(1), fused_op(*a, **k))[1]
        with torch.no_grad():
            ops.FUSED_OFFSET_MASK = True
            y_fused = m(x)
            assert len(calls) == 1
            ops.FUSED_OFFSET_MASK = False
            y_plain = m(x)
            assert len(calls) == 1
    finally:
        ops.FUSED_OFFSET_MASK = saved
        ops.dcnv4_fused_offset_forward = fused_op
    close(y_fused, y_plain, FWD_TOL[torch.float16], "S/B/L-style module, fused offsets vs separate Linear")
    assert ops.device_status() == 0
