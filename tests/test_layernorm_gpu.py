"""Channels-last LayerNorm kernel against torch.nn.functional.layer_norm computed in fp32."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("rows,C", [(1, 64), (7, 64), (4099, 64), (513, 128), (300, 256), (77, 512), (33, 768),
                                    (5, 1024), (9, 96), (11, 1280 // 2), (3, 8), (2, 2048)])
def test_layernorm_matches_fp32_reference(rows, C, dtype):
    from dcnv4_b200 import ops
    if dtype == torch.float32 and C > 1024:
        pytest.skip("fp32 rows above 1024 channels are outside the kernel's range")
    torch.manual_seed(rows * 131 + C)
    x = (torch.randn(rows, C, device=DEV) * 3 + 1.5).to(dtype)
    for pdt in {torch.float32, dtype}:
        w = torch.randn(C, device=DEV).to(pdt)
        b = torch.randn(C, device=DEV).to(pdt)
        assert ops.layer_norm_supported(x, w)
        y = ops.layer_norm_forward(x, w, b, 1e-6)
        ref = F.layer_norm(x.float(), (C,), w.float(), b.float(), 1e-6)
        tol = {torch.float32: dict(rtol=1e-5, atol=1e-5), torch.float16: dict(rtol=2e-3, atol=2e-3),
               torch.bfloat16: dict(rtol=1.6e-2, atol=1.6e-2)}[dtype]
        torch.testing.assert_close(y.float(), ref, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("rows,C", [(5, 32), (4099, 32), (777, 64), (33, 320)])
def test_layernorm_with_gelu_matches_the_two_step_formulation(rows, C, dtype):
    """y = GELU(LayerNorm(x)) in one pass equals LayerNorm (rounded to the storage type) followed by GELU."""
    from dcnv4_b200 import ops
    torch.manual_seed(rows + C)
    x = (torch.randn(rows, C, device=DEV) * 2 - 0.5).to(dtype)
    w, b = torch.randn(C, device=DEV).to(dtype), torch.randn(C, device=DEV).to(dtype)
    y = ops.layer_norm_forward(x, w, b, 1e-6, "gelu")
    ref = F.gelu(F.layer_norm(x.float(), (C,), w.float(), b.float(), 1e-6).to(dtype).float())
    tol = {torch.float32: dict(rtol=1e-5, atol=1e-5), torch.float16: dict(rtol=2e-3, atol=2e-3),
           torch.bfloat16: dict(rtol=1.6e-2, atol=1.6e-2)}[dtype]
    torch.testing.assert_close(y.float(), ref, **tol)
    with pytest.raises(ValueError):
        ops.layer_norm_forward(x, w, b, 1e-6, "relu")


def test_stem_layer_fused_norm_matches_the_stock_modules():
    """FlashInternImage's stem (conv -> LayerNorm -> GELU -> conv -> LayerNorm) with the fused
    LayerNorm+GELU pass equals the same modules run one by one."""
    from dcnv4_b200.flash_intern_image import LayerNorm, StemLayer
    torch.manual_seed(3)
    stem = StemLayer(3, 64, "GELU", "LN").to(DEV).half().eval()
    with torch.no_grad():
        for ln in (stem.norm1[1], stem.norm2[1]):
            ln.weight.uniform_(0.5, 1.5)
            ln.bias.normal_(0, 0.3)
        x = torch.randn(4, 3, 64, 96, device=DEV).half()
        fast = stem(x)
        LayerNorm.use_library_kernel = False
        try:
            slow = stem(x)
        finally:
            LayerNorm.use_library_kernel = True
    assert fast.shape == (4, 16, 24, 64) and fast.is_contiguous()
    torch.testing.assert_close(fast.float(), slow.float(), rtol=2e-2, atol=2e-2)
    assert stem.state_dict().keys() >= {"norm1.1.weight", "norm1.1.bias", "norm2.1.weight", "norm2.1.bias"}


def test_layernorm_module_falls_back_when_autograd_needs_it():
    from dcnv4_b200.flash_intern_image import LayerNorm
    ln = LayerNorm(64, eps=1e-6).to(DEV)
    x = torch.randn(10, 5, 64, device=DEV, requires_grad=True)
    y = ln(x)                       # autograd path (stock kernel)
    y.sum().backward()
    assert x.grad is not None and ln.weight.grad is not None
    with torch.no_grad():
        y2 = ln(x)                  # library kernel
    torch.testing.assert_close(y2, y.detach(), rtol=1e-5, atol=1e-5)
    assert not torch.equal(torch.zeros(1), torch.ones(1))
    xs = torch.randn(4, 7, device=DEV)          # 7 channels: unsupported -> stock path, no error
    with torch.no_grad():
        assert LayerNorm(7).to(DEV)(xs).shape == xs.shape


def test_layernorm_rejects_what_it_cannot_do():
    from dcnv4_b200 import ops
    x = torch.randn(4, 12, device=DEV, dtype=torch.float16)   # 24 bytes per row
    w = torch.ones(12, device=DEV, dtype=torch.float16)
    assert not ops.layer_norm_supported(x, w)
    with pytest.raises(ValueError):
        ops.layer_norm_forward(x, w, w, 1e-6)
    with pytest.raises(ValueError):
        big = torch.randn(2, 4096, device=DEV, dtype=torch.float16)
        ops.layer_norm_forward(big, torch.ones(4096, device=DEV, dtype=torch.float16),
                               torch.ones(4096, device=DEV, dtype=torch.float16), 1e-6)
