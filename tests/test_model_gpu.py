"""FlashInternImage on the GPU: the model built on the CUDA DCNv4 op equals the same model with
the op replaced by the CPU oracle; fp16 inference and a training step run."""
import pytest
import torch

from oracle import cref

pytestmark = pytest.mark.gpu
DEV = "cuda"


class _OracleDCN(torch.autograd.Function):
    """DCNv4Function stand-in that computes the forward with the CPU oracle."""

    @staticmethod
    def forward(ctx, x, om, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, step, rc):
        out = cref.dcnv4_forward(x.float().cpu(), om.float().cpu(), kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, rc)
        return out.to(device=x.device, dtype=x.dtype)


def test_tiny_model_matches_oracle_composition(monkeypatch):
    from dcnv4_b200 import flash_intern_image as fii
    from dcnv4_b200.modules import dcnv4 as dcn_mod
    torch.manual_seed(0)
    model = fii.FlashInternImage(channels=32, depths=(1, 1, 2, 1), groups=(2, 4, 8, 16), num_classes=10,
                                 offset_scale=1.0, drop_path_rate=0.0).to(DEV).eval()
    with torch.no_grad():     # give the zero-initialised offset/mask layers something to do
        for m in model.modules():
            if isinstance(m, dcn_mod.DCNv4):
                m.offset_mask.weight.normal_(0, 0.2)
                m.offset_mask.bias.uniform_(0, 1)
    x = torch.randn(2, 3, 64, 96, device=DEV)
    with torch.no_grad():
        y = model(x)
        monkeypatch.setattr(dcn_mod, "DCNv4Function", _OracleDCN)
        y_ref = model(x)
    assert y.shape == (2, 10)
    torch.testing.assert_close(y, y_ref, rtol=1e-3, atol=1e-4)


def test_flash_intern_image_t_fp16_inference_and_train_step():
    from dcnv4_b200.flash_intern_image import flash_intern_image
    torch.manual_seed(0)
    model = flash_intern_image("t").to(DEV)
    x = torch.randn(4, 3, 224, 224, device=DEV)
    model.eval()
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.float16):
        y = model(x)
    assert y.shape == (4, 1000) and y.dtype == torch.float16 and torch.isfinite(y).all()
    model.half()
    with torch.no_grad():
        y16 = model(x.half())
    assert torch.isfinite(y16).all()
    torch.testing.assert_close(y16.float(), y.float(), rtol=5e-2, atol=5e-2)

    model.float().train()
    opt = torch.optim.SGD(model.parameters(), lr=1e-3)
    labels = torch.randint(0, 1000, (4,), device=DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = torch.nn.functional.cross_entropy(model(x).float(), labels)
    loss.backward()
    g = model.levels[0].blocks[0].dcn.offset_mask.weight.grad
    assert g is not None and torch.isfinite(g).all() and torch.isfinite(loss)
    opt.step()
