"""FlashInternImage on the GPU: the model built on the CUDA DCNv4 op equals the same model with
the op replaced by the CPU oracle; fp16 inference and a training step run."""
import pytest
import torch

from oracle import cref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_every_dcn_layer_of_a_tiny_model_matches_the_oracle():
    """Run a small FlashInternImage once, capture what each DCNv4 layer saw and produced, and
    recompute every layer from its own weights with the CPU oracle as the core.  (Comparing only
    the logits would mix in the amplification of 1e-6 differences by the random-init layers.)"""
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
    seen = []
    hooks = [m.register_forward_hook(lambda mod, args, kwargs, out: seen.append((mod, args, kwargs, out)),
                                     with_kwargs=True)
             for m in model.modules() if isinstance(m, dcn_mod.DCNv4)]
    x = torch.randn(2, 3, 64, 96, device=DEV)
    with torch.no_grad():
        y = model(x)
    for h in hooks:
        h.remove()
    assert y.shape == (2, 10) and torch.isfinite(y).all()
    assert len(seen) == 5
    for mod, args, kwargs, out in seen:
        inp = args[0]
        H, W = kwargs.get("shape") or args[1]
        normed = None
        if kwargs.get("norm") is not None:           # the layer asked for (result, norm(result))
            out, normed = out
        N, L, C = inp.shape
        with torch.no_grad():
            v = mod.value_proj(inp).reshape(N, H, W, C)
            om = mod.offset_mask(inp).reshape(N, H, W, -1)
            core = cref.dcnv4_forward(v.cpu(), om.cpu(), 3, 3, 1, 1, 1, 1, 1, 1, mod.group, mod.group_channels,
                                      mod.offset_scale, 0)
            ref = mod.output_proj(core.to(DEV).float().reshape(N, L, C))
            if kwargs.get("residual") is not None:      # the block lets the module add its skip path
                ref = kwargs["residual"] + ref
        torch.testing.assert_close(out, ref, rtol=1e-3, atol=1e-4)
        if normed is not None:
            torch.testing.assert_close(normed, kwargs["norm"](out), rtol=1e-4, atol=1e-5)


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


def test_batchnorm_folding_and_graphed_inference_reproduce_the_eager_model():
    import copy
    from dcnv4_b200.flash_intern_image import GraphedInference, flash_intern_image, fold_batchnorm_
    torch.manual_seed(3)
    model = flash_intern_image("t").to(DEV).eval()
    with torch.no_grad():          # non-trivial BatchNorm statistics
        for m in model.modules():
            if isinstance(m, torch.nn.BatchNorm2d):
                m.running_mean.normal_(0, 0.5)
                m.running_var.uniform_(0.5, 2.0)
                m.weight.uniform_(0.5, 1.5)
                m.bias.normal_(0, 0.2)
    x = torch.randn(3, 3, 224, 224, device=DEV)
    tf32 = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False     # compare the folding itself, not TF32 rounding of scaled weights
    try:
        with torch.no_grad():
            y = model(x)
            folded = fold_batchnorm_(copy.deepcopy(model))
            y_folded = folded(x)
    finally:
        torch.backends.cudnn.allow_tf32 = tf32
    torch.testing.assert_close(y_folded, y, rtol=1e-3, atol=2e-4)
    # graph replay vs eager: same kernels except for cuDNN/cuBLAS algorithm choices (TF32 convolutions)
    graphed = GraphedInference(folded, x)
    y_graph = graphed(x).clone()
    torch.testing.assert_close(y_graph, y_folded, rtol=1e-2, atol=1e-3)
    x2 = torch.randn_like(x)
    with torch.no_grad():
        y2 = graphed(x2).clone()
        torch.testing.assert_close(y2, folded(x2), rtol=1e-2, atol=1e-3)
    assert not torch.allclose(y2, y_graph)      # the replay really consumed the new input
