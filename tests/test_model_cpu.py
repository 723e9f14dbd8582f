"""FlashInternImage restatement: structure checks that need no GPU (construction only)."""
import pytest
import torch

from dcnv4_b200.flash_intern_image import CONFIGS, DownsampleLayer, StemLayer, flash_intern_image


@pytest.mark.parametrize("size,millions", [("t", 30), ("s", 50), ("b", 97), ("l", 223)])
def test_parameter_counts_match_the_published_model_sizes(size, millions):
    # README.md:29-32 of the reference: 30M / 50M / 97M / 223M parameters
    n = sum(p.numel() for p in flash_intern_image(size).parameters()) / 1e6
    assert abs(n - millions) < 1.0


def test_state_dict_keys_follow_the_reference_naming():
    m = flash_intern_image("s")
    keys = set(m.state_dict())
    for k in ("patch_embed.conv1.weight", "patch_embed.norm1.1.weight", "patch_embed.norm2.1.bias",
              "levels.0.blocks.0.norm1.0.weight", "levels.0.blocks.0.dcn.offset_mask.weight",
              "levels.0.blocks.0.dcn.offset_mask_dw.weight", "levels.0.blocks.0.dcn.value_proj.bias",
              "levels.0.blocks.0.dcn.output_proj.weight", "levels.0.blocks.0.gamma1", "levels.0.blocks.0.mlp.fc1.weight",
              "levels.0.downsample.conv.weight", "levels.0.downsample.norm.1.weight",
              "levels.3.blocks.3.mlp.fc2.weight", "conv_head.0.weight", "conv_head.1.0.weight", "head.bias"):
        assert k in keys, k
    assert "levels.0.norm.0.weight" not in keys            # post-norm models have no block-level norm
    assert "levels.0.norm.0.weight" in set(flash_intern_image("t").state_dict())
    assert "levels.3.downsample.conv.weight" not in keys   # the last level does not downsample


def test_offset_mask_layers_start_at_zero_and_have_padded_width():
    m = flash_intern_image("t")
    widths = []
    for lvl, G in zip(m.levels, CONFIGS["t"]["groups"]):
        dcn = lvl.blocks[0].dcn
        assert float(dcn.offset_mask.weight.abs().sum()) == 0.0 and float(dcn.offset_mask.bias.abs().sum()) == 0.0
        widths.append(dcn.offset_mask.out_features)
        assert dcn.group == G and dcn.group_channels == 16
    assert widths == [112, 216, 432, 864]


def test_stem_and_downsample_shapes_on_cpu():
    stem = StemLayer(3, 64).eval()
    x = torch.randn(2, 3, 64, 48)
    y = stem(x)
    assert y.shape == (2, 16, 12, 64) and y.is_contiguous()
    down = DownsampleLayer(64).eval()
    z, shape = down(y.view(2, 16 * 12, 64), (16, 12))
    assert shape == (8, 6) and z.shape == (2, 48, 128)


def test_fused_linear_predicates_reject_cpu_and_odd_inputs():
    """The helpers that decide whether the fused tensor-core kernels apply: never on CPU tensors,
    never for shapes the kernels do not cover -- the stock PyTorch path then runs and gives the
    same interface (a tensor, or a (y, norm(y)) pair)."""
    import torch
    from dcnv4_b200 import ops
    lin = torch.nn.Linear(64, 128)
    norm = torch.nn.LayerNorm(128, eps=1e-6)
    x = torch.randn(5, 7, 64)
    assert not ops.linear_supported(x, lin.weight)
    assert ops._norm_fusable(norm, 128, torch.float32)          # shape rule only; dtype / device gate elsewhere
    assert not ops._norm_fusable(norm, 128, torch.float16)      # parameters must match the activations' dtype
    assert not ops._norm_fusable(torch.nn.LayerNorm(160), 160, torch.float32)     # above 128: multiples of 64
    assert not ops._norm_fusable(torch.nn.LayerNorm(512), 512, torch.float32)     # a row must fit one tile
    assert not ops._norm_fusable(torch.nn.LayerNorm(128, elementwise_affine=False), 128, torch.float32)
    with torch.no_grad():
        y = ops.linear_module_forward(x, lin)
        torch.testing.assert_close(y, lin(x))
        r = torch.randn(5, 7, 128)
        y2, z2 = ops.linear_module_forward(x, lin, r, "gelu", norm)
        want = r + torch.nn.functional.gelu(lin(x))
        torch.testing.assert_close(y2, want)
        torch.testing.assert_close(z2, norm(want))


def test_layers_chain_their_layernorms_without_changing_the_result():
    """InternImageBlock hands each layer the already-normalised input and the next LayerNorm;
    on CPU everything falls back to the stock modules, so the chained forward must equal the
    plain layer-by-layer formula exactly."""
    import torch
    from dcnv4_b200 import flash_intern_image as fii
    torch.manual_seed(0)
    layer_cls = fii.InternImageLayer

    class Core(torch.nn.Module):      # stands in for DCNv4 (CUDA only): same call signature
        def __init__(self, channels, **kw):
            super().__init__()
            self.proj = torch.nn.Linear(channels, channels)

        def forward(self, x, shape=None, residual=None, norm=None):
            y = self.proj(x)
            y = y if residual is None else residual + y
            return y if norm is None else (y, norm(y))

    blk = fii.InternImageBlock(core_op=Core, channels=32, depth=3, groups=2, downsample=False, drop_path=0.0).eval()
    x = torch.randn(2, 16, 32)
    with torch.no_grad():
        got, _ = blk(x, (4, 4))
        want = x
        for layer in blk.blocks:
            want = want + layer.dcn(layer.norm1(want), (4, 4))
            want = want + layer.mlp(layer.norm2(want), (4, 4))
        want = blk.norm(want)
    torch.testing.assert_close(got, want)
    assert isinstance(blk.blocks[0], layer_cls)


@pytest.mark.parametrize("size", ["t", "s", "b", "l"])
def test_state_dict_matches_the_reference_model_key_for_key(size):
    """Every parameter / buffer name and shape of the reference's own FlashInternImage
    (classification/models/flash_intern_image.py:235-770, built with the released settings; fixture
    written by tests/golden/make_state_dict_fixture.py) exists here with the same shape, and nothing
    else does: a released checkpoint loads with strict=True."""
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "flash_intern_image_state_dicts.json")) as f:
        want = json.load(f)[size]
    got = {k: list(v.shape) for k, v in flash_intern_image(size).state_dict().items()}
    assert set(got) == set(want), (sorted(set(want) - set(got))[:5], sorted(set(got) - set(want))[:5])
    bad = [k for k in want if got[k] != want[k]]
    assert not bad, [(k, got[k], want[k]) for k in bad[:5]]


def test_fused_projection_cache_is_dropped_when_parameters_may_have_changed_unseen():
    """The stacked value/offset-mask weights are keyed on version counters, which writes through
    `.data` bypass; train(), load_state_dict() and _reset_parameters() drop the cache."""
    from dcnv4_b200 import DCNv4, ops
    mod = DCNv4(channels=64, group=4)
    paired = mod.__dict__["_paired_proj"] = ops.PairedLinear(mod.value_proj, mod.offset_mask)
    for action in (lambda: mod.train(False), lambda: mod.load_state_dict(mod.state_dict()),
                   mod._reset_parameters, mod.invalidate_fused_weights):
        paired._key = ("stale",)
        paired._weight = torch.zeros(1)
        action()
        assert paired._key is None and paired._weight is None


def test_fused_offset_policy_thresholds(monkeypatch):
    """The module fuses the offset/mask Linear into the sampling kernel from 128 channels up at any batch
    and for narrower layers only when there are many rows per SM; the switch turns it off."""
    from dcnv4_b200 import ops
    monkeypatch.setattr(ops, "_sm_count", lambda device: 148)
    monkeypatch.setattr(ops, "_FUSED_OFFSET_ENV", "")
    monkeypatch.setattr(ops, "FUSED_OFFSET_MASK", True)
    assert ops.fused_offset_pays(100, 128, "cuda:0")
    assert ops.fused_offset_pays(256 * 56 * 56, 64, "cuda:0")
    assert not ops.fused_offset_pays(64 * 56 * 56, 64, "cuda:0")
    monkeypatch.setattr(ops, "_FUSED_OFFSET_ENV", "1")
    assert ops.fused_offset_pays(1, 64, "cuda:0")
    monkeypatch.setattr(ops, "FUSED_OFFSET_MASK", False)
    assert not ops.fused_offset_pays(10 ** 9, 512, "cuda:0")


def test_cpu_input_is_refused_by_the_operator_not_by_the_fusion_policy():
    """No CPU fallback: a CPU tensor reaches the operator's own check (RuntimeError naming CUDA)."""
    from dcnv4_b200.modules import DCNv4
    m = DCNv4(channels=64, group=4).eval()
    with torch.no_grad(), pytest.raises(RuntimeError, match="CUDA"):
        m(torch.randn(1, 16, 64))
