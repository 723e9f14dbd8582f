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
    for k in ("patch_embed.conv1.weight", "patch_embed.norm1.0.running_mean", "patch_embed.norm2.0.weight",
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
