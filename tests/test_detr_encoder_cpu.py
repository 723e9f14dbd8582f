"""Deformable-DETR encoder restatement, parts that need no GPU: the grid_sample attention path
equals the C oracle of the operator, parameter names follow the mmcv modules, reference points
follow Deformable-DETR's rule."""
import torch

from dcnv4_b200 import detr_encoder as de
from oracle import cref, inputs as oin

LEVELS = ((12, 16), (6, 8), (3, 4))


def test_torch_attention_path_equals_the_operator_oracle():
    torch.manual_seed(0)
    t = oin.fda_inputs(2, LEVELS, 4, 16, 4, Len_q=50, seed=3, loc_lo=-0.2, loc_hi=1.2)
    L, P = len(LEVELS), 4
    loc = t["sampling_loc_attn"][..., : 2 * L * P].reshape(2, 50, 4, L, P, 2)
    logits = t["sampling_loc_attn"][..., 2 * L * P:]
    w = logits.softmax(-1).reshape(2, 50, 4, L, P)
    got = de.multi_scale_deformable_attn_torch(t["value"].double(), t["spatial_shapes"], loc.double(), w.double())
    ref = cref.fda_forward(t["value"], t["spatial_shapes"], t["level_start_index"], t["sampling_loc_attn"], P)
    torch.testing.assert_close(got, ref, rtol=1e-5, atol=1e-5)


def test_parameter_names_follow_the_mmcv_modules():
    layer = de.DeformableDetrEncoderLayer(embed_dims=64, num_heads=4, num_levels=3, num_points=4, feedforward_channels=128)
    keys = set(layer.state_dict())
    for k in ("attentions.0.sampling_offsets.weight", "attentions.0.attention_weights.bias",
              "attentions.0.value_proj.weight", "attentions.0.output_proj.bias", "ffns.0.layers.0.0.weight",
              "ffns.0.layers.1.bias", "norms.0.weight", "norms.1.bias"):
        assert k in keys, k
    assert len(keys) == 16
    attn = layer.attentions[0]
    assert float(attn.sampling_offsets.weight.abs().sum()) == 0.0 and float(attn.attention_weights.bias.abs().sum()) == 0.0
    bias = attn.sampling_offsets.bias.view(4, 3, 4, 2)
    torch.testing.assert_close(bias[0, 0, :, 0], torch.tensor([1.0, 2.0, 3.0, 4.0]))   # head 0 looks along +x


def test_encoder_runs_on_cpu_and_reference_points_are_position_centres():
    torch.manual_seed(1)
    enc = de.DeformableDetrEncoder(num_layers=2, embed_dims=64, num_heads=4, num_levels=3, num_points=4,
                                   feedforward_channels=128, dropout=0.0, use_flash=True).eval()
    feats = [torch.randn(2, 64, h, w) for h, w in LEVELS]
    pos = [torch.randn(2, 64, h, w) for h, w in LEVELS]
    with torch.no_grad():
        mem = enc(feats, pos)          # CPU tensors: the grid_sample path runs even with use_flash on
    assert mem.shape == (sum(h * w for h, w in LEVELS), 2, 64) and torch.isfinite(mem).all()
    ref = de.DeformableDetrEncoder.get_reference_points(LEVELS, torch.ones(2, 3, 2))
    assert ref.shape == (2, mem.shape[0], 3, 2)
    torch.testing.assert_close(ref[0, 0, 0], torch.tensor([0.5 / 16, 0.5 / 12]))
    torch.testing.assert_close(ref[0, 12 * 16, 1], torch.tensor([0.5 / 8, 0.5 / 6]))
    # padding masks: padded values are zeroed and reference points use the valid extent
    masks = [torch.zeros(2, h, w, dtype=torch.bool) for h, w in LEVELS]
    for m in masks:
        m[1, :, m.shape[2] // 2:] = True
    with torch.no_grad():
        mem2 = enc(feats, pos, masks)
    torch.testing.assert_close(mem2[:, 0], mem[:, 0])              # image 0 has no padding: unchanged
    assert not torch.allclose(mem2[:, 1], mem[:, 1])
