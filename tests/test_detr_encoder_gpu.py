"""Deformable-DETR encoder layer on the GPU: the flash path (one packed tensor, softmax inside the
kernel) equals the layer's own parts composed around the CPU oracle, and the grid_sample path."""
import pytest
import torch

from oracle import cref

pytestmark = pytest.mark.gpu
DEV = "cuda"
LEVELS = ((20, 30), (10, 15), (5, 8), (3, 4))


def _setup(dropout=0.0):
    from dcnv4_b200 import detr_encoder as de
    torch.manual_seed(2)
    layer = de.DeformableDetrEncoderLayer(embed_dims=256, num_heads=8, num_levels=4, num_points=4,
                                          feedforward_channels=512, dropout=dropout, use_flash=True).to(DEV).eval()
    with torch.no_grad():
        layer.attentions[0].sampling_offsets.weight.normal_(0, 0.05)
        layer.attentions[0].attention_weights.weight.normal_(0, 0.05)
    shapes = torch.tensor(LEVELS, dtype=torch.int64, device=DEV)
    sizes = shapes[:, 0] * shapes[:, 1]
    starts = torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))
    Len = int(sizes.sum())
    x = torch.randn(Len, 2, 256, device=DEV)
    pos = torch.randn(Len, 2, 256, device=DEV) * 0.1
    ref_pts = de.DeformableDetrEncoder.get_reference_points(LEVELS, torch.ones(2, 4, 2, device=DEV))
    mask = torch.zeros(2, Len, dtype=torch.bool, device=DEV)
    mask[1, -40:] = True
    return de, layer, x, pos, ref_pts, shapes, starts, mask


def test_encoder_layer_flash_path_matches_parts_around_the_oracle():
    de, layer, x, pos, ref_pts, shapes, starts, mask = _setup()
    attn = layer.attentions[0]
    with torch.no_grad():
        y = layer(x, query_pos=pos, key_padding_mask=mask, reference_points=ref_pts, spatial_shapes=shapes,
                  level_start_index=starts)
        q = (x + pos).permute(1, 0, 2)
        value = attn.value_proj(x.permute(1, 0, 2)).masked_fill(mask[..., None], 0.0).view(2, -1, 8, 32)
        off = attn.sampling_offsets(q).view(2, -1, 8, 4, 4, 2)
        logits = attn.attention_weights(q).view(2, -1, 8, 16)
        norm = torch.stack([shapes[..., 1], shapes[..., 0]], -1)
        loc = (ref_pts[:, :, None, :, None, :] + off / norm[None, None, None, :, None, :]).flatten(-3)
        sla = torch.cat([loc, logits], -1)
        core = cref.fda_forward(value.cpu(), shapes.cpu(), starts.cpu(), sla.cpu(), 4).to(DEV).float()
        a = attn.output_proj(core).permute(1, 0, 2) + x
        h = layer.norms[0](a)
        ref = layer.norms[1](layer.ffns[0](h))
    torch.testing.assert_close(y, ref, rtol=1e-3, atol=2e-4)
    # the grid_sample path of the same layer agrees as well
    attn.use_flash = False
    with torch.no_grad():
        y2 = layer(x, query_pos=pos, key_padding_mask=mask, reference_points=ref_pts, spatial_shapes=shapes,
                   level_start_index=starts)
    attn.use_flash = True
    torch.testing.assert_close(y, y2, rtol=1e-3, atol=2e-4)


def test_encoder_trains_through_the_flash_operator_and_runs_in_fp16():
    de, layer, x, pos, ref_pts, shapes, starts, mask = _setup()
    x = x.clone().requires_grad_(True)
    y = layer(x, query_pos=pos, reference_points=ref_pts, spatial_shapes=shapes, level_start_index=starts)
    y.square().mean().backward()
    attn = layer.attentions[0]
    assert torch.isfinite(x.grad).all() and float(attn.sampling_offsets.weight.grad.abs().sum()) > 0
    assert float(attn.value_proj.weight.grad.abs().sum()) > 0
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.float16):
        y16 = layer(x, query_pos=pos, reference_points=ref_pts, spatial_shapes=shapes, level_start_index=starts)
    torch.testing.assert_close(y16.float(), y.detach(), rtol=3e-2, atol=3e-2)
    enc = de.DeformableDetrEncoder(num_layers=2, embed_dims=256, feedforward_channels=512, dropout=0.0).to(DEV).eval()
    feats = [torch.randn(2, 256, h, w, device=DEV) for h, w in LEVELS]
    with torch.no_grad():
        mem = enc(feats, [torch.zeros_like(f) for f in feats])
    assert mem.shape == (x.shape[0], 2, 256) and torch.isfinite(mem).all()
