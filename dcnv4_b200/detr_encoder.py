"""Deformable-DETR / DINO encoder around the flash deformable-attention operator, without mmcv.

The reference wires its operator into mmdet through `FlashMultiScaleDeformableAttention`
(detection/mmdet_custom/models/dense_heads/msda.py:218-369), a subclass of mmcv's
`MultiScaleDeformableAttention` whose flash branch is left unfinished (`assert False`,
msda.py:350-351); the layer and encoder around it come from mmcv / mmdet
(`BaseTransformerLayer` with operation order self_attn, norm, ffn, norm, and
`DeformableDetrTransformerEncoder.get_reference_points`).  mmcv is not a dependency of this
package, so the three pieces are restated here on plain `torch.nn`, with

* the parameter names of the mmcv modules (`attentions.0.sampling_offsets.weight`,
  `ffns.0.layers.0.0.weight`, `norms.1.bias`, ...), so that encoder weights of released
  Deformable-DETR / DINO checkpoints load key for key;
* the forward contract of msda.py:246-369 (sequence-first tensors unless `batch_first`,
  `query_pos` added to the query, `key_padding_mask` zeroing padded values, 2- or 4-component
  reference points, dropout + identity at the end);
* `use_flash=True` finished: sampling locations and attention logits are packed into the one
  tensor the operator takes and the softmax over levels x points runs inside the kernel
  (`FlashDeformAttnFunction`); `use_flash=False` is a grid_sample formulation that also runs on
  the CPU and serves as the reference in the tests.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .functions import FlashDeformAttnFunction


def multi_scale_deformable_attn_torch(value: torch.Tensor, spatial_shapes: torch.Tensor,
                                      sampling_locations: torch.Tensor, attention_weights: torch.Tensor) -> torch.Tensor:
    """value (B, Len_in, heads, D); sampling_locations (B, Len_q, heads, L, P, 2) normalised (x, y);
    attention_weights (B, Len_q, heads, L, P), already normalised.  Returns (B, Len_q, heads*D).
    Per level: bilinear sampling with pixel centres at half-integers and zero padding, the pixel
    convention of the operator (DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:185-198)."""
    B, _, H, D = value.shape
    _, Lq, _, L, P, _ = sampling_locations.shape
    sizes = [(int(h), int(w)) for h, w in spatial_shapes.tolist()]
    out = value.new_zeros(B * H, D, Lq)
    start = 0
    for lvl, (h, w) in enumerate(sizes):
        v = value[:, start:start + h * w].permute(0, 2, 3, 1).reshape(B * H, D, h, w)
        start += h * w
        grid = (2 * sampling_locations[:, :, :, lvl] - 1).permute(0, 2, 1, 3, 4).reshape(B * H, Lq, P, 2)
        sampled = F.grid_sample(v, grid, mode="bilinear", padding_mode="zeros", align_corners=False)  # (BH, D, Lq, P)
        wgt = attention_weights[:, :, :, lvl].permute(0, 2, 1, 3).reshape(B * H, 1, Lq, P)
        out = out + (sampled * wgt).sum(-1)
    return out.view(B, H * D, Lq).transpose(1, 2).contiguous()


class FlashMultiScaleDeformableAttention(nn.Module):
    """Multi-scale deformable attention with the constructor and forward contract of the
    reference's mmdet plug-in (msda.py:233-369) and the parameter names of the mmcv module it
    extends."""

    def __init__(self, embed_dims: int = 256, num_heads: int = 8, num_levels: int = 4, num_points: int = 4,
                 im2col_step: int = 64, dropout: float = 0.1, batch_first: bool = False, use_flash: bool = True,
                 use_softmax: bool = True):
        super().__init__()
        if embed_dims % num_heads != 0:
            raise ValueError(f"embed_dims must be divisible by num_heads, but got {embed_dims} and {num_heads}")
        self.embed_dims, self.num_heads, self.num_levels, self.num_points = embed_dims, num_heads, num_levels, num_points
        self.im2col_step, self.batch_first = im2col_step, batch_first
        self.use_flash, self.use_softmax = use_flash, use_softmax
        if use_flash and not use_softmax:
            raise ValueError("the flash operator normalises the attention weights itself: use_softmax must stay on")
        self.dropout = nn.Dropout(dropout)
        self.sampling_offsets = nn.Linear(embed_dims, num_heads * num_levels * num_points * 2)
        self.attention_weights = nn.Linear(embed_dims, num_heads * num_levels * num_points)
        self.value_proj = nn.Linear(embed_dims, embed_dims)
        self.output_proj = nn.Linear(embed_dims, embed_dims)
        self.init_weights()

    def init_weights(self) -> None:
        """Offsets start on a ring of directions, one per head, scaled by the point index; attention
        weights start uniform; projections xavier (the initialisation of the mmcv module, which is also
        that of DCNv4_op/DCNv4/modules/flash_deform_attn.py:64-82)."""
        nn.init.constant_(self.sampling_offsets.weight, 0.0)
        thetas = torch.arange(self.num_heads, dtype=torch.float32) * (2.0 * math.pi / self.num_heads)
        grid = torch.stack([thetas.cos(), thetas.sin()], -1)
        grid = (grid / grid.abs().max(-1, keepdim=True)[0]).view(self.num_heads, 1, 1, 2)
        grid = grid.repeat(1, self.num_levels, self.num_points, 1)
        for i in range(self.num_points):
            grid[:, :, i, :] *= i + 1
        with torch.no_grad():
            self.sampling_offsets.bias.copy_(grid.view(-1))
        nn.init.constant_(self.attention_weights.weight, 0.0)
        nn.init.constant_(self.attention_weights.bias, 0.0)
        nn.init.xavier_uniform_(self.value_proj.weight)
        nn.init.constant_(self.value_proj.bias, 0.0)
        nn.init.xavier_uniform_(self.output_proj.weight)
        nn.init.constant_(self.output_proj.bias, 0.0)

    def forward(self, query, key=None, value=None, identity=None, query_pos=None, key_padding_mask=None,
                reference_points=None, spatial_shapes=None, level_start_index=None, **kwargs):
        if value is None:
            value = query
        if identity is None:
            identity = query
        if query_pos is not None:
            query = query + query_pos
        if not self.batch_first:                      # (num_query, bs, C) -> (bs, num_query, C)
            query = query.permute(1, 0, 2)
            value = value.permute(1, 0, 2)
        bs, num_query, _ = query.shape
        _, num_value, _ = value.shape
        assert int((spatial_shapes[:, 0] * spatial_shapes[:, 1]).sum()) == num_value

        value = self.value_proj(value)
        if key_padding_mask is not None:
            value = value.masked_fill(key_padding_mask[..., None], 0.0)
        value = value.view(bs, num_value, self.num_heads, -1)
        offsets = self.sampling_offsets(query).view(bs, num_query, self.num_heads, self.num_levels, self.num_points, 2)
        logits = self.attention_weights(query).view(bs, num_query, self.num_heads, self.num_levels * self.num_points)
        if reference_points.shape[-1] == 2:
            normalizer = torch.stack([spatial_shapes[..., 1], spatial_shapes[..., 0]], -1)
            locations = reference_points[:, :, None, :, None, :] + offsets / normalizer[None, None, None, :, None, :]
        elif reference_points.shape[-1] == 4:
            locations = (reference_points[:, :, None, :, None, :2]
                         + offsets / self.num_points * reference_points[:, :, None, :, None, 2:] * 0.5)
        else:
            raise ValueError(f"Last dim of reference_points must be 2 or 4, but get {reference_points.shape[-1]} instead.")
        locations = locations.to(offsets.dtype)

        if self.use_flash and value.is_cuda:
            packed = torch.cat([locations.flatten(-3), logits], dim=-1).to(value.dtype)
            output = FlashDeformAttnFunction.apply(value.contiguous(), spatial_shapes, level_start_index,
                                                   packed.contiguous(), self.im2col_step, self.num_points)
        else:
            weights = logits.softmax(-1) if self.use_softmax else logits
            weights = weights.view(bs, num_query, self.num_heads, self.num_levels, self.num_points)
            output = multi_scale_deformable_attn_torch(value, spatial_shapes, locations, weights)
        output = self.output_proj(output)
        if not self.batch_first:
            output = output.permute(1, 0, 2)
        return self.dropout(output) + identity


class FFN(nn.Module):
    """Two-layer feed-forward block with residual; module tree of mmcv's FFN, hence the parameter
    names `layers.0.0.*` (first Linear, inside a Sequential with its activation and dropout) and
    `layers.1.*`."""

    def __init__(self, embed_dims: int = 256, feedforward_channels: int = 1024, ffn_drop: float = 0.1):
        super().__init__()
        self.layers = nn.Sequential(
            nn.Sequential(nn.Linear(embed_dims, feedforward_channels), nn.ReLU(inplace=True), nn.Dropout(ffn_drop)),
            nn.Linear(feedforward_channels, embed_dims),
            nn.Dropout(ffn_drop))

    def forward(self, x, identity=None):
        return (x if identity is None else identity) + self.layers(x)


class DeformableDetrEncoderLayer(nn.Module):
    """self_attn -> norm -> ffn -> norm, the operation order of Deformable-DETR's encoder layers;
    parameter names of mmcv's BaseTransformerLayer (`attentions.0`, `ffns.0`, `norms.0/1`)."""

    def __init__(self, embed_dims: int = 256, num_heads: int = 8, num_levels: int = 4, num_points: int = 4,
                 feedforward_channels: int = 1024, dropout: float = 0.1, use_flash: bool = True):
        super().__init__()
        self.attentions = nn.ModuleList([FlashMultiScaleDeformableAttention(
            embed_dims, num_heads, num_levels, num_points, dropout=dropout, batch_first=False, use_flash=use_flash)])
        self.ffns = nn.ModuleList([FFN(embed_dims, feedforward_channels, dropout)])
        self.norms = nn.ModuleList([nn.LayerNorm(embed_dims), nn.LayerNorm(embed_dims)])

    def forward(self, query, query_pos=None, key_padding_mask=None, reference_points=None, spatial_shapes=None,
                level_start_index=None):
        query = self.attentions[0](query, query_pos=query_pos, key_padding_mask=key_padding_mask,
                                   reference_points=reference_points, spatial_shapes=spatial_shapes,
                                   level_start_index=level_start_index)
        query = self.norms[0](query)
        query = self.ffns[0](query)
        return self.norms[1](query)


class DeformableDetrEncoder(nn.Module):
    """Stack of encoder layers over the flattened multi-level feature maps, with the reference
    points Deformable-DETR gives its encoder queries: every position attends around its own
    location in every level."""

    def __init__(self, num_layers: int = 6, embed_dims: int = 256, num_heads: int = 8, num_levels: int = 4,
                 num_points: int = 4, feedforward_channels: int = 1024, dropout: float = 0.1, use_flash: bool = True):
        super().__init__()
        self.layers = nn.ModuleList([DeformableDetrEncoderLayer(embed_dims, num_heads, num_levels, num_points,
                                                                feedforward_channels, dropout, use_flash)
                                     for _ in range(num_layers)])
        self.level_embeds = nn.Parameter(torch.empty(num_levels, embed_dims))
        nn.init.normal_(self.level_embeds)

    @staticmethod
    def get_reference_points(spatial_shapes: Sequence[Tuple[int, int]], valid_ratios: torch.Tensor) -> torch.Tensor:
        """Centres of all positions of all levels, normalised by the valid (un-padded) extent of their
        own level and re-scaled to every level's valid extent: (bs, sum H_l*W_l, num_levels, 2) as (x, y)."""
        device, dtype = valid_ratios.device, valid_ratios.dtype
        pts = []
        for lvl, (h, w) in enumerate(spatial_shapes):
            ys, xs = torch.meshgrid(torch.linspace(0.5, h - 0.5, h, dtype=dtype, device=device),
                                    torch.linspace(0.5, w - 0.5, w, dtype=dtype, device=device), indexing="ij")
            ys = ys.reshape(-1)[None] / (valid_ratios[:, None, lvl, 1] * h)
            xs = xs.reshape(-1)[None] / (valid_ratios[:, None, lvl, 0] * w)
            pts.append(torch.stack((xs, ys), -1))
        ref = torch.cat(pts, 1)
        return ref[:, :, None] * valid_ratios[:, None]

    def forward(self, feats: List[torch.Tensor], pos_embeds: List[torch.Tensor],
                masks: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """feats / pos_embeds: per level (bs, C, H_l, W_l); masks: per level (bs, H_l, W_l), True = padding.
        Returns the encoded memory (sum H_l*W_l, bs, C)."""
        shapes = [(int(f.shape[2]), int(f.shape[3])) for f in feats]
        bs = feats[0].shape[0]
        flat, pos, flat_masks, ratios = [], [], [], []
        for lvl, (f, pe) in enumerate(zip(feats, pos_embeds)):
            flat.append(f.flatten(2).transpose(1, 2))
            pos.append(pe.flatten(2).transpose(1, 2) + self.level_embeds[lvl].view(1, 1, -1))
            if masks is not None:
                m = masks[lvl]
                flat_masks.append(m.flatten(1))
                valid_h = (~m[:, :, 0]).sum(1).to(f.dtype) / m.shape[1]
                valid_w = (~m[:, 0, :]).sum(1).to(f.dtype) / m.shape[2]
                ratios.append(torch.stack([valid_w, valid_h], -1))
            else:
                ratios.append(f.new_ones(bs, 2))
        x = torch.cat(flat, 1).transpose(0, 1)            # (sum HW, bs, C)
        query_pos = torch.cat(pos, 1).transpose(0, 1)
        key_padding_mask = torch.cat(flat_masks, 1) if masks is not None else None
        valid_ratios = torch.stack(ratios, 1)              # (bs, L, 2)
        spatial_shapes = torch.tensor(shapes, dtype=torch.int64, device=x.device)
        sizes = spatial_shapes[:, 0] * spatial_shapes[:, 1]
        level_start_index = torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))
        reference_points = self.get_reference_points(shapes, valid_ratios)
        for layer in self.layers:
            x = layer(x, query_pos=query_pos, key_padding_mask=key_padding_mask, reference_points=reference_points,
                      spatial_shapes=spatial_shapes, level_start_index=level_start_index)
        return x
