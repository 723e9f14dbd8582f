"""`DCNv4` module with the reference's constructor, parameter names and forward contract
(DCNv4_op/DCNv4/modules/dcnv4.py:28-153), so released checkpoints load unchanged:
`offset_mask`, `value_proj`, `output_proj`, optional `offset_mask_dw` and
`center_feature_scale_proj_{weight,bias}`.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn.init import constant_, xavier_uniform_

from .. import ops
from ..functions import DCNv4Function


class CenterFeatureScaleModule(nn.Module):
    """sigmoid(linear(query)) per group (DCNv4_op/DCNv4/modules/dcnv4.py:18-26)."""

    def forward(self, query, center_feature_scale_proj_weight, center_feature_scale_proj_bias):
        return F.linear(query, weight=center_feature_scale_proj_weight,
                        bias=center_feature_scale_proj_bias).sigmoid()


class DCNv4(nn.Module):
    def __init__(self, channels=64, kernel_size=3, stride=1, pad=1, dilation=1, group=4,
                 offset_scale=1.0, dw_kernel_size=None, center_feature_scale=False,
                 remove_center=False, output_bias=True, without_pointwise=False, **kwargs):
        super().__init__()
        if channels % group != 0:
            raise ValueError(f"channels must be divisible by group, but got {channels} and {group}")
        _d_per_group = channels // group
        assert _d_per_group % 16 == 0

        self.offset_scale = offset_scale
        self.channels = channels
        self.kernel_size = kernel_size
        self.stride = stride
        self.dilation = dilation
        self.pad = pad
        self.group = group
        self.group_channels = channels // group
        self.dw_kernel_size = dw_kernel_size
        self.center_feature_scale = center_feature_scale
        self.remove_center = int(remove_center)
        self.without_pointwise = without_pointwise

        self.K = group * (kernel_size * kernel_size - self.remove_center)
        if dw_kernel_size is not None:
            self.offset_mask_dw = nn.Conv2d(channels, channels, dw_kernel_size, stride=1,
                                            padding=(dw_kernel_size - 1) // 2, groups=channels)
        self.offset_mask = nn.Linear(channels, int(math.ceil((self.K * 3) / 8) * 8))
        if not without_pointwise:
            self.value_proj = nn.Linear(channels, channels)
            self.output_proj = nn.Linear(channels, channels, bias=output_bias)
        self._reset_parameters()

        if center_feature_scale:
            self.center_feature_scale_proj_weight = nn.Parameter(
                torch.zeros((group, channels), dtype=torch.float))
            self.center_feature_scale_proj_bias = nn.Parameter(
                torch.tensor(0.0, dtype=torch.float).view((1,)).repeat(group, ))
            self.center_feature_scale_module = CenterFeatureScaleModule()

    def invalidate_fused_weights(self) -> None:
        """Drop the stacked value/offset-mask weights of the inference path.  Needed only after
        writing a parameter through `.data`, which PyTorch's version counters do not see."""
        paired = self.__dict__.get("_paired_proj")
        if paired is not None:
            paired.invalidate()

    def train(self, mode: bool = True):
        self.invalidate_fused_weights()
        return super().train(mode)

    def _load_from_state_dict(self, *args, **kwargs):
        self.invalidate_fused_weights()
        return super()._load_from_state_dict(*args, **kwargs)

    def _reset_parameters(self):
        self.invalidate_fused_weights()
        constant_(self.offset_mask.weight.data, 0.)
        constant_(self.offset_mask.bias.data, 0.)
        if not self.without_pointwise:
            xavier_uniform_(self.value_proj.weight.data)
            constant_(self.value_proj.bias.data, 0.)
            xavier_uniform_(self.output_proj.weight.data)
            if self.output_proj.bias is not None:
                constant_(self.output_proj.bias.data, 0.)

    def _blend_fusable(self, x, x_proj) -> bool:
        w = self.center_feature_scale_proj_weight
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or x_proj.requires_grad or w.requires_grad)
        return (not needs_grad and not torch.is_autocast_enabled() and x.dtype == x_proj.dtype
                and self.center_feature_scale_proj_bias.dtype == w.dtype
                and ops.center_scale_blend_supported(x, w, self.group_channels))

    def _offsets_fusable(self, input) -> bool:
        """Inference on 16-bit CUDA tensors in the configuration the fused kernel is written for (3x3,
        stride 1, pad 1, dilation 1, all nine points, 16 channels per group), at a size where it pays."""
        params = [self.offset_mask.weight] + ([] if self.without_pointwise else [self.value_proj.weight])
        needs_grad = torch.is_grad_enabled() and (input.requires_grad or any(p.requires_grad for p in params))
        return (input.is_cuda and input.is_contiguous() and input.numel() > 0
                and input.dtype in (torch.float16, torch.bfloat16) and self.offset_mask.weight.dtype == input.dtype
                and not needs_grad and not torch.is_autocast_enabled()
                and not self.remove_center and self.kernel_size == 3 and self.stride == 1 and self.pad == 1
                and self.dilation == 1 and self.group_channels == 16
                and ops.fused_offset_pays(input.numel() // input.shape[-1], self.channels, input.device))

    def forward(self, input, shape=None, residual=None, norm=None):
        """input (N, L, C) with L = H*W; `shape` = (H, W) when the map is not square.
        Returns (N, L, C).  Two extensions over the reference signature serve the layer that
        embeds this module: `residual` (N, L, C) is added to the result, and with `norm` (an
        nn.LayerNorm over C) the pair `(result, norm(result))` is returned; at inference both are
        fused into the output projection."""
        N, L, C = input.shape
        if shape is not None:
            H, W = shape
        else:
            H, W = int(L ** 0.5), int(L ** 0.5)

        fuse = self._offsets_fusable(input)
        paired = None
        if not fuse and not self.without_pointwise and self.dw_kernel_size is None:
            # both projections read the layer input: at inference they are one tensor-core product
            paired = self.__dict__.get("_paired_proj")
            if paired is None or paired.first is not self.value_proj or paired.second is not self.offset_mask:
                paired = self.__dict__["_paired_proj"] = ops.PairedLinear(self.value_proj, self.offset_mask)
            if not (input.is_contiguous() and paired.usable(input)):
                paired = None
        offset_mask = offset_mask_input = None
        if paired is not None:
            x, offset_mask = paired(input)
            x = x.reshape(N, H, W, -1)
            offset_mask = offset_mask.reshape(N, H, W, -1)
        else:
            x = input
            if not self.without_pointwise:
                x = ops.linear_module_forward(x, self.value_proj) if fuse else self.value_proj(x)
            x = x.reshape(N, H, W, -1)
            if self.dw_kernel_size is not None:
                offset_mask_input = self.offset_mask_dw(input.view(N, H, W, C).permute(0, 3, 1, 2))
                offset_mask_input = offset_mask_input.permute(0, 2, 3, 1).reshape(N, L, C)
            else:
                offset_mask_input = input
            # inference: the sampling kernel computes the offset/mask rows itself from the Linear's input
            if fuse and not offset_mask_input.is_contiguous():
                offset_mask_input = offset_mask_input.contiguous()
            fuse = fuse and ops.fused_offset_supported(x, offset_mask_input, self.offset_mask.weight,
                                                       self.offset_mask.bias, self.group, self.group_channels)
            if not fuse:
                offset_mask = self.offset_mask(offset_mask_input).reshape(N, H, W, -1)

        x_proj = x
        if offset_mask is None:
            x = ops.dcnv4_fused_offset_forward(x, offset_mask_input, self.offset_mask.weight, self.offset_mask.bias,
                                               self.group, self.group_channels, self.offset_scale)
        else:
            x = DCNv4Function.apply(
                x, offset_mask, self.kernel_size, self.kernel_size, self.stride, self.stride,
                self.pad, self.pad, self.dilation, self.dilation, self.group, self.group_channels,
                self.offset_scale, 256, self.remove_center)

        if self.center_feature_scale and self._blend_fusable(x, x_proj):
            # inference: Linear + sigmoid + repeat + blend in one pass over x and x_proj
            x = ops.center_scale_blend_forward(x, x_proj.contiguous(), self.center_feature_scale_proj_weight,
                                               self.center_feature_scale_proj_bias)
        elif self.center_feature_scale:
            scale = self.center_feature_scale_module(
                x, self.center_feature_scale_proj_weight, self.center_feature_scale_proj_bias)
            scale = scale[..., None].repeat(1, 1, 1, 1, self.channels // self.group).flatten(-2)
            x = x * (1 - scale) + x_proj * scale

        x = x.view(N, L, -1)
        if not self.without_pointwise:
            return ops.linear_module_forward(x, self.output_proj, residual, "none", norm)
        x = x if residual is None else residual + x
        return x if norm is None else (x, norm(x))
