"""`DCNv4Function`: autograd glue with the reference's argument list and gradient tuple
(DCNv4_op/DCNv4/functions/dcnv4_func.py:62-129).

Differences from the reference, all internal: there is no launch-spec lookup (`findspec`,
`find_spec_bwd`, `table.py`) -- the kernels derive their geometry from the shapes -- and
`im2col_step` is validated but does not chunk the batch.
"""
from __future__ import annotations

import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from .. import ops

try:  # torch >= 2.4
    from torch.amp import custom_bwd as _custom_bwd, custom_fwd as _custom_fwd

    def custom_fwd(fn):
        return _custom_fwd(fn, device_type="cuda")

    def custom_bwd(fn):
        return _custom_bwd(fn, device_type="cuda")
except ImportError:  # pragma: no cover
    from torch.cuda.amp import custom_bwd, custom_fwd


class DCNv4Function(Function):
    @staticmethod
    @custom_fwd
    def forward(ctx, input, offset_mask, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w,
                dilation_h, dilation_w, group, group_channels, offset_scale, im2col_step,
                remove_center):
        ctx.kernel_h, ctx.kernel_w = kernel_h, kernel_w
        ctx.stride_h, ctx.stride_w = stride_h, stride_w
        ctx.pad_h, ctx.pad_w = pad_h, pad_w
        ctx.dilation_h, ctx.dilation_w = dilation_h, dilation_w
        ctx.group, ctx.group_channels = group, group_channels
        ctx.offset_scale = offset_scale
        ctx.im2col_step = im2col_step
        ctx.remove_center = remove_center
        output = ops.dcnv4_forward(input, offset_mask, kernel_h, kernel_w, stride_h, stride_w,
                                   pad_h, pad_w, dilation_h, dilation_w, group, group_channels,
                                   offset_scale, im2col_step, remove_center, softmax=False)
        ctx.save_for_backward(input, offset_mask)
        return output

    @staticmethod
    @once_differentiable
    @custom_bwd
    def backward(ctx, grad_output):
        input, offset_mask = ctx.saved_tensors
        grad_input, grad_offset_mask = ops.dcnv4_backward(
            input, offset_mask, ctx.kernel_h, ctx.kernel_w, ctx.stride_h, ctx.stride_w,
            ctx.pad_h, ctx.pad_w, ctx.dilation_h, ctx.dilation_w, ctx.group, ctx.group_channels,
            ctx.offset_scale, ctx.im2col_step, grad_output.contiguous(), ctx.remove_center,
            softmax=False)
        return (grad_input, grad_offset_mask) + (None,) * 13
