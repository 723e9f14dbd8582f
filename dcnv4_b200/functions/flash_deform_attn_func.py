"""`FlashDeformAttnFunction`: autograd glue with the reference's argument list
(DCNv4_op/DCNv4/functions/flash_deform_attn_func.py:69-114).

The reference refuses to import on compute capability 10.0 (its shared-memory table stops
at 9.0, flash_deform_attn_func.py:21-36); this module has no such gate.
"""
from __future__ import annotations

import warnings

import torch
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from .. import ops


def _autocast_fp16(fn):
    # Building the decorator on a host without CUDA (CPU-side tests import this module) makes PyTorch
    # warn that it disables autocast; there is nothing to run on such a host anyway.
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return torch.autocast("cuda", enabled=True, dtype=torch.float16)(fn)


class FlashDeformAttnFunction(Function):
    # The reference decorates forward with autocast(fp16) (flash_deform_attn_func.py:71).  Autocast
    # only re-types the inputs of PyTorch operators that have an autocast rule; neither the
    # reference's extension call nor this library's has one, so the operator runs in the dtype of
    # the tensors it is given, with or without the decorator.  It is kept so that any PyTorch
    # operator a subclass adds to forward sees the same autocast state as in the reference.
    @staticmethod
    @_autocast_fp16
    def forward(ctx, value, value_spatial_shapes, value_level_start_index, sampling_loc_attn,
                im2col_step, K=8):
        ctx.im2col_step = im2col_step
        ctx.K = K
        output = ops.flash_deform_attn_forward(value, value_spatial_shapes, value_level_start_index,
                                               sampling_loc_attn, im2col_step, K)
        ctx.save_for_backward(value, value_spatial_shapes, value_level_start_index, sampling_loc_attn)
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        value, shapes, starts, sampling_loc_attn = ctx.saved_tensors
        grad_value, grad_sla = ops.flash_deform_attn_backward(
            value, shapes, starts, sampling_loc_attn, grad_output.contiguous(), ctx.im2col_step, ctx.K)
        return grad_value, None, None, grad_sla, None, None
