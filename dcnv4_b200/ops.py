"""Tensor-level entry points over the C ABI (the role of the reference's `DCNv4.ext` module,
DCNv4_op/src/vision.cpp:14-21): validate torch tensors the way the reference host wrappers
do (DCNv4_op/src/cuda/dcnv4_cuda.cu:26-60, DCNv4_op/src/cuda/flash_deform_attn_cuda.cu:26-58),
allocate outputs with torch (device memory and streams are torch's job here, nothing else),
and call the library on the current CUDA stream.
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError(f"dcnv4_b200 supports float32/float16/bfloat16 tensors, got {t.dtype}") from None


def _check_tensor(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} tensor has to be contiguous")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _check_step(batch: int, im2col_step: int) -> None:
    step = min(batch, int(im2col_step))
    if step <= 0 or batch % step != 0:
        raise RuntimeError(f"batch({batch}) must divide im2col_step({step})")


def dcnv4_forward(value, p_offset, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w,
                  dilation_h, dilation_w, group, group_channels, offset_scale, im2col_step,
                  remove_center, d_stride=None, block_thread=None, softmax=False) -> torch.Tensor:
    """Positional signature of the reference's `ext.dcnv4_forward` (DCNv4_op/src/dcnv4.h:64-83).
    `im2col_step` is validated like the reference does and otherwise unused (the whole batch
    is one launch); `d_stride` / `block_thread` are accepted and ignored."""
    _check_tensor(value, "input")
    _check_tensor(p_offset, "offset")
    if value.dim() != 4 or p_offset.dim() != 4:
        raise RuntimeError("input and offset_mask must be (N,H,W,C) and (N,Ho,Wo,P) tensors")
    if p_offset.dtype != value.dtype:
        raise RuntimeError("input and offset_mask must have the same dtype")
    N, H, W, C = value.shape
    if C != group * group_channels:
        raise RuntimeError(
            f"Input channels and group times group channels wont match: ({C} vs {group * group_channels}).")
    _check_step(N, im2col_step)
    L = _lib.lib()
    Ho = L.dcnv4b200_out_size(H, pad_h, dilation_h, kernel_h, stride_h)
    Wo = L.dcnv4b200_out_size(W, pad_w, dilation_w, kernel_w, stride_w)
    if tuple(p_offset.shape[:3]) != (N, Ho, Wo):
        raise RuntimeError(f"offset_mask must be (N,{Ho},{Wo},P), got {tuple(p_offset.shape)}")
    out = torch.empty((N, Ho, Wo, C), dtype=value.dtype, device=value.device)
    with torch.cuda.device(value.device):
        rc = L.dcnv4b200_fwd(value.data_ptr(), p_offset.data_ptr(), out.data_ptr(), _code(value),
                             N, H, W, group, group_channels, kernel_h, kernel_w, stride_h, stride_w,
                             pad_h, pad_w, dilation_h, dilation_w, float(offset_scale),
                             int(remove_center), p_offset.shape[3], int(bool(softmax)), _stream(value))
    _lib.check(rc, "dcnv4_forward")
    return out


def dcnv4_backward(value, p_offset, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w,
                   dilation_h, dilation_w, group, group_channels, offset_scale, im2col_step,
                   grad_output, remove_center, d_stride=None, block_thread=None,
                   softmax=False) -> List[torch.Tensor]:
    """Positional signature of `ext.dcnv4_backward` (DCNv4_op/src/dcnv4.h:85-107).  Returns
    [grad_input, grad_offset_mask] in the dtype of `value` (bf16 included; the reference
    raises a type error for bf16, DCNv4_op/src/cuda/dcnv4_cuda.cu:133-139,161)."""
    _check_tensor(value, "input")
    _check_tensor(p_offset, "offset")
    _check_tensor(grad_output, "grad_output")
    if p_offset.dtype != value.dtype or grad_output.dtype != value.dtype:
        raise RuntimeError("input, offset_mask and grad_output must have the same dtype")
    N, H, W, C = value.shape
    if C != group * group_channels:
        raise RuntimeError(
            f"Input channels and group times group channels wont match: ({C} vs {group * group_channels}).")
    _check_step(N, im2col_step)
    L = _lib.lib()
    Ho = L.dcnv4b200_out_size(H, pad_h, dilation_h, kernel_h, stride_h)
    Wo = L.dcnv4b200_out_size(W, pad_w, dilation_w, kernel_w, stride_w)
    if grad_output.numel() != N * Ho * Wo * C or tuple(p_offset.shape[:3]) != (N, Ho, Wo):
        raise RuntimeError("grad_output / offset_mask shape does not match the output size")
    code = _code(value)
    grad_input = torch.empty_like(value)
    grad_offset = torch.empty_like(p_offset)
    ws_bytes = L.dcnv4b200_bwd_workspace_bytes(code, N, H, W, group, group_channels)
    ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device=value.device) if ws_bytes else None
    with torch.cuda.device(value.device):
        rc = L.dcnv4b200_bwd(value.data_ptr(), p_offset.data_ptr(), grad_output.data_ptr(),
                             grad_input.data_ptr(), grad_offset.data_ptr(),
                             ws.data_ptr() if ws is not None else None, ws_bytes, code,
                             N, H, W, group, group_channels, kernel_h, kernel_w, stride_h, stride_w,
                             pad_h, pad_w, dilation_h, dilation_w, float(offset_scale),
                             int(remove_center), p_offset.shape[3], int(bool(softmax)), _stream(value))
    _lib.check(rc, "dcnv4_backward")
    return [grad_input, grad_offset]


def _check_fda(value, spatial_shapes, level_start_index, sampling_loc_attn, K) -> Tuple[int, ...]:
    _check_tensor(value, "value")
    _check_tensor(spatial_shapes, "spatial_shapes")
    _check_tensor(level_start_index, "level_start_index")
    _check_tensor(sampling_loc_attn, "sampling_loc_attn")
    if spatial_shapes.dtype != torch.int64 or level_start_index.dtype != torch.int64:
        raise RuntimeError("spatial_shapes and level_start_index must be int64 tensors")
    if value.dim() != 4 or sampling_loc_attn.dim() != 4:
        raise RuntimeError("value must be (B,Len_in,G,D) and sampling_loc_attn (B,Len_q,G,3*L*K)")
    if sampling_loc_attn.dtype != value.dtype:
        raise RuntimeError("value and sampling_loc_attn must have the same dtype")
    B, Len_in, G, D = value.shape
    L = spatial_shapes.shape[0]
    Len_q = sampling_loc_attn.shape[1]
    if tuple(sampling_loc_attn.shape) != (B, Len_q, G, 3 * L * K):
        raise RuntimeError(
            f"sampling_loc_attn must be ({B},Len_q,{G},{3 * L * K}), got {tuple(sampling_loc_attn.shape)}")
    return B, Len_in, G, D, L, Len_q


def flash_deform_attn_forward(value, spatial_shapes, level_start_index, sampling_loc_attn,
                              im2col_step=64, K=8, d_stride=None, block_thread=None) -> torch.Tensor:
    """Positional signature of `ext.flash_deform_attn_forward` (DCNv4_op/src/dcnv4.h:19-38).
    Returns (B, Len_q, G*D)."""
    B, Len_in, G, D, L, Len_q = _check_fda(value, spatial_shapes, level_start_index, sampling_loc_attn, K)
    _check_step(B, im2col_step)
    out = torch.empty((B, Len_q, G * D), dtype=value.dtype, device=value.device)
    with torch.cuda.device(value.device):
        rc = _lib.lib().fdab200_fwd(value.data_ptr(), spatial_shapes.data_ptr(), level_start_index.data_ptr(),
                                    sampling_loc_attn.data_ptr(), out.data_ptr(), _code(value),
                                    B, Len_in, G, D, L, Len_q, K, _stream(value))
    _lib.check(rc, "flash_deform_attn_forward")
    return out


def flash_deform_attn_backward(value, spatial_shapes, level_start_index, sampling_loc_attn, grad_output,
                               im2col_step=64, K=8, d_stride=None, block_thread=None) -> List[torch.Tensor]:
    """Positional signature of `ext.flash_deform_attn_backward` (DCNv4_op/src/dcnv4.h:40-62).
    Returns [grad_value, grad_sampling_loc_attn] in the dtype of `value`."""
    B, Len_in, G, D, L, Len_q = _check_fda(value, spatial_shapes, level_start_index, sampling_loc_attn, K)
    _check_tensor(grad_output, "grad_output")
    if grad_output.dtype != value.dtype or grad_output.numel() != B * Len_q * G * D:
        raise RuntimeError("grad_output must be (B,Len_q,G*D) in the dtype of value")
    _check_step(B, im2col_step)
    lib = _lib.lib()
    code = _code(value)
    grad_value = torch.empty_like(value)
    grad_sla = torch.empty_like(sampling_loc_attn)
    ws_bytes = lib.fdab200_bwd_workspace_bytes(code, B, Len_in, G, D)
    ws = torch.empty(ws_bytes // 4, dtype=torch.float32, device=value.device) if ws_bytes else None
    with torch.cuda.device(value.device):
        rc = lib.fdab200_bwd(value.data_ptr(), spatial_shapes.data_ptr(), level_start_index.data_ptr(),
                             sampling_loc_attn.data_ptr(), grad_output.data_ptr(), grad_value.data_ptr(),
                             grad_sla.data_ptr(), ws.data_ptr() if ws is not None else None, ws_bytes,
                             code, B, Len_in, G, D, L, Len_q, K, _stream(value))
    _lib.check(rc, "flash_deform_attn_backward")
    return [grad_value, grad_sla]


def layer_norm_forward(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float,
                       activation: str = "none") -> torch.Tensor:
    """LayerNorm over the last dimension of a contiguous CUDA tensor with the library's
    channels-last kernel (forward only; no autograd), optionally followed by GELU (erf form) in
    the same pass.  Raises ValueError for sizes the kernel does not cover -- callers that want a
    fallback check `layer_norm_supported` first."""
    if activation not in ("none", "gelu"):
        raise ValueError("activation must be 'none' or 'gelu'")
    _check_tensor(x, "input")
    _check_tensor(weight, "weight")
    _check_tensor(bias, "bias")
    C = x.shape[-1]
    if weight.numel() != C or bias.numel() != C or weight.dtype != bias.dtype:
        raise RuntimeError("weight and bias must have the size of the last dimension and one dtype")
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        rc = _lib.lib().dcnv4b200_layernorm_act_fwd(x.data_ptr(), weight.data_ptr(), bias.data_ptr(), y.data_ptr(),
                                                    _code(x), _code(weight), x.numel() // max(C, 1), C, float(eps),
                                                    1 if activation == "gelu" else 0, _stream(x))
    _lib.check(rc, "layer_norm_forward")
    return y


def center_scale_blend_supported(x: torch.Tensor, weight: torch.Tensor, D: int) -> bool:
    """True when `center_scale_blend_forward` covers this input (dtype, size, layout)."""
    if not (x.is_cuda and x.is_contiguous() and x.dtype in _DTYPES and x.numel() > 0):
        return False
    C, es = x.shape[-1], x.element_size()
    G = weight.shape[0]
    return (C == G * D and (D * es) % 16 == 0 and C <= (1024 if es == 4 else 2048) and G <= 128
            and weight.is_cuda and weight.is_contiguous() and weight.dtype in (torch.float32, x.dtype)
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def center_scale_blend_forward(x: torch.Tensor, x_proj: torch.Tensor, weight: torch.Tensor,
                               bias: torch.Tensor) -> torch.Tensor:
    """`x * (1 - s) + x_proj * s` with `s = sigmoid(x @ weight.T + bias)` repeated over each group's
    channels: the centre-feature-scale blend of the DCNv4 module in one pass (forward only; no autograd).
    x, x_proj (..., G*D) contiguous; weight (G, G*D); bias (G)."""
    for t, n in ((x, "x"), (x_proj, "x_proj"), (weight, "weight"), (bias, "bias")):
        _check_tensor(t, n)
    G, C = weight.shape
    if x.shape != x_proj.shape or x.shape[-1] != C or x.dtype != x_proj.dtype or C % G != 0 \
            or bias.numel() != G or bias.dtype != weight.dtype:
        raise RuntimeError("x and x_proj must be (..., G*D) in one dtype, weight (G, G*D), bias (G)")
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        rc = _lib.lib().dcnv4b200_center_scale_blend_fwd(x.data_ptr(), x_proj.data_ptr(), weight.data_ptr(),
                                                         bias.data_ptr(), out.data_ptr(), _code(x), _code(weight),
                                                         x.numel() // C, G, C // G, _stream(x))
    _lib.check(rc, "center_scale_blend_forward")
    return out


def layer_norm_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """True when `layer_norm_forward` covers this input (dtype, size, layout)."""
    if not (x.is_cuda and x.is_contiguous() and x.dtype in _DTYPES and x.numel() > 0):
        return False
    C, es = x.shape[-1], x.element_size()
    if (C * es) % 16 != 0 or C > (1024 if es == 4 else 2048):
        return False
    return weight is not None and weight.is_cuda and weight.dtype in (torch.float32, x.dtype) \
        and x.data_ptr() % 16 == 0


def linear_forward(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   residual: Optional[torch.Tensor] = None, activation: str = "none") -> torch.Tensor:
    """y = act(x @ weight.T + bias) [+ residual] in one tensor-core kernel (forward only; no
    autograd; fp16 / bf16).  `activation` is "none" or "gelu" (erf form, as nn.GELU()).  Raises
    ValueError / RuntimeError for inputs the kernel does not cover -- callers that want a
    fallback check `linear_supported` first."""
    _check_tensor(x, "input")
    _check_tensor(weight, "weight")
    if activation not in ("none", "gelu"):
        raise ValueError("activation must be 'none' or 'gelu'")
    N, K = weight.shape
    if x.shape[-1] != K or weight.dtype != x.dtype:
        raise RuntimeError("weight must be (out_features, in_features) in the dtype of the input")
    for t, name in ((bias, "bias"), (residual, "residual")):
        if t is not None:
            _check_tensor(t, name)
            if t.dtype != x.dtype:
                raise RuntimeError(f"{name} must have the dtype of the input")
    M = x.numel() // max(K, 1)
    if bias is not None and bias.numel() != N:
        raise RuntimeError("bias must have out_features elements")
    if residual is not None and residual.numel() != M * N:
        raise RuntimeError("residual must have the shape of the output")
    y = torch.empty(x.shape[:-1] + (N,), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().dcnv4b200_linear_fwd(x.data_ptr(), weight.data_ptr(),
                                             bias.data_ptr() if bias is not None else None,
                                             residual.data_ptr() if residual is not None else None,
                                             y.data_ptr(), _code(x), M, N, K, 1 if activation == "gelu" else 0,
                                             _stream(x))
    _lib.check(rc, "linear_forward")
    return y


def linear_layer_norm_forward(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                              residual: Optional[torch.Tensor], ln_weight: torch.Tensor, ln_bias: torch.Tensor,
                              eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(y, LayerNorm(y)) with y = x @ weight.T + bias [+ residual], one tensor-core kernel
    (forward only; fp16 / bf16; out_features at most 256 and a multiple of 32, of 64 above 128)."""
    _check_tensor(x, "input")
    _check_tensor(weight, "weight")
    N, K = weight.shape
    if x.shape[-1] != K or weight.dtype != x.dtype:
        raise RuntimeError("weight must be (out_features, in_features) in the dtype of the input")
    for t, name in ((bias, "bias"), (residual, "residual"), (ln_weight, "ln_weight"), (ln_bias, "ln_bias")):
        if t is not None:
            _check_tensor(t, name)
            if t.dtype != x.dtype:
                raise RuntimeError(f"{name} must have the dtype of the input")
    M = x.numel() // max(K, 1)
    if (bias is not None and bias.numel() != N) or ln_weight.numel() != N or ln_bias.numel() != N:
        raise RuntimeError("bias and LayerNorm parameters must have out_features elements")
    if residual is not None and residual.numel() != M * N:
        raise RuntimeError("residual must have the shape of the output")
    y = torch.empty(x.shape[:-1] + (N,), dtype=x.dtype, device=x.device)
    z = torch.empty_like(y)
    with torch.cuda.device(x.device):
        rc = _lib.lib().dcnv4b200_linear_ln_fwd(x.data_ptr(), weight.data_ptr(),
                                                bias.data_ptr() if bias is not None else None,
                                                residual.data_ptr() if residual is not None else None,
                                                y.data_ptr(), ln_weight.data_ptr(), ln_bias.data_ptr(), float(eps),
                                                z.data_ptr(), _code(x), M, N, K, _stream(x))
    _lib.check(rc, "linear_layer_norm_forward")
    return y, z


def linear_pair_forward(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                        n1: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Two Linear layers over the same input in one tensor-core product: `weight` is the two
    weights stacked along the output dimension, `n1` (a multiple of 64) the first layer's
    out_features.  Returns (x @ W1.T + b1, x @ W2.T + b2) as two contiguous tensors (forward
    only; fp16 / bf16)."""
    _check_tensor(x, "input")
    _check_tensor(weight, "weight")
    N, K = weight.shape
    if x.shape[-1] != K or weight.dtype != x.dtype or not 0 < n1 < N:
        raise RuntimeError("weight must be (n1 + n2, in_features) in the dtype of the input")
    if bias is not None:
        _check_tensor(bias, "bias")
        if bias.dtype != x.dtype or bias.numel() != N:
            raise RuntimeError("bias must have n1 + n2 elements in the dtype of the input")
    M = x.numel() // max(K, 1)
    y1 = torch.empty(x.shape[:-1] + (n1,), dtype=x.dtype, device=x.device)
    y2 = torch.empty(x.shape[:-1] + (N - n1,), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().dcnv4b200_linear_pair_fwd(x.data_ptr(), weight.data_ptr(),
                                                  bias.data_ptr() if bias is not None else None,
                                                  y1.data_ptr(), n1, y2.data_ptr(), N - n1, _code(x), M, K,
                                                  _stream(x))
    _lib.check(rc, "linear_pair_forward")
    return y1, y2


def fused_offset_supported(value: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                           bias: Optional[torch.Tensor], group: int, group_channels: int) -> bool:
    """True when `dcnv4_fused_offset_forward` covers these tensors (the kernel is specialised for
    3x3 / stride 1 / pad 1 / dilation 1, which the caller checks)."""
    if not (value.is_cuda and value.dtype in (torch.float16, torch.bfloat16) and value.is_contiguous()
            and value.dim() == 4 and value.numel() > 0 and value.data_ptr() % 32 == 0):
        return False
    if not (x.is_cuda and x.dtype == value.dtype and x.is_contiguous() and x.data_ptr() % 16 == 0):
        return False
    if not (weight.is_cuda and weight.dtype == value.dtype and weight.is_contiguous() and weight.dim() == 2
            and weight.data_ptr() % 16 == 0):
        return False
    if bias is not None and not (bias.is_cuda and bias.dtype == value.dtype and bias.is_contiguous()
                                 and bias.numel() == weight.shape[0]):
        return False
    N, H, W, C = value.shape
    rows, K = weight.shape
    return (group_channels == 16 and C == 16 * group and 0 < group <= 128
            and K % 8 == 0 and x.shape[-1] == K and x.numel() == N * H * W * K and rows >= 27 * group
            and value.numel() < 2 ** 31)


def dcnv4_fused_offset_forward(value: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                               bias: Optional[torch.Tensor], group: int, group_channels: int,
                               offset_scale: float) -> torch.Tensor:
    """`dcnv4_forward(value, linear(x, weight, bias), 3, 3, 1, 1, 1, 1, 1, 1, group, group_channels,
    offset_scale, ...)` in one kernel: the offset/mask rows are computed by the CTA that samples
    for them and are never stored (forward only; fp16 / bf16).  value (N,H,W,C), x (N,H*W,K) or
    (N,H,W,K), weight (P,K) with P >= 27*group, bias (P) or None."""
    for t, name in ((value, "input"), (x, "offset_mask input"), (weight, "weight")):
        _check_tensor(t, name)
    if value.dim() != 4:
        raise RuntimeError("input must be an (N,H,W,C) tensor")
    N, H, W, C = value.shape
    if C != group * group_channels:
        raise RuntimeError(
            f"Input channels and group times group channels wont match: ({C} vs {group * group_channels}).")
    rows, K = weight.shape
    if x.dtype != value.dtype or weight.dtype != value.dtype or x.shape[-1] != K or x.numel() != N * H * W * K:
        raise RuntimeError("offset_mask input must be (N,H*W,K) and weight (P,K), in the dtype of the input")
    if bias is not None:
        _check_tensor(bias, "bias")
        if bias.dtype != value.dtype or bias.numel() != rows:
            raise RuntimeError("bias must have one element per weight row, in the dtype of the input")
    out = torch.empty_like(value)
    with torch.cuda.device(value.device):
        rc = _lib.lib().dcnv4b200_fwd_fused_offset(value.data_ptr(), x.data_ptr(), weight.data_ptr(),
                                                   bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                                   _code(value), N, H, W, group, group_channels, K, rows,
                                                   float(offset_scale), _stream(value))
    _lib.check(rc, "dcnv4_fused_offset_forward")
    return out


class PairedLinear:
    """Inference-time cache of two nn.Linear layers that read the same input, stacked for
    `linear_pair_forward`.  The stacked copy is rebuilt whenever a parameter changed (version
    counters), moved or changed dtype.  Writes through `.data` (`param.data.copy_()` in an EMA
    update, `constant_(w.data)`) do not bump a version counter: the owning module therefore
    calls `invalidate()` from `train()`, `_load_from_state_dict()` and `_reset_parameters()`, and
    code that writes `.data` by other routes must call it too."""

    def __init__(self, first: "torch.nn.Linear", second: "torch.nn.Linear"):
        self.first, self.second = first, second
        self._key, self._weight, self._bias = None, None, None

    def invalidate(self) -> None:
        self._key, self._weight, self._bias = None, None, None

    def usable(self, x: torch.Tensor) -> bool:
        a, b = self.first, self.second
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or a.weight.requires_grad or b.weight.requires_grad)
        return (FUSED_LINEAR and not needs_grad and not torch.is_autocast_enabled() and linear_supported(x, a.weight)
                and b.weight.dtype == x.dtype and b.weight.is_cuda and a.in_features == b.in_features
                and a.in_features <= FUSED_LINEAR_MAX_K and a.out_features % 64 == 0 and b.out_features % 8 == 0
                and (a.bias is None) == (b.bias is None) and (a.bias is None or a.bias.dtype == x.dtype))

    def __call__(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        a, b = self.first, self.second
        params = [t for t in (a.weight, b.weight, a.bias, b.bias) if t is not None]
        key = tuple((t.data_ptr(), t._version, t.dtype, t.device) for t in params)
        if key != self._key:
            with torch.no_grad():
                self._weight = torch.cat([a.weight, b.weight], 0).contiguous()
                self._bias = None if a.bias is None else torch.cat([a.bias, b.bias], 0).contiguous()
            self._key = key
        return linear_pair_forward(x, self._weight, self._bias, a.out_features)


def linear_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """True when `linear_forward` covers this input (dtype, size, layout)."""
    if not (x.is_cuda and x.is_contiguous() and x.dtype in (torch.float16, torch.bfloat16) and x.numel() > 0):
        return False
    if weight is None or not weight.is_cuda or weight.dtype != x.dtype or not weight.is_contiguous():
        return False
    N, K = weight.shape
    return N % 8 == 0 and K % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0


FUSED_LINEAR = True  # benchmarks turn this off to time the stock nn.Linear / GELU / add kernels
# The fused kernel streams both operands through one SM's shared memory (no 2-CTA tiles), which
# bounds long reductions by L2 bandwidth: measured against cuBLAS + separate element-wise kernels
# it wins up to K = 1024 and loses at K = 2048 (FlashInternImage-T stage-4 fc2: 45 vs 36 us).
FUSED_LINEAR_MAX_K = 1024
# DCNv4 module at inference: compute the offset/mask rows inside the sampling kernel
# (`dcnv4_fused_offset_forward`) instead of storing them from the paired projection.  Measured on a
# B200, fp16, value projection + fused kernel against paired projection + sampling kernel, us:
#   batch 256: 56x56x64 330 / 338, 28x28x128 175 / 193, 14x14x256 100 / 114, 7x7x512 68 / 67;
#   batch 32:  60 / 56, 40 / 42, 33 / 37, 30 / 37.
# It pays from 128 channels upward at any batch and at 64 channels only for large batches, hence the
# two thresholds.  Environment variable DCNV4B200_FUSED_OFFSET=0 turns it off, =1 forces it wherever
# the kernel applies (tests).
_FUSED_OFFSET_ENV = os.environ.get("DCNV4B200_FUSED_OFFSET", "")
FUSED_OFFSET_MASK = _FUSED_OFFSET_ENV != "0"
FUSED_OFFSET_MIN_CHANNELS = 128
FUSED_OFFSET_MIN_ROWS_NARROW = 4096  # rows per SM below which 64-channel layers keep the two-step path


def fused_offset_pays(rows: int, channels: int, device) -> bool:
    """Whether the module should take the fused kernel for a layer of this size (see above)."""
    if not FUSED_OFFSET_MASK:
        return False
    if _FUSED_OFFSET_ENV == "1" or channels >= FUSED_OFFSET_MIN_CHANNELS:
        return True
    return rows >= FUSED_OFFSET_MIN_ROWS_NARROW * _sm_count(device)


# The LayerNorm epilogue needs a whole row in one tile, i.e. one CTA per 128 rows: below this many
# rows per SM the separate kernels (narrower tiles, more CTAs) are faster.
LN_FUSION_MIN_ROWS_PER_SM = 64


def linear_module_forward(x: torch.Tensor, lin: "torch.nn.Linear", residual: Optional[torch.Tensor] = None,
                          activation: str = "none", norm: Optional["torch.nn.LayerNorm"] = None):
    """`y = residual + act(lin(x))` for an nn.Linear, and with `norm` (an nn.LayerNorm over the
    output features) the pair `(y, norm(y))`.  One fused tensor-core kernel when autograd is not
    needed and the kernel covers the input, else the stock PyTorch operations (same result up
    to fp rounding: the fused kernel rounds at the same points)."""
    needs_grad = torch.is_grad_enabled() and (x.requires_grad or lin.weight.requires_grad)
    fused = (FUSED_LINEAR and not needs_grad and not torch.is_autocast_enabled() and linear_supported(x, lin.weight)
             and lin.in_features <= FUSED_LINEAR_MAX_K
             and (lin.bias is None or (lin.bias.dtype == x.dtype and lin.bias.data_ptr() % 16 == 0))
             and (residual is None or (residual.dtype == x.dtype and residual.is_contiguous()
                                       and residual.data_ptr() % 16 == 0)))
    # The LayerNorm epilogue needs a whole row in one tile, i.e. one tile per 128 rows: with row
    # tiles for fewer than half of the SMs the separate kernels (narrower tiles, more CTAs) are
    # faster (measured on FlashInternImage-T stage 3: 98 tiles fused wins, 49 tiles it loses).
    if (fused and norm is not None and activation == "none" and _norm_fusable(norm, lin.out_features, x.dtype)
            and x.numel() // lin.in_features >= LN_FUSION_MIN_ROWS_PER_SM * _sm_count(x.device)):
        return linear_layer_norm_forward(x, lin.weight, lin.bias, residual, norm.weight, norm.bias, norm.eps)
    if fused:
        y = linear_forward(x, lin.weight, lin.bias, residual, activation)
    else:
        y = torch.nn.functional.linear(x, lin.weight, lin.bias)
        if activation == "gelu":
            y = torch.nn.functional.gelu(y)
        if residual is not None:
            y = residual + y
    return y if norm is None else (y, norm(y))


_SM_COUNT = {}


def _sm_count(device) -> int:
    idx = torch.device(device).index
    idx = torch.cuda.current_device() if idx is None else idx
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def _norm_fusable(norm, features: int, dtype: torch.dtype) -> bool:
    return (isinstance(norm, torch.nn.LayerNorm) and norm.elementwise_affine and norm.bias is not None
            and tuple(norm.normalized_shape) == (features,) and features <= 256
            and features % (64 if features > 128 else 32) == 0
            and norm.weight.dtype == dtype and norm.bias.dtype == dtype
            and norm.weight.data_ptr() % 16 == 0 and norm.bias.data_ptr() % 16 == 0)


def bias_act_(x: torch.Tensor, bias: torch.Tensor, activation: str = "none") -> torch.Tensor:
    """In place: x = act(x + bias) over the last dimension of a contiguous fp16 / bf16 CUDA
    tensor (forward only).  `activation` is "none" or "gelu" (erf form)."""
    _check_tensor(x, "input")
    _check_tensor(bias, "bias")
    if activation not in ("none", "gelu"):
        raise ValueError("activation must be 'none' or 'gelu'")
    C = x.shape[-1]
    if bias.numel() != C or bias.dtype != x.dtype:
        raise RuntimeError("bias must have the size of the last dimension and the dtype of the input")
    with torch.cuda.device(x.device):
        rc = _lib.lib().dcnv4b200_bias_act_fwd(x.data_ptr(), bias.data_ptr(), x.data_ptr(), _code(x),
                                               x.numel() // max(C, 1), C, 1 if activation == "gelu" else 0,
                                               _stream(x))
    _lib.check(rc, "bias_act_")
    return x


def conv2d_bias_act(x: torch.Tensor, conv: "torch.nn.Conv2d", activation: str = "none") -> torch.Tensor:
    """act(conv(x)) for a biased nn.Conv2d on a channels-last image batch: at inference in fp16 /
    bf16 the bias and the activation are applied in place by one pass over the convolution's
    output instead of PyTorch's separate broadcast addition and activation kernels."""
    F = torch.nn.functional
    needs_grad = torch.is_grad_enabled() and (x.requires_grad or conv.weight.requires_grad)
    if (FUSED_LINEAR and not needs_grad and not torch.is_autocast_enabled() and x.is_cuda and conv.bias is not None
            and x.dtype in (torch.float16, torch.bfloat16) and conv.weight.dtype == x.dtype
            and conv.bias.dtype == x.dtype and conv.out_channels % 8 == 0 and conv.padding_mode == "zeros"
            and conv.bias.data_ptr() % 16 == 0):
        y = F.conv2d(x, conv.weight, None, conv.stride, conv.padding, conv.dilation, conv.groups)
        rows = y.permute(0, 2, 3, 1)            # channels-last storage seen as (N, H, W, C)
        if rows.is_contiguous() and y.data_ptr() % 16 == 0:
            bias_act_(rows, conv.bias, activation)
            return y
        y = y + conv.bias.view(1, -1, 1, 1)
    else:
        y = conv(x)
    return F.gelu(y) if activation == "gelu" else y


def dcnv4_corners(p_offset, H, W, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, dilation_h,
                  dilation_w, group, offset_scale, remove_center) -> torch.Tensor:
    """(N,Ho,Wo,G,K,2) int32 corner indices the kernels select (test aid)."""
    _check_tensor(p_offset, "offset")
    N, Ho, Wo, P = p_offset.shape
    K = kernel_h * kernel_w - int(bool(remove_center))
    corners = torch.empty((N, Ho, Wo, group, K, 2), dtype=torch.int32, device=p_offset.device)
    with torch.cuda.device(p_offset.device):
        rc = _lib.lib().dcnv4b200_fwd_corners(p_offset.data_ptr(), corners.data_ptr(), _code(p_offset),
                                              N, H, W, group, kernel_h, kernel_w, stride_h, stride_w,
                                              pad_h, pad_w, dilation_h, dilation_w, float(offset_scale),
                                              int(remove_center), P, _stream(p_offset))
    _lib.check(rc, "dcnv4_corners")
    return corners


def flash_deform_attn_corners(spatial_shapes, sampling_loc_attn, K) -> torch.Tensor:
    """(B,Len_q,G,L*K,2) int32 corner indices the kernels select (test aid)."""
    _check_tensor(sampling_loc_attn, "sampling_loc_attn")
    B, Len_q, G, _ = sampling_loc_attn.shape
    L = spatial_shapes.shape[0]
    corners = torch.empty((B, Len_q, G, L * K, 2), dtype=torch.int32, device=sampling_loc_attn.device)
    with torch.cuda.device(sampling_loc_attn.device):
        rc = _lib.lib().fdab200_fwd_corners(spatial_shapes.data_ptr(), sampling_loc_attn.data_ptr(),
                                            corners.data_ptr(), _code(sampling_loc_attn), B, G, L, Len_q, K,
                                            _stream(sampling_loc_attn))
    _lib.check(rc, "flash_deform_attn_corners")
    return corners


def device_status() -> int:
    """Read-and-clear the current device's kernel status word (synchronises; test aid)."""
    import ctypes as C
    v = C.c_int(0)
    _lib.check(_lib.lib().dcnv4b200_device_status(C.byref(v)), "device_status")
    return v.value
