"""ctypes front end of the plain-C oracle (`dcn_oracle.c`).

TEST INFRASTRUCTURE ONLY (see the package docstring).  All functions take and
return CPU torch tensors; inputs are widened to float32 (after whatever storage
rounding the caller applied), results are float64.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np
import torch

from . import build as _build

SKIPPED = -(2 ** 31)  # corner marker of a point that failed the range test

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(_build.build())
        _lib.oracle_dcnv4_out_size.restype = C.c_int
        for name in ("oracle_dcnv4_forward", "oracle_dcnv4_backward",
                     "oracle_fda_forward", "oracle_fda_backward"):
            getattr(_lib, name).restype = C.c_int
    return _lib


def _f32(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().to(torch.float32).numpy())


def _i64(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().to(torch.int64).numpy())


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def dcnv4_out_hw(H, W, kh, kw, sh, sw, ph, pw, dh, dw) -> Tuple[int, int]:
    """Output size rule of the reference host wrapper (DCNv4_op/src/cuda/dcnv4_cuda.cu:48-52)."""
    return ((H + 2 * ph - (dh * (kh - 1) + 1)) // sh + 1,
            (W + 2 * pw - (dw * (kw - 1) + 1)) // sw + 1)


def dcnv4_forward(value, offset_mask, kh, kw, sh, sw, ph, pw, dh, dw, G, D,
                  offset_scale, remove_center, softmax=False, want_corners=False):
    """DCNv4 forward (DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:142-244) -> float64 (N,Ho,Wo,G*D)."""
    N, H, W, Cc = value.shape
    assert Cc == G * D
    Ho, Wo = dcnv4_out_hw(H, W, kh, kw, sh, sw, ph, pw, dh, dw)
    Ppad = offset_mask.shape[-1]
    K = kh * kw - int(bool(remove_center))
    v, om = _f32(value), _f32(offset_mask)
    out = np.empty((N, Ho, Wo, Cc), dtype=np.float64)
    corners = np.empty((N, Ho, Wo, G, K, 2), dtype=np.int32) if want_corners else None
    rc = lib().oracle_dcnv4_forward(
        _p(v), _p(om), _p(out), _p(corners), N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw,
        C.c_float(offset_scale), int(remove_center), Ppad, int(softmax))
    if rc != 0:
        raise ValueError("oracle_dcnv4_forward: bad arguments")
    out_t = torch.from_numpy(out)
    return (out_t, torch.from_numpy(corners)) if want_corners else out_t


def dcnv4_backward(value, offset_mask, grad_out, kh, kw, sh, sw, ph, pw, dh, dw, G, D,
                   offset_scale, remove_center, softmax=False):
    """DCNv4 backward (DCNv4_op/src/cuda/dcnv4_col2im_cuda.cuh:196-366) -> float64 grads."""
    N, H, W, Cc = value.shape
    Ppad = offset_mask.shape[-1]
    v, om, go = _f32(value), _f32(offset_mask), _f32(grad_out)
    gv = np.empty(v.shape, dtype=np.float64)
    gom = np.empty(om.shape, dtype=np.float64)
    rc = lib().oracle_dcnv4_backward(
        _p(v), _p(om), _p(go), _p(gv), _p(gom), N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw,
        C.c_float(offset_scale), int(remove_center), Ppad, int(softmax))
    if rc != 0:
        raise ValueError("oracle_dcnv4_backward: bad arguments")
    return torch.from_numpy(gv), torch.from_numpy(gom)


def fda_forward(value, spatial_shapes, level_start_index, sampling_loc_attn, K,
                want_corners=False):
    """FlashDeformAttn forward (DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:129-209)."""
    B, Len_in, G, D = value.shape
    Len_q = sampling_loc_attn.shape[1]
    L = spatial_shapes.shape[0]
    assert sampling_loc_attn.shape[-1] == 3 * L * K
    v, sla = _f32(value), _f32(sampling_loc_attn)
    ss, ls = _i64(spatial_shapes), _i64(level_start_index)
    out = np.empty((B, Len_q, G * D), dtype=np.float64)
    corners = np.empty((B, Len_q, G, L * K, 2), dtype=np.int32) if want_corners else None
    rc = lib().oracle_fda_forward(_p(v), _p(ss), _p(ls), _p(sla), _p(out), _p(corners),
                                  B, Len_in, G, D, L, Len_q, K)
    if rc != 0:
        raise ValueError("oracle_fda_forward: bad arguments")
    out_t = torch.from_numpy(out)
    return (out_t, torch.from_numpy(corners)) if want_corners else out_t


def fda_backward(value, spatial_shapes, level_start_index, sampling_loc_attn, grad_out, K):
    """FlashDeformAttn backward (DCNv4_op/src/cuda/flash_deform_col2im_cuda.cuh:171-318)."""
    B, Len_in, G, D = value.shape
    Len_q = sampling_loc_attn.shape[1]
    L = spatial_shapes.shape[0]
    v, sla, go = _f32(value), _f32(sampling_loc_attn), _f32(grad_out)
    ss, ls = _i64(spatial_shapes), _i64(level_start_index)
    gv = np.empty(v.shape, dtype=np.float64)
    gs = np.empty(sla.shape, dtype=np.float64)
    rc = lib().oracle_fda_backward(_p(v), _p(ss), _p(ls), _p(sla), _p(go), _p(gv), _p(gs),
                                   B, Len_in, G, D, L, Len_q, K)
    if rc != 0:
        raise ValueError("oracle_fda_backward: bad arguments")
    return torch.from_numpy(gv), torch.from_numpy(gs)
