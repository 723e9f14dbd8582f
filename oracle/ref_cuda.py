"""Front end of the reference's own CUDA extension built by oracle/build_ref.py.

TEST / BENCHMARK INFRASTRUCTURE ONLY.  Used for (a) golden vectors of FlashDeformAttn, which the
reference cannot produce on CPU, (b) a second parity target for DCNv4, (c) timing "the kernel to
beat" beside ours.  The launch specs (d_stride, block_thread) the reference's Python layer would
pick are restated here: its tuned table covers the 56x56 and 28x28 benchmark shapes
(DCNv4_op/DCNv4/functions/table.py), everything else follows its divisor heuristic
(DCNv4_op/DCNv4/functions/dcnv4_func.py:28-60, flash_deform_attn_func.py:45-67).
"""
from __future__ import annotations

from . import build_ref

_ext = None

# "BxHxWxGxC" -> (d_stride, block_thread): the reference's tuned entries for the benchmark shapes
_FWD_TABLE = {(64, 56, 56, 4, 16): (8, 448), (64, 28, 28, 8, 16): (8, 448)}
_BWD_TABLE = {(64, 56, 56, 4, 16): (1, 256), (64, 28, 28, 8, 16): (1, 128)}


def ext():
    global _ext
    if _ext is None:
        _ext = build_ref.load()
    return _ext


def available() -> bool:
    import os
    return os.path.exists(build_ref.LIB)


def _largest_multiplier(total: int, per_query_threads: int, limit: int) -> int:
    best = 1
    for m in range(1, 65):
        if total % m == 0 and m * per_query_threads <= limit:
            best = m
    return best


def dcnv4_spec(B, H, W, G, D, backward=False):
    key = (B, H, W, G, D)
    table = _BWD_TABLE if backward else _FWD_TABLE
    if key in table:
        return table[key]
    if backward:
        d_stride = 2 if D >= 64 else 1
        m = _largest_multiplier(B * H * W, G * D // d_stride, 256)
    else:
        d_stride = 8
        m = _largest_multiplier(B * H * W, G * D // d_stride, 512)
    return d_stride, m * G * D // d_stride


def fda_spec(B, Q, G, D, backward=False):
    if backward:
        d_stride = 2 if D >= 64 else 1
        m = _largest_multiplier(B * Q, G * D // d_stride, 256)
    else:
        d_stride = 8
        m = _largest_multiplier(B * Q, G * D // d_stride, 512)
    return d_stride, m * G * D // d_stride


def dcnv4_forward(value, offset_mask, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, remove_center, im2col_step=256):
    ds, bt = dcnv4_spec(value.shape[0], value.shape[1], value.shape[2], G, D)
    return ext().dcnv4_forward(value, offset_mask, kh, kw, sh, sw, ph, pw, dh, dw, G, D, float(scale),
                               im2col_step, int(remove_center), ds, bt, False)


def dcnv4_backward(value, offset_mask, grad_out, kh, kw, sh, sw, ph, pw, dh, dw, G, D, scale, remove_center,
                   im2col_step=256):
    ds, bt = dcnv4_spec(value.shape[0], value.shape[1], value.shape[2], G, D, backward=True)
    return ext().dcnv4_backward(value, offset_mask, kh, kw, sh, sw, ph, pw, dh, dw, G, D, float(scale),
                                im2col_step, grad_out, int(remove_center), ds, bt, False)


def fda_forward(value, shapes, starts, sla, K, im2col_step=64):
    ds, bt = fda_spec(value.shape[0], sla.shape[1], value.shape[2], value.shape[3])
    return ext().flash_deform_attn_forward(value, shapes, starts, sla, im2col_step, K, ds, bt)


def fda_backward(value, shapes, starts, sla, grad_out, K, im2col_step=64):
    ds, bt = fda_spec(value.shape[0], sla.shape[1], value.shape[2], value.shape[3], backward=True)
    return ext().flash_deform_attn_backward(value, shapes, starts, sla, grad_out, im2col_step, K, ds, bt)
