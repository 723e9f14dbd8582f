"""grid_sample-based CPU formulation of the four ops (second opinion + timed CPU baseline).

TEST INFRASTRUCTURE ONLY (see the package docstring).

This is the algorithm of the reference's pure-PyTorch core
(classification/ops_dcnv3/functions/dcnv3_func.py:172-220: build sampling
locations, normalise them to [-1,1], `F.grid_sample(bilinear, zeros,
align_corners=False)`, weight by the mask and sum over the points), restated
for the packed DCNv4 `offset_mask` layout and written against un-padded pixel
coordinates.  `grid_sample` with `align_corners=False` maps a normalised
coordinate g to pixel (g+1)*size/2 - 0.5 and treats out-of-map corners as zero,
which is exactly the reference kernels' convention (pixel centres at integers,
corners outside the map contribute nothing, DCNv4_op/src/cuda/common.h:74-90).

FlashDeformAttn has no PyTorch formula inside the reference; the same
grid_sample construction per level plus a softmax over the L*K logits restates
DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:152-198.  Gradients come from
autograd in both cases.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def unpack_offset_mask(offset_mask: torch.Tensor, G: int, K: int):
    """Split the packed (N,Ho,Wo,Ppad) tensor into offsets (N,Ho,Wo,G,K,2) [x,y] and
    masks (N,Ho,Wo,G,K).  Per group the layout is 2K offsets then K masks
    (DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:163,169-171,219-225)."""
    N, Ho, Wo, _ = offset_mask.shape
    g = offset_mask[..., : G * K * 3].reshape(N, Ho, Wo, G, 3 * K)
    return g[..., : 2 * K].reshape(N, Ho, Wo, G, K, 2), g[..., 2 * K:]


def dcnv4_core(value, offset_mask, kh, kw, sh, sw, ph, pw, dh, dw, G, D,
               offset_scale, remove_center, softmax=False):
    """DCNv4 forward on any device/dtype through grid_sample.  value (N,H,W,G*D)."""
    N, H, W, C = value.shape
    Ho = (H + 2 * ph - (dh * (kh - 1) + 1)) // sh + 1
    Wo = (W + 2 * pw - (dw * (kw - 1) + 1)) // sw + 1
    dt, dev = value.dtype, value.device
    taps = [(i, j) for i in range(kw) for j in range(kh)
            if not (remove_center and i == kw // 2 and j == kh // 2)]
    K = len(taps)
    off, mask = unpack_offset_mask(offset_mask, G, K)
    if softmax:
        mask = mask.softmax(-1)
    cw, ch = (dw * (kw - 1)) // 2, (dh * (kh - 1)) // 2
    xs = torch.arange(Wo, dtype=dt, device=dev) * sw + (cw - pw) - cw * offset_scale
    ys = torch.arange(Ho, dtype=dt, device=dev) * sh + (ch - ph) - ch * offset_scale
    ti = torch.tensor([t[0] * dw for t in taps], dtype=dt, device=dev)
    tj = torch.tensor([t[1] * dh for t in taps], dtype=dt, device=dev)
    # pixel coordinates (N,Ho,Wo,G,K)
    px = xs.view(1, 1, Wo, 1, 1) + (ti.view(1, 1, 1, 1, K) + off[..., 0]) * offset_scale
    py = ys.view(1, Ho, 1, 1, 1) + (tj.view(1, 1, 1, 1, K) + off[..., 1]) * offset_scale
    gx = (2 * px + 1) / W - 1
    gy = (2 * py + 1) / H - 1
    grid = torch.stack((gx, gy), -1)                       # (N,Ho,Wo,G,K,2)
    grid = grid.permute(0, 3, 1, 2, 4, 5).reshape(N * G, Ho * Wo, K, 2)
    img = value.reshape(N, H * W, G, D).permute(0, 2, 3, 1).reshape(N * G, D, H, W)
    sampled = F.grid_sample(img, grid, mode="bilinear", padding_mode="zeros",
                            align_corners=False)          # (N*G, D, Q, K)
    m = mask.permute(0, 3, 1, 2, 4).reshape(N * G, 1, Ho * Wo, K)
    out = (sampled * m).sum(-1)                            # (N*G, D, Q)
    return out.reshape(N, G, D, Ho * Wo).permute(0, 3, 1, 2).reshape(N, Ho, Wo, C)


def fda_core(value, spatial_shapes, level_start_index, sampling_loc_attn, K):
    """FlashDeformAttn forward through grid_sample.  value (B,Len_in,G,D);
    sampling_loc_attn (B,Len_q,G,3*L*K) -> (B,Len_q,G*D)."""
    B, Len_in, G, D = value.shape
    Len_q = sampling_loc_attn.shape[1]
    L = int(spatial_shapes.shape[0])
    LK = L * K
    loc = sampling_loc_attn[..., : 2 * LK].reshape(B, Len_q, G, L, K, 2)
    prob = sampling_loc_attn[..., 2 * LK:].softmax(-1).reshape(B, Len_q, G, L, K)
    shapes = [(int(h), int(w)) for h, w in spatial_shapes.tolist()]
    starts = [int(s) for s in level_start_index.tolist()]
    out = None
    for l, (Hl, Wl) in enumerate(shapes):
        img = value[:, starts[l]: starts[l] + Hl * Wl].permute(0, 2, 3, 1).reshape(B * G, D, Hl, Wl)
        grid = (2 * loc[:, :, :, l] - 1).permute(0, 2, 1, 3, 4).reshape(B * G, Len_q, K, 2)
        sampled = F.grid_sample(img, grid, mode="bilinear", padding_mode="zeros",
                                align_corners=False)      # (B*G, D, Len_q, K)
        w = prob[:, :, :, l].permute(0, 2, 1, 3).reshape(B * G, 1, Len_q, K)
        part = (sampled * w).sum(-1)
        out = part if out is None else out + part
    return out.reshape(B, G, D, Len_q).permute(0, 3, 1, 2).reshape(B, Len_q, G * D)


def dcnv4_fwd_bwd(value, offset_mask, grad_out, *args, **kw):
    """Forward + autograd backward; returns (out, grad_value, grad_offset_mask)."""
    v = value.detach().clone().requires_grad_(True)
    om = offset_mask.detach().clone().requires_grad_(True)
    out = dcnv4_core(v, om, *args, **kw)
    gv, gom = torch.autograd.grad(out, (v, om), grad_out)
    return out.detach(), gv, gom


def fda_fwd_bwd(value, spatial_shapes, level_start_index, sampling_loc_attn, grad_out, K):
    """Forward + autograd backward; returns (out, grad_value, grad_sampling_loc_attn)."""
    v = value.detach().clone().requires_grad_(True)
    s = sampling_loc_attn.detach().clone().requires_grad_(True)
    out = fda_core(v, spatial_shapes, level_start_index, s, K)
    gv, gs = torch.autograd.grad(out, (v, s), grad_out)
    return out.detach(), gv, gs
