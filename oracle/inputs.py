"""Seeded synthetic inputs with the benchmark configurations' shapes and distributions.

TEST INFRASTRUCTURE ONLY (see the package docstring).  The real datasets the
reference evaluates on are not available offline; these tensors reproduce the
shapes of FlashInternImage's stages and of a Deformable-DETR encoder and the
value distributions the benchmark configurations state (inputs ~N(0,1), offsets
~N(0,1) pixels, masks ~U(0,1), locations ~U(0,1), logits ~N(0,1)).
"""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch

# FlashInternImage-T stage shapes at 224x224 (H=W, C, G), group_channels 16.
STAGES_T = ((56, 64, 4), (28, 128, 8), (14, 256, 16), (7, 512, 32))
# Deformable-DETR encoder levels whose sizes sum to 20,197 positions.
DETR_LEVELS = ((100, 152), (50, 76), (25, 38), (13, 19))
# The variant that sums to 19,947 positions.
DETR_LEVELS_ALT = ((100, 150), (50, 75), (25, 38), (13, 19))


def padded_offset_dim(G: int, K: int) -> int:
    """ceil(3*G*K/8)*8, the packed offset_mask width (DCNv4_op/DCNv4/modules/dcnv4.py:79-82)."""
    return int(math.ceil(G * K * 3 / 8) * 8)


def dcnv4_inputs(N: int, H: int, W: int, G: int, D: int, *, kh=3, kw=3, sh=1, sw=1, ph=1,
                 pw=1, dh=1, dw=1, remove_center=0, seed=0, offset_std=1.0,
                 dtype=torch.float32, device="cpu") -> Dict[str, torch.Tensor]:
    """value ~N(0,1); per group 2K offsets ~N(0,offset_std) px then K masks ~U(0,1);
    pad columns zero; grad_out ~N(0,1).  Generated in fp32 on CPU, then cast/moved."""
    g = torch.Generator().manual_seed(seed)
    K = kh * kw - int(bool(remove_center))
    Ho = (H + 2 * ph - (dh * (kh - 1) + 1)) // sh + 1
    Wo = (W + 2 * pw - (dw * (kw - 1) + 1)) // sw + 1
    Ppad = padded_offset_dim(G, K)
    value = torch.randn(N, H, W, G * D, generator=g)
    off = torch.randn(N, Ho, Wo, G, 2 * K, generator=g) * offset_std
    msk = torch.rand(N, Ho, Wo, G, K, generator=g)
    om = torch.zeros(N, Ho, Wo, Ppad)
    om[..., : G * K * 3] = torch.cat((off, msk), -1).reshape(N, Ho, Wo, G * K * 3)
    grad_out = torch.randn(N, Ho, Wo, G * D, generator=g)
    return {"value": value.to(device=device, dtype=dtype),
            "offset_mask": om.to(device=device, dtype=dtype),
            "grad_out": grad_out.to(device=device, dtype=dtype)}


def level_tensors(levels) -> Tuple[torch.Tensor, torch.Tensor, int]:
    shapes = torch.tensor(levels, dtype=torch.int64)
    sizes = shapes[:, 0] * shapes[:, 1]
    starts = torch.cat((sizes.new_zeros(1), sizes.cumsum(0)[:-1]))
    return shapes, starts, int(sizes.sum())


def fda_inputs(B: int, levels, G: int, D: int, K: int, *, Len_q=None, seed=0,
               loc_lo=0.0, loc_hi=1.0, dtype=torch.float32, device="cpu"):
    """value ~N(0,1) (B,Len_in,G,D); sampling locations ~U(loc_lo,loc_hi) normalised,
    logits ~N(0,1), packed as [x,y]*(L*K) then L*K logits; grad_out ~N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    shapes, starts, Len_in = level_tensors(levels)
    L = len(levels)
    Len_q = Len_in if Len_q is None else Len_q
    value = torch.randn(B, Len_in, G, D, generator=g)
    loc = torch.rand(B, Len_q, G, L * K * 2, generator=g) * (loc_hi - loc_lo) + loc_lo
    logits = torch.randn(B, Len_q, G, L * K, generator=g)
    sla = torch.cat((loc, logits), -1)
    grad_out = torch.randn(B, Len_q, G * D, generator=g)
    return {"value": value.to(device=device, dtype=dtype),
            "spatial_shapes": shapes.to(device), "level_start_index": starts.to(device),
            "sampling_loc_attn": sla.to(device=device, dtype=dtype),
            "grad_out": grad_out.to(device=device, dtype=dtype)}


def dcnv4_bytes(N, H, W, G, D, Ho, Wo, Ppad, elem_size) -> Tuple[int, int]:
    """Algorithmic bytes (each tensor counted once) of one forward and one backward."""
    C = G * D
    fwd = elem_size * (N * H * W * C + N * Ho * Wo * Ppad + N * Ho * Wo * C)
    bwd = elem_size * (2 * N * H * W * C + 2 * N * Ho * Wo * Ppad + N * Ho * Wo * C)
    return fwd, bwd


def fda_bytes(B, Len_in, Len_q, G, D, L, K, elem_size) -> Tuple[int, int]:
    fwd = elem_size * (B * Len_in * G * D + B * Len_q * G * L * K * 3 + B * Len_q * G * D)
    bwd = fwd + elem_size * (B * Len_in * G * D + B * Len_q * G * L * K * 3)
    return fwd, bwd
