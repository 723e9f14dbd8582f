"""Canary guard bands: every output, gradient and workspace buffer handed to the C ABI sits between
two sentinel-filled bands; after the call the bands must be untouched and the payload fully written
(no sentinel left).  Catches stray writes that parity checks on the payload alone would miss."""
import pytest
import torch

from dcnv4_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"
GUARD = 4096  # bytes on each side
SENTINEL = 0x5A


class Guarded:
    """A device buffer of `nbytes` (16-byte aligned payload) with guard bands on both sides."""

    def __init__(self, nbytes):
        self.nbytes = nbytes
        self.raw = torch.full((GUARD + nbytes + GUARD,), SENTINEL, dtype=torch.uint8, device=DEV)
        assert self.raw.data_ptr() % 16 == 0

    @property
    def ptr(self):
        return self.raw.data_ptr() + GUARD

    def payload(self, dtype, shape):
        return self.raw[GUARD:GUARD + self.nbytes].view(dtype).view(shape)

    def check(self, what, expect_fully_written=True):
        assert bool((self.raw[:GUARD] == SENTINEL).all()), f"{what}: bytes before the buffer were overwritten"
        assert bool((self.raw[GUARD + self.nbytes:] == SENTINEL).all()), f"{what}: bytes after the buffer were overwritten"
        if expect_fully_written and self.nbytes >= 8:
            words = self.raw[GUARD:GUARD + self.nbytes // 8 * 8].view(torch.int64)
            untouched = words == int.from_bytes(bytes([SENTINEL]) * 8, "little")
            assert not bool(untouched.any()), f"{what}: part of the buffer was never written"


@pytest.mark.parametrize("dtype,code", [(torch.float32, _lib.F32), (torch.float16, _lib.F16), (torch.bfloat16, _lib.BF16)],
                         ids=["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("shape", [(3, 9, 11, 3, 16), (2, 14, 14, 16, 16), (1, 7, 7, 32, 16), (2, 5, 6, 2, 48)],
                         ids=lambda s: "x".join(map(str, s)))
def test_dcnv4_buffers_are_written_exactly(shape, dtype, code):
    from oracle import inputs as oin
    N, H, W, G, D = shape
    lib = _lib.lib()
    t = oin.dcnv4_inputs(N, H, W, G, D, seed=5, offset_std=3.0, dtype=dtype, device=DEV)
    es = t["value"].element_size()
    P = t["offset_mask"].shape[-1]
    out = Guarded(t["value"].numel() * es)
    gv = Guarded(t["value"].numel() * es)
    gom = Guarded(t["offset_mask"].numel() * es)
    ws_bytes = lib.dcnv4b200_bwd_workspace_bytes(code, N, H, W, G, D)
    ws = Guarded(max(ws_bytes, 16))
    scal = (N, H, W, G, D, 3, 3, 1, 1, 1, 1, 1, 1, 1.0, 0, P, 0)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.dcnv4b200_fwd(t["value"].data_ptr(), t["offset_mask"].data_ptr(), out.ptr, code, *scal, st) == 0
    assert lib.dcnv4b200_bwd(t["value"].data_ptr(), t["offset_mask"].data_ptr(), t["grad_out"].data_ptr(), gv.ptr,
                             gom.ptr, ws.ptr if ws_bytes else None, ws_bytes, code, *scal, st) == 0
    torch.cuda.synchronize()
    out.check("out")
    gv.check("grad_value")
    gom.check("grad_offset_mask")
    ws.check("workspace", expect_fully_written=bool(ws_bytes))
    assert torch.isfinite(out.payload(dtype, t["value"].shape).float()).all()


@pytest.mark.parametrize("dtype,code", [(torch.float32, _lib.F32), (torch.float16, _lib.F16)], ids=["fp32", "fp16"])
@pytest.mark.parametrize("case", [(2, ((6, 8), (3, 4)), 2, 16, 4, 37), (1, ((5, 7), (4, 4), (2, 3)), 3, 8, 8, 19),
                                  (1, ((20, 30), (10, 15)), 8, 32, 4, 301)], ids=["two_levels", "ragged_rows", "detr_like"])
def test_flash_deform_attn_buffers_are_written_exactly(case, dtype, code):
    from oracle import inputs as oin
    B, levels, G, D, K, Lq = case
    lib = _lib.lib()
    t = oin.fda_inputs(B, levels, G, D, K, Len_q=Lq, seed=9, loc_lo=-0.2, loc_hi=1.2, dtype=dtype, device=DEV)
    es = t["value"].element_size()
    Len_in, L = t["value"].shape[1], len(levels)
    out = Guarded(B * Lq * G * D * es)
    gv = Guarded(t["value"].numel() * es)
    gs = Guarded(t["sampling_loc_attn"].numel() * es)
    ws_bytes = lib.fdab200_bwd_workspace_bytes(code, B, Len_in, G, D)
    ws = Guarded(max(ws_bytes, 16))
    st = torch.cuda.current_stream().cuda_stream
    dims = (code, B, Len_in, G, D, L, Lq, K, st)
    assert lib.fdab200_fwd(t["value"].data_ptr(), t["spatial_shapes"].data_ptr(), t["level_start_index"].data_ptr(),
                           t["sampling_loc_attn"].data_ptr(), out.ptr, *dims) == 0
    assert lib.fdab200_bwd(t["value"].data_ptr(), t["spatial_shapes"].data_ptr(), t["level_start_index"].data_ptr(),
                           t["sampling_loc_attn"].data_ptr(), t["grad_out"].data_ptr(), gv.ptr, gs.ptr,
                           ws.ptr if ws_bytes else None, ws_bytes, *dims) == 0
    torch.cuda.synchronize()
    out.check("out")
    gv.check("grad_value")
    gs.check("grad_sampling_loc_attn")
    ws.check("workspace", expect_fully_written=bool(ws_bytes))


def test_layernorm_buffer_is_written_exactly():
    lib = _lib.lib()
    x = torch.randn(1001, 64, device=DEV, dtype=torch.float16)
    w = torch.ones(64, device=DEV, dtype=torch.float16)
    y = Guarded(x.numel() * 2)
    assert lib.dcnv4b200_layernorm_fwd(x.data_ptr(), w.data_ptr(), w.data_ptr(), y.ptr, _lib.F16, _lib.F16,
                                       1001, 64, 1e-6, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    y.check("layernorm out")
