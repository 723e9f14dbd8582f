"""Golden vectors produced by the reference's own CUDA kernels on a B200
(tests/golden/make_golden_ref_cuda.py -> tests/golden/ref_cuda_golden.npz): they pin the CPU
oracle (no GPU needed) and, on the GPU, this library's kernels -- including FlashDeformAttn, for
which the reference has no CPU formula."""
import os

import numpy as np
import pytest
import torch

from oracle import cref, inputs as oin

PATH = os.path.join(os.path.dirname(__file__), "golden", "ref_cuda_golden.npz")
Z = np.load(PATH) if os.path.exists(PATH) else None
needs_file = pytest.mark.skipif(Z is None, reason="ref_cuda_golden.npz not generated yet")
FDA = sorted({k.split("/")[1] for k in Z.files if k.startswith("fda/")}) if Z is not None else []
DCN = sorted({k.split("/")[1] for k in Z.files if k.startswith("dcn/")}) if Z is not None else []

# the reference kernels compute in fp32: compare at fp32 tolerances (forward 1e-4/1e-5 relaxed by
# the kernels' own rounding, backward 1e-3 because both sides accumulate with atomics)
FWD = dict(rtol=2e-4, atol=2e-5)
BWD = dict(rtol=2e-3, atol=2e-4)


def _fda_inputs(name, device="cpu"):
    s = Z[f"fda/{name}/spec"]
    B, G, D, K, Lq, seed = (int(x) for x in s[:6])
    levels = tuple((int(s[6 + 2 * i]), int(s[7 + 2 * i])) for i in range((len(s) - 6) // 2))
    return oin.fda_inputs(B, levels, G, D, K, Len_q=Lq, seed=seed, loc_lo=0.02, loc_hi=0.98, device=device), K


def _dcn_inputs(name, device="cpu"):
    N, HW, G, D, seed, step = (int(x) for x in Z[f"dcn/{name}/spec"])
    return oin.dcnv4_inputs(N, HW, HW, G, D, seed=seed, device=device), (N, HW, G, D, step)


@needs_file
@pytest.mark.parametrize("name", FDA)
def test_oracle_matches_reference_cuda_fda(name):
    t, K = _fda_inputs(name)
    out = cref.fda_forward(t["value"], t["spatial_shapes"], t["level_start_index"], t["sampling_loc_attn"], K)
    gv, gs = cref.fda_backward(t["value"], t["spatial_shapes"], t["level_start_index"], t["sampling_loc_attn"],
                               t["grad_out"], K)
    torch.testing.assert_close(out[:, ::8], torch.from_numpy(Z[f"fda/{name}/out"]).double(), **FWD)
    torch.testing.assert_close(gv[:, ::8], torch.from_numpy(Z[f"fda/{name}/grad_value"]).double(), **BWD)
    # location gradients carry a factor H_l / W_l (up to 30 here)
    torch.testing.assert_close(gs[:, ::8], torch.from_numpy(Z[f"fda/{name}/grad_sla"]).double(), rtol=2e-3, atol=5e-3)


@needs_file
@pytest.mark.parametrize("name", [n for n in DCN if n != "n64_56"])   # the 64x56x56 case is sized for the GPU
def test_oracle_matches_reference_cuda_dcnv4(name):
    t, (N, HW, G, D, step) = _dcn_inputs(name)
    a = (3, 3, 1, 1, 1, 1, 1, 1, G, D, 1.0, 0)
    out = cref.dcnv4_forward(t["value"], t["offset_mask"], *a)
    gv, gom = cref.dcnv4_backward(t["value"], t["offset_mask"], t["grad_out"], *a)
    C = G * D
    torch.testing.assert_close(out.reshape(-1, C)[::step], torch.from_numpy(Z[f"dcn/{name}/out"]).double(), **FWD)
    torch.testing.assert_close(gv.reshape(-1, C)[::step], torch.from_numpy(Z[f"dcn/{name}/grad_value"]).double(), **BWD)
    torch.testing.assert_close(gom.reshape(-1, gom.shape[-1])[::step],
                               torch.from_numpy(Z[f"dcn/{name}/grad_offset_mask"]).double(), **BWD)


@needs_file
@pytest.mark.gpu
@pytest.mark.parametrize("name", FDA)
def test_kernels_match_reference_cuda_fda(name):
    from dcnv4_b200 import ops
    t, K = _fda_inputs(name, "cuda")
    out = ops.flash_deform_attn_forward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                        t["sampling_loc_attn"], 64, K)
    gv, gs = ops.flash_deform_attn_backward(t["value"], t["spatial_shapes"], t["level_start_index"],
                                            t["sampling_loc_attn"], t["grad_out"], 64, K)
    torch.testing.assert_close(out[:, ::8].cpu(), torch.from_numpy(Z[f"fda/{name}/out"]), **FWD)
    torch.testing.assert_close(gv[:, ::8].cpu(), torch.from_numpy(Z[f"fda/{name}/grad_value"]), **BWD)
    torch.testing.assert_close(gs[:, ::8].cpu(), torch.from_numpy(Z[f"fda/{name}/grad_sla"]), rtol=2e-3, atol=5e-3)


@needs_file
@pytest.mark.gpu
@pytest.mark.parametrize("name", DCN)
def test_kernels_match_reference_cuda_dcnv4(name):
    from dcnv4_b200 import ops
    t, (N, HW, G, D, step) = _dcn_inputs(name, "cuda")
    out = ops.dcnv4_forward(t["value"], t["offset_mask"], 3, 3, 1, 1, 1, 1, 1, 1, G, D, 1.0, 256, 0)
    gv, gom = ops.dcnv4_backward(t["value"], t["offset_mask"], 3, 3, 1, 1, 1, 1, 1, 1, G, D, 1.0, 256,
                                 t["grad_out"], 0)
    C = G * D
    torch.testing.assert_close(out.reshape(-1, C)[::step].cpu(), torch.from_numpy(Z[f"dcn/{name}/out"]), **FWD)
    torch.testing.assert_close(gv.reshape(-1, C)[::step].cpu(), torch.from_numpy(Z[f"dcn/{name}/grad_value"]), **BWD)
    torch.testing.assert_close(gom.reshape(-1, gom.shape[-1])[::step].cpu(),
                               torch.from_numpy(Z[f"dcn/{name}/grad_offset_mask"]), **BWD)
