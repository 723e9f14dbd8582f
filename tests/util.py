"""Shared helpers of the parity tests: tolerances and oracle calls on storage-rounded inputs."""
import torch

from oracle import cref

# Forward tolerances: fp32 as the acceptance criterion states (rel 1e-4 / abs 1e-5 against the
# fp64 oracle); fp16 rel 1e-2 (with the abs 1e-3 the reference's own scripts use,
# DCNv4_op/scripts/test_dcnv4.py:116); bf16 has 3 fewer mantissa bits than fp16.
FWD_TOL = {torch.float32: dict(rtol=1e-4, atol=1e-5),
           torch.float16: dict(rtol=1e-2, atol=1e-3),
           torch.bfloat16: dict(rtol=2e-2, atol=1e-2)}
# Backward: fp32 rel 1e-3 (atomic accumulation order differs run to run); the abs term covers
# sums that cancel to ~0.
BWD_TOL = {torch.float32: dict(rtol=1e-3, atol=1e-4),
           torch.float16: dict(rtol=1e-2, atol=4e-3),
           torch.bfloat16: dict(rtol=2e-2, atol=3e-2)}


def close(actual, expected, tol, what=""):
    torch.testing.assert_close(actual.detach().double().cpu(), expected.double().cpu(), msg=lambda m: f"{what}: {m}", **tol)


def dcn_args(spec):
    """spec dict -> positional tail (kh..remove_center) shared by oracle and ops."""
    return (spec["kh"], spec["kw"], spec["sh"], spec["sw"], spec["ph"], spec["pw"], spec["dh"], spec["dw"],
            spec["G"], spec["D"], spec["scale"], spec["rc"])


def oracle_dcn(t, spec, softmax=False, corners=False):
    """Run the C oracle on exactly the values the GPU sees (already rounded to storage dtype)."""
    v, om, go = (t[k].detach().float().cpu() for k in ("value", "offset_mask", "grad_out"))
    a = dcn_args(spec)
    fwd = cref.dcnv4_forward(v, om, *a, softmax=softmax, want_corners=corners)
    gv, gom = cref.dcnv4_backward(v, om, go, *a, softmax=softmax)
    return fwd, gv, gom


def oracle_fda(t, K, corners=False):
    v, sla, go = (t[k].detach().float().cpu() for k in ("value", "sampling_loc_attn", "grad_out"))
    ss, ls = t["spatial_shapes"].cpu(), t["level_start_index"].cpu()
    fwd = cref.fda_forward(v, ss, ls, sla, K, want_corners=corners)
    gv, gs = cref.fda_backward(v, ss, ls, sla, go, K)
    return fwd, gv, gs
