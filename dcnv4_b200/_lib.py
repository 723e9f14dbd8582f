"""ctypes loader of the in-tree CUDA library (`dcnv4_b200/_C/libdcnv4_b200.so`).

There is no CPU fallback and no other backend: if the library is missing or a call is
made without a CUDA tensor, an exception is raised.  Build the library with
`python -m dcnv4_b200.build`.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_C", "libdcnv4_b200.so")
ABI_VERSION = 1

F32, F16, BF16 = 0, 1, 2

_lib = None
_lock = threading.Lock()

_i, _f, _p, _z = C.c_int, C.c_float, C.c_void_p, C.c_size_t
_DCN_SCALARS = [_i] * 13 + [_f, _i, _i, _i]  # N,H,W,G,D,kh,kw,sh,sw,ph,pw,dh,dw, scale, rc, Ppad, softmax

_SIGNATURES = {
    "dcnv4b200_abi_version": (_i, []),
    "dcnv4b200_strerror": (C.c_char_p, [_i]),
    "dcnv4b200_out_size": (_i, [_i] * 5),
    "dcnv4b200_fwd": (_i, [_p, _p, _p, _i] + _DCN_SCALARS + [_p]),
    "dcnv4b200_bwd_workspace_bytes": (_z, [_i] * 6),
    "dcnv4b200_bwd": (_i, [_p] * 6 + [_z, _i] + _DCN_SCALARS + [_p]),
    "fdab200_fwd": (_i, [_p] * 5 + [_i] * 8 + [_p]),
    "fdab200_bwd_workspace_bytes": (_z, [_i] * 5),
    "fdab200_bwd": (_i, [_p] * 8 + [_z] + [_i] * 8 + [_p]),
    "dcnv4b200_fwd_corners": (_i, [_p, _p, _i] + [_i] * 12 + [_f, _i, _i, _p]),
    "fdab200_fwd_corners": (_i, [_p, _p, _p] + [_i] * 6 + [_p]),
    "dcnv4b200_layernorm_fwd": (_i, [_p, _p, _p, _p, _i, _i, C.c_longlong, _i, _f, _p]),
    "dcnv4b200_layernorm_act_fwd": (_i, [_p, _p, _p, _p, _i, _i, C.c_longlong, _i, _f, _i, _p]),
    "dcnv4b200_center_scale_blend_fwd": (_i, [_p, _p, _p, _p, _p, _i, _i, C.c_longlong, _i, _i, _p]),
    "dcnv4b200_linear_fwd": (_i, [_p, _p, _p, _p, _p, _i, C.c_longlong, _i, _i, _i, _p]),
    "dcnv4b200_bias_act_fwd": (_i, [_p, _p, _p, _i, C.c_longlong, _i, _i, _p]),
    "dcnv4b200_linear_pair_fwd": (_i, [_p, _p, _p, _p, _i, _p, _i, _i, C.c_longlong, _i, _p]),
    "dcnv4b200_fwd_fused_offset": (_i, [_p] * 5 + [_i] * 8 + [_f, _p]),
    "dcnv4b200_linear_ln_fwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _f, _p, _i, C.c_longlong, _i, _i, _p]),
    "dcnv4b200_device_status": (_i, [C.POINTER(_i)]),
    "dcnv4b200_bwd_static_scratch_max_elements": (_z, []),
    "dcnv4b200_bwd_static_scratch": (_i, [_p] * 5 + [_i] + _DCN_SCALARS + [_p]),
}


class LibraryError(RuntimeError):
    """The CUDA library is missing, stale, or rejected a call."""


def exported_symbols():
    """Names every build of the library must export (the declarations of include/dcnv4_b200.h)."""
    return tuple(_SIGNATURES)


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise LibraryError(
                    f"{LIB_PATH} not found: the dcnv4_b200 CUDA library is not built "
                    "(run `python -m dcnv4_b200.build`); there is no CPU fallback")
            handle = C.CDLL(LIB_PATH)
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(handle, name)  # AttributeError if the symbol is missing
                fn.restype, fn.argtypes = res, args
            got = handle.dcnv4b200_abi_version()
            if got != ABI_VERSION:
                raise LibraryError(f"ABI mismatch: library {got}, python {ABI_VERSION}; rebuild the library")
            _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    """Map a library return code to the exception type the reference raises for the same
    condition: argument problems -> RuntimeError (AT_ASSERTM in
    DCNv4_op/src/cuda/dcnv4_cuda.cu:34-60), unsupported parameter values -> ValueError
    (std::invalid_argument in DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:282-296)."""
    if rc == 0:
        return
    msg = lib().dcnv4b200_strerror(rc).decode()
    if rc in (-6, -8):
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg} (code {rc})")
