"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header declares,
and rejects bad arguments before touching a GPU (no compute call is made here)."""
import ctypes as C
import os
import re

import pytest

import __graft_entry__ as entry
from dcnv4_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    entry.build()
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dcnv4_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:dcnv4b200|fdab200)_\w+)\s*\(", text)))


def test_header_and_loader_agree(lib):
    decl = declared_symbols()
    assert decl, "header declares nothing?"
    assert sorted(_lib.exported_symbols()) == decl
    for name in decl:
        assert hasattr(lib, name), f"library does not export {name}"


def test_version_strerror_out_size(lib):
    assert lib.dcnv4b200_abi_version() == 1
    assert b"NULL" in lib.dcnv4b200_strerror(-1)
    assert lib.dcnv4b200_strerror(12345) is not None
    assert lib.dcnv4b200_out_size(56, 1, 1, 3, 1) == 56
    assert lib.dcnv4b200_out_size(15, 1, 1, 3, 2) == 8
    assert lib.dcnv4b200_out_size(12, 2, 2, 3, 1) == 12
    assert lib.dcnv4b200_out_size(2, 0, 1, 5, 1) == 0


def test_workspace_sizes(lib):
    assert lib.dcnv4b200_bwd_workspace_bytes(_lib.F32, 64, 56, 56, 4, 16) == 0
    assert lib.dcnv4b200_bwd_workspace_bytes(_lib.F16, 64, 56, 56, 4, 16) == 64 * 56 * 56 * 64 * 4
    assert lib.fdab200_bwd_workspace_bytes(_lib.BF16, 8, 20197, 8, 32) == 8 * 20197 * 256 * 4
    assert lib.fdab200_bwd_workspace_bytes(_lib.F32, 8, 20197, 8, 32) == 0


def _fwd(lib, value=0x1000, om=0x2000, out=0x3000, dtype=0, N=1, H=8, W=8, G=2, D=16, kh=3, kw=3, sh=1, sw=1,
         ph=1, pw=1, dh=1, dw=1, scale=1.0, rc=0, P=56, softmax=0):
    return lib.dcnv4b200_fwd(value, om, out, dtype, N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw,
                             scale, rc, P, softmax, None)


def test_rejects_bad_arguments_without_launching(lib):
    # every one of these returns before any CUDA call (pointers are never dereferenced)
    assert _fwd(lib, value=None) == -1
    assert _fwd(lib, om=0x2004) == -4
    assert _fwd(lib, dtype=7) == -2
    assert _fwd(lib, N=0) == -3
    assert _fwd(lib, H=1, W=1, ph=0, pw=0) == -3          # empty output
    assert _fwd(lib, P=54) == -7                          # not a multiple of 8
    assert _fwd(lib, P=48) == -7                          # < 3*K*G
    assert _fwd(lib, D=6) == -8
    assert _fwd(lib, dtype=1, D=20) == -8                 # fp16 needs multiples of 8
    assert _fwd(lib, G=2000, P=54000) == -6               # one query row exceeds the staging budget
    assert _fwd(lib, N=70000, H=200, W=200) == -9         # query count needs more than 31 bits
    rc = lib.fdab200_fwd(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 0, 1, 10, 1, 8, 9, 1, 1, None)
    assert rc == -6                                       # more than 8 levels
    rc = lib.dcnv4b200_bwd(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, None, 0, 1, 1, 8, 8, 2, 16,
                           3, 3, 1, 1, 1, 1, 1, 1, 1.0, 0, 56, 0, None)
    assert rc == -5                                       # fp16 backward needs the workspace


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.LibraryError, match="no CPU fallback"):
        _lib.lib()


def test_ops_refuse_cpu_tensors():
    import torch
    from dcnv4_b200 import ops
    v = torch.zeros(1, 4, 4, 32)
    om = torch.zeros(1, 4, 4, 56)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.dcnv4_forward(v, om, 3, 3, 1, 1, 1, 1, 1, 1, 2, 16, 1.0, 256, 0)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.flash_deform_attn_forward(torch.zeros(1, 4, 1, 16), torch.tensor([[2, 2]]), torch.tensor([0]),
                                      torch.zeros(1, 3, 1, 12), 64, 4)
