"""Generate tests/golden/flash_intern_image_state_dicts.json from the reference's own model file.

    python tests/golden/make_state_dict_fixture.py /path/to/reference

The reference's `classification/models/flash_intern_image.py` is imported UNMODIFIED by file
path and instantiated with the released settings of its four classification configs
(classification/configs/flash_intern_image_{t,s,b}_1k_224.yaml, ..._l_22kto1k_384.yaml).  Its two
imports that are not installed here are stood in for: `timm.models.layers` (`trunc_normal_`,
`DropPath`: initialisation and stochastic depth, neither changes a parameter's name or shape) and
the compiled `DCNv4` package, for which this repository's drop-in package of the same name is
used (the reference builds its core operator with `getattr(DCNv4, core_op)`,
classification/models/flash_intern_image.py:634).  The result is the complete map
parameter/buffer name -> shape for each size, which `tests/test_model_cpu.py` compares with the
restatement in `dcnv4_b200/flash_intern_image.py`, so released checkpoints load key for key.
"""
from __future__ import annotations

import importlib.util
import json
import os
import sys
import types

import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

# released settings: MODEL.FLASH_INTERN_IMAGE of the four yaml files
RELEASED = {
    "t": dict(channels=64, depths=[4, 4, 18, 4], groups=[4, 8, 16, 32], offset_scale=1.0, mlp_ratio=4.0,
              drop_path_rate=0.1),
    "s": dict(channels=80, depths=[4, 4, 21, 4], groups=[5, 10, 20, 40], layer_scale=1e-5, offset_scale=1.0,
              mlp_ratio=4.0, post_norm=True, dw_kernel_size=3, drop_path_rate=0.4),
    "b": dict(channels=112, depths=[4, 4, 21, 4], groups=[7, 14, 28, 56], layer_scale=1e-5, offset_scale=0.5,
              mlp_ratio=4.0, post_norm=True, dw_kernel_size=3, drop_path_rate=0.5),
    "l": dict(channels=160, depths=[5, 5, 22, 5], groups=[10, 20, 40, 80], layer_scale=1e-5, offset_scale=2.0,
              mlp_ratio=4.0, post_norm=True, dw_kernel_size=3, dcn_output_bias=True, mlp_fc2_bias=True,
              drop_path_rate=0.1),
}


def load_reference_model_module(ref_root: str):
    class DropPath(nn.Module):
        def __init__(self, p=0.0):
            super().__init__()

        def forward(self, x):
            return x

    layers = types.ModuleType("timm.models.layers")
    layers.trunc_normal_ = lambda t, std=0.02, **kw: nn.init.normal_(t, std=std)
    layers.DropPath = DropPath
    for name in ("timm", "timm.models"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["timm.models.layers"] = layers
    import DCNv4  # noqa: F401  (this repository's drop-in package of the reference's name)
    path = os.path.join(ref_root, "classification", "models", "flash_intern_image.py")
    spec = importlib.util.spec_from_file_location("ref_flash_intern_image", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str):
    ref = load_reference_model_module(ref_root)
    out = {}
    for size, kw in RELEASED.items():
        model = ref.FlashInternImage(core_op="DCNv4", num_classes=1000, **kw)
        out[size] = {k: list(v.shape) for k, v in model.state_dict().items()}
        print(size, len(out[size]), "entries,", sum(p.numel() for p in model.parameters()), "parameters")
    path = os.path.join(HERE, "flash_intern_image_state_dicts.json")
    with open(path, "w") as f:
        json.dump(out, f, separators=(",", ":"), sort_keys=True)
    print(path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    from oracle import ref_core
    root = sys.argv[1] if len(sys.argv) > 1 else ref_core.reference_root()
    if root is None:
        raise SystemExit("usage: make_state_dict_fixture.py /path/to/reference (or set DCNV4_REFERENCE_ROOT)")
    main(root)
