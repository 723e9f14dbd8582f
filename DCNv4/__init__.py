"""Drop-in alias: `import DCNv4` resolves to the B200 implementation, so callers written
against the reference package (e.g. `getattr(DCNv4, core_op)` in
classification/models/flash_intern_image.py:634) run unchanged."""
from dcnv4_b200 import DCNv4, DCNv4Function, FlashDeformAttn, FlashDeformAttnFunction, ext  # noqa: F401

__all__ = ["DCNv4Function", "FlashDeformAttnFunction", "DCNv4", "FlashDeformAttn", "ext"]
