from .dcnv4 import DCNv4
from .flash_deform_attn import FlashDeformAttn

__all__ = ["DCNv4", "FlashDeformAttn"]
