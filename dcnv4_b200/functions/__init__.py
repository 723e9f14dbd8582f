from .dcnv4_func import DCNv4Function
from .flash_deform_attn_func import FlashDeformAttnFunction

__all__ = ["DCNv4Function", "FlashDeformAttnFunction"]
