"""dcnv4_b200: B200 (sm_100a) implementation of the DCNv4 / FlashDeformAttn operator path.

Public surface = the reference package's (DCNv4_op/DCNv4/__init__.py:1-2):
`DCNv4Function`, `FlashDeformAttnFunction`, `DCNv4`, `FlashDeformAttn`, plus `ext`, a
stand-in for the reference's compiled `DCNv4.ext` module with the same four positional
functions.  Importing the package does not touch the GPU; the CUDA library is loaded on
first use and its absence is an error (there is no CPU path).
"""
from . import ops as ext
from .functions import DCNv4Function, FlashDeformAttnFunction
from .modules import DCNv4, FlashDeformAttn

__all__ = ["DCNv4Function", "FlashDeformAttnFunction", "DCNv4", "FlashDeformAttn", "ext"]
__version__ = "0.1.0"
