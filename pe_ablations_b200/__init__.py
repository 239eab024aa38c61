"""B200-native fused positional-encoding attention (sm_100a) behind the reference's module API.

``ops.pe_attention`` is the functional entry point over the C ABI in
``include/pe_attn.h``; ``modules`` holds drop-in replacements for the
reference's three attention classes.  Importing the package loads the in-tree
CUDA library and fails loudly if it has not been built.
"""

from . import _lib  # noqa: F401  (raises if the CUDA library is missing)
from .ops import attention_flops, check_device_status, pe_attention  # noqa: F401

__all__ = ["pe_attention", "check_device_status", "attention_flops"]
