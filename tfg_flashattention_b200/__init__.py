"""B200-native FlashAttention forward behind the reference project's `custom_flash_attn` entry point.

    from tfg_flashattention_b200 import custom_flash_attn
    o = custom_flash_attn.forward(q, k, v)            # the reference's call, unchanged

`install_as_custom_flash_attn()` registers the module under the top-level name the reference
imports (`import custom_flash_attn`, src/py/model_inference.py:13), so its code runs unmodified.
"""
import sys

from . import custom_flash_attn  # noqa: F401

__all__ = ["custom_flash_attn", "install_as_custom_flash_attn"]


def install_as_custom_flash_attn() -> None:
    sys.modules["custom_flash_attn"] = custom_flash_attn
