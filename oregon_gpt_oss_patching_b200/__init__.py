"""B200-native GPT-OSS attention forward/backward (sinks, GQA, causal / sliding window).

Public surface, matching the reference project's two modules:

* ``attention_kernel``: ``attention``, ``triton_flash_attention`` / ``b200_flash_attention``; plus
  ``attention_varlen`` for documents packed back to back (no counterpart in the reference)
* ``patching``: ``patch_flash_attention``, ``unpatch_flash_attention`` (imports transformers)
"""
from .attention_kernel import attention, attention_varlen, b200_flash_attention, triton_flash_attention  # noqa: F401

__all__ = ["attention", "attention_varlen", "b200_flash_attention", "triton_flash_attention"]
__version__ = "0.1.0"
