"""Monkey-patch HF's GPT-OSS eager attention with the B200 kernels.

Same three names and behaviour as the reference's ``patching.py:1-10``: the original
function is captured at import time, ``patch_flash_attention()`` assigns the module global
``modeling_gpt_oss.eager_attention_forward`` (which ``GptOssAttention.forward`` looks up at
call time when ``attn_implementation == "eager"``), ``unpatch_flash_attention()`` restores it.
"""
from transformers.models.gpt_oss import modeling_gpt_oss

from .attention_kernel import triton_flash_attention

_original_eager_attention_forward = modeling_gpt_oss.eager_attention_forward


def patch_flash_attention():
    modeling_gpt_oss.eager_attention_forward = triton_flash_attention


def unpatch_flash_attention():
    modeling_gpt_oss.eager_attention_forward = _original_eager_attention_forward
