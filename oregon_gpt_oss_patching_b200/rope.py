"""Rotary position embedding in front of the patched attention, as one kernel per tensor.

``GptOssAttention.forward`` rotates the query and key projections with ``apply_rotary_pos_emb``
(``transformers/models/gpt_oss/modeling_gpt_oss.py:226-242``, called at ``:318-319``) right before it calls the
function the reference patches.  The original is seven elementwise tensor operations per tensor -- each a
pass over memory, plus as many again in the backward -- on (B, H, S, d) views of the (B, S, H, d) projection
output.  ``b200_apply_rotary_pos_emb`` has the same signature and result and runs one pass per tensor
(``b200attn_rope``), reading the strided view where it lies and writing the result with the same strides, which
the attention kernels consume in place; the backward is the same kernel with the rotation reversed.
``patch_rotary_embedding`` assigns it to the module global, exactly as the attention patch does.
"""
from __future__ import annotations

import ctypes

import torch

from . import _cabi

__all__ = ["b200_apply_rotary_pos_emb", "patch_rotary_embedding", "unpatch_rotary_embedding", "rope"]


def _launch(x, out, cos, sin, inverse: bool) -> None:
    B, Hh, S, d = x.shape
    tx, to = _cabi.tensor4(x, "bhsd"), _cabi.tensor4(out, "bhsd")
    cb = 0 if cos.shape[0] == 1 else cos.stride(0)
    dev = x.device
    rc = _cabi.load().b200attn_rope(ctypes.byref(tx), ctypes.byref(to), cos.data_ptr(), sin.data_ptr(), cb, cos.stride(1),
                                    B, Hh, S, 1 if inverse else 0, dev.index, torch.cuda.current_stream(dev).cuda_stream)
    _cabi.check(rc, "b200attn_rope")


def _like(x):
    """An uninitialised tensor with the shape AND the strides of ``x`` (a (B,S,H,d) buffer viewed as (B,H,S,d) stays one)."""
    return torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)


class _rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        if not x.is_cuda or x.dtype != torch.bfloat16 or x.shape[-1] != 64:
            raise RuntimeError("rope: needs a CUDA bfloat16 tensor with head_dim 64 (the sm_100a library is the only code path)")
        if x.stride(-1) != 1 or any(s % 8 for s in x.stride()[:-1]) or x.data_ptr() % 16:
            x = x.contiguous()
        cos, sin = cos.to(torch.bfloat16).contiguous(), sin.to(torch.bfloat16).contiguous()
        if cos.shape != sin.shape or cos.dim() != 3 or cos.shape[-1] != 32 or cos.shape[1] != x.shape[2] or cos.shape[0] not in (1, x.shape[0]):
            raise RuntimeError("rope: cos / sin must be (B or 1, S, 32)")
        out = _like(x)
        _launch(x, out, cos, sin, inverse=False)
        ctx.save_for_backward(cos, sin)
        return out

    @staticmethod
    def backward(ctx, dout):
        cos, sin = ctx.saved_tensors
        if dout.stride(-1) != 1 or any(s % 8 for s in dout.stride()[:-1]) or dout.data_ptr() % 16:
            dout = dout.contiguous()
        # (B, S, H, d) memory behind a (B, H, S, d) view: what the projection's backward wants to reshape for free
        B, Hh, S, d = dout.shape
        dx = torch.empty(B, S, Hh, d, dtype=dout.dtype, device=dout.device).transpose(1, 2)
        _launch(dout, dx, cos, sin, inverse=True)
        return dx, None, None


rope = _rope.apply


def b200_apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    """Same signature and result as ``modeling_gpt_oss.apply_rotary_pos_emb`` (``:237-242``) for (B, H, S, 64) q and k."""
    if unsqueeze_dim != 1:
        raise RuntimeError("b200_apply_rotary_pos_emb: only the (B, H, S, d) layout (unsqueeze_dim=1) is supported")
    return rope(q, cos, sin), rope(k, cos, sin)


_original_apply_rotary_pos_emb = None


def patch_rotary_embedding():
    global _original_apply_rotary_pos_emb
    from transformers.models.gpt_oss import modeling_gpt_oss
    if _original_apply_rotary_pos_emb is None:
        _original_apply_rotary_pos_emb = modeling_gpt_oss.apply_rotary_pos_emb
    modeling_gpt_oss.apply_rotary_pos_emb = b200_apply_rotary_pos_emb


def unpatch_rotary_embedding():
    from transformers.models.gpt_oss import modeling_gpt_oss
    if _original_apply_rotary_pos_emb is not None:
        modeling_gpt_oss.apply_rotary_pos_emb = _original_apply_rotary_pos_emb
