"""The one-pass rotary embedding (`b200attn_rope`) on the GPU, through the C ABI and through the patch point."""
import pytest
import torch

from oracle.rope_fp32 import apply_rotary, rotary_tables
from oregon_gpt_oss_patching_b200.rope import (b200_apply_rotary_pos_emb, patch_rotary_embedding, rope,
                                               unpatch_rotary_embedding)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max())


@pytest.mark.parametrize("B,H,S,table_batch", [(2, 64, 300, 2), (1, 8, 1, 1), (3, 5, 129, 1)])
def test_forward_and_backward_match_the_fp32_oracle_on_model_layout_views(B, H, S, table_batch):
    g = torch.Generator().manual_seed(S)
    x = torch.randn(B, S, H, 64, generator=g).to(device=DEV, dtype=torch.bfloat16).transpose(1, 2)   # as the projection's view
    dy = torch.randn(B, H, S, 64, generator=g).to(device=DEV, dtype=torch.bfloat16)
    cos, sin = (t.to(device=DEV, dtype=torch.bfloat16) for t in rotary_tables(S, batch=table_batch, scaling=1.2, offset=1000))
    xg = x.detach().clone().requires_grad_(True)
    y = rope(xg, cos, sin)
    assert y.shape == x.shape and y.stride() == xg.stride()        # same layout out as in: consumed in place downstream
    y.backward(dy)
    torch.cuda.synchronize()
    ref_y = apply_rotary(x.float(), cos.float(), sin.float())
    ref_dx = apply_rotary(dy.float(), cos.float(), -sin.float())
    assert rel(y, ref_y) < 4e-3 and rel(xg.grad, ref_dx) < 4e-3      # one bf16 rounding of an fp32 result
    assert xg.grad.transpose(1, 2).is_contiguous()                 # (B,S,H,d) memory: the projection's backward reshapes it for free


def test_patch_point_and_attention_downstream():
    from transformers.models.gpt_oss import modeling_gpt_oss
    from oregon_gpt_oss_patching_b200.attention_kernel import attention
    original = modeling_gpt_oss.apply_rotary_pos_emb
    B, S, Hq, Hkv = 1, 256, 16, 2
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, S, Hq, 64, generator=g).to(device=DEV, dtype=torch.bfloat16).transpose(1, 2)
    k = torch.randn(B, S, Hkv, 64, generator=g).to(device=DEV, dtype=torch.bfloat16).transpose(1, 2)
    v = torch.randn(B, S, Hkv, 64, generator=g).to(device=DEV, dtype=torch.bfloat16).transpose(1, 2)
    cos, sin = (t.to(device=DEV, dtype=torch.bfloat16) for t in rotary_tables(S))
    patch_rotary_embedding()
    try:
        assert modeling_gpt_oss.apply_rotary_pos_emb is b200_apply_rotary_pos_emb
        q1, k1 = modeling_gpt_oss.apply_rotary_pos_emb(q, k, cos, sin)
    finally:
        unpatch_rotary_embedding()
    assert modeling_gpt_oss.apply_rotary_pos_emb is original
    q0, k0 = original(q, k, cos, sin)
    assert rel(q1, q0) < 2e-2 and rel(k1, k0) < 2e-2                # the original rounds every intermediate to bf16
    # the rotated views go straight into the attention kernels (no copy: strides are taken as they are)
    sinks = torch.zeros(Hq, device=DEV, dtype=torch.bfloat16)
    o1 = attention(q1, k1, v, sinks, 0.125, 128, None)
    o0 = attention(q0.contiguous(), k0.contiguous(), v, sinks, 0.125, 128, None)
    assert rel(o1, o0) < 2e-2
