"""The rotary-embedding restatement against the installed Hugging Face function (CPU, fp32)."""
import torch

from oracle.rope_fp32 import apply_rotary, rotary_tables


def test_restatement_matches_the_hugging_face_function():
    from transformers.models.gpt_oss.modeling_gpt_oss import apply_rotary_pos_emb
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 8, 37, 64, generator=g).transpose(1, 2).contiguous().transpose(1, 2)   # (B,S,H,d) memory, as in the model
    k = torch.randn(2, 2, 37, 64, generator=g)
    cos, sin = rotary_tables(37, batch=2, scaling=1.3)
    q_ref, k_ref = apply_rotary_pos_emb(q, k, cos, sin)
    assert torch.equal(apply_rotary(q, cos, sin), q_ref) and torch.equal(apply_rotary(k, cos, sin), k_ref)


def test_the_inverse_rotation_is_the_gradient():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, 3, 20, 64, generator=g, requires_grad=True)
    cos, sin = rotary_tables(20)
    dy = torch.randn(1, 3, 20, 64, generator=g)
    apply_rotary(x, cos, sin).backward(dy)
    assert torch.allclose(x.grad, apply_rotary(dy, cos, -sin), atol=1e-6)
