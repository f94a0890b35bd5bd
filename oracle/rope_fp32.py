"""fp32 restatement of the rotary position embedding in front of the attention path (TEST INFRASTRUCTURE ONLY).

Restates ``transformers/models/gpt_oss/modeling_gpt_oss.py:226-242`` (``_apply_rotary_emb``,
``apply_rotary_pos_emb``; checked against transformers 5.5.0): the head dimension is split in two halves,
``first' = first * cos - second * sin``, ``second' = second * cos + first * sin``, with cos / sin of shape
(B, S, d/2) broadcast over the heads of a (B, H, S, d) tensor.  ``tests/test_rope_oracle.py`` pins it to the
installed function itself.
"""
import torch


def rotary_tables(S: int, d: int = 64, base: float = 150000.0, batch: int = 1, scaling: float = 1.0, offset: int = 0):
    """cos / sin tables (batch, S, d/2) in fp32 for positions offset .. offset+S-1 (plain RoPE frequencies; the values only
    need to look like the model's, the kernels take any table)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    pos = torch.arange(offset, offset + S, dtype=torch.float32)
    ang = pos[:, None] * inv_freq[None, :]
    return (ang.cos() * scaling)[None].expand(batch, -1, -1).contiguous(), (ang.sin() * scaling)[None].expand(batch, -1, -1).contiguous()


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: (B, H, S, d); cos, sin: (B or 1, S, d/2)."""
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)          # :238-239
    first, second = torch.chunk(x, 2, dim=-1)              # :231
    return torch.cat((first * cos - second * sin, second * cos + first * sin), dim=-1)   # :232-234
