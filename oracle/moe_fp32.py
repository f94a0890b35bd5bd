"""fp32 restatement of the GPT-OSS mixture-of-experts block (TEST INFRASTRUCTURE ONLY).

The arithmetic lives in ``transformers`` (the reference pins ``transformers>=4.55.0``,
``requirements.txt:4``; checked here against 5.5.0), ``models/gpt_oss/modeling_gpt_oss.py``:

* ``GptOssExperts._apply_gate`` ``:76-82``  -- interleaved (gate, up) columns, gate clamped from above at 7,
  up clamped to [-7, 7], ``(up + 1) * gate * sigmoid(1.702 * gate)``;
* ``GptOssExperts.forward`` ``:84-114``     -- per expert: gather its tokens, ``x @ gate_up_proj[e] + bias``,
  gate, ``@ down_proj[e] + bias``, times the routing weight of (token, choice), ``index_add_`` into the output.

The restatement below is the same loop without in-place updates; gradients come from autograd.  Pinned by
``tests/golden/moe_*.npz``, which ``tests/golden/make_golden_moe.py`` produced by running the unmodified
``GptOssExperts`` module in fp32 on the same seeded inputs.
"""
from __future__ import annotations

import dataclasses

import torch

GLU_ALPHA = 1.702   # GptOssExperts.alpha  (modeling_gpt_oss.py:73)
GLU_LIMIT = 7.0     # GptOssExperts.limit  (modeling_gpt_oss.py:74)


@dataclasses.dataclass(frozen=True)
class MoeCase:
    name: str
    tokens: int
    hidden: int
    intermediate: int
    experts: int
    top_k: int
    seed: int = 0
    unused_expert: int = -1      # an expert no token is routed to (-1: none)


MOE_CASES = {
    "moe_small": MoeCase("moe_small", tokens=48, hidden=64, intermediate=48, experts=4, top_k=2, seed=11),
    "moe_ragged": MoeCase("moe_ragged", tokens=70, hidden=72, intermediate=40, experts=5, top_k=3, seed=12, unused_expert=2),
}


def make_moe_inputs(case: MoeCase, dtype=torch.float32, device="cpu"):
    """Seeded inputs with bf16-representable values: hidden, router_indices, routing_weights, the four
    parameters and the upstream gradient.  Weights are scaled so that the pre-activations spread over both
    clamps of the gate (some beyond +-7)."""
    g = torch.Generator().manual_seed(case.seed)
    T, H, I, E, k = case.tokens, case.hidden, case.intermediate, case.experts, case.top_k

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(torch.float32)

    hidden = rnd(T, H)
    w1 = rnd(E, H, 2 * I, scale=3.0 / H ** 0.5)
    b1 = rnd(E, 2 * I, scale=0.5)
    w2 = rnd(E, I, H, scale=1.0 / I ** 0.5)
    b2 = rnd(E, H, scale=0.5)
    logits = torch.randn(T, E, generator=g)
    if case.unused_expert >= 0:
        logits[:, case.unused_expert] = -1e9
    top_val, idx = torch.topk(logits, k, dim=-1)
    weights = torch.softmax(top_val, dim=-1).to(torch.bfloat16).to(torch.float32)
    dout = rnd(T, H)
    out = [hidden, idx, weights, w1, b1, w2, b2, dout]
    return [t.to(device) if t.dtype == torch.int64 else t.to(device=device, dtype=dtype) for t in out]


def apply_gate(gate_up: torch.Tensor) -> torch.Tensor:
    """modeling_gpt_oss.py:76-82."""
    gate, up = gate_up[..., ::2], gate_up[..., 1::2]
    gate = gate.clamp(min=None, max=GLU_LIMIT)
    up = up.clamp(min=-GLU_LIMIT, max=GLU_LIMIT)
    glu = gate * torch.sigmoid(gate * GLU_ALPHA)
    return (up + 1) * glu


def round_through(x: torch.Tensor, dtype) -> torch.Tensor:
    """x rounded to `dtype` (back in x's own dtype) with the identity as its derivative."""
    return x if dtype is None else x + (x.to(dtype).to(x.dtype) - x).detach()


def moe_experts_forward(hidden, idx, weights, w1, b1, w2, b2, preact_dtype=None):
    """modeling_gpt_oss.py:84-114: the loop over the experts, with an out-of-place ``index_add`` so that autograd
    can differentiate with respect to everything (fp32, so the order of the additions only moves the last bit).

    ``preact_dtype``: where the module runs in bf16 its pre-activation ``gate_up`` IS a bf16 tensor, and the gate's
    derivative is discontinuous at the clamps (7 and +-7): a value that fp32 puts at 7.01 and bf16 at 7.0 has its
    gradient switched on.  With wide pre-activations a few such elements per token move the max-norm of
    dhidden / dw1 by several per cent, whatever the implementation.  Passing ``torch.bfloat16`` rounds the
    pre-activation at that one place (identity derivative), which is the fair reference for a bf16 pipeline;
    the golden fixtures are plain fp32 (``None``)."""
    out = torch.zeros_like(hidden)
    for e in range(w1.shape[0]):
        token, choice = (idx == e).nonzero(as_tuple=True)                 # :103 `torch.where(expert_mask[e])`
        if token.numel() == 0:                                            # :93-97 only experts that were hit
            continue
        gate_up = hidden[token] @ w1[e] + b1[e]                           # :104-105
        gate_up = round_through(gate_up, preact_dtype)
        gated = apply_gate(gate_up)                                       # :106
        y = gated @ w2[e] + b2[e]                                         # :107
        out = out.index_add(0, token, y * weights[token, choice, None])   # :108-109
    return out


def moe_experts_fwd_bwd(hidden, idx, weights, w1, b1, w2, b2, dout, preact_dtype=None):
    """Output and the gradients of everything differentiable, in the dtype of the inputs."""
    leaves = [t.detach().clone().requires_grad_(True) for t in (hidden, weights, w1, b1, w2, b2)]
    h_, wt_, w1_, b1_, w2_, b2_ = leaves
    out = moe_experts_forward(h_, idx, wt_, w1_, b1_, w2_, b2_, preact_dtype)
    out.backward(dout)
    return {"out": out.detach(), "dhidden": h_.grad, "dweights": wt_.grad, "dw1": w1_.grad, "db1": b1_.grad,
            "dw2": w2_.grad, "db2": b2_.grad}
