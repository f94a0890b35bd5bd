"""Mixture-of-experts block on the CPU: the fp32 restatement against the fixtures the unmodified Hugging Face
module produced, and the routing bookkeeping of the product path (pure tensor operations, no GPU needed)."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle.moe_fp32 import MOE_CASES, MoeCase, apply_gate, make_moe_inputs, moe_experts_fwd_bwd
from oregon_gpt_oss_patching_b200.moe_experts import padded_rows, route

TOL = 2e-6   # fp32 restatement vs fp32 module: summation-order differences only


@pytest.mark.parametrize("name", list(MOE_CASES))
def test_restatement_matches_the_hugging_face_module(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    res = moe_experts_fwd_bwd(*make_moe_inputs(MOE_CASES[name]))
    for key, val in res.items():
        ref = torch.from_numpy(z[key])
        assert val.shape == ref.shape, key
        assert float((val - ref).abs().max() / ref.abs().max()) < TOL, key


def test_unused_expert_gets_zero_gradients():
    case = MOE_CASES["moe_ragged"]
    res = moe_experts_fwd_bwd(*make_moe_inputs(case))
    e = case.unused_expert
    for key in ("dw1", "db1", "dw2", "db2"):
        assert float(res[key][e].abs().max()) == 0.0


def test_gate_clamps_are_exercised_by_the_fixtures():
    hidden, idx, weights, w1, b1, w2, b2, dout = make_moe_inputs(MOE_CASES["moe_small"])
    gate_up = torch.einsum("th,thn->tn", hidden, w1[idx[:, 0]]) + b1[idx[:, 0]]
    assert float(gate_up[..., ::2].max()) > 7.0 and float(gate_up[..., 1::2].abs().max()) > 7.0
    assert torch.isfinite(apply_gate(gate_up)).all()


@pytest.mark.parametrize("tokens,top_k,experts", [(48, 2, 4), (70, 3, 5), (1, 4, 32), (300, 4, 8)])
def test_routing_bookkeeping(tokens, top_k, experts):
    g = torch.Generator().manual_seed(tokens)
    logits = torch.randn(tokens, experts, generator=g)
    if experts > 4:
        logits[:, 1] = -1e9                                   # an expert nobody is routed to
    val, idx = torch.topk(logits, top_k, dim=-1)
    weights = torch.softmax(val, -1)
    r = route(idx, weights, experts)
    off = r.offsets.tolist()
    assert r.rows == padded_rows(tokens * top_k, experts) and r.rows % 128 == 0 and off[-1] <= r.rows
    assert off[0] == 0 and all(o % 128 == 0 for o in off) and all(b >= a for a, b in zip(off, off[1:]))
    counts = torch.bincount(idx.reshape(-1), minlength=experts).tolist()
    for e in range(experts):
        seg = r.row_token[off[e]:off[e + 1]]
        assert int((seg >= 0).sum()) == counts[e]
        assert bool((seg[:counts[e]] >= 0).all())             # real rows first, padding behind them
        assert seg[:counts[e]].tolist() == sorted(seg[:counts[e]].tolist())   # stable: token order kept
    assert bool((r.row_token[off[-1]:] == -1).all())
    # pos is the inverse map, and every sorted row carries its pair's weight
    for t in range(tokens):
        for j in range(top_k):
            row = int(r.pos[t, j])
            e = int(idx[t, j])
            assert off[e] <= row < off[e + 1] and int(r.row_token[row]) == t
            assert float(r.row_weight[row]) == float(weights[t, j])
    assert float(r.row_weight.sum()) == pytest.approx(float(weights.sum()), rel=1e-5)


def test_rounding_the_preactivation_moves_gradients_at_the_clamps():
    """Why the GPU tests at model-like widths compare with ``preact_dtype=torch.bfloat16``: rounding that one tensor
    leaves the output within bf16 precision but switches gradient elements next to the clamps on or off."""
    case = MoeCase("wide", tokens=256, hidden=128, intermediate=192, experts=8, top_k=4, seed=5)
    inputs = make_moe_inputs(case)
    plain = moe_experts_fwd_bwd(*inputs)
    rounded = moe_experts_fwd_bwd(*inputs, preact_dtype=torch.bfloat16)
    err = {k: float((rounded[k] - plain[k]).abs().max() / plain[k].abs().max()) for k in plain}
    assert err["out"] < 1e-2 and err["dw2"] < 1e-2
    assert err["dw1"] > 2e-2          # far beyond rounding noise: whole elements flipped
