"""Documents packed back to back in one row (`attention_varlen`, offsets in the `cu_seqlens` convention).

The reference has no such entry; the checker is the dense fp32 oracle with the same-document mask
transformers builds for packed rows.  Documents start at arbitrary (not tile-aligned) rows, include
one-token and empty documents, and the packed tensors are also passed as the strided views HF hands
over.  The results of a document must not depend on its neighbours: the packed call equals separate
calls bit for bit.
"""
import types

import pytest
import torch

from gpu_util import TOL_DSINKS, TOL_TENSOR, run_b200
from oracle import AttnCase, attention_fwd_bwd_dense, make_inputs, rel_err
from oregon_gpt_oss_patching_b200 import attention_varlen, triton_flash_attention
from oregon_gpt_oss_patching_b200.attention_kernel import last_status

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_varlen(q, k, v, do, sinks, scale, window, bounds):
    q = q.detach().requires_grad_(True)
    k = k.detach().requires_grad_(True)
    v = v.detach().requires_grad_(True)
    s = sinks.detach().clone().requires_grad_(True)
    o = attention_varlen(q, k, v, s, scale, window, bounds)
    o.backward(do)
    return {"o": o.detach(), "dq": q.grad, "dk": k.grad, "dv": v.grad, "dsinks": s.grad}


@pytest.mark.parametrize("window,Hq,Hkv", [(128, 16, 2), (0, 16, 2), (64, 8, 2), (128, 8, 8)])
def test_packed_documents_match_the_masked_dense_oracle(window, Hq, Hkv):
    bounds = [0, 1, 131, 131, 388, 452, 1000, 1017]       # lengths 1, 130, 0, 257, 64, 548, 17
    case = AttnCase("t", B=1, S=bounds[-1], Hq=Hq, Hkv=Hkv, window=window, seed=5)
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    res = _run_varlen(q, k, v, do, sinks, case.scale, window, torch.tensor(bounds, dtype=torch.int32, device=DEV))
    ref = attention_fwd_bwd_dense(q, k, v, sinks, do, case.scale, window, cu_seqlens=bounds)
    for key in ("o", "dq", "dk", "dv"):
        assert rel_err(res[key].float(), ref[key]) < TOL_TENSOR, (key, rel_err(res[key].float(), ref[key]))
    assert rel_err(res["dsinks"].float(), ref["dsinks"]) < TOL_DSINKS
    # and nothing leaks between neighbours: every document alone gives the same bits
    for a, b in zip(bounds, bounds[1:]):
        if b == a:
            continue
        one = run_b200(q[:, :, a:b].contiguous(), k[:, :, a:b].contiguous(), v[:, :, a:b].contiguous(),
                       do[:, a:b].contiguous(), sinks, case.scale, window)
        assert torch.equal(one["o"], res["o"][:, a:b]) and torch.equal(one["dq"], res["dq"][:, :, a:b])
        assert torch.equal(one["dk"], res["dk"][:, :, a:b]) and torch.equal(one["dv"], res["dv"][:, :, a:b])
    assert last_status(DEV) == 0


def test_adapter_takes_cu_seq_lens_and_strided_views():
    """HF's padding-free collation: batch 1, `cu_seq_lens_q` in the keyword arguments, q/k/v as transposed
    views of (1,T,H,d) projections."""
    bounds = [0, 300, 301, 700]
    case = AttnCase("t", B=1, S=700, Hq=16, Hkv=2, window=128, seed=6)
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    qv, kv, vv = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (q, k, v))      # (1,H,T,d) views of (1,T,H,d)
    module = types.SimpleNamespace(sinks=sinks.to(torch.bfloat16), sliding_window=128, num_key_value_groups=8, training=True)
    cu = torch.tensor(bounds, dtype=torch.int32, device=DEV)
    out, weights = triton_flash_attention(module, qv, kv, vv, None, scaling=case.scale, dropout=0.0,
                                          cu_seq_lens_q=cu, cu_seq_lens_k=cu, max_length_q=400, max_length_k=400)
    ref = attention_fwd_bwd_dense(q, k, v, module.sinks, do, case.scale, 128, cu_seqlens=bounds)
    assert weights is None and out.shape == (1, 700, 16, 64)
    assert rel_err(out.float(), ref["o"]) < TOL_TENSOR
    # without the offsets the same call is one long document, as in the reference
    whole, _ = triton_flash_attention(module, qv, kv, vv, None, scaling=case.scale, dropout=0.0)
    ref_whole = attention_fwd_bwd_dense(q, k, v, module.sinks, do, case.scale, 128)
    assert rel_err(whole.float(), ref_whole["o"]) < TOL_TENSOR
    assert not torch.equal(whole, out)


def test_bad_offsets_are_rejected():
    case = AttnCase("t", B=1, S=64, Hq=8, Hkv=1, seed=7)
    q, k, v, _, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    for bad in ([0, 70], [1, 64], [0, 40, 30, 64], [0]):
        with pytest.raises(ValueError):
            attention_varlen(q, k, v, sinks, case.scale, 0, bad)
    with pytest.raises(ValueError):
        attention_varlen(q.expand(2, -1, -1, -1), k.expand(2, -1, -1, -1), v.expand(2, -1, -1, -1), sinks, case.scale, 0, [0, 64])
