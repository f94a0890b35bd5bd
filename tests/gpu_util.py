"""Helpers shared by the GPU parity tests (everything goes through the C ABI via the package)."""
import ctypes

import torch

from oracle import attention_fwd_bwd_blockwise, make_inputs, rel_err
from oregon_gpt_oss_patching_b200 import _cabi
from oregon_gpt_oss_patching_b200.attention_kernel import attention, last_status

# north-star tolerances: bf16 results vs the fp32 eager result, max|a-b|/max|b|
TOL_TENSOR = 2e-2   # O, dQ, dK, dV
TOL_DSINKS = 1e-2   # dSinks
TOL_LSE = 2e-3      # LSE is fp32 output computed from bf16 inputs


def run_b200(q, k, v, do, sinks, scale, window, seqlens=None):
    """q,k,v (B,H,S,d) and do (B,S,Hq,d): bf16 cuda tensors.  Returns dict of results (cuda)."""
    q = q.detach().requires_grad_(True)
    k = k.detach().requires_grad_(True)
    v = v.detach().requires_grad_(True)
    s = sinks.detach().clone().requires_grad_(True)
    sl = None if seqlens is None else torch.as_tensor(seqlens, dtype=torch.int32, device=q.device)
    o = attention(q, k, v, s, scale, window, sl)
    o.backward(do)
    return {"o": o.detach(), "dq": q.grad, "dk": k.grad, "dv": v.grad, "dsinks": s.grad}


def assert_close_valid(res, ref, lens, S, tol=TOL_TENSOR, tol_ds=TOL_DSINKS):
    """Compare on rows inside each sequence (padding rows: o and dq must be exactly zero)."""
    errs = {}
    for key in ("dk", "dv"):
        errs[key] = rel_err(res[key].float(), ref[key])
    errs["dsinks"] = rel_err(res["dsinks"].float(), ref["dsinks"])
    for key, kind in (("o", "bshd"), ("dq", "bhsd")):
        worst = 0.0
        denom = ref[key].abs().max().item()
        for b, L in enumerate(lens):
            got = res[key][b, :L] if kind == "bshd" else res[key][b, :, :L]
            want = ref[key][b, :L] if kind == "bshd" else ref[key][b, :, :L]
            worst = max(worst, (got.float().cpu().double() - want.cpu().double()).abs().max().item() / denom)
            pad = res[key][b, L:] if kind == "bshd" else res[key][b, :, L:]
            assert pad.numel() == 0 or float(pad.float().abs().max()) == 0.0, f"{key}: padding rows not zero"
        errs[key] = worst
    for key in ("o", "dq", "dk", "dv"):
        assert errs[key] < tol, (key, errs)
    assert errs["dsinks"] < tol_ds, errs
    assert not any(torch.isnan(res[k_].float()).any().item() for k_ in res), "NaN in results"
    return errs


def oracle_on_gpu(q, k, v, do, sinks, scale, window, seqlens=None, slices=None, row_block=2048):
    """fp32 blockwise oracle evaluated on the GPU (as the checker) on the bf16-rounded inputs."""
    return attention_fwd_bwd_blockwise(q.float(), k.float(), v.float(), sinks.float(), do.float(), scale, window,
                                       seqlens, dtype=torch.float32, row_block=row_block, slices=slices)
