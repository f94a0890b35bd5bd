"""fp32 restatement of GPT-OSS eager attention (forward and backward).

TEST INFRASTRUCTURE ONLY -- see ``oracle/__init__.py``.

Two implementations of the same function:

``attention_fwd_bwd_dense``
    Follows ``transformers/models/gpt_oss/modeling_gpt_oss.py:245-273`` line by
    line (repeat K/V over the query-head group :254-255 via ``repeat_kv``
    :214-223, ``QK^T * scaling`` :256, additive mask :257-258, sink column
    concatenated :260-261, row max subtracted :266, softmax :267, sink column
    dropped :268, ``P V`` :270, transpose to (B,S,Hq,d) :271) and lets autograd
    produce the gradients, exactly as the reference's CPU path does.  It
    materialises the (B,Hq,S,S+1) logits, so it is for small S only.

``attention_fwd_bwd_blockwise``
    The closed-form backward of the same function, evaluated per (batch,
    KV-head group) slice and per block of query rows so that memory stays
    bounded at long S.  It is the formula the reference's flash kernel uses
    (``attention_kernel.py:53-98`` forward, ``:111-120`` delta,
    ``:173-176`` dSinks, ``:190-214`` dV/dP/dS/dK/dQ) but with every product in
    the tensor's own precision (fp32 or fp64) and no tiling approximations.

Mask semantics (identical in both):  key j is visible to query i of sequence b
iff ``j <= i`` (``masking_utils.py:78``), ``j > i - window`` when a window is
set (``masking_utils.py:96-97``; the reference kernel's ``too_old`` test,
``attention_kernel.py:71``) and ``j < seqlen[b]`` (right padding).  Rows
``i >= seqlen[b]`` are padding: their output is defined as zero and they take
no part in any gradient.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional, Sequence

import numpy as np
import torch

__all__ = [
    "AttnCase", "CONFIGS", "attention_fwd_bwd_dense", "attention_fwd_bwd_blockwise",
    "visible_mask", "make_inputs", "rel_err", "visible_pairs", "algorithmic_flops",
    "algorithmic_bytes",
]


# --------------------------------------------------------------------------------------
# workload descriptions
# --------------------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class AttnCase:
    """One attention workload: shapes, mask and input distribution."""
    name: str
    B: int
    S: int
    Hq: int = 64
    Hkv: int = 8
    d: int = 64
    window: int = 0            # 0 = full causal
    input_scale: float = 1.0   # Q,K,V,dO ~ input_scale * N(0,1)
    seqlens: Optional[tuple] = None  # right-padded lengths, None = all S
    seed: int = 0

    @property
    def scale(self) -> float:
        return 1.0 / math.sqrt(self.d)

    def lengths(self) -> list:
        return list(self.seqlens) if self.seqlens is not None else [self.S] * self.B


def _padded_lengths(seed: int = 0, n: int = 8, lo: int = 1024, hi: int = 16384) -> tuple:
    return tuple(int(x) for x in np.random.default_rng(seed).integers(lo, hi + 1, n))


# The benchmark configurations.  "cfg3_full" is the full-causal layer at the
# same S=16K shape as the sliding-window one.
CONFIGS = {
    "cfg1": AttnCase("cfg1", B=1, S=512, window=128),
    "cfg2": AttnCase("cfg2", B=4, S=4096, window=0, input_scale=0.5),
    "cfg3": AttnCase("cfg3", B=2, S=16384, window=128),
    "cfg3_full": AttnCase("cfg3_full", B=2, S=16384, window=0),
    "cfg4_swa": AttnCase("cfg4_swa", B=8, S=16384, window=128, seqlens=_padded_lengths()),
    "cfg4_full": AttnCase("cfg4_full", B=8, S=16384, window=0, seqlens=_padded_lengths()),
}


def make_inputs(case: AttnCase, dtype=torch.float32, device="cpu", zero_pad_do: bool = True):
    """Seeded synthetic inputs for ``case``.

    Values are drawn in fp32 on the CPU with a ``torch.Generator`` (so they do
    not depend on the device) and then cast/moved.  Layouts follow what the
    attention module receives: q (B,Hq,S,d), k,v (B,Hkv,S,d), dO (B,S,Hq,d),
    sinks (Hq,).  Rows of dO at padded positions are zeroed, because a loss that
    ignores padding sends no gradient there.
    """
    g = torch.Generator(device="cpu").manual_seed(case.seed)
    B, S, Hq, Hkv, d = case.B, case.S, case.Hq, case.Hkv, case.d
    q = torch.randn(B, Hq, S, d, generator=g) * case.input_scale
    k = torch.randn(B, Hkv, S, d, generator=g) * case.input_scale
    v = torch.randn(B, Hkv, S, d, generator=g) * case.input_scale
    do = torch.randn(B, S, Hq, d, generator=g) * case.input_scale
    sinks = torch.randn(Hq, generator=g)
    if zero_pad_do and case.seqlens is not None:
        for b, L in enumerate(case.seqlens):
            do[b, L:] = 0
    out = [t.to(dtype).to(device) for t in (q, k, v, do)]
    return (*out, sinks.to(device))


# --------------------------------------------------------------------------------------
# masks and work counts
# --------------------------------------------------------------------------------------
def visible_mask(S: int, window: int, seqlen: Optional[int] = None, device="cpu",
                 row0: int = 0, rows: Optional[int] = None) -> torch.Tensor:
    """Boolean (rows, S) matrix, True where query ``row0+r`` may attend to key j."""
    rows = S - row0 if rows is None else rows
    i = torch.arange(row0, row0 + rows, device=device)[:, None]
    j = torch.arange(S, device=device)[None, :]
    m = j <= i
    if window:
        m = m & (j > i - window)
    if seqlen is not None:
        m = m & (j < seqlen) & (i < seqlen)
    return m


def visible_pairs(L: int, window: int) -> int:
    """Number of (query, key) pairs that are not masked for one head of length L."""
    if not window or L <= window:
        return L * (L + 1) // 2
    return window * L - window * (window - 1) // 2


def algorithmic_flops(case: AttnCase) -> dict:
    """Matmul flops on visible pairs only: 2 products forward, 5 backward."""
    pairs = sum(visible_pairs(L, case.window) for L in case.lengths())
    fwd = 4 * case.d * case.Hq * pairs
    bwd = 10 * case.d * case.Hq * pairs
    return {"fwd": fwd, "bwd": bwd, "total": fwd + bwd, "pairs_per_head": pairs}


def algorithmic_bytes(case: AttnCase, elt: int = 2) -> dict:
    """Every operand and result once at padded size (bf16 tensors, fp32 LSE/delta)."""
    qb = case.B * case.Hq * case.S * case.d * elt
    kb = case.B * case.Hkv * case.S * case.d * elt
    row = case.B * case.Hq * case.S * 4
    fwd = qb + 2 * kb + qb + row                      # R Q,K,V ; W O,LSE
    bwd = (qb + 2 * kb + qb + qb + row) + (qb + 2 * kb)  # R Q,K,V,O,dO,LSE ; W dQ,dK,dV
    return {"fwd": fwd, "bwd": bwd, "total": fwd + bwd,
            "delta": 2 * qb + row, "dsinks": 2 * row}


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / max|b| -- the error measure used for every tolerance in the tests."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    denom = b.abs().max().item()
    return (a - b).abs().max().item() / (denom if denom > 0 else 1.0)


# --------------------------------------------------------------------------------------
# dense restatement of transformers' eager_attention_forward (+ autograd backward)
# --------------------------------------------------------------------------------------
def _repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    # modeling_gpt_oss.py:214-223
    B, H, S, d = x.shape
    if n_rep == 1:
        return x
    return x[:, :, None].expand(B, H, n_rep, S, d).reshape(B, H * n_rep, S, d)


def attention_fwd_bwd_dense(q, k, v, sinks, do, scale: float, window: int = 0,
                            seqlens: Optional[Sequence[int]] = None, dtype=torch.float32,
                            cu_seqlens: Optional[Sequence[int]] = None):
    """Eager attention and its autograd gradients on dense (S,S) logits.

    Returns ``dict(o, lse, dq, dk, dv, dsinks)``; o is (B,S,Hq,d); lse is the
    log of the softmax denominator including the sink term, (B,Hq,S).
    With ``cu_seqlens`` (ascending offsets, 0 first, S last) the rows hold documents packed back to
    back and a token sees only its own document: the causal / sliding-window mask AND-ed with
    "same document", which is what transformers builds for packed rows
    (``masking_utils.py``: ``packed_sequence_mask_function`` and-ed into the mask function).
    """
    q = q.detach().to(dtype).requires_grad_(True)
    k = k.detach().to(dtype).requires_grad_(True)
    v = v.detach().to(dtype).requires_grad_(True)
    sinks = sinks.detach().to(dtype).requires_grad_(True)
    do = do.detach().to(dtype)
    B, Hq, S, d = q.shape
    G = Hq // k.shape[1]
    neg = torch.finfo(dtype).min
    masks = []
    for b in range(B):
        L = None if seqlens is None else int(seqlens[b])
        masks.append(visible_mask(S, window, L, device=q.device))
    vis = torch.stack(masks)[:, None]                                   # (B,1,S,S)
    if cu_seqlens is not None:
        ends = torch.as_tensor([int(x) for x in cu_seqlens][1:], device=q.device)
        doc = torch.bucketize(torch.arange(S, device=q.device), ends, right=True)
        vis = vis & (doc[:, None] == doc[None, :])
    add_mask = torch.zeros(B, 1, S, S, dtype=dtype, device=q.device).masked_fill(~vis, neg)

    ks, vs = _repeat_kv(k, G), _repeat_kv(v, G)                         # :254-255
    logits = torch.matmul(q, ks.transpose(2, 3)) * scale + add_mask      # :256-258
    sink_col = sinks.reshape(1, -1, 1, 1).expand(B, -1, S, -1)          # :260
    comb = torch.cat([logits, sink_col], dim=-1)                        # :261
    comb = comb - comb.max(dim=-1, keepdim=True).values                 # :266
    probs = torch.softmax(comb, dim=-1, dtype=comb.dtype)               # :267
    scores = probs[..., :-1]                                            # :268
    o = torch.matmul(scores, vs).transpose(1, 2).contiguous()           # :270-271
    if seqlens is not None:                                             # padding rows -> 0
        rowvalid = torch.stack([torch.arange(S, device=q.device) < int(L) for L in seqlens])
        o = o * rowvalid[:, :, None, None].to(dtype)
    lse = torch.logsumexp(torch.cat([logits, sink_col], dim=-1), dim=-1)
    o.backward(do)
    return {"o": o.detach(), "lse": lse.detach(), "dq": q.grad, "dk": k.grad, "dv": v.grad,
            "dsinks": sinks.grad}


# --------------------------------------------------------------------------------------
# closed-form blockwise forward + backward (bounded memory)
# --------------------------------------------------------------------------------------
def attention_fwd_bwd_blockwise(q, k, v, sinks, do, scale: float, window: int = 0,
                                seqlens: Optional[Sequence[int]] = None, dtype=torch.float32,
                                row_block: int = 1024, slices: Optional[Sequence[tuple]] = None):
    """Same function as ``attention_fwd_bwd_dense`` without (S,S) storage.

    Works slice by slice over (batch b, KV head g) -- attention is independent
    across them, dK/dV sum over the G query heads of a group and dSinks sums
    over batch -- and over blocks of ``row_block`` query rows.  Only the keys a
    row block can see are touched.  ``slices`` restricts the work to a list of
    (b, g) pairs (the other entries of the results stay zero; dsinks then only
    holds those slices' contribution).
    """
    B, Hq, S, d = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    dev = q.device
    o = torch.zeros(B, S, Hq, d, dtype=dtype, device=dev)
    lse = torch.zeros(B, Hq, S, dtype=dtype, device=dev)
    dq = torch.zeros(B, Hq, S, d, dtype=dtype, device=dev)
    dk = torch.zeros(B, Hkv, S, d, dtype=dtype, device=dev)
    dv = torch.zeros(B, Hkv, S, d, dtype=dtype, device=dev)
    dsinks = torch.zeros(Hq, dtype=dtype, device=dev)
    todo = slices if slices is not None else [(b, g) for b in range(B) for g in range(Hkv)]
    for (b, g) in todo:
        L = S if seqlens is None else int(seqlens[b])
        hs = slice(g * G, (g + 1) * G)
        sink = sinks[hs].to(dtype)                                     # (G,)
        kg = k[b, g].to(dtype)
        vg = v[b, g].to(dtype)
        for r0 in range(0, L, row_block):
            r1 = min(r0 + row_block, L)
            c0 = max(0, r0 - window + 1) if window else 0
            c1 = r1
            qb = q[b, hs, r0:r1].to(dtype)                             # (G,R,d)
            dob = do[b, r0:r1, hs].to(dtype).transpose(0, 1)           # (G,R,d)
            kk, vv = kg[c0:c1], vg[c0:c1]                              # (C,d)
            s = torch.matmul(qb, kk.t()) * scale                       # (G,R,C)
            i = torch.arange(r0, r1, device=dev)[:, None]
            j = torch.arange(c0, c1, device=dev)[None, :]
            vis = j <= i
            if window:
                vis = vis & (j > i - window)
            s = s.masked_fill(~vis, float("-inf"))
            m = torch.maximum(s.max(dim=-1).values, sink[:, None])     # (G,R)
            p_un = torch.exp(s - m[..., None])
            z = p_un.sum(-1) + torch.exp(sink[:, None] - m)
            p = p_un / z[..., None]                                    # (G,R,C)
            ob = torch.matmul(p, vv)                                   # (G,R,d)
            o[b, r0:r1, hs] = ob.transpose(0, 1)
            lse[b, hs, r0:r1] = m + torch.log(z)
            # backward
            delta = (dob * ob).sum(-1)                                 # (G,R)
            p_sink = torch.exp(sink[:, None] - (m + torch.log(z)))
            dsinks[hs] += -(p_sink * delta).sum(-1)
            dv[b, g, c0:c1] += torch.matmul(p.transpose(1, 2), dob).sum(0)
            dp = torch.matmul(dob, vv.t())
            ds = p * (dp - delta[..., None])
            dq[b, hs, r0:r1] = torch.matmul(ds, kk) * scale
            dk[b, g, c0:c1] += torch.matmul(ds.transpose(1, 2), qb).sum(0) * scale
    return {"o": o, "lse": lse, "dq": dq, "dk": dk, "dv": dv, "dsinks": dsinks}
