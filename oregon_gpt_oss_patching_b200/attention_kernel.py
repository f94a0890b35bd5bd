"""GPT-OSS attention forward/backward on B200, as a drop-in for the reference's callable.

Mirrors the reference's ``attention_kernel.py``: an ``_attention`` autograd function
(reference ``attention_kernel.py:220-344``), ``attention = _attention.apply`` (``:347``) and
the HF-compatible adapter (``triton_flash_attention``, ``:348-358``; exported here under the
same name and as ``b200_flash_attention``).  The device work is done by the hand-written
sm_100a kernels behind the C ABI of ``libb200attn.so``; this module only prepares tensor
views, allocates outputs with torch and passes raw pointers.  There is no other code path:
if the library is missing or rejects the call, an exception is raised.

Differences from the reference, all deliberate:

* ``attention_mask`` is honoured (the reference ignores it, ``attention_kernel.py:353-358``):
  ``None``, a 2-D (B,S) keep-mask or HF's 4-D additive mask are reduced to per-sequence valid
  lengths, which assumes right padding.  Rows past a sequence's length produce zeros and
  receive/contribute no gradient.  With ``None`` the behaviour is exactly the reference's.
* q/k/v are consumed with whatever outer strides they have (no pad / contiguous copies,
  reference ``:233-239``); the output is written directly in (B,S,Hq,d) (no transpose copy,
  ``:272``) and dO is read in that layout (no copy, ``:290-292``).
* dK/dV are accumulated in fp32 with a single writer per element and dSinks is reduced in a
  fixed order, so results are deterministic (the reference uses global atomics, ``:176``,
  ``:201-212``).
* only bf16 tensors and head_dim 64 (the GPT-OSS configuration) are supported.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _cabi

__all__ = ["attention", "attention_varlen", "b200_flash_attention", "triton_flash_attention", "seqlens_from_mask",
           "last_status", "check_status"]

_status_words: dict = {}


def _status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that kernels OR an error bit into when a bounded wait gave up."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def last_status(device=None) -> int:
    """Synchronise and return the device status word.

    0 = nothing went wrong so far; bit ``_cabi.STATUS_WAIT_TIMEOUT`` = a kernel gave up a bounded
    wait; bit ``_cabi.STATUS_NONPREFIX_MASK`` = a padding mask that is not right-padded was passed.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(_status_word(device).item())


def check_status(device=None) -> None:
    """Synchronise and raise ``RuntimeError`` if the device status word is non-zero (then clear it)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    code = last_status(device)
    if code == 0:
        return
    _status_word(device).zero_()
    what = []
    if code & _cabi.STATUS_WAIT_TIMEOUT:
        what.append("a kernel abandoned a bounded wait")
    if code & _cabi.STATUS_NONPREFIX_MASK:
        what.append("an attention mask was not right-padded (a real token follows a padding token): "
                    "only prefix masks can be reduced to sequence lengths")
    raise RuntimeError(f"b200attn status {code}: " + "; ".join(what or ["unknown status bits"]))


def _as_view(t: torch.Tensor) -> torch.Tensor:
    """Return ``t`` if the kernels can address it in place, else a contiguous copy."""
    st = t.stride()
    ok = st[-1] == 1 and t.data_ptr() % 16 == 0 and all(
        (s % 8 == 0 and s >= 0) or n == 1 for s, n in zip(st[:-1], t.shape[:-1]))
    ok = ok and all(s > 0 or n == 1 for s, n in zip(st[:-1], t.shape[:-1]))
    return t if ok else t.contiguous()


def seqlens_from_mask(attention_mask: Optional[torch.Tensor], B: int, S: int) -> Optional[torch.Tensor]:
    """Valid length of each right-padded sequence as an int32 device tensor, or None.

    Accepts a (B,S) keep-mask (bool or 0/1) or HF's additive (B,1,S,S) mask, where position i
    is a real token iff it may attend to itself (mask[b,0,i,i] == 0).  No host synchronisation:
    a mask that is NOT right-padded (left padding, packed documents -- a real token after a
    padding token) cannot be expressed as a length; it is detected on the device and reported
    through the status word (``_cabi.STATUS_NONPREFIX_MASK``), which ``check_status`` /
    ``B200ATTN_CHECK_STATUS=1`` turn into an exception.
    """
    if attention_mask is None:
        return None
    m = attention_mask
    if m.dim() == 2:
        keep = m if m.dtype == torch.bool else m != 0
    elif m.dim() == 4:
        diag = torch.diagonal(m[:, 0], dim1=-2, dim2=-1)
        keep = diag if m.dtype == torch.bool else diag == 0
    else:
        raise ValueError(f"attention_mask must be 2-D or 4-D, got shape {tuple(m.shape)}")
    if keep.shape[0] != B or keep.shape[-1] != S:
        raise ValueError(f"attention_mask shape {tuple(attention_mask.shape)} does not match B={B}, S={S}")
    if keep.is_cuda and S > 1:
        bad = (keep[:, 1:] & ~keep[:, :-1]).any()
        _status_word(keep.device).bitwise_or_(bad.to(torch.int32) * _cabi.STATUS_NONPREFIX_MASK)
    return keep.sum(dim=-1, dtype=torch.int32).contiguous()


def _params(q, k, v, o, lse, sinks_f32, scale, window, seqlens) -> _cabi.Params:
    B, Hq, S, d = q.shape
    p = _cabi.Params()
    p.B, p.Hq, p.Hkv, p.S, p.d = B, Hq, k.shape[1], S, d
    p.window = int(window)
    p.scale = float(scale)
    p.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    p.stream = torch.cuda.current_stream(q.device).cuda_stream
    p.status = _status_word(q.device).data_ptr()
    p.seqlens = seqlens.data_ptr() if seqlens is not None else None
    p.sinks = sinks_f32.data_ptr()
    p.q, p.k, p.v = _cabi.tensor4(q, "bhsd"), _cabi.tensor4(k, "bhsd"), _cabi.tensor4(v, "bhsd")
    p.o = _cabi.tensor4(o, "bshd")
    p.lse = lse.data_ptr()
    return p


def _check_inputs(q, k, v, sinks):
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("b200 attention needs CUDA tensors (there is no CPU path)")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError(f"b200 attention supports bfloat16 q/k/v only, got {q.dtype}, {k.dtype}, {v.dtype}")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be (B, H, S, d)")
    B, Hq, S, d = q.shape
    if k.shape != v.shape or k.shape[0] != B or k.shape[2] != S or k.shape[3] != d:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    if sinks is None or sinks.numel() != Hq:
        raise ValueError("sinks must hold one logit per query head")


class _attention(torch.autograd.Function):
    """forward(q, k, v, sinks, sm_scale, bandwidth, seqlens) -> o (B,S,Hq,d).

    Same argument order as the reference's ``_attention.forward`` (``attention_kernel.py:222``)
    with its unused ``start_q`` slot carrying the per-sequence valid lengths instead.
    """

    @staticmethod
    def forward(ctx, q, k, v, sinks, sm_scale, bandwidth, seqlens):
        _check_inputs(q, k, v, sinks)
        lib = _cabi.load()
        q, k, v = _as_view(q), _as_view(k), _as_view(v)
        B, Hq, S, d = q.shape
        window = int(bandwidth) if bandwidth else 0
        o = torch.empty((B, S, Hq, d), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, _cabi.padded_len(S)), dtype=torch.float32, device=q.device)
        sinks_f32 = sinks.detach().to(torch.float32).contiguous()
        if seqlens is not None:
            seqlens = seqlens.to(device=q.device, dtype=torch.int32).contiguous()
        p = _params(q, k, v, o, lse, sinks_f32, sm_scale, window, seqlens)
        _cabi.check(lib.b200attn_fwd(ctypes.byref(p)), "b200attn_fwd")
        ctx.save_for_backward(q, k, v, sinks, o, lse, seqlens)
        ctx.sm_scale = float(sm_scale)
        ctx.window = window
        _maybe_check_status(q.device)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, sinks, o, lse, seqlens = ctx.saved_tensors
        lib = _cabi.load()
        do = _as_view(do if do.dtype == q.dtype else do.to(q.dtype))
        B, Hq, S, d = q.shape
        dq = torch.empty((B, Hq, S, d), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, k.shape[1], S, d), dtype=k.dtype, device=q.device)
        dv = torch.empty((B, k.shape[1], S, d), dtype=v.dtype, device=q.device)
        delta = torch.empty((_cabi.DELTA_PLANES,) + tuple(lse.shape), dtype=torch.float32, device=q.device)
        dsinks = torch.empty((Hq,), dtype=torch.float32, device=q.device)
        sinks_f32 = sinks.detach().to(torch.float32).contiguous()
        p = _params(q, k, v, o, lse, sinks_f32, ctx.sm_scale, ctx.window, seqlens)
        p.d_o = _cabi.tensor4(do, "bshd")
        p.dq, p.dk, p.dv = _cabi.tensor4(dq, "bhsd"), _cabi.tensor4(dk, "bhsd"), _cabi.tensor4(dv, "bhsd")
        p.delta = delta.data_ptr()
        p.dsinks = dsinks.data_ptr()
        partial = torch.empty((int(lib.b200attn_dsinks_scratch_floats(ctypes.byref(p))),), dtype=torch.float32,
                              device=q.device)
        p.dsinks_partial = partial.data_ptr()
        _cabi.check(lib.b200attn_bwd(ctypes.byref(p)), "b200attn_bwd")
        _maybe_check_status(q.device)
        return dq, dk, dv, dsinks.to(sinks.dtype), None, None, None


def _maybe_check_status(device) -> None:
    # Opt-in (it synchronises): turn a device-side give-up into an exception right away.
    if os.environ.get("B200ATTN_CHECK_STATUS") == "1":
        check_status(device)


attention = _attention.apply


def _doc_bounds(cu_seqlens, total: int) -> list:
    """Document boundaries as a validated list of Python ints (a device tensor is read back once)."""
    bounds = [int(x) for x in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
    if len(bounds) < 2 or bounds[0] != 0 or bounds[-1] != total or any(b1 < b0 for b0, b1 in zip(bounds, bounds[1:])):
        raise ValueError(f"cu_seqlens must rise from 0 to the packed length {total}, got {bounds}")
    return bounds


class _attention_varlen(torch.autograd.Function):
    """forward(q, k, v, sinks, sm_scale, bandwidth, cu_seqlens) -> o (1,T,Hq,d) for packed documents.

    q (1,Hq,T,d) and k, v (1,Hkv,T,d) hold several documents back to back along the position axis;
    ``cu_seqlens`` (n_docs+1 ascending offsets, 0 first and T last: the convention of the varlen
    flash-attention interfaces HF passes as ``cu_seq_lens_q``) says where each starts.  A token attends
    only inside its own document (causal, sliding window and sink as in ``attention``).  The reference
    has no such entry (it ignores masks and position ids, ``attention_kernel.py:353-358``, so packed
    documents attend to each other there).

    Every document is one call of the same kernels on views of the packed tensors -- a document's rows
    are contiguous along the position axis whatever the outer strides, and the tensor maps of a call
    end at the document's last row, so loads past it read zeros and stores are clipped; nothing is
    copied or padded.  dSinks is the sum of the documents' contributions, added in document order.
    """

    @staticmethod
    def forward(ctx, q, k, v, sinks, sm_scale, bandwidth, cu_seqlens):
        _check_inputs(q, k, v, sinks)
        if q.shape[0] != 1:
            raise ValueError("packed documents come as one row: q (1,Hq,T,d), k/v (1,Hkv,T,d)")
        lib = _cabi.load()
        q, k, v = _as_view(q), _as_view(k), _as_view(v)
        _, Hq, T, d = q.shape
        bounds = _doc_bounds(cu_seqlens, T)
        window = int(bandwidth) if bandwidth else 0
        o = torch.empty((1, T, Hq, d), dtype=q.dtype, device=q.device)
        docs = [(a, b) for a, b in zip(bounds, bounds[1:]) if b > a]
        pads = [_cabi.padded_len(b - a) for a, b in docs]
        lse = torch.empty((Hq * sum(pads),), dtype=torch.float32, device=q.device)
        sinks_f32 = sinks.detach().to(torch.float32).contiguous()
        off = 0
        for (a, b), pad in zip(docs, pads):
            p = _params(q[:, :, a:b], k[:, :, a:b], v[:, :, a:b], o[:, a:b], lse[off:off + Hq * pad], sinks_f32,
                        sm_scale, window, None)
            _cabi.check(lib.b200attn_fwd(ctypes.byref(p)), "b200attn_fwd")
            off += Hq * pad
        ctx.save_for_backward(q, k, v, sinks, o, lse)
        ctx.sm_scale, ctx.window, ctx.docs, ctx.pads = float(sm_scale), window, docs, pads
        _maybe_check_status(q.device)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, sinks, o, lse = ctx.saved_tensors
        lib = _cabi.load()
        do = _as_view(do if do.dtype == q.dtype else do.to(q.dtype))
        _, Hq, T, d = q.shape
        Hkv = k.shape[1]
        dq = torch.empty((1, Hq, T, d), dtype=q.dtype, device=q.device)
        dk = torch.empty((1, Hkv, T, d), dtype=k.dtype, device=q.device)
        dv = torch.empty((1, Hkv, T, d), dtype=v.dtype, device=q.device)
        sinks_f32 = sinks.detach().to(torch.float32).contiguous()
        dsinks = torch.zeros((max(len(ctx.docs), 1), Hq), dtype=torch.float32, device=q.device)
        delta = torch.empty((_cabi.DELTA_PLANES * Hq * max(ctx.pads, default=0),), dtype=torch.float32, device=q.device)
        partial = None
        off = 0
        for i, ((a, b), pad) in enumerate(zip(ctx.docs, ctx.pads)):
            p = _params(q[:, :, a:b], k[:, :, a:b], v[:, :, a:b], o[:, a:b], lse[off:off + Hq * pad], sinks_f32,
                        ctx.sm_scale, ctx.window, None)
            p.d_o = _cabi.tensor4(do[:, a:b], "bshd")
            p.dq, p.dk, p.dv = (_cabi.tensor4(t[:, :, a:b], "bhsd") for t in (dq, dk, dv))
            p.delta = delta.data_ptr()          # scratch of one document at a time: calls run in stream order
            p.dsinks = dsinks[i].data_ptr()
            need = int(lib.b200attn_dsinks_scratch_floats(ctypes.byref(p)))
            if partial is None or partial.numel() < need:
                partial = torch.empty((need,), dtype=torch.float32, device=q.device)
            p.dsinks_partial = partial.data_ptr()
            _cabi.check(lib.b200attn_bwd(ctypes.byref(p)), "b200attn_bwd")
            off += Hq * pad
        _maybe_check_status(q.device)
        return dq, dk, dv, dsinks.sum(dim=0).to(sinks.dtype), None, None, None


attention_varlen = _attention_varlen.apply


def b200_flash_attention(
    module,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    scaling: float,
    dropout: float = 0.0,
    **kwargs,
):
    """Replacement for ``modeling_gpt_oss.eager_attention_forward`` (same signature and return).

    Reads ``module.sinks`` and ``module.sliding_window`` like the reference adapter
    (``attention_kernel.py:348-358``); ``dropout`` and the extra keyword arguments HF passes
    (``sliding_window``, ``s_aux``, ``position_ids`` ...) are ignored as they are there, except
    ``cu_seq_lens_q``: with batch 1 and more than one document it selects ``attention_varlen``.
    Returns ``(attn_output (B,S,Hq,d), None)``.
    """
    B, _, S, _ = query.shape
    cu = kwargs.get("cu_seq_lens_q")
    if cu is not None and B == 1 and len(cu) > 2:       # HF's padding-free collation: documents packed in one row
        return attention_varlen(query, key, value, module.sinks, scaling, module.sliding_window, cu), None
    seqlens = seqlens_from_mask(attention_mask, B, S)
    return attention(query, key, value, module.sinks, scaling, module.sliding_window, seqlens), None


# the reference's public name, so that `from attention_kernel import triton_flash_attention` ports 1:1
triton_flash_attention = b200_flash_attention
