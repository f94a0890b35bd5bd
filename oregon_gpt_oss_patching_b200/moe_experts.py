"""GPT-OSS mixture-of-experts block on B200, as a drop-in for Hugging Face's ``GptOssExperts.forward``.

The reference project trains the model with Hugging Face's expert block
(``transformers/models/gpt_oss/modeling_gpt_oss.py:84-114``): a Python loop over the experts that finds
each expert's tokens with ``torch.where`` (a host synchronisation per expert), gathers them, multiplies,
applies the gated activation through strided slices, multiplies again and scatter-adds with bf16 atomics.
Once attention is fast this loop is the largest part of a fine-tuning step.  Here the same arithmetic runs
as grouped GEMMs on the tensor cores over token rows sorted by expert, behind the C ABI of
``include/b200moe.h``:

    forward    rows sorted by expert -> X_s;  Y1 = X_s W1_e + b1_e and H = glu(Y1) from one launch;  Y2 = H W2_e + b2_e;
               out[t] = sum_j w[t, j] * Y2[row of (t, j)]
    backward   dW2_e = H_e^T dY2_e, dH = dY2 W2_e^T, dY1 = glu'(Y1) dH, dW1_e = X_e^T dY1_e, dX_s = dY1 W1_e^T,
               bias gradients as per-expert column sums, d w[t, j] = <d out[t], Y2[row of (t, j)]>

The routing bookkeeping (a stable sort of the (token, choice) pairs by expert, segment offsets rounded up
to 128 rows) is one more launch (``b200moe_route``; ``route`` states the same thing in torch tensor operations and
serves the CPU tests); nothing synchronises with the host.  There is no other code path: if the library is
missing or rejects a call an exception is raised.

Differences from the Hugging Face loop, all deliberate: sums over a token's experts and over an expert's
rows are taken in fp32 in a fixed order (bit-reproducible; ``index_add_`` is not), the gated activation is
evaluated in fp32 from the bf16 pre-activation, and an expert index equal to ``num_experts`` (the masking
index of expert-parallel runs) is not supported.
"""
from __future__ import annotations

import ctypes
from typing import NamedTuple

import torch

from . import _cabi
from .attention_kernel import _status_word

__all__ = ["moe_experts", "b200_experts_forward", "patch_moe_experts", "unpatch_moe_experts", "route", "route_on_device", "padded_rows",
           "set_gemm_ctas"]


class Routing(NamedTuple):
    offsets: torch.Tensor     # int32 (E + 1): first row of each expert's segment, multiples of 128
    row_token: torch.Tensor   # int32 (rows): token of each sorted row, -1 for padding rows
    pos: torch.Tensor         # int32 (T, k): sorted row of each (token, choice)
    row_weight: torch.Tensor  # fp32 (rows): routing weight of each sorted row, 0 for padding rows
    rows: int


def padded_rows(pairs: int, num_experts: int) -> int:
    """Rows of the sorted buffer: enough for any routing of ``pairs`` (token, choice) pairs (no host sync needed)."""
    align = _cabi.MOE_ROW_ALIGN
    return (pairs + num_experts * (align - 1) + align - 1) // align * align


def route(router_indices: torch.Tensor, routing_weights: torch.Tensor, num_experts: int) -> Routing:
    """Sort the (token, choice) pairs by expert (stable: token order is kept inside an expert)."""
    T, k = router_indices.shape
    dev = router_indices.device
    align = _cabi.MOE_ROW_ALIGN
    flat = router_indices.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    # first sorted pair of each expert by binary search (bincount would synchronise, index_add_ uses atomics)
    first = torch.searchsorted(sorted_e, torch.arange(num_experts + 1, device=dev))
    counts = first[1:] - first[:-1]
    first = first[:-1]
    padded = (counts + (align - 1)) // align * align
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=dev)
    offsets[1:] = torch.cumsum(padded, 0)
    dest = offsets[sorted_e] + (torch.arange(T * k, device=dev) - first[sorted_e])
    rows = padded_rows(T * k, num_experts)
    row_token = torch.full((rows,), -1, dtype=torch.int32, device=dev)
    row_token[dest] = (order // k).to(torch.int32)
    pos = torch.empty(T * k, dtype=torch.int32, device=dev)
    pos[order] = dest.to(torch.int32)
    row_weight = torch.zeros(rows, dtype=torch.float32, device=dev)
    row_weight[dest] = routing_weights.reshape(-1).to(torch.float32)[order]
    return Routing(offsets.to(torch.int32), row_token, pos.view(T, k), row_weight, rows)


ROUTE_KERNEL_MAX_EXPERTS = 256


def route_on_device(router_indices: torch.Tensor, weights_f32: torch.Tensor, num_experts: int) -> Routing:
    """The same bookkeeping as ``route`` in one launch of this library (``b200moe_route``): bit-identical outputs."""
    T, k = router_indices.shape
    dev = router_indices.device
    rows = padded_rows(T * k, num_experts)
    idx = router_indices.to(torch.int64).contiguous()
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    row_token = torch.empty(rows, dtype=torch.int32, device=dev)
    pos = torch.empty(T, k, dtype=torch.int32, device=dev)
    row_weight = torch.empty(rows, dtype=torch.float32, device=dev)
    rc = _cabi.load().b200moe_route(_ptr(idx), _ptr(weights_f32), T, k, num_experts, rows, _ptr(offsets), _ptr(row_token), _ptr(pos),
                                    _ptr(row_weight), dev.index, _stream(dev))
    _cabi.check(rc, "b200moe_route")
    return Routing(offsets, row_token, pos, row_weight, rows)


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


# Persistent CTAs of the grouped GEMM (0 = one per SM).  A data-parallel trainer whose gradient all-reduce runs beside
# the backward pass can leave the collective's SMs free: ``set_gemm_ctas(132)``.
_gemm_ctas = 0


def set_gemm_ctas(n: int) -> None:
    global _gemm_ctas
    _gemm_ctas = max(0, int(n))


def grouped_gemm(op: int, a, b, d, offsets, *, bias=None, glu_out=None, M=0, N=0, K=0) -> None:
    """One ``b200moe_grouped_gemm`` call on the current stream (see include/b200moe.h for the three forms)."""
    dev = a.device
    p = _cabi.MoeGemmParams(op=op, num_groups=offsets.numel() - 1, rows=a.shape[0], M=M, N=N, K=K,
                            offsets=offsets.data_ptr(), a=a.data_ptr(), b=b.data_ptr(),
                            bias=None if bias is None else bias.data_ptr(), d=d.data_ptr(), device=dev.index,
                            stream=torch.cuda.current_stream(dev).cuda_stream, status=_status_word(dev).data_ptr(),
                            glu_out=None if glu_out is None else glu_out.data_ptr(), max_ctas=_gemm_ctas)
    _cabi.check(_cabi.load().b200moe_grouped_gemm(ctypes.byref(p)), "b200moe_grouped_gemm")


def _check(hidden, router_indices, routing_weights, w1, b1, w2, b2):
    if not hidden.is_cuda:
        raise RuntimeError("moe_experts needs CUDA tensors (the sm_100a library is the only code path)")
    for name, t in (("hidden_states", hidden), ("gate_up_proj", w1), ("gate_up_proj_bias", b1), ("down_proj", w2),
                    ("down_proj_bias", b2)):
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"moe_experts: {name} must be bfloat16, got {t.dtype}")
    E, H, I2 = w1.shape
    if w2.shape != (E, I2 // 2, H) or b1.shape != (E, I2) or b2.shape != (E, H) or hidden.shape[-1] != H:
        raise RuntimeError("moe_experts: parameter shapes do not match GptOssExperts")
    if H % 8 or (I2 // 2) % 8 or E > 256:
        raise RuntimeError("moe_experts: hidden and intermediate sizes must be multiples of 8, at most 256 experts")
    if router_indices.shape != routing_weights.shape or router_indices.shape[0] != hidden.shape[0]:
        raise RuntimeError("moe_experts: router_indices / routing_weights must be (tokens, top_k)")


class _moe_experts(torch.autograd.Function):
    """out = GptOssExperts.forward(hidden, router_indices, routing_weights) with the module's four parameters."""

    @staticmethod
    def forward(ctx, hidden, router_indices, routing_weights, w1, b1, w2, b2):
        _check(hidden, router_indices, routing_weights, w1, b1, w2, b2)
        lib = _cabi.load()
        dev = hidden.device
        hidden = hidden.contiguous()
        w1, b1, w2, b2 = w1.contiguous(), b1.contiguous(), w2.contiguous(), b2.contiguous()
        T, H = hidden.shape
        E, _, I2 = w1.shape
        I = I2 // 2
        k = router_indices.shape[1]
        weights = routing_weights.to(torch.float32).contiguous()
        r = (route_on_device(router_indices, weights, E) if E <= ROUTE_KERNEL_MAX_EXPERTS
             else route(router_indices, routing_weights, E))
        rows, di, st = r.rows, dev.index, _stream(dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        xs = torch.empty(rows, H, **bf)
        _cabi.check(lib.b200moe_gather_rows(_ptr(hidden), _ptr(r.row_token), None, _ptr(xs), rows, H, di, st), "b200moe_gather_rows")
        y1 = torch.empty(rows, I2, **bf)
        h = torch.empty(rows, I, **bf)
        if I2 % 16 == 0:   # the gated activation leaves the first GEMM's epilogue (rows past the last expert stay unwritten, and unread)
            grouped_gemm(_cabi.MOE_ROWS_NN, xs, w1, y1, r.offsets, bias=b1, glu_out=h, N=I2, K=H)
        else:
            grouped_gemm(_cabi.MOE_ROWS_NN, xs, w1, y1, r.offsets, bias=b1, N=I2, K=H)
            _cabi.check(lib.b200moe_glu(_ptr(y1), _ptr(h), rows, I, di, st), "b200moe_glu")
        y2 = torch.empty(rows, H, **bf)
        grouped_gemm(_cabi.MOE_ROWS_NN, h, w2, y2, r.offsets, bias=b2, N=H, K=I)
        out = torch.empty(T, H, **bf)
        _cabi.check(lib.b200moe_combine_rows(_ptr(y2), _ptr(r.pos), _ptr(weights), _ptr(out), T, k, H, di, st), "b200moe_combine_rows")
        ctx.save_for_backward(xs, y1, h, y2, w1, w2, r.offsets, r.row_token, r.pos, r.row_weight)
        ctx.weights_dtype = routing_weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        xs, y1, h, y2, w1, w2, offsets, row_token, pos, row_weight = ctx.saved_tensors
        lib = _cabi.load()
        dev = dout.device
        dout = dout.contiguous()
        T, H = dout.shape
        E, _, I2 = w1.shape
        I = I2 // 2
        k = pos.shape[1]
        rows, di, st = xs.shape[0], dev.index, _stream(dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        d_weights = torch.empty(T, k, dtype=torch.float32, device=dev)
        _cabi.check(lib.b200moe_row_dot(_ptr(dout), _ptr(y2), _ptr(pos), _ptr(d_weights), T, k, H, di, st), "b200moe_row_dot")
        dy2 = torch.empty(rows, H, **bf)
        _cabi.check(lib.b200moe_gather_rows(_ptr(dout), _ptr(row_token), _ptr(row_weight), _ptr(dy2), rows, H, di, st), "b200moe_gather_rows")
        db2 = torch.empty(E, H, **bf)
        _cabi.check(lib.b200moe_bias_grad(_ptr(dy2), _ptr(offsets), _ptr(db2), E, H, di, st), "b200moe_bias_grad")
        dw2 = torch.empty(E, I, H, **bf)
        grouped_gemm(_cabi.MOE_INNER_TN, h, dy2, dw2, offsets, M=I, N=H)
        dh = torch.empty(rows, I, **bf)
        grouped_gemm(_cabi.MOE_ROWS_NT, dy2, w2, dh, offsets, N=I, K=H)
        dy1 = torch.empty(rows, I2, **bf)
        _cabi.check(lib.b200moe_glu_bwd(_ptr(y1), _ptr(dh), _ptr(dy1), rows, I, di, st), "b200moe_glu_bwd")
        db1 = torch.empty(E, I2, **bf)
        _cabi.check(lib.b200moe_bias_grad(_ptr(dy1), _ptr(offsets), _ptr(db1), E, I2, di, st), "b200moe_bias_grad")
        dw1 = torch.empty(E, H, I2, **bf)
        grouped_gemm(_cabi.MOE_INNER_TN, xs, dy1, dw1, offsets, M=H, N=I2)
        dxs = torch.empty(rows, H, **bf)
        grouped_gemm(_cabi.MOE_ROWS_NT, dy1, w1, dxs, offsets, N=H, K=I2)
        dhidden = torch.empty(T, H, **bf)
        _cabi.check(lib.b200moe_combine_rows(_ptr(dxs), _ptr(pos), None, _ptr(dhidden), T, k, H, di, st), "b200moe_combine_rows")
        return dhidden, None, d_weights.to(ctx.weights_dtype), dw1, db1, dw2, db2


moe_experts = _moe_experts.apply


def b200_experts_forward(self, hidden_states: torch.Tensor, router_indices=None, routing_weights=None) -> torch.Tensor:
    """Same signature and result as ``GptOssExperts.forward`` (modeling_gpt_oss.py:84-114)."""
    shape = hidden_states.shape
    out = moe_experts(hidden_states.reshape(-1, shape[-1]), router_indices, routing_weights, self.gate_up_proj,
                      self.gate_up_proj_bias, self.down_proj, self.down_proj_bias)
    return out.view(shape)


_original_experts_forward = None


def patch_moe_experts():
    """Route every ``GptOssExperts`` through the grouped-GEMM path (``unpatch_moe_experts`` restores the original)."""
    global _original_experts_forward
    from transformers.models.gpt_oss import modeling_gpt_oss
    if _original_experts_forward is None:
        _original_experts_forward = modeling_gpt_oss.GptOssExperts.forward
    modeling_gpt_oss.GptOssExperts.forward = b200_experts_forward


def unpatch_moe_experts():
    from transformers.models.gpt_oss import modeling_gpt_oss
    if _original_experts_forward is not None:
        modeling_gpt_oss.GptOssExperts.forward = _original_experts_forward
