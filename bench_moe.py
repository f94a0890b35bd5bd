#!/usr/bin/env python
"""`bench.py --workload moe`: forward + backward of one GPT-OSS mixture-of-experts block on one B200.

Workload: the gpt-oss-20b layer (hidden 2880, intermediate 2880, 32 experts, 4 per token) on `--moe-tokens`
tokens (default 8192 = one sequence of the fine-tuning configuration), random bf16 weights, routing from
random logits (nearly balanced; stated because real routers are not).  A step is `moe_experts` forward and
backward: 15 launches of this library's kernels (6 grouped GEMMs -- the first forward one also writes the gated
activation -- 8 memory-bound ones and the routing kernel).

`value` counts the algorithmic FLOPs of the six matrix products over the real (token, choice) pairs,
2 * pairs * 3 * H * I each for forward, input gradient and weight gradient; `roofline` is the grouped GEMM
against the measured dense bf16 peak, from CUDA events around the six GEMM launches of every timed step;
`contenders` are Hugging Face's own two implementations of the block (the per-expert loop,
`experts_implementation="eager"`, and `torch._grouped_mm`, `"grouped_mm"`) on the same weights and inputs in
the same process; `cpu_baseline` is Hugging Face's loop in fp32 on the host cores on a bounded sample of tokens.
"""
from __future__ import annotations

import ctypes
import json
import time

import torch

H, I, E, TOPK = 2880, 2880, 32, 4


def _inputs(tokens, device, seed=0):
    g = torch.Generator().manual_seed(seed)
    w1 = (torch.randn(E, H, 2 * I, generator=g) * (2.0 / H ** 0.5)).to(torch.bfloat16)
    b1 = (torch.randn(E, 2 * I, generator=g) * 0.1).to(torch.bfloat16)
    w2 = (torch.randn(E, I, H, generator=g) * (1.0 / I ** 0.5)).to(torch.bfloat16)
    b2 = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16)
    hidden = torch.randn(tokens, H, generator=g).to(torch.bfloat16)
    dout = torch.randn(tokens, H, generator=g).to(torch.bfloat16)
    val, idx = torch.topk(torch.randn(tokens, E, generator=g), TOPK, dim=-1)
    weights = torch.softmax(val, -1).to(torch.bfloat16)
    return [t.to(device) for t in (hidden, idx, weights, w1, b1, w2, b2, dout)]


def block_flops(pairs: int) -> float:
    return 3.0 * 2.0 * pairs * (H * 2 * I + I * H)


def _hf_module(params, implementation, device, dtype):
    from transformers.models.gpt_oss.configuration_gpt_oss import GptOssConfig
    from transformers.models.gpt_oss.modeling_gpt_oss import GptOssExperts
    cfg = GptOssConfig(hidden_size=H, intermediate_size=I, num_local_experts=E, num_experts_per_tok=TOPK)
    cfg._experts_implementation = implementation
    with torch.device("meta"):
        mod = GptOssExperts(cfg)
    mod = mod.to_empty(device=device).to(dtype)
    w1, b1, w2, b2 = params
    with torch.no_grad():
        mod.gate_up_proj.copy_(w1)
        mod.gate_up_proj_bias.copy_(b1)
        mod.down_proj.copy_(w2)
        mod.down_proj_bias.copy_(b2)
    return mod


def _time(fn, steps, warm, stream):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(steps):
        fn()
    b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def run_moe(args, rank, world, local_rank):
    from bench import ClockSampler, load_peaks
    from oregon_gpt_oss_patching_b200 import _cabi, moe_experts as me
    from oregon_gpt_oss_patching_b200.attention_kernel import last_status

    if world > 1 and rank != 0:
        return   # one block on one GPU: the other ranks have nothing to add
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    stream = torch.cuda.current_stream(dev)
    peaks = load_peaks()
    tokens = args.moe_tokens
    hidden, idx, weights, w1, b1, w2, b2, dout = _inputs(tokens, dev)
    pairs = tokens * TOPK
    flops = block_flops(pairs)

    # ---- the six grouped GEMMs alone, for the roofline of the dominant kernel ----
    r = me.route(idx, weights, E)
    rows = r.rows
    bf = dict(dtype=torch.bfloat16, device=dev)
    xs, y1, hh, y2 = (torch.randn(rows, n, **bf) for n in (H, 2 * I, I, H))
    xs[r.row_token < 0] = 0
    y2[r.row_token < 0] = 0
    dw1, dw2 = torch.empty(E, H, 2 * I, **bf), torch.empty(E, I, H, **bf)
    y1b = torch.empty_like(y1)
    gemms = [
        ("fwd_gate_up", lambda: me.grouped_gemm(_cabi.MOE_ROWS_NN, xs, w1, y1, r.offsets, bias=b1, glu_out=hh, N=2 * I, K=H), H * 2 * I),
        ("fwd_down", lambda: me.grouped_gemm(_cabi.MOE_ROWS_NN, hh, w2, y2, r.offsets, bias=b2, N=H, K=I), I * H),
        ("dgrad_down", lambda: me.grouped_gemm(_cabi.MOE_ROWS_NT, y2, w2, hh, r.offsets, N=I, K=H), I * H),
        ("dgrad_gate_up", lambda: me.grouped_gemm(_cabi.MOE_ROWS_NT, y1, w1, xs, r.offsets, N=H, K=2 * I), H * 2 * I),
        ("wgrad_down", lambda: me.grouped_gemm(_cabi.MOE_INNER_TN, hh, y2, dw2, r.offsets, M=I, N=H), I * H),
        ("wgrad_gate_up", lambda: me.grouped_gemm(_cabi.MOE_INNER_TN, xs, y1, dw1, r.offsets, M=H, N=2 * I), H * 2 * I),
    ]

    if args.capture:   # profiler target
        for _ in range(args.warmup + args.steps):
            for _, fn, _ in gemms:
                fn()
        torch.cuda.synchronize()
        print(json.dumps({"capture": "moe", "passes": args.warmup + args.steps}))
        return

    leaves = [t.clone().requires_grad_(True) for t in (hidden, weights, w1, b1, w2, b2)]

    def step():
        for t in leaves:
            t.grad = None
        out = me.moe_experts(leaves[0], idx, leaves[1], leaves[2], leaves[3], leaves[4], leaves[5])
        out.backward(dout)
        return out

    steps, warm = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_step = _time(step, steps, warm, stream)
    gemm_ms = {name: _time(fn, steps, warm, stream) for name, fn, _ in gemms}
    clocks = sampler.stop()
    if last_status(dev) != 0:
        raise RuntimeError("a kernel abandoned a bounded wait (status word non-zero)")
    gemm_tflops = {name: 2.0 * pairs * mnk / (gemm_ms[name] * 1e-3) / 1e12 for name, _, mnk in gemms}
    total_gemm_ms = sum(gemm_ms.values())
    achieved = flops / (total_gemm_ms * 1e-3) / 1e12

    # ---- the memory-bound kernels alone, against the HBM peak (bytes = every operand and result once) ----
    lib = _cabi.load()
    st = ctypes.c_void_p(stream.cuda_stream)
    di = dev.index
    ptr = lambda t_: None if t_ is None else ctypes.c_void_p(t_.data_ptr())   # noqa: E731
    out_t, dots = torch.empty(tokens, H, **bf), torch.empty(tokens, TOPK, dtype=torch.float32, device=dev)
    db1, db2 = torch.empty(E, 2 * I, **bf), torch.empty(E, H, **bf)
    w32 = weights.float().contiguous()
    real = pairs   # rows that carry a (token, choice) pair; padding rows are written, not read
    aux = [
        ("gather_rows", lambda: lib.b200moe_gather_rows(ptr(hidden), ptr(r.row_token), None, ptr(xs), rows, H, di, st), 2 * (real + rows) * H),
        ("gather_rows_scaled", lambda: lib.b200moe_gather_rows(ptr(dout), ptr(r.row_token), ptr(r.row_weight), ptr(y2), rows, H, di, st), 2 * (real + rows) * H),
        ("glu_bwd", lambda: lib.b200moe_glu_bwd(ptr(y1), ptr(hh), ptr(y1b), rows, I, di, st), 2 * rows * 5 * I),
        ("combine_rows", lambda: lib.b200moe_combine_rows(ptr(y2), ptr(r.pos), ptr(w32), ptr(out_t), tokens, TOPK, H, di, st), 2 * (real + tokens) * H),
        ("row_dot", lambda: lib.b200moe_row_dot(ptr(dout), ptr(y2), ptr(r.pos), ptr(dots), tokens, TOPK, H, di, st), 2 * (real + tokens) * H),
        ("bias_grad_gate_up", lambda: lib.b200moe_bias_grad(ptr(y1), ptr(r.offsets), ptr(db1), E, 2 * I, di, st), 2 * rows * 2 * I),
        ("bias_grad_down", lambda: lib.b200moe_bias_grad(ptr(y2), ptr(r.offsets), ptr(db2), E, H, di, st), 2 * rows * H),
    ]
    aux_rec = {}
    for name, fn, nbytes in aux:
        ms = _time(fn, steps, warm, stream)
        aux_rec[name] = {"ms": round(ms, 4), "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1), "frac_of_hbm_peak": round(nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 3)}

    # ---- end to end: activations from pinned host memory, results back ----
    host_in = [hidden.cpu().pin_memory(), dout.cpu().pin_memory()]
    host_out = [torch.empty(tokens, H, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dev_hidden = torch.empty_like(hidden).requires_grad_(True)
    dev_dout = torch.empty_like(dout)

    def step_e2e():
        with torch.no_grad():
            dev_hidden.copy_(host_in[0], non_blocking=True)
        dev_dout.copy_(host_in[1], non_blocking=True)
        dev_hidden.grad = None
        for t in leaves[1:]:
            t.grad = None
        out = me.moe_experts(dev_hidden, idx, leaves[1], leaves[2], leaves[3], leaves[4], leaves[5])
        out.backward(dev_dout)
        host_out[0].copy_(out.detach(), non_blocking=True)
        host_out[1].copy_(dev_hidden.grad, non_blocking=True)

    ms_e2e = _time(step_e2e, steps, warm, stream)
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # ---- contenders: Hugging Face's own implementations on the same weights ----
    contenders = {}
    if not args.no_contender:
        for impl in ("grouped_mm", "eager"):
            try:
                mod = _hf_module((w1, b1, w2, b2), impl, dev, torch.bfloat16)
                h_in = hidden.clone().requires_grad_(True)
                w_in = weights.clone().requires_grad_(True)

                def hf_step():
                    for p_ in mod.parameters():
                        p_.grad = None
                    h_in.grad = None
                    w_in.grad = None
                    mod(h_in, idx, w_in).backward(dout)

                ms = _time(hf_step, max(3, steps // 4), 2, stream)
                contenders["hf_" + impl] = {"ms_per_step": round(ms, 3), "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
                                            "vs_b200": round(ms / ms_step, 3)}
                del mod
            except Exception as exc:   # noqa: BLE001
                contenders["hf_" + impl] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:120]}"}
            torch.cuda.empty_cache()

    line = {
        "metric": "moe_block_fwd_bwd_tflops", "value": round(flops / (ms_step * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": 1, "steps": steps, "warmup": warm, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"moe: one gpt-oss-20b expert block, {tokens} tokens, top-{TOPK} of {E} experts, hidden {H}, "
                               f"intermediate {I}; fwd+bwd", "tokens": tokens, "routing": "top-k of random logits (nearly balanced)",
                   "l2": "weights (1.6 GB) and activations larger than L2 (no flush)",
                   "flops": "3 * 2 * pairs * (H*2I + I*H)"},
        "tokens_per_s": round(tokens / (ms_step * 1e-3), 1),
        "clocks": clocks,
        "e2e": {"value": round(flops / (ms_e2e * 1e-3) / 1e12, 2), "unit": "TFLOP/s", "ms_per_step": round(ms_e2e, 3),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": 15 * steps,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": round(achieved / peaks["bf16_tflops"], 4), "kernel": "moe_grouped_gemm_kernel (six launches per step)",
                     "peak_source": peaks["source"], "traffic": None},
        "kernels": {name: {"ms": round(gemm_ms[name], 4), "tflops": round(gemm_tflops[name], 1)} for name, _, _ in gemms},
        "memory_bound_kernels": aux_rec,
        "other_ms_per_step": round(ms_step - total_gemm_ms, 4),
        "contenders": contenders,
    }
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_sample()
    print(json.dumps(line), flush=True)


def summary_record(device_index: int, tokens: int = 8192, steps: int = 10) -> dict:
    """A compact record of the expert block for the attention benchmark's N = 1 line: this library's forward + backward
    and transformers' default implementation (`torch._grouped_mm`) on the same weights and inputs."""
    from oregon_gpt_oss_patching_b200 import moe_experts as me
    dev = torch.device("cuda", device_index)
    stream = torch.cuda.current_stream(dev)
    hidden, idx, weights, w1, b1, w2, b2, dout = _inputs(tokens, dev)
    flops = block_flops(tokens * TOPK)
    leaves = [t.requires_grad_(True) for t in (hidden, weights, w1, b1, w2, b2)]

    def step():
        for t in leaves:
            t.grad = None
        me.moe_experts(leaves[0], idx, *leaves[1:]).backward(dout)

    ms = _time(step, steps, 3, stream)
    rec = {"workload": f"one gpt-oss-20b expert block, {tokens} tokens, top-{TOPK} of {E}, fwd+bwd (`bench.py --workload moe` has the full line)",
           "ms_per_step": round(ms, 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 1)}
    for t in leaves:
        t.grad = None
    try:
        mod = _hf_module((w1.detach(), b1.detach(), w2.detach(), b2.detach()), "grouped_mm", dev, torch.bfloat16)
        h_in, w_in = hidden.detach().clone().requires_grad_(True), weights.detach().clone().requires_grad_(True)

        def hf_step():
            for p_ in mod.parameters():
                p_.grad = None
            h_in.grad = None
            w_in.grad = None
            mod(h_in, idx, w_in).backward(dout)

        hf_ms = _time(hf_step, max(3, steps // 3), 2, stream)
        rec["hf_grouped_mm"] = {"ms_per_step": round(hf_ms, 3), "vs_b200": round(hf_ms / ms, 3)}
    except Exception as exc:   # noqa: BLE001
        rec["hf_grouped_mm"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:120]}"}
    return rec


def cpu_sample(tokens: int = 256) -> dict:
    """Hugging Face's per-expert loop (fp32) on the host cores: forward + backward of the same block on `tokens` tokens."""
    torch.set_num_threads(max(1, torch.get_num_threads()))
    hidden, idx, weights, w1, b1, w2, b2, dout = [t.float() if t.is_floating_point() else t for t in _inputs(tokens, "cpu", seed=1)]
    mod = _hf_module((w1, b1, w2, b2), "eager", "cpu", torch.float32)
    hidden.requires_grad_(True)
    times = []
    for _ in range(3):
        for p_ in mod.parameters():
            p_.grad = None
        t0 = time.perf_counter()
        mod(hidden, router_indices=idx, routing_weights=weights).backward(dout)
        times.append(time.perf_counter() - t0)
    dt = sorted(times)[1]
    return {"value": round(block_flops(tokens * TOPK) / dt / 1e12, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "kind": "reference", "sample": f"{tokens} tokens through transformers' GptOssExperts (eager loop, fp32), fwd+bwd, median of 3, {dt:.2f} s"}
