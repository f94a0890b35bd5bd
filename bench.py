#!/usr/bin/env python
"""Benchmark of the GPT-OSS attention forward+backward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3] [--impl b200|reference]

A step is one forward + backward pass of one attention layer over one batch of synthetic
input (seeded N(0,1) tensors with the shapes of the named workload).  The default workload is
the sliding-window layer at S=16K (B=2, 64 query / 8 KV heads, head_dim 64, window 128, bf16)
the headline metric is quoted on.  With N > 1 (launched by torchrun, one process per GPU) every
rank runs the same per-GPU workload on its own (batch x KV-group) units -- attention needs no
exchange between units, so there is no collective on the data path; only the timing is
reduced (max over ranks).  One JSON line is printed by rank 0.

At N = 1 the line also carries `moe_block` (the expert block that follows attention in every layer: this library's
grouped-GEMM path next to transformers' own, see bench_moe.py) and `triton_reference`: the reference project's own Triton kernel run
through its stock `attention()` on the same GPU, same seeded inputs and same event protocol
(imported from `--reference-path`, `$REFERENCE_PATH` or `baseline/_ref`; "unavailable" with the
reason when it cannot be imported), and `cpu_baseline_cfg1`: the unmodified `transformers`
eager attention in fp32 on the CPU-runnable configuration.  At N > 1 it carries `strong`: the
named configurations sharded by KV-head group across the ranks (total work fixed).

`--impl reference` times the reference's CPU path for the same function (fp32 eager attention
evaluated slice by slice by the oracle port) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


# --------------------------------------------------------------------------------------------
def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples the SM clock and the throttle reasons through NVML while the timed region runs.

    A thread polls every 10 ms (nvidia-smi's own loop starts too slowly for sub-second regions);
    falls back to one nvidia-smi query when NVML cannot be loaded.
    """
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.samples, self.reason_bits = [], 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.gpu_index]) if visible and visible.split(",")[0].isdigit() else self.gpu_index
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._poll, daemon=True)
        self._thread.start()

    def _poll(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            except Exception:
                try:
                    self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                except Exception:
                    pass
            self._stop.wait(0.01)

    def stop(self) -> dict:
        if self._nvml is None:
            return self._smi_once()
        self._stop.set()
        self._thread.join(timeout=2)
        reasons = sorted(name for name, bit in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.samples), "reasons": reasons, "source": "nvml"}

    def _smi_once(self) -> dict:
        try:
            out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits",
                                  "-i", str(self.gpu_index)], capture_output=True, text=True, timeout=10).stdout
            sm, mx = (float(x) for x in out.strip().split(","))
            return {"sm_mhz": sm, "sm_max_mhz": mx, "samples": 1, "reasons": [], "source": "nvidia-smi (after the region)"}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["clock query unavailable"]}


# --------------------------------------------------------------------------------------------
# work accounting per kernel (algorithmic = visible pairs only; every tensor once)
# --------------------------------------------------------------------------------------------
def kernel_work(case, algorithmic_flops, algorithmic_bytes):
    fl = algorithmic_flops(case)
    pairs = fl["pairs_per_head"]
    unit = case.d * case.Hq * pairs           # flops of one d-deep product over all visible pairs / 2
    qb = case.B * case.Hq * case.S * case.d * 2
    kb = case.B * case.Hkv * case.S * case.d * 2
    row = case.B * case.Hq * case.S * 4
    return {
        "fwd": {"flops": 4 * unit, "bytes": 2 * qb + 2 * kb + row},
        "bwd_preprocess": {"flops": 0, "bytes": 2 * qb + 2 * row},
        "bwd_dsinks": {"flops": 0, "bytes": row // 32 + 4 * case.Hq},
        "bwd_dkdv": {"flops": 8 * unit, "bytes": 2 * qb + 2 * kb + 2 * row + 2 * kb},
        "bwd_dq": {"flops": 6 * unit, "bytes": 2 * qb + 2 * kb + 2 * row + qb},
        # narrow windows: one kernel makes dK, dV and dQ (S, dP once), after a preprocess that also clears dQ
        "bwd_preprocess_fused": {"flops": 0, "bytes": 2 * qb + 2 * row + qb},
        "bwd_fused": {"flops": 10 * unit, "bytes": 2 * qb + 2 * kb + 2 * row + 2 * kb + qb},
    }


def shape_case(shape: str):
    """--shape B,S,window: a GPT-OSS-shaped case (64 query / 8 KV heads, head_dim 64) of another size."""
    from oracle import AttnCase
    B, S, window = (int(x) for x in shape.split(","))
    return AttnCase(f"B{B}_S{S}_W{window}", B=B, S=S, window=window)


def resident_problem(lib, q, k, v, do, sinks, seqlens, scale, window, device_index, stream):
    """C-ABI parameter block for device-resident inputs, with every output and scratch buffer allocated.

    q (B,Hq,S,d), k/v (B,Hkv,S,d), do (B,S,Hq,d): bf16 device tensors (any outer strides).  Returns the block
    and a dict that keeps the buffers alive.
    """
    import ctypes
    from oregon_gpt_oss_patching_b200 import _cabi
    dev = q.device
    B, Hq, S, d = q.shape
    Hkv = k.shape[1]
    S_pad = _cabi.padded_len(S)
    keep = {
        "o": torch.empty(B, S, Hq, d, dtype=torch.bfloat16, device=dev),
        "lse": torch.empty(B, Hq, S_pad, dtype=torch.float32, device=dev),
        "delta": torch.empty((_cabi.DELTA_PLANES, B, Hq, S_pad), dtype=torch.float32, device=dev),
        "dq": torch.empty(B, Hq, S, d, dtype=torch.bfloat16, device=dev),
        "dk": torch.empty(B, Hkv, S, d, dtype=torch.bfloat16, device=dev),
        "dv": torch.empty(B, Hkv, S, d, dtype=torch.bfloat16, device=dev),
        "dsinks": torch.empty(Hq, dtype=torch.float32, device=dev),
        "status": torch.zeros(1, dtype=torch.int32, device=dev),
        "sinks_f32": sinks.float().contiguous(),
        "inputs": (q, k, v, do, seqlens),
    }
    p = _cabi.Params()
    p.B, p.Hq, p.Hkv, p.S, p.d, p.window, p.scale, p.device = B, Hq, Hkv, S, d, window, scale, device_index
    p.stream, p.status, p.sinks = stream.cuda_stream, keep["status"].data_ptr(), keep["sinks_f32"].data_ptr()
    p.seqlens = seqlens.data_ptr() if seqlens is not None else None
    p.q, p.k, p.v = (_cabi.tensor4(t, "bhsd") for t in (q, k, v))
    p.o, p.d_o = _cabi.tensor4(keep["o"], "bshd"), _cabi.tensor4(do, "bshd")
    p.lse, p.delta = keep["lse"].data_ptr(), keep["delta"].data_ptr()
    p.dq, p.dk, p.dv = (_cabi.tensor4(keep[x], "bhsd") for x in ("dq", "dk", "dv"))
    keep["partial"] = torch.empty(int(lib.b200attn_dsinks_scratch_floats(ctypes.byref(p))), dtype=torch.float32, device=dev)
    p.dsinks, p.dsinks_partial = keep["dsinks"].data_ptr(), keep["partial"].data_ptr()
    return p, keep


def run_b200(args, rank, world, local_rank):
    from oracle import CONFIGS, algorithmic_bytes, algorithmic_flops, make_inputs
    import ctypes
    from oregon_gpt_oss_patching_b200 import _cabi
    from oregon_gpt_oss_patching_b200.attention_kernel import attention, last_status

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    case = CONFIGS[args.workload] if not args.shape else shape_case(args.shape)
    lib = _cabi.load()
    peaks = load_peaks()

    # per-rank inputs: same shapes on every rank, different seed per rank (independent units)
    import dataclasses
    case_r = dataclasses.replace(case, seed=case.seed + rank)
    q, k, v, do, sinks = make_inputs(case_r, dtype=torch.bfloat16, device="cpu")
    seqlens = None if case.seqlens is None else torch.tensor(case.seqlens, dtype=torch.int32, device=dev)
    # the pinned staging buffers of the end-to-end leg are first touched by a thread bound to the GPU's own
    # NUMA node (when this process is allowed to run there): the copies, not the kernels, set that leg's time
    numa = bind_to_gpu_numa_node(local_rank)
    host = [t.pin_memory() for t in (q, k, v, do)]
    qd, kd, vd, dod = (t.to(dev) for t in host)
    sinks = sinks.to(dev)
    B, Hq, S, d = qd.shape
    Hkv = kd.shape[1]
    S_pad = _cabi.padded_len(S)

    # device-resident buffers for the kernel-level timing (direct C-ABI calls, no allocation inside)
    stream = torch.cuda.current_stream(dev)
    p, keep = resident_problem(lib, qd, kd, vd, dod, sinks, seqlens, case.scale, case.window, local_rank, stream)
    status = keep["status"]
    pref = ctypes.byref(p)
    if lib.b200attn_bwd_dq_is_fused(pref):
        # window <= 128: the dkdv stage is the one backward kernel (dK, dV and dQ); the dq stage would return at once
        stages = [("fwd", lib.b200attn_fwd), ("bwd_preprocess_fused", lib.b200attn_bwd_preprocess),
                  ("bwd_fused", lib.b200attn_bwd_dkdv), ("bwd_dsinks", lib.b200attn_bwd_dsinks)]
    else:
        stages = [("fwd", lib.b200attn_fwd), ("bwd_preprocess", lib.b200attn_bwd_preprocess),
                  ("bwd_dkdv", lib.b200attn_bwd_dkdv), ("bwd_dq", lib.b200attn_bwd_dq),
                  ("bwd_dsinks", lib.b200attn_bwd_dsinks)]

    def step_resident(events=None):
        for idx, (name, fn) in enumerate(stages):
            if events is not None:
                events[idx].record(stream)
            rc = fn(pref)
            if rc != 0:
                raise RuntimeError(f"{name}: {_cabi.strerror(rc)}")
        if events is not None:
            events[len(stages)].record(stream)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(dev)

    if args.capture:   # profiler target: a few passes of the five kernels and nothing else
        for _ in range(args.warmup + args.steps):
            step_resident()
        barrier()
        if status.item() != 0:
            raise RuntimeError("a kernel abandoned a bounded wait (status word non-zero)")
        print(json.dumps({"capture": case.name, "passes": args.warmup + args.steps}))
        return

    for _ in range(max(args.warmup, 3)):
        step_resident()
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- timed region 1: inputs resident in HBM, K steps, per-stage events inside -------------
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(stages) + 1)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin.record(stream)
    for it in range(args.steps):
        step_resident(ev[it])
    t_end.record(stream)
    barrier()
    ms_total = t_begin.elapsed_time(t_end)
    clocks = sampler.stop() if rank == 0 else None
    stage_ms = {name: sum(ev[it][i].elapsed_time(ev[it][i + 1]) for it in range(args.steps)) / args.steps
                for i, (name, _) in enumerate(stages)}
    if status.item() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait (status word non-zero)")

    # ---- timed region 2: end to end through the public API with host buffers ------------------
    # Every step copies its inputs from pinned host memory, runs attention() forward + backward and
    # copies every result back to pinned host memory.  The three phases of consecutive steps run on
    # three streams (upload / compute / download) with two sets of device buffers, so a step's
    # upload overlaps the previous step's kernels and the download of the one before.
    sk = sinks.clone().requires_grad_(True)
    up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [[torch.empty_like(t, device=dev) for t in host] for _ in range(2)]
    outs_host = [[torch.empty(shape, dtype=dt, pin_memory=True) for shape, dt in
                  (((B, S, Hq, d), torch.bfloat16), (tuple(qd.shape), torch.bfloat16), (tuple(kd.shape), torch.bfloat16),
                   (tuple(vd.shape), torch.bfloat16), ((Hq,), torch.float32))] for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]   # inputs of a slot no longer needed by compute
    e2e_count = 0

    def step_e2e():
        nonlocal e2e_count
        slot = e2e_count % 2
        e2e_count += 1
        with torch.cuda.stream(up):
            up.wait_event(consumed[slot])            # the step that used this slot two steps ago is done with it
            for dst, src in zip(dev_in[slot], host):
                dst.copy_(src, non_blocking=True)
            uploaded[slot].record(up)
        stream.wait_event(uploaded[slot])
        stream.wait_event(downloaded[slot])          # results of this slot's previous use have left the device
        qx, kx, vx, dox = (t.detach() for t in dev_in[slot])
        qx.requires_grad_(True); kx.requires_grad_(True); vx.requires_grad_(True)
        sk.grad = None
        out = attention(qx, kx, vx, sk, case.scale, case.window, seqlens)
        out.backward(dox)
        res = (out.detach(), qx.grad, kx.grad, vx.grad, sk.grad.float())
        computed[slot].record(stream)
        consumed[slot].record(stream)
        with torch.cuda.stream(down):
            down.wait_event(computed[slot])
            for h_, t in zip(outs_host[slot], res):
                h_.copy_(t, non_blocking=True)
                t.record_stream(down)
            downloaded[slot].record(down)

    e2e_steps = max(4, min(args.steps, 20))
    for _ in range(2):
        step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        step_e2e()
    stream.wait_stream(up)
    stream.wait_stream(down)                         # the last downloads are inside the timed region
    e1.record(stream)
    barrier()
    ms_e2e = e0.elapsed_time(e1) / e2e_steps
    outs_host = outs_host[0]
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = sum(t.numel() * t.element_size() for t in outs_host)

    # ---- reduce timing: max over ranks -----------------------------------------------------
    tm = torch.tensor([ms_total, ms_e2e] + [stage_ms[n] for n, _ in stages], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(tm, op=torch.distributed.ReduceOp.MAX)
    ms_total, ms_e2e = tm[0].item(), tm[1].item()
    stage_ms = {n: tm[2 + i].item() for i, (n, _) in enumerate(stages)}
    ms_step = ms_total / args.steps

    strong = None
    if world > 1 and not args.no_strong:
        strong = {name: strong_scaling_record(name, lib, rank, world, local_rank, dev, stream, max(5, min(args.steps, 50)))
                  for name in ("cfg2", "cfg3")}

    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    fl = algorithmic_flops(case)
    by = algorithmic_bytes(case)
    tokens = sum(case.lengths())
    value = fl["total"] * world / (ms_step * 1e-3) / 1e12
    work = kernel_work(case, algorithmic_flops, algorithmic_bytes)
    kernels = {}
    for name, _ in stages:
        t = stage_ms[name] * 1e-3
        w = work[name]
        kernels[name] = {"ms": round(stage_ms[name], 5), "gbs": round(w["bytes"] / t / 1e9, 1),
                         "tflops": round(w["flops"] / t / 1e12, 2)}
    top = max(stage_ms, key=stage_ms.get)
    w, t = work[top], stage_ms[top] * 1e-3
    t_hbm, t_tc = w["bytes"] / (peaks["hbm_gbs"] * 1e9), w["flops"] / (peaks["bf16_tflops"] * 1e12)
    if t_hbm >= t_tc:
        roof = {"bound": "hbm", "achieved": round(w["bytes"] / t / 1e9, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s"}
    else:
        roof = {"bound": "tensor", "achieved": round(w["flops"] / t / 1e12, 2), "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s"}
    roof["frac"] = round(roof["achieved"] / roof["peak"], 4)
    roof["kernel"] = top
    roof["peak_source"] = peaks["source"]
    roof["traffic"] = ncu_traffic_bytes(args.workload, top)
    t_min = max(by["total"] / (peaks["hbm_gbs"] * 1e9), fl["total"] / (peaks["bf16_tflops"] * 1e12))

    line = {
        "metric": "attn_fwd_bwd_tflops", "value": round(value, 3), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: B={case.B}/GPU S={case.S} Hq={case.Hq} Hkv={case.Hkv} d={case.d} "
                               f"window={case.window} sinks; fwd+bwd of one attention layer",
                   "global_batch": case.B * world, "seq_len": case.S,
                   "parallelism": f"{world} x independent (batch x KV-group) units, no collective",
                   "l2": "inputs larger than L2 (no flush)", "flops": "14*d*Hq*visible_pairs"},
        "tokens_per_s": round(tokens * world / (ms_step * 1e-3), 1),
        "whole_path_roofline_frac": round(t_min / (ms_step * 1e-3), 4),
        "frac_of_bf16_peak": round(value / world / peaks["bf16_tflops"], 4),
        "clocks": clocks,
        "e2e": {"value": round(fl["total"] * world / (ms_e2e * 1e-3) / 1e12, 4), "unit": "TFLOP/s",
                "ms_per_step": round(ms_e2e, 3), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": len(stages) * args.steps,
        "roofline": roof,
        "kernels": kernels,
        "host_numa": numa,
    }
    if strong is not None:
        line["strong"] = strong
    if world == 1 and not args.no_contender:
        line["triton_reference"] = triton_contender(args, case, (qd, kd, vd, dod, sinks), seqlens, stream)
    if world == 1 and not args.no_contender and not args.shape:
        # the rotary pass in front of attention: one kernel per tensor, read + write once, against the HBM peak
        try:
            from oregon_gpt_oss_patching_b200.rope import rope
            ang = torch.arange(S, device=dev, dtype=torch.float32)[:, None] / (150000.0 ** (torch.arange(0, d, 2, device=dev) / d))[None, :]
            cos, sin = ang.cos()[None].to(torch.bfloat16), ang.sin()[None].to(torch.bfloat16)
            q_view = qd.transpose(1, 2).contiguous().transpose(1, 2)     # (B,S,H,d) memory, as the projection leaves it
            ms_rope = time_steps(lambda: rope(q_view, cos, sin), 20, stream)
            nbytes = 2 * q_view.numel() * 2
            line["rope"] = {"ms": round(ms_rope, 4), "gbs": round(nbytes / (ms_rope * 1e-3) / 1e9, 1),
                            "frac_of_hbm_peak": round(nbytes / (ms_rope * 1e-3) / 1e9 / peaks["hbm_gbs"], 3),
                            "what": f"b200attn_rope on q of this workload ({q_view.numel() * 2 >> 20} MiB, (B,S,H,d) memory viewed (B,H,S,d))"}
            del q_view
        except Exception as exc:   # noqa: BLE001
            line["rope"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}
        # the block that follows attention in every layer, measured in the same process (a record, not the headline)
        torch.cuda.empty_cache()
        try:
            from bench_moe import summary_record
            line["moe_block"] = summary_record(local_rank)
        except Exception as exc:   # noqa: BLE001
            line["moe_block"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_sample(args.workload, budget_s=args.cpu_budget)
        line["cpu_baseline_cfg1"] = cpu_hf_eager_cfg1()
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def ncu_traffic_bytes(workload, kernel):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of `kernel` on `workload`, from the ncu
    captures summarised in profiles/ncu_traffic.json (absent entry = not captured: null)."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            entry = json.load(f)["traffic"].get(workload, {}).get(kernel)
        return None if entry is None else int(entry["dram_read_bytes"]) + int(entry["dram_write_bytes"])
    except Exception:
        return None


def bind_to_gpu_numa_node(gpu_index: int) -> dict:
    """Restrict this process to the CPUs of the NUMA node the GPU hangs off, if it may run there.

    Pinned host memory is placed on the node of the thread that first touches it; with several ranks
    staging gigabytes per step, buffers on the far socket halve the copy bandwidth.  Best effort: any
    failure (no sysfs entry, node outside the allowed CPU set) leaves the affinity as it was.
    """
    info = {"gpu_node": None, "bound": False}
    try:
        bus = torch.cuda.get_device_properties(gpu_index).pci_bus_id
        dom = torch.cuda.get_device_properties(gpu_index).pci_domain_id
        devn = torch.cuda.get_device_properties(gpu_index).pci_device_id
        with open(f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{devn:02x}.0/numa_node") as f:
            node = int(f.read().strip())
        info["gpu_node"] = node
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        target = cpus & allowed
        info["allowed_cpus"] = len(allowed)
        if target and target != allowed:
            os.sched_setaffinity(0, target)
            info["bound"] = True
        elif target:
            info["bound"] = "already local"
    except Exception as e:
        info["note"] = f"{type(e).__name__}"
    return info


def time_steps(fn, steps, stream, warm=3):
    """Average ms per call of fn: warm-up calls first (JIT compilation excluded), CUDA events on `stream`."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def triton_contender(args, case, tensors, seqlens, stream):
    """The reference's Triton kernel on this GPU: same device-resident inputs, forward+backward through its own
    autograd function; this library timed the same way (through `attention()`) right after it."""
    from baseline import triton_ref
    from oracle import algorithmic_flops
    from oregon_gpt_oss_patching_b200.attention_kernel import attention
    mod, where = triton_ref.load(args.reference_path or None)
    if mod is None:
        return {"unavailable": where}
    q, k, v, do, sinks = tensors
    sinks_model = sinks.to(torch.bfloat16)     # the attention module holds its sinks in the model dtype
    steps = max(3, min(args.steps, 20))
    try:
        ms_ref = time_steps(lambda: triton_ref.fwd_bwd(mod, q, k, v, do, sinks_model, case.scale, case.window), steps, stream)
    except Exception as e:
        return {"unavailable": f"the reference kernel did not run here: {type(e).__name__}: {str(e)[:160]}"}

    def b200_step():
        qq, kk, vv, ss = (t.detach().requires_grad_(True) for t in (q, k, v, sinks_model))
        attention(qq, kk, vv, ss, case.scale, case.window, seqlens).backward(do)

    ms_b200 = time_steps(b200_step, steps, stream)
    fl = algorithmic_flops(case)["total"]
    return {"ms_per_step": round(ms_ref, 4), "tflops": round(fl / ms_ref / 1e9, 2),
            "b200_same_protocol_ms": round(ms_b200, 4), "vs_b200": round(ms_ref / ms_b200, 3),
            "steps": steps, "where": os.path.relpath(where, ROOT) if where.startswith(ROOT) else where,
            "protocol": "device-resident bf16 inputs, fwd+bwd through each implementation's autograd function, "
                        "3 warm-up calls (JIT excluded), CUDA events; the reference ignores padding masks"}


def strong_scaling_record(name, lib, rank, world, local_rank, dev, stream, steps):
    """One named configuration sharded by KV-head group over the ranks: total work fixed, no collective.

    Every rank builds the same seeded inputs on its own GPU, takes its groups (all batches), and runs the five
    kernels on that share; the time is the max over ranks, the throughput the configuration's algorithmic
    flops over that time.
    """
    import ctypes
    from oracle import CONFIGS, algorithmic_flops
    from oregon_gpt_oss_patching_b200 import _cabi
    from oregon_gpt_oss_patching_b200.sharding import shard_by_group
    import torch.distributed as dist
    case = CONFIGS[name]
    if world > case.Hkv or case.Hkv % world:
        return {"unavailable": f"{world} ranks do not divide {case.Hkv} KV-head groups"}
    g = torch.Generator(device=dev).manual_seed(case.seed)
    mk = lambda *shape: (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * case.input_scale).to(torch.bfloat16)
    q, k, v = mk(case.B, case.Hq, case.S, case.d), mk(case.B, case.Hkv, case.S, case.d), mk(case.B, case.Hkv, case.S, case.d)
    do = mk(case.B, case.S, case.Hq, case.d)
    sinks = torch.randn(case.Hq, generator=g, device=dev)
    (qs, ks, vs, dos, ss), (g0, g1) = shard_by_group(q, k, v, do, sinks, rank, world)
    p, keep = resident_problem(lib, qs, ks, vs, dos, ss, None, case.scale, case.window, local_rank, stream)
    fns = (lib.b200attn_fwd, lib.b200attn_bwd_preprocess, lib.b200attn_bwd_dkdv, lib.b200attn_bwd_dq, lib.b200attn_bwd_dsinks)

    def step():
        for fn in fns:
            rc = fn(ctypes.byref(p))
            if rc != 0:
                raise RuntimeError(_cabi.strerror(rc))

    for _ in range(3):
        step()
    torch.cuda.synchronize(dev)
    dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize(dev)
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if keep["status"].item() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait (status word non-zero)")
    ms = t.item()
    fl = algorithmic_flops(case)["total"]
    return {"scaling": "strong", "ms_per_step": round(ms, 5), "value": round(fl / ms / 1e9, 2), "unit": "TFLOP/s",
            "groups_per_rank": g1 - g0, "steps": steps,
            "note": "whole configuration split by KV-head group, max over ranks, inputs resident"}


# --------------------------------------------------------------------------------------------
# CPU arms (oracle port of the reference's eager path) -- the only place the oracle is executed
# --------------------------------------------------------------------------------------------
def use_all_host_threads() -> int:
    """The CPU arms use every core this process may run on (torchrun sets OMP_NUM_THREADS=1 by default)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_slices(case, n):
    units = [(b, g) for b in range(case.B) for g in range(case.Hkv)]
    return units[:max(1, min(n, len(units)))]


def cpu_step(case, tensors, slices):
    from oracle import attention_fwd_bwd_blockwise
    q, k, v, do, sinks = tensors
    attention_fwd_bwd_blockwise(q, k, v, sinks, do, case.scale, case.window, case.seqlens, slices=slices,
                                row_block=1024)


def slice_flops(case, slices):
    from oracle import visible_pairs
    lens = case.lengths()
    G = case.Hq // case.Hkv
    return sum(14 * case.d * G * visible_pairs(lens[b], case.window) for b, _ in slices)


def cpu_sample(workload, budget_s=15.0):
    """Time the oracle port on a bounded number of (batch, KV-group) slices of the workload."""
    from oracle import CONFIGS, make_inputs
    case = CONFIGS[workload]
    use_all_host_threads()
    tensors = make_inputs(case, dtype=torch.float32, device="cpu")
    one = cpu_slices(case, 1)
    t0 = time.perf_counter()
    cpu_step(case, tensors, one)
    t_one = time.perf_counter() - t0
    n = max(1, min(case.B * case.Hkv, int(budget_s / max(t_one, 1e-3))))
    sl = cpu_slices(case, n)
    t0 = time.perf_counter()
    cpu_step(case, tensors, sl)
    dt = time.perf_counter() - t0
    return {"value": round(slice_flops(case, sl) / dt / 1e12, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "kind": "port", "sample": f"{len(sl)} of {case.B * case.Hkv} (batch, KV-group) slices of {workload}, "
                                      f"fp32 blockwise eager oracle, {dt:.2f} s"}


def cpu_hf_eager_cfg1(runs: int = 5) -> dict:
    """The CPU path the reference project falls back to, unmodified: `transformers`' eager_attention_forward
    (models/gpt_oss/modeling_gpt_oss.py:245-273) in fp32, forward + autograd backward, on the CPU-runnable
    configuration exactly (B=1, S=512, 64/8 heads, window 128).  Median of `runs` after one warm-up run."""
    import types
    from oracle import CONFIGS, algorithmic_flops, make_inputs, visible_mask
    try:
        from transformers.models.gpt_oss.modeling_gpt_oss import eager_attention_forward
    except Exception as e:
        return {"unavailable": f"transformers' gpt_oss model cannot be imported: {type(e).__name__}"}
    case = CONFIGS["cfg1"]
    threads = use_all_host_threads()
    q, k, v, do, sinks = make_inputs(case, dtype=torch.float32, device="cpu")
    vis = visible_mask(case.S, case.window)[None, None]
    add = torch.zeros(1, 1, case.S, case.S).masked_fill(~vis, torch.finfo(torch.float32).min)
    times = []
    for i in range(runs + 1):
        qq, kk, vv, ss = (t.clone().requires_grad_(True) for t in (q, k, v, sinks))
        module = types.SimpleNamespace(num_key_value_groups=case.Hq // case.Hkv, sinks=ss, training=False)
        t0 = time.perf_counter()
        o, _ = eager_attention_forward(module, qq, kk, vv, add, scaling=case.scale, dropout=0.0)
        o.backward(do)
        if i > 0:
            times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": round(algorithmic_flops(case)["total"] / med / 1e12, 6), "unit": "TFLOP/s", "ms": round(med * 1e3, 2),
            "cores": threads, "os_cpu_count": os.cpu_count(), "kind": "reference",
            "sample": f"cfg1 whole (B=1 S=512 window 128, fp32), transformers eager_attention_forward fwd+bwd, median of {runs}"}


def run_reference(args, rank):
    if rank != 0:
        return
    from oracle import CONFIGS, algorithmic_flops, make_inputs
    case = CONFIGS[args.workload]
    use_all_host_threads()
    tensors = make_inputs(case, dtype=torch.float32, device="cpu")
    cpu_step(case, tensors, cpu_slices(case, 1))   # first touch (allocator, thread pool)
    t0 = time.perf_counter()
    cpu_step(case, tensors, cpu_slices(case, 1))
    t_one = time.perf_counter() - t0
    steps, warm = args.steps, max(args.warmup, 1)
    # bound the whole run to a few minutes: slices per step from a per-run budget
    budget = 120.0
    n = max(1, min(case.B * case.Hkv, int(budget / max(t_one, 1e-3) / (steps + warm))))
    sl = cpu_slices(case, n)
    for _ in range(warm):
        cpu_step(case, tensors, sl)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(case, tensors, sl)
    dt = (time.perf_counter() - t0) / steps
    value = slice_flops(case, sl) / dt / 1e12
    sample = f"{len(sl)} of {case.B * case.Hkv} (batch, KV-group) slices of {args.workload} per step, fp32 blockwise eager oracle"
    line = {"impl": "reference", "metric": "attn_fwd_bwd_tflops", "value": round(value, 5), "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": round(dt * 1e3, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: bounded sample", "seq_len": case.S, "sample": sample},
            "cpu_baseline": {"value": round(value, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                             "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "cpu_baseline_cfg1": cpu_hf_eager_cfg1(),
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg3")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--shape", default="", help="B,S,window: run this shape instead of a named workload")
    ap.add_argument("--capture", action="store_true", help="only run warmup+steps passes of the kernels (for ncu)")
    ap.add_argument("--reference-path", default="", help="directory holding the reference's attention_kernel.py "
                    "(default: $REFERENCE_PATH, then baseline/_ref)")
    ap.add_argument("--no-contender", action="store_true", help="skip the reference-Triton-kernel arm")
    ap.add_argument("--no-strong", action="store_true", help="skip the sharded (strong-scaling) records at N > 1")
    ap.add_argument("--moe-tokens", type=int, default=8192, help="tokens of `--workload moe` (one expert block, fwd+bwd)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU implementation")
    if args.workload == "moe":   # the block after attention in every layer: a separate line, not the headline metric
        from bench_moe import run_moe
        run_moe(args, rank, world, local_rank)
        return
    run_b200(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
