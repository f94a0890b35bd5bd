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
    }


def shape_case(shape: str):
    """--shape B,S,window: a GPT-OSS-shaped case (64 query / 8 KV heads, head_dim 64) of another size."""
    from oracle import AttnCase
    B, S, window = (int(x) for x in shape.split(","))
    return AttnCase(f"B{B}_S{S}_W{window}", B=B, S=S, window=window)


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
    host = [t.pin_memory() for t in (q, k, v, do)]
    qd, kd, vd, dod = (t.to(dev) for t in host)
    sinks = sinks.to(dev)
    B, Hq, S, d = qd.shape
    Hkv = kd.shape[1]
    S_pad = _cabi.padded_len(S)

    # device-resident buffers for the kernel-level timing (direct C-ABI calls, no allocation inside)
    o = torch.empty(B, S, Hq, d, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(B, Hq, S_pad, dtype=torch.float32, device=dev)
    delta = torch.empty((_cabi.DELTA_PLANES,) + tuple(lse.shape), dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    dsinks = torch.empty(Hq, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    p = _cabi.Params()
    p.B, p.Hq, p.Hkv, p.S, p.d, p.window, p.scale, p.device = B, Hq, Hkv, S, d, case.window, case.scale, local_rank
    stream = torch.cuda.current_stream(dev)
    sinks_f32 = sinks.float().contiguous()
    p.stream, p.status, p.sinks = stream.cuda_stream, status.data_ptr(), sinks_f32.data_ptr()
    p.seqlens = seqlens.data_ptr() if seqlens is not None else None
    p.q, p.k, p.v = (_cabi.tensor4(t, "bhsd") for t in (qd, kd, vd))
    p.o, p.d_o, p.lse, p.delta = _cabi.tensor4(o, "bshd"), _cabi.tensor4(dod, "bshd"), lse.data_ptr(), delta.data_ptr()
    p.dq, p.dk, p.dv = (_cabi.tensor4(t, "bhsd") for t in (dq, dk, dv))
    part = torch.empty(int(lib.b200attn_dsinks_scratch_floats(ctypes.byref(p))), dtype=torch.float32, device=dev)
    p.dsinks, p.dsinks_partial = dsinks.data_ptr(), part.data_ptr()
    stages = [("fwd", lib.b200attn_fwd), ("bwd_preprocess", lib.b200attn_bwd_preprocess),
              ("bwd_dkdv", lib.b200attn_bwd_dkdv), ("bwd_dq", lib.b200attn_bwd_dq),
              ("bwd_dsinks", lib.b200attn_bwd_dsinks)]
    pref = ctypes.byref(p)

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
    roof["traffic"] = NCU_TRAFFIC_BYTES.get((args.workload, top))
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
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_sample(args.workload, budget_s=args.cpu_budget)
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (workload, kernel) -> bytes; absent = not captured.
NCU_TRAFFIC_BYTES: dict = {
    # cfg3 launches = 4x the rows of the captured B=1, S=8192, window-128 case (traffic grows with rows)
    ("cfg3", "fwd"): 4 * (83_966_464 + 23_717_632),
    ("cfg3", "bwd_dkdv"): 4 * (167_820_800 + 11_823_872),
    ("cfg3", "bwd_dq"): 4 * (155_429_120 + 38_473_216),
    # cfg2 launches = 4x the rows of the captured B=1, S=4096 full-causal case
    ("cfg2", "fwd"): 4 * (42_022_144 + 2_042_112),
    ("cfg2", "bwd_dkdv"): 4 * (84_045_568 + 5_633_536),
    ("cfg2", "bwd_dq"): 4 * (77_636_096 + 10_991_872),
}


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
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU implementation")
    run_b200(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
