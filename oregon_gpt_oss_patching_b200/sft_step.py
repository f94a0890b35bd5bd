"""One supervised-fine-tuning step of a gpt-oss-architecture model with the patched attention.

Stands in, for measurement purposes, for the reference's training entry point (``sft.py:16-53``
launched by ``scripts/run_full_sft.sh`` with ``configs/sft_full.yaml`` / ``configs/zero3.yaml``):
the model is built from ``GptOssConfig`` with random bf16 weights (no checkpoint, no dataset:
token ids are uniform over the vocabulary), attention is patched exactly as the reference does
(``sft.py:18``), gradient checkpointing is on (``sft_full.yaml:13``), batch 1 per GPU and
``max_length`` 8192 (``sft_full.yaml:16,18``); the expert block runs through this library's grouped GEMMs unless
``--moe hf`` / ``--moe hf_eager`` asks for transformers' own implementations.  Data parallelism is plain replication with a
bucketed NCCL all-reduce of the bf16 gradients (torch DDP) instead of DeepSpeed ZeRO-3, and the
optimizer is state-free SGD, so that one replica (41.8 GB weights + 41.8 GB gradients for the 20b
architecture) fits one 180 GB GPU.

    python -m oregon_gpt_oss_patching_b200.sft_step [--layers 24] [--seq 8192] [--steps 3] [--unpatched] [--moe b200|hf|hf_eager]
    torchrun --nproc-per-node N -m oregon_gpt_oss_patching_b200.sft_step ...

Prints one JSON line (rank 0): tokens/s/GPU, ms/step, peak memory.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch


def build_model(layers: int, experts: int, vocab: int, device, seed: int = 0, experts_implementation=None):
    from transformers import GptOssConfig, GptOssForCausalLM
    cfg = GptOssConfig(num_hidden_layers=layers, num_local_experts=experts, vocab_size=vocab,
                       layer_types=["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(layers)],
                       attention_dropout=0.0, use_cache=False)
    cfg._attn_implementation = "eager"   # the patch point is the eager function (patching.py:6-7 of the reference)
    if experts_implementation is not None:
        cfg._experts_implementation = experts_implementation
    torch.manual_seed(seed)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            model = GptOssForCausalLM(cfg)
    finally:
        torch.set_default_dtype(prev)
    with torch.no_grad():
        for layer in model.model.layers:
            layer.self_attn.sinks.normal_()
    model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False})
    model.train()
    return model, cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--vocab", type=int, default=201088)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--unpatched", action="store_true", help="HF eager attention instead of the B200 kernels")
    ap.add_argument("--moe", default="b200", choices=["b200", "hf", "hf_eager"],
                    help="expert block: this library's grouped GEMMs, transformers' default (torch._grouped_mm where it "
                         "can dispatch), or transformers' per-expert loop")
    ap.add_argument("--no-allreduce", action="store_true", help="attribution run: data-parallel replicas that skip the gradient "
                    "all-reduce (the difference to a normal run is the part of the all-reduce that backward does not hide)")
    ap.add_argument("--gemm-ctas", type=int, default=0, help="persistent CTAs of the grouped GEMM (0 = one per SM); fewer "
                    "leaves SMs to the all-reduce that runs beside the backward pass")
    ap.add_argument("--hf-rope", action="store_true", help="keep transformers' rotary embedding (default: the one-pass kernel, "
                    "whenever the attention is patched)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)

    from . import patching
    if not args.unpatched:
        patching.patch_flash_attention()
        if not args.hf_rope:
            from . import rope
            rope.patch_rotary_embedding()

    from . import moe_experts
    if args.moe == "b200":
        moe_experts.patch_moe_experts()
        moe_experts.set_gemm_ctas(args.gemm_ctas)

    model, cfg = build_model(args.layers, args.experts, args.vocab, dev, experts_implementation="eager" if args.moe == "hf_eager" else None)
    n_params = sum(p.numel() for p in model.parameters())
    net = model
    if world > 1 and not args.no_allreduce:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], gradient_as_bucket_view=True,
                                                        bucket_cap_mb=512, static_graph=True)
    g = torch.Generator().manual_seed(rank)
    ids = torch.randint(0, args.vocab, (1, args.seq), generator=g).to(dev)

    def step():
        out = net(input_ids=ids, labels=ids, use_cache=False)
        out.loss.backward()
        with torch.no_grad():
            params = [p for p in model.parameters() if p.grad is not None]
            torch._foreach_add_(params, [p.grad for p in params], alpha=-args.lr)
            for p in params:
                p.grad = None
        return out.loss.detach()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(dev)
    if world > 1:
        torch.distributed.barrier()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
    status = 0
    if not args.unpatched or args.moe == "b200":
        from .attention_kernel import last_status
        status = int(last_status(dev))
    if rank == 0:
        print(json.dumps({
            "metric": "sft_tokens_per_s_per_gpu", "value": round(args.seq / (ms.item() * 1e-3), 1), "unit": "tokens/s/GPU",
            "n_gpus": world, "ms_per_step": round(ms.item(), 1), "steps": args.steps, "warmup": args.warmup,
            "attention": "hf_eager" if args.unpatched else "b200",
            "rope": "hf" if (args.unpatched or args.hf_rope) else "b200",
            "moe": args.moe if args.moe != "hf" else "hf:" + str(getattr(cfg, "_experts_implementation", None)), "loss": round(float(loss), 4), "kernel_status": status,
            "config": {"layers": args.layers, "experts": args.experts, "vocab": args.vocab, "seq_len": args.seq,
                       "params_b": round(n_params / 1e9, 2), "batch_per_gpu": 1, "gemm_ctas": args.gemm_ctas, "grad_checkpointing": True,
                       "optimizer": "sgd (state-free)", "dp": ("replicas, all-reduce skipped (attribution run)" if args.no_allreduce else "replicas + NCCL all-reduce (DDP)") if world > 1 else "none"},
            "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2**30, 1), "data": "synthetic",
            "wall_s": round(time.perf_counter() - t0, 1)}), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
