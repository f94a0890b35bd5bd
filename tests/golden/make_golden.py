"""Generate the golden fixtures in this directory from the reference itself.

Run once, in a container that has the reference checkout and ``transformers``:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/reference

Two independent producers are run on the same seeded inputs, both in fp32 on
the CPU:

* ``hf``     -- the unmodified ``transformers`` function
  ``models/gpt_oss/modeling_gpt_oss.py:245-273`` (``eager_attention_forward``),
  fed the additive mask HF's own mask functions describe
  (``masking_utils.py:78`` and ``:96-97``), gradients by autograd.  This is the
  function the reference's ``patching.py:4`` saves as the original and the one
  its un-patched path runs.
* ``triton`` -- the reference's ``attention_kernel.py`` (``_attention`` at
  ``:220-344``) executed by Triton's CPU interpreter.  It ignores padding, so
  for padded cases only rows inside each sequence are comparable.

The fixtures hold the inputs (rounded to bf16-representable values and stored
as their 16-bit patterns, so that a bf16 kernel sees exactly the same numbers)
and both producers' outputs.  Nothing here is imported by the library.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.eager_fp32 import AttnCase, make_inputs, visible_mask  # noqa: E402

# name -> case.  Small enough that every fixture stays a few hundred KB.
CASES = {
    "full_s128": AttnCase("full_s128", B=1, S=128, Hq=4, Hkv=1, window=0, seed=1),
    "full_s200_2kv": AttnCase("full_s200_2kv", B=1, S=200, Hq=4, Hkv=2, window=0, seed=2),
    "swa64_s200": AttnCase("swa64_s200", B=1, S=200, Hq=4, Hkv=1, window=64, seed=3),
    "swa128_s320": AttnCase("swa128_s320", B=1, S=320, Hq=2, Hkv=1, window=128, seed=4),
    "pad_swa128": AttnCase("pad_swa128", B=2, S=256, Hq=2, Hkv=1, window=128, seqlens=(256, 130), seed=5),
    "pad_full": AttnCase("pad_full", B=2, S=256, Hq=2, Hkv=1, window=0, seqlens=(200, 77), seed=6),
}
# The CPU-runnable benchmark configuration: only a digest is stored.
CFG1 = AttnCase("cfg1", B=1, S=512, Hq=64, Hkv=8, window=128, seed=0)


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def to_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def run_hf(case, q, k, v, do, sinks):
    from transformers.models.gpt_oss.modeling_gpt_oss import eager_attention_forward
    q, k, v, sinks = (t.clone().requires_grad_(True) for t in (q, k, v, sinks))
    B, S = case.B, case.S
    lens = case.lengths()
    vis = torch.stack([visible_mask(S, case.window, L if case.seqlens else None) for L in lens])[:, None]
    add = torch.zeros(B, 1, S, S).masked_fill(~vis, torch.finfo(torch.float32).min)
    module = types.SimpleNamespace(num_key_value_groups=case.Hq // case.Hkv, sinks=sinks, training=False)
    o, _ = eager_attention_forward(module, q, k, v, add, scaling=case.scale, dropout=0.0)
    o.backward(do)
    return {"o": o.detach(), "dq": q.grad, "dk": k.grad, "dv": v.grad, "dsinks": sinks.grad}


def run_triton(ref_dir, case, q, k, v, do, sinks):
    sys.path.insert(0, ref_dir)
    import attention_kernel as ak  # the reference's module

    class Ctx:  # stands in for autograd's context so that LSE can be read back
        def save_for_backward(self, *ts):
            self.saved_tensors = ts

    ctx = Ctx()
    window = case.window if case.window else None
    o = ak._attention.forward(ctx, q, k, v, sinks, case.scale, window, None)
    dq, dk, dv, ds, *_ = ak._attention.backward(ctx, do)
    lse = ctx.saved_tensors[5][:, :, :case.S]
    return {"o": o, "dq": dq, "dk": dk, "dv": dv, "dsinks": ds, "lse": lse}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of nlp-uoregon/oregon_gpt_oss_patching")
    ap.add_argument("--skip-cfg1-triton", action="store_true")
    args = ap.parse_args()
    torch.manual_seed(0)
    for name, case in CASES.items():
        q, k, v, do, sinks = make_inputs(case)
        q, k, v, do, sinks = (bf16_round(t) for t in (q, k, v, do, sinks))
        hf = run_hf(case, q, k, v, do, sinks)
        tr = run_triton(args.reference, case, q, k, v, do, sinks)
        blob = {"q_bits": to_bits(q), "k_bits": to_bits(k), "v_bits": to_bits(v),
                "do_bits": to_bits(do), "sinks_bits": to_bits(sinks),
                "meta": np.array([case.B, case.S, case.Hq, case.Hkv, case.d, case.window], np.int64),
                "seqlens": np.array(case.lengths(), np.int32),
                "has_padding": np.array(case.seqlens is not None)}
        for key, val in hf.items():
            blob["hf_" + key] = val.numpy().astype(np.float32)
        # The Triton producer's full outputs would double the fixture; keep its LSE (HF has
        # none), dSinks, a strided sample of the rest, and how far it is from HF on valid rows.
        blob["triton_lse"] = tr["lse"].detach().numpy().astype(np.float32)
        blob["triton_dsinks"] = tr["dsinks"].detach().numpy().astype(np.float32)
        blob["triton_o_sample"] = tr["o"][:, ::7].detach().numpy().astype(np.float32)
        blob["triton_dq_sample"] = tr["dq"][:, :, ::7].detach().numpy().astype(np.float32)
        blob["triton_dk_sample"] = tr["dk"][:, :, ::7].detach().numpy().astype(np.float32)
        blob["triton_dv_sample"] = tr["dv"][:, :, ::7].detach().numpy().astype(np.float32)
        agree = {}
        for key in ("o", "dq", "dk", "dv", "dsinks"):
            a, b = tr[key].detach(), hf[key]
            if case.seqlens is not None and key in ("o", "dq"):
                worst = 0.0
                for bi, L in enumerate(case.seqlens):
                    aa = a[bi, :L] if key == "o" else a[bi, :, :L]
                    bb = b[bi, :L] if key == "o" else b[bi, :, :L]
                    worst = max(worst, float((aa - bb).abs().max() / b.abs().max()))
            else:
                worst = float((a - b).abs().max() / b.abs().max())
            agree[key] = worst
        blob["hf_vs_triton_rel"] = np.array([agree[x] for x in ("o", "dq", "dk", "dv", "dsinks")])
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
        print(f"{name}: wrote; hf-vs-triton rel (o,dq,dk,dv,dsinks) "
              + " ".join(f"{agree[x]:.1e}" for x in ("o", "dq", "dk", "dv", "dsinks")))

    # cfg1 digest: sums and a strided sample instead of the full 8 MB tensors
    case = CFG1
    q, k, v, do, sinks = make_inputs(case)
    hf = run_hf(case, q, k, v, do, sinks)
    blob = {"meta": np.array([case.B, case.S, case.Hq, case.Hkv, case.d, case.window], np.int64)}
    producers = {"hf": hf}
    if not args.skip_cfg1_triton:
        producers["triton"] = run_triton(args.reference, case, q, k, v, do, sinks)
    for pname, res in producers.items():
        for key in ("o", "dq", "dk", "dv", "dsinks"):
            t = res[key].detach().double()
            blob[f"{pname}_{key}_sum"] = np.array(t.sum().item())
            blob[f"{pname}_{key}_abssum"] = np.array(t.abs().sum().item())
            blob[f"{pname}_{key}_absmax"] = np.array(t.abs().max().item())
        blob[f"{pname}_dsinks"] = res["dsinks"].detach().numpy().astype(np.float32)
        blob[f"{pname}_o_sample"] = res["o"][0, ::31, ::9, :].detach().numpy().astype(np.float32)
        blob[f"{pname}_dq_sample"] = res["dq"][0, ::9, ::31, :].detach().numpy().astype(np.float32)
        blob[f"{pname}_dk_sample"] = res["dk"][0, :, ::31, :].detach().numpy().astype(np.float32)
        blob[f"{pname}_dv_sample"] = res["dv"][0, :, ::31, :].detach().numpy().astype(np.float32)
    blob["input_abssum"] = np.array([t.double().abs().sum().item() for t in (q, k, v, do, sinks)])
    np.savez_compressed(os.path.join(HERE, "cfg1_digest.npz"), **blob)
    print("cfg1 digest written")


if __name__ == "__main__":
    main()
