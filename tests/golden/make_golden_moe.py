"""Generate the mixture-of-experts golden fixtures from the unmodified Hugging Face module.

Run once, in a container that has ``transformers``:

    python tests/golden/make_golden_moe.py

For every case of ``oracle.moe_fp32.MOE_CASES`` it builds ``GptOssExperts``
(``transformers/models/gpt_oss/modeling_gpt_oss.py:62-114``) in fp32 on the CPU, loads the seeded parameters,
runs its own ``forward`` (the per-expert loop with ``torch.where`` / ``index_add_``) and autograd, and stores
the output and every gradient.  Inputs are not stored: ``make_moe_inputs`` regenerates them from the seed.
Nothing here is imported by the library.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle.moe_fp32 import MOE_CASES, make_moe_inputs  # noqa: E402


def run_hf(case):
    from transformers.models.gpt_oss.configuration_gpt_oss import GptOssConfig
    from transformers.models.gpt_oss.modeling_gpt_oss import GptOssExperts

    hidden, idx, weights, w1, b1, w2, b2, dout = make_moe_inputs(case)
    cfg = GptOssConfig(hidden_size=case.hidden, intermediate_size=case.intermediate, num_local_experts=case.experts,
                       num_experts_per_tok=case.top_k)
    mod = GptOssExperts(cfg).to(torch.float32)
    with torch.no_grad():
        mod.gate_up_proj.copy_(w1)
        mod.gate_up_proj_bias.copy_(b1)
        mod.down_proj.copy_(w2)
        mod.down_proj_bias.copy_(b2)
    hidden.requires_grad_(True)
    weights.requires_grad_(True)
    out = mod(hidden, router_indices=idx, routing_weights=weights)
    out.backward(dout)
    return {"out": out.detach(), "dhidden": hidden.grad, "dweights": weights.grad, "dw1": mod.gate_up_proj.grad,
            "db1": mod.gate_up_proj_bias.grad, "dw2": mod.down_proj.grad, "db2": mod.down_proj_bias.grad}


def main():
    import transformers
    for name, case in MOE_CASES.items():
        res = run_hf(case)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, transformers_version=np.array(transformers.__version__),
                            **{k: v.numpy() for k, v in res.items()})
        print(name, {k: tuple(v.shape) for k, v in res.items()}, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
