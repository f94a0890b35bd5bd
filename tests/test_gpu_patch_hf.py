"""The drop-in boundary: HF's GptOss model with and without the patch (tiny random model, GPU).

Mirrors how the reference is used (sft.py:18: patch, then train): the same model and batch run
un-patched (HF eager attention, fp32 and bf16) and patched (bf16, B200 kernels); loss and every
parameter gradient -- the sink logits included -- must agree with the fp32 eager run to bf16
accuracy, and no worse than HF's own bf16 eager path does.
"""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tiny_model(dtype):
    from transformers import GptOssConfig, GptOssForCausalLM
    cfg = GptOssConfig(vocab_size=512, hidden_size=128, intermediate_size=128, num_hidden_layers=2,
                       num_attention_heads=8, num_key_value_heads=2, head_dim=64, sliding_window=64,
                       # every expert is used by every token: top-k routing is discontinuous, and a one-ulp
                       # difference between two bf16 attention paths can otherwise flip a token's experts
                       num_local_experts=4, num_experts_per_tok=4, max_position_embeddings=1024,
                       layer_types=["sliding_attention", "full_attention"], attention_dropout=0.0)
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    model = GptOssForCausalLM(cfg).to(DEV)
    with torch.no_grad():
        for layer in model.model.layers:
            layer.self_attn.sinks.normal_()      # sinks are created uninitialised
    return model.to(dtype)


def _run(model, ids, mask, labels):
    model.zero_grad(set_to_none=True)
    out = model(input_ids=ids, attention_mask=mask, labels=labels, use_cache=False)
    out.loss.backward()
    return out.loss.detach().float(), {n: p.grad.detach().float().clone() for n, p in model.named_parameters() if p.grad is not None}


def _rel(a, b):
    return (a - b).abs().max().item() / max(b.abs().max().item(), 1e-12)


def test_patched_model_matches_unpatched_eager():
    from oregon_gpt_oss_patching_b200 import patching
    from transformers.models.gpt_oss import modeling_gpt_oss
    g = torch.Generator().manual_seed(1)
    B, S = 2, 200
    ids = torch.randint(0, 512, (B, S), generator=g).to(DEV)
    mask = torch.ones(B, S, dtype=torch.long, device=DEV)
    mask[1, 137:] = 0                                   # right padding
    labels = ids.clone()
    labels[mask == 0] = -100

    ref_model = _tiny_model(torch.float32)
    bf_model = copy.deepcopy(ref_model).to(torch.bfloat16)
    loss_ref, grads_ref = _run(ref_model, ids, mask, labels)
    loss_eager, grads_eager = _run(bf_model, ids, mask, labels)

    original = modeling_gpt_oss.eager_attention_forward
    patching.patch_flash_attention()
    try:
        assert modeling_gpt_oss.eager_attention_forward is not original
        loss_b200, grads_b200 = _run(bf_model, ids, mask, labels)
    finally:
        patching.unpatch_flash_attention()
    assert modeling_gpt_oss.eager_attention_forward is original

    assert abs(loss_b200.item() - loss_ref.item()) < 2e-2 * abs(loss_ref.item())
    assert set(grads_b200) == set(grads_ref)
    worst_b200 = worst_eager = 0.0
    table = {name: (_rel(grads_b200[name], grads_ref[name]), _rel(grads_eager[name], grads_ref[name])) for name in grads_ref}
    for name, (e_b200, e_eager) in table.items():
        worst_b200, worst_eager = max(worst_b200, e_b200), max(worst_eager, e_eager)
    for name, (e_b200, e_eager) in table.items():
        assert e_b200 < max(5e-2, 2.0 * e_eager), (name, e_b200, e_eager, sorted(table.items(), key=lambda kv: -kv[1][0])[:6])
    sink_names = [n for n in grads_ref if n.endswith("sinks")]
    assert len(sink_names) == 2
    for n in sink_names:
        assert _rel(grads_b200[n], grads_ref[n]) < 3e-2, n
    print(f"loss fp32 {loss_ref.item():.5f} bf16-eager {loss_eager.item():.5f} bf16-b200 {loss_b200.item():.5f}; "
          f"worst grad error vs fp32: b200 {worst_b200:.2e}, HF bf16 eager {worst_eager:.2e}")


def test_adapter_signature_and_return_contract():
    """(out, None) with out (B,S,Hq,d), sinks and window read from the module, extra kwargs ignored."""
    import types
    from oregon_gpt_oss_patching_b200 import triton_flash_attention
    from oracle import AttnCase, make_inputs
    case = AttnCase("t", B=1, S=130, Hq=8, Hkv=2, window=64, seed=2)
    q, k, v, _, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    module = types.SimpleNamespace(sinks=sinks.to(torch.bfloat16), sliding_window=64, num_key_value_groups=4, training=True)
    out, weights = triton_flash_attention(module, q, k, v, None, scaling=case.scale, dropout=0.0,
                                          sliding_window=64, s_aux=module.sinks, position_ids=None)
    assert weights is None and out.shape == (1, 130, 8, 64) and out.is_contiguous() and out.dtype == torch.bfloat16
