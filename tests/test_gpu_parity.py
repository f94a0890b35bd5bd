"""CUDA path vs the oracle and the reference-made golden fixtures.  All through the C ABI."""
import ctypes

import pytest
import torch

from conftest import GOLDEN_CASES, load_golden
from gpu_util import (TOL_DSINKS, TOL_LSE, TOL_TENSOR, assert_close_valid, oracle_on_gpu, run_b200)
from oracle import CONFIGS, AttnCase, make_inputs, rel_err
from oregon_gpt_oss_patching_b200 import _cabi
from oregon_gpt_oss_patching_b200.attention_kernel import attention, last_status

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_umma_building_blocks(mode):
    lib = _cabi.load()
    g = torch.Generator().manual_seed(mode)
    a = torch.randn(128, 128 if mode == 1 else 64, generator=g).to(torch.bfloat16).to(DEV)
    b = torch.randn(128, 64, generator=g).to(torch.bfloat16).to(DEV)
    n = 64 if mode == 1 else 128
    d = torch.full((128, n), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = lib.b200attn_umma_selftest(mode, a.data_ptr(), b.data_ptr(), d.data_ptr(), status.data_ptr(), 0, None)
    torch.cuda.synchronize()
    assert rc == 0 and status.item() == 0
    ref = a.float() @ (b.float() if mode == 1 else b.float().t())
    if mode == 2:   # one more k-step from unswizzled side operands: the first 16 columns again
        ref = ref + a.float()[:, :16] @ b.float()[:, :16].t()
    assert rel_err(d, ref) < 1e-5


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_fixture_parity(name):
    g = load_golden(name)
    q, k, v, do = (g[x].to(torch.bfloat16).to(DEV) for x in ("q", "k", "v", "do"))
    res = run_b200(q, k, v, do, g["sinks"].to(DEV), g["scale"], g["window"], g["seqlens"])
    lens = g["seqlens"] or [g["S"]] * g["B"]
    ref = {key: g["hf_" + key] for key in ("o", "dq", "dk", "dv", "dsinks")}
    assert_close_valid(res, ref, lens, g["S"])
    assert last_status(DEV) == 0


@pytest.mark.parametrize("name", ["full_s200_2kv", "pad_swa128"])
def test_lse_and_delta_stage(name):
    """Forward LSE vs the reference kernel's; preprocess stage delta vs rowsum(dO*O)."""
    g = load_golden(name)
    lib = _cabi.load()
    q, k, v, do = (g[x].to(torch.bfloat16).to(DEV) for x in ("q", "k", "v", "do"))
    B, Hq, S, d = q.shape
    sinks = g["sinks"].to(DEV).float()
    sl = torch.tensor(g["seqlens"], dtype=torch.int32, device=DEV) if g["seqlens"] else None
    o = torch.empty(B, S, Hq, d, dtype=torch.bfloat16, device=DEV)
    S_pad = _cabi.padded_len(S)
    lse = torch.full((B, Hq, S_pad), float("nan"), device=DEV)
    delta = torch.full((_cabi.DELTA_PLANES, B, Hq, S_pad), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    p = _cabi.Params()
    p.B, p.Hq, p.Hkv, p.S, p.d, p.window, p.scale, p.device = B, Hq, k.shape[1], S, d, g["window"], g["scale"], 0
    p.stream, p.status, p.sinks = None, status.data_ptr(), sinks.data_ptr()
    p.seqlens = sl.data_ptr() if sl is not None else None
    p.q, p.k, p.v = (_cabi.tensor4(t, "bhsd") for t in (q, k, v))
    p.o, p.d_o, p.lse, p.delta = _cabi.tensor4(o, "bshd"), _cabi.tensor4(do, "bshd"), lse.data_ptr(), delta.data_ptr()
    part = torch.empty(int(lib.b200attn_dsinks_scratch_floats(ctypes.byref(p))), device=DEV)
    dsinks = torch.empty(Hq, device=DEV)
    p.dsinks_partial, p.dsinks = part.data_ptr(), dsinks.data_ptr()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    p.dq, p.dk, p.dv = (_cabi.tensor4(t, "bhsd") for t in (dq, dk, dv))
    assert lib.b200attn_fwd(ctypes.byref(p)) == 0
    # the stages in the order b200attn_bwd runs them (for a narrow window the dkdv stage also makes dQ and the
    # dq stage returns at once)
    assert lib.b200attn_bwd_dq_is_fused(ctypes.byref(p)) == (1 if 0 < g["window"] <= 128 else 0)
    assert lib.b200attn_bwd_preprocess(ctypes.byref(p)) == 0
    assert lib.b200attn_bwd_dkdv(ctypes.byref(p)) == 0
    assert lib.b200attn_bwd_dq(ctypes.byref(p)) == 0
    assert lib.b200attn_bwd_dsinks(ctypes.byref(p)) == 0
    torch.cuda.synchronize()
    assert status.item() == 0
    lens = g["seqlens"] or [S] * B
    want_delta = (do.float() * o.float()).sum(-1).transpose(1, 2)  # (B,Hq,S)
    for b, L in enumerate(lens):
        assert rel_err(lse[b, :, :L], g["triton_lse"][b, :, :L]) < TOL_LSE
        assert rel_err(delta[0, b, :, :L], want_delta[b, :, :L]) < 1e-5
        assert float(delta[0, b, :, L:].abs().max() if L < S_pad else 0.0) == 0.0
        if lib.b200attn_bwd_dq_is_fused(ctypes.byref(p)):   # second plane: the sink's probability per row, 0 in padding
            want_w = torch.exp(sinks[:, None] - lse[b, :, :L])
            assert rel_err(delta[1, b, :, :L], want_w) < 1e-5
            assert float(delta[1, b, :, L:].abs().max() if L < S_pad else 0.0) == 0.0
    assert rel_err(dsinks, g["hf_dsinks"]) < TOL_DSINKS


@pytest.mark.parametrize("S,window,Hq,Hkv,B", [
    (64, 0, 8, 1, 1), (1, 0, 2, 1, 1), (127, 0, 2, 2, 2), (129, 128, 8, 1, 1), (255, 64, 4, 2, 1),
    (384, 128, 8, 1, 2), (640, 0, 16, 2, 1), (513, 256, 8, 4, 1), (1000, 128, 8, 1, 1), (300, 1, 2, 1, 1),
    # windows either side of the switch of the dK/dV kernel variants (256),
    # an odd group size (one query head per work item), and enough work items for several rounds per CTA
    (1000, 200, 6, 2, 2), (1500, 256, 8, 1, 2), (1500, 257, 8, 2, 1), (20000, 128, 8, 1, 1), (9000, 100, 3, 1, 2),
    # either side of the dQ (1024) and forward (4096) switches between persistent and one-item kernels
    (3000, 1024, 8, 2, 1), (3000, 1025, 8, 2, 1), (6000, 4096, 4, 1, 1), (6000, 4097, 4, 1, 1),
])
def test_odd_shapes_vs_oracle(S, window, Hq, Hkv, B):
    case = AttnCase("t", B=B, S=S, Hq=Hq, Hkv=Hkv, window=window, seed=100 + S)
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    res = run_b200(q, k, v, do, sinks, case.scale, window)
    ref = oracle_on_gpu(q, k, v, do, sinks, case.scale, window, row_block=256)
    assert_close_valid(res, ref, [S] * B, S)
    assert last_status(DEV) == 0


@pytest.mark.parametrize("window", [0, 128, 200])
def test_ragged_padding(window):
    lens = (700, 1, 129, 512)
    case = AttnCase("t", B=4, S=768, Hq=8, Hkv=2, window=window, seqlens=lens, seed=7)
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    res = run_b200(q, k, v, do, sinks, case.scale, window, lens)
    ref = oracle_on_gpu(q, k, v, do, sinks, case.scale, window, lens, row_block=256)
    assert_close_valid(res, ref, lens, 768)
    # gradient sent to padding rows must not matter
    do2 = do.clone()
    do2[1, 1:] = 3.0
    res2 = run_b200(q, k, v, do2, sinks, case.scale, window, lens)
    for key in res:
        assert torch.equal(res[key], res2[key]), key


def test_hf_strided_value_layout_and_bshd_views():
    """V as HF hands it over with use_cache=False: a (B,S,Hkv,d) buffer viewed as (B,Hkv,S,d)."""
    case = AttnCase("t", B=2, S=320, Hq=16, Hkv=2, window=128, seed=5)
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    v_strided = v.transpose(1, 2).contiguous().transpose(1, 2)
    q_strided = q.transpose(1, 2).contiguous().transpose(1, 2)
    assert not v_strided.is_contiguous()
    a = run_b200(q, k, v, do, sinks, case.scale, 128)
    b = run_b200(q_strided, k, v_strided, do, sinks, case.scale, 128)
    for key in a:
        assert torch.equal(a[key], b[key]), key
    # dO arriving as a non-contiguous view
    do_view = do.transpose(1, 2).contiguous().transpose(1, 2)
    c = run_b200(q, k, v, do_view, sinks, case.scale, 128)
    for key in a:
        assert torch.equal(a[key], c[key]), key


def test_bitwise_deterministic():
    case = AttnCase("t", B=2, S=1024, Hq=16, Hkv=2, window=0, seed=9)
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    a = run_b200(q, k, v, do, sinks, case.scale, 0)
    b = run_b200(q, k, v, do, sinks, case.scale, 0)
    for key in a:
        assert torch.equal(a[key], b[key]), key


def test_cfg1_shape_bf16():
    case = CONFIGS["cfg1"]
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    res = run_b200(q, k, v, do, sinks, case.scale, case.window)
    ref = oracle_on_gpu(q, k, v, do, sinks, case.scale, case.window)
    errs = assert_close_valid(res, ref, [case.S], case.S)
    print("cfg1 errors", errs)


def test_large_sink_and_extreme_logits_stay_finite():
    case = AttnCase("t", B=1, S=256, Hq=4, Hkv=1, window=0, seed=3, input_scale=4.0)
    q, k, v, do, _ = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    sinks = torch.tensor([60.0, -60.0, 0.0, 5.0], device=DEV)
    res = run_b200(q, k, v, do, sinks, case.scale, 0)
    ref = oracle_on_gpu(q, k, v, do, sinks, case.scale, 0)
    assert_close_valid(res, ref, [256], 256, tol_tile=None)


def test_packed_window_layer_with_extreme_sinks_and_logits():
    """The 8-heads-per-group, window-128 kernels exponentiate against the sink logit and redo rows that would
    overflow: logits far above and far below the sink, and an early sequence end, must all come out right."""
    case = AttnCase("t", B=2, S=700, Hq=16, Hkv=2, window=128, seed=31, input_scale=4.0, seqlens=(700, 333))
    q, k, v, do, _ = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    sinks = torch.tensor([60.0, -60.0, 0.0, 5.0, -120.0, 120.0, 30.0, -30.0] * 2, device=DEV)
    res = run_b200(q, k, v, do, sinks, case.scale, 128, case.seqlens)
    ref = oracle_on_gpu(q, k, v, do, sinks, case.scale, 128, case.seqlens)
    assert_close_valid(res, ref, case.lengths(), 700, tol_tile=None)
    assert last_status(DEV) == 0


# ---- the benchmark configurations at full size ------------------------------------------------
# The dense oracle cannot hold S x S logits at these sizes; the blockwise fp32 oracle is run on
# the GPU over every (batch, KV-group) slice, so all five results -- dSinks included, which needs
# every slice -- are compared everywhere, whole-tensor and tile by tile, plus size-independent
# properties of the result (finite, padding rows exactly zero, backward exactly linear in dO).
def _check_config(case, check_linearity=True, row_block=1024):
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    lens = case.lengths()
    res = run_b200(q, k, v, do, sinks, case.scale, case.window, case.seqlens)
    ref = oracle_on_gpu(q, k, v, do, sinks, case.scale, case.window, case.seqlens, row_block=row_block)
    errs = assert_close_valid(res, ref, lens, case.S)
    del ref
    for key in res:
        assert torch.isfinite(res[key].float()).all(), key
    for b, L in enumerate(lens):
        if L < case.S:
            assert float(res["dk"][b, :, L:].float().abs().max()) == 0.0 and float(res["dv"][b, :, L:].float().abs().max()) == 0.0
    if check_linearity:
        # backward is linear in dO: doubling dO doubles every gradient exactly (powers of two are exact in bf16)
        res2 = run_b200(q, k, v, do * 2, sinks, case.scale, case.window, case.seqlens)
        for key in ("dq", "dk", "dv", "dsinks"):
            assert torch.equal(res2[key].float(), res[key].float() * 2), key
    assert last_status(DEV) == 0
    return res, errs


def test_cfg2_full_causal_full_size():
    _, errs = _check_config(CONFIGS["cfg2"])
    print("cfg2 errors", errs)


def test_cfg3_sliding_window_full_size():
    _, errs = _check_config(CONFIGS["cfg3"], row_block=2048)
    print("cfg3 errors", errs)


@pytest.mark.parametrize("name", ["cfg4_swa", "cfg4_full"])
def test_cfg4_padded_batch_full_size(name):
    _, errs = _check_config(CONFIGS[name], check_linearity=(name == "cfg4_swa"))
    print(name, "errors", errs)


def test_cfg3_full_causal_at_16k():
    _, errs = _check_config(CONFIGS["cfg3_full"], check_linearity=False)
    print("cfg3_full errors", errs)
