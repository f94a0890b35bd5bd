"""The oracle against the reference-made golden fixtures (CPU only)."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR, load_golden, valid_rows_view
from oracle import (CONFIGS, AttnCase, algorithmic_bytes, algorithmic_flops,
                    attention_fwd_bwd_blockwise, attention_fwd_bwd_dense, make_inputs, rel_err,
                    visible_mask, visible_pairs)
from oracle.c_ref import attention_fwd_bwd_c

TOL = 2e-6  # fp32 restatement vs fp32 reference run: rounding-order differences only


def _check_against_golden(res, g, tol=TOL):
    lens = g["seqlens"] or [g["S"]] * g["B"]
    for key in ("dk", "dv", "dsinks"):
        assert rel_err(res[key], g["hf_" + key]) < tol, key
    for b, L in enumerate(lens):
        assert rel_err(valid_rows_view(res["o"], "bshd", b, L), valid_rows_view(g["hf_o"], "bshd", b, L)) < tol
        assert rel_err(valid_rows_view(res["dq"], "bhsd", b, L), valid_rows_view(g["hf_dq"], "bhsd", b, L)) < tol
        assert rel_err(res["lse"][b, :, :L], g["triton_lse"][b, :, :L]) < tol
    assert rel_err(res["dsinks"], g["triton_dsinks"]) < tol


def test_fixture_producers_agree(golden):
    # transformers' eager function and the reference's Triton kernel, both run in fp32
    assert float(golden["hf_vs_triton_rel"].max()) < TOL


def test_dense_matches_golden(golden):
    g = golden
    res = attention_fwd_bwd_dense(g["q"], g["k"], g["v"], g["sinks"], g["do"], g["scale"], g["window"], g["seqlens"])
    _check_against_golden(res, g)


@pytest.mark.parametrize("row_block", [37, 128, 1024])
def test_blockwise_matches_golden(golden, row_block):
    g = golden
    res = attention_fwd_bwd_blockwise(g["q"], g["k"], g["v"], g["sinks"], g["do"], g["scale"], g["window"],
                                      g["seqlens"], row_block=row_block)
    _check_against_golden(res, g)


def test_c_restatement_matches_golden(golden):
    g = golden
    res = attention_fwd_bwd_c(g["q"].numpy(), g["k"].numpy(), g["v"].numpy(), g["sinks"].numpy(),
                              g["do"].numpy(), g["scale"], g["window"], g["seqlens"])
    _check_against_golden({k: torch.from_numpy(v) for k, v in res.items()}, g)


def test_cfg1_digest():
    z = np.load(os.path.join(GOLDEN_DIR, "cfg1_digest.npz"))
    case = CONFIGS["cfg1"]
    q, k, v, do, sinks = make_inputs(case)
    got = np.array([t.double().abs().sum().item() for t in (q, k, v, do, sinks)])
    np.testing.assert_allclose(got, z["input_abssum"], rtol=1e-9)  # generator drift guard
    res = attention_fwd_bwd_blockwise(q, k, v, sinks, do, case.scale, case.window, row_block=256)
    for prod in ("hf", "triton"):
        assert rel_err(res["dsinks"], torch.from_numpy(z[f"{prod}_dsinks"])) < TOL
        assert rel_err(res["o"][0, ::31, ::9, :], torch.from_numpy(z[f"{prod}_o_sample"])) < TOL
        assert rel_err(res["dq"][0, ::9, ::31, :], torch.from_numpy(z[f"{prod}_dq_sample"])) < TOL
        assert rel_err(res["dk"][0, :, ::31, :], torch.from_numpy(z[f"{prod}_dk_sample"])) < TOL
        assert rel_err(res["dv"][0, :, ::31, :], torch.from_numpy(z[f"{prod}_dv_sample"])) < TOL
        for key in ("o", "dq", "dk", "dv"):
            assert abs(res[key].double().abs().sum().item() / float(z[f"{prod}_{key}_abssum"]) - 1) < 1e-5


def test_fp64_blockwise_close_to_fp32():
    case = AttnCase("t", B=1, S=160, Hq=4, Hkv=2, window=64, seed=11)
    q, k, v, do, sinks = make_inputs(case)
    a = attention_fwd_bwd_blockwise(q, k, v, sinks, do, case.scale, case.window, dtype=torch.float64)
    b = attention_fwd_bwd_blockwise(q, k, v, sinks, do, case.scale, case.window, dtype=torch.float32)
    for key in ("o", "dq", "dk", "dv", "dsinks", "lse"):
        assert rel_err(b[key], a[key]) < TOL


def test_slices_argument_is_a_partition():
    case = AttnCase("t", B=2, S=96, Hq=4, Hkv=2, window=0, seed=12)
    q, k, v, do, sinks = make_inputs(case)
    full = attention_fwd_bwd_blockwise(q, k, v, sinks, do, case.scale)
    acc = None
    for b in range(2):
        for g in range(2):
            part = attention_fwd_bwd_blockwise(q, k, v, sinks, do, case.scale, slices=[(b, g)])
            acc = part if acc is None else {k_: acc[k_] + part[k_] for k_ in acc}
    for key in full:
        assert rel_err(acc[key], full[key]) < 1e-6


def test_window_keeps_exactly_w_keys_including_self():
    m = visible_mask(300, 128)
    assert int(m[299].sum()) == 128 and bool(m[299, 299]) and bool(m[299, 172]) and not bool(m[299, 171])
    assert int(m[5].sum()) == 6
    assert int(visible_mask(300, 0)[299].sum()) == 300


def test_sink_only_enters_the_denominator():
    # a huge sink logit drives the output to zero but never produces NaN
    case = AttnCase("t", B=1, S=32, Hq=2, Hkv=1, seed=13)
    q, k, v, do, _ = make_inputs(case)
    res = attention_fwd_bwd_dense(q, k, v, torch.tensor([60.0, -60.0]), do, case.scale)
    assert torch.isfinite(res["o"]).all() and res["o"][:, :, 0].abs().max() < 1e-12
    assert abs(res["dsinks"][1].item()) < 1e-12


def test_work_counts_match_the_published_table():
    assert visible_pairs(512, 128) == 57408
    assert algorithmic_flops(CONFIGS["cfg2"])["pairs_per_head"] == 33562624
    assert algorithmic_flops(CONFIGS["cfg3"])["pairs_per_head"] == 4178048
    assert abs(algorithmic_flops(CONFIGS["cfg2"])["total"] / 1.9246e12 - 1) < 1e-3
    assert abs(algorithmic_bytes(CONFIGS["cfg3"])["total"] / 1829e6 - 1) < 2e-3
    assert CONFIGS["cfg4_swa"].seqlens == (14090, 10808, 8875, 5168, 5752, 1653, 2179, 1277)


@pytest.mark.parametrize("window", [0, 16])
def test_packed_documents_equal_the_documents_taken_one_by_one(window):
    """The same-document mask of the dense oracle == running every document alone (dSinks adds up)."""
    bounds = [0, 1, 40, 40, 97, 128]
    case = AttnCase("t", B=1, S=bounds[-1], Hq=4, Hkv=2, window=window, seed=21)
    q, k, v, do, sinks = make_inputs(case)
    packed = attention_fwd_bwd_dense(q, k, v, sinks, do, case.scale, window, cu_seqlens=bounds)
    dsinks = torch.zeros_like(packed["dsinks"])
    for a, b in zip(bounds, bounds[1:]):
        if b == a:
            continue
        one = attention_fwd_bwd_dense(q[:, :, a:b], k[:, :, a:b], v[:, :, a:b], sinks, do[:, a:b], case.scale, window)
        assert rel_err(packed["o"][:, a:b], one["o"]) < TOL and rel_err(packed["lse"][:, :, a:b], one["lse"]) < TOL
        for key in ("dq", "dk", "dv"):
            assert rel_err(packed[key][:, :, a:b], one[key]) < TOL, key
        dsinks += one["dsinks"]
    assert rel_err(packed["dsinks"], dsinks) < TOL
