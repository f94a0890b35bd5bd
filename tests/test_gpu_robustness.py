"""Robustness of the CUDA path: the give-up path of the bounded waits, guard bands around every
buffer the kernels write, masks the length reduction cannot express, and the sharded (by KV-head
group) form of a call reproducing the single call bit for bit.  Nothing here faults, traps or hangs
a GPU: the one wait that runs out is a few hundred microseconds long and returns a status."""
import ctypes

import pytest
import torch

from gpu_util import assert_close_valid, oracle_on_gpu, run_b200
from oracle import AttnCase, make_inputs
from oregon_gpt_oss_patching_b200 import _cabi
from oregon_gpt_oss_patching_b200.attention_kernel import (attention, check_status, last_status, seqlens_from_mask,
                                                           _status_word)
from oregon_gpt_oss_patching_b200.sharding import shard_by_group

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---- (i) a bounded wait that runs out -----------------------------------------------------------
def test_a_wait_that_runs_out_returns_a_status_and_leaves_the_device_usable():
    lib = _cabi.load()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert lib.b200attn_wait_selftest(1_000_000, status.data_ptr(), 0, None) == 0   # ~0.5 ms of SM clock
    torch.cuda.synchronize()
    assert status.item() == _cabi.STATUS_WAIT_TIMEOUT
    assert lib.b200attn_wait_selftest(0, status.data_ptr(), 0, None) == -1          # limit out of range
    assert lib.b200attn_wait_selftest(10**12, status.data_ptr(), 0, None) == -1
    # tensor memory was released and the context is intact: the tensor-core self-test and an attention call pass
    a = torch.randn(128, 64).to(torch.bfloat16).to(DEV)
    b = torch.randn(128, 64).to(torch.bfloat16).to(DEV)
    d = torch.empty(128, 128, device=DEV)
    status.zero_()
    assert lib.b200attn_umma_selftest(0, a.data_ptr(), b.data_ptr(), d.data_ptr(), status.data_ptr(), 0, None) == 0
    torch.cuda.synchronize()
    assert status.item() == 0 and torch.allclose(d, a.float() @ b.float().t(), atol=1e-3)
    case = AttnCase("t", B=1, S=300, Hq=8, Hkv=1, window=128, seed=11)
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    res = run_b200(q, k, v, do, sinks, case.scale, case.window)
    assert_close_valid(res, oracle_on_gpu(q, k, v, do, sinks, case.scale, case.window), [300], 300)
    assert last_status(DEV) == 0


# ---- (ii) guard bands ---------------------------------------------------------------------------
SENTINEL_BF16 = 0x7FC1             # a NaN pattern no kernel produces, as int16
GAP = 8                            # sentinel rows between heads / after the last position


def _guarded_bf16(B, H, S, d, layout):
    """A (B,H,S,d) view [bhsd] or (B,S,H,d) view [bshd] inside a sentinel-filled buffer with GAP extra
    positions after every S and a band before and after the whole buffer."""
    band = 4096
    inner = (B, H, S + GAP, d) if layout == "bhsd" else (B, S + GAP, H, d)
    n = 1
    for x in inner:
        n *= x
    raw = torch.full((band + n + band,), SENTINEL_BF16, dtype=torch.int16, device=DEV)
    body = raw[band:band + n].view(torch.bfloat16).view(inner)
    view = body[:, :, :S] if layout == "bhsd" else body[:, :S]
    mask = torch.ones_like(raw, dtype=torch.bool)
    m_body = mask[band:band + n].view(inner)
    (m_body[:, :, :S] if layout == "bhsd" else m_body[:, :S]).fill_(False)
    return raw, view, mask


def _guarded_f32(numel):
    band = 1024
    raw = torch.full((band + numel + band,), float("nan"), device=DEV)
    raw.view(torch.int32).fill_(0x7FC00123)
    mask = torch.ones(raw.numel(), dtype=torch.bool, device=DEV)
    mask[band:band + numel] = False
    return raw, raw[band:band + numel], mask


@pytest.mark.parametrize("S,window,lens", [
    (1, 0, None), (127, 128, None), (129, 128, None), (1000, 128, None), (1000, 0, None),
    (300, 128, (300, 1, 129)), (300, 0, (17, 300, 128)), (520, 1024, None), (700, 5000, None),
])
def test_nothing_is_written_outside_the_buffers(S, window, lens):
    lib = _cabi.load()
    B = 3 if lens else 2
    Hq, Hkv, d = 8, 2, 64
    case = AttnCase("t", B=B, S=S, Hq=Hq, Hkv=Hkv, window=window, seqlens=lens, seed=40 + S)
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    S_pad = _cabi.padded_len(S)
    bufs = {"o": _guarded_bf16(B, Hq, S, d, "bshd"), "dq": _guarded_bf16(B, Hq, S, d, "bhsd"),
            "dk": _guarded_bf16(B, Hkv, S, d, "bhsd"), "dv": _guarded_bf16(B, Hkv, S, d, "bhsd")}
    p = _cabi.Params()
    p.B, p.Hq, p.Hkv, p.S, p.d, p.window, p.scale, p.device = B, Hq, Hkv, S, d, window, case.scale, 0
    fl = {"lse": _guarded_f32(B * Hq * S_pad), "delta": _guarded_f32(_cabi.DELTA_PLANES * B * Hq * S_pad),
          "dsinks": _guarded_f32(Hq)}
    fl["partial"] = _guarded_f32(int(lib.b200attn_dsinks_scratch_floats(ctypes.byref(p))))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    sinks_f = sinks.float().contiguous()
    sl = None if lens is None else torch.tensor(lens, dtype=torch.int32, device=DEV)
    p.stream, p.status, p.sinks = None, status.data_ptr(), sinks_f.data_ptr()
    p.seqlens = sl.data_ptr() if sl is not None else None
    p.q, p.k, p.v = (_cabi.tensor4(t, "bhsd") for t in (q, k, v))
    p.o, p.d_o = _cabi.tensor4(bufs["o"][1], "bshd"), _cabi.tensor4(do, "bshd")
    p.dq, p.dk, p.dv = (_cabi.tensor4(bufs[x][1], "bhsd") for x in ("dq", "dk", "dv"))
    p.lse, p.delta = fl["lse"][1].data_ptr(), fl["delta"][1].data_ptr()
    p.dsinks, p.dsinks_partial = fl["dsinks"][1].data_ptr(), fl["partial"][1].data_ptr()
    assert lib.b200attn_fwd(ctypes.byref(p)) == 0
    assert lib.b200attn_bwd(ctypes.byref(p)) == 0
    torch.cuda.synchronize()
    assert status.item() == 0
    for name, (raw, view, mask) in bufs.items():
        assert bool((raw[mask] == SENTINEL_BF16).all()), f"{name}: bytes outside the tensor were written"
        assert not torch.isnan(view.float()).any(), f"{name}: not fully written"
    for name, (raw, view, mask) in fl.items():
        assert bool((raw.view(torch.int32)[mask] == 0x7FC00123).all()), f"{name}: bytes outside the buffer were written"
    assert not torch.isnan(fl["lse"][1]).any() and not torch.isnan(fl["dsinks"][1]).any()
    # and the results in those strided, guarded buffers are the right ones
    res = {"o": bufs["o"][1], "dq": bufs["dq"][1], "dk": bufs["dk"][1], "dv": bufs["dv"][1], "dsinks": fl["dsinks"][1]}
    ref = oracle_on_gpu(q, k, v, do, sinks, case.scale, window, lens, row_block=256)
    assert_close_valid(res, ref, case.lengths(), S)


# ---- (iii) masks that are not right-padded ------------------------------------------------------
def test_left_padded_and_packed_masks_are_reported_not_silently_misread():
    B, S = 2, 64
    _status_word(torch.device(DEV)).zero_()
    right = torch.ones(B, S, dtype=torch.bool, device=DEV)
    right[1, 40:] = False
    assert seqlens_from_mask(right, B, S).tolist() == [64, 40]
    assert last_status(DEV) == 0
    check_status(DEV)                                   # nothing to report
    left = right.flip(-1)                               # padding first: a real token follows a padding token
    seqlens_from_mask(left, B, S)
    assert last_status(DEV) == _cabi.STATUS_NONPREFIX_MASK
    with pytest.raises(RuntimeError, match="not right-padded"):
        check_status(DEV)
    assert last_status(DEV) == 0                        # cleared by check_status
    # HF's additive 4-D form of a mask with a hole
    holed = torch.zeros(B, 1, S, S, device=DEV)
    holed[0, 0, 10, 10] = torch.finfo(torch.float32).min
    seqlens_from_mask(holed, B, S)
    with pytest.raises(RuntimeError, match="not right-padded"):
        check_status(DEV)


# ---- (iv) a call sharded by KV-head group equals the single call --------------------------------
@pytest.mark.parametrize("window,world", [(128, 2), (0, 4), (128, 8)])
def test_group_sharded_calls_reproduce_the_single_call_bit_for_bit(window, world):
    """What N ranks would each compute (their KV-head groups, all batches; views into the full tensors,
    so non-contiguous heads) concatenated == the one-GPU result, dSinks included: no reduction exists."""
    case = AttnCase("t", B=2, S=1500, Hq=64, Hkv=8, window=window, seed=77)
    q, k, v, do, sinks = make_inputs(case, dtype=torch.bfloat16, device=DEV)
    full = run_b200(q, k, v, do, sinks, case.scale, window)
    G = case.Hq // case.Hkv
    for rank in range(world):
        (qs, ks, vs, dos, ss), (g0, g1) = shard_by_group(q, k, v, do, sinks, rank, world)
        part = run_b200(qs, ks, vs, dos, ss, case.scale, window)
        assert torch.equal(part["o"], full["o"][:, :, g0 * G:g1 * G])
        assert torch.equal(part["dq"], full["dq"][:, g0 * G:g1 * G])
        assert torch.equal(part["dk"], full["dk"][:, g0:g1]) and torch.equal(part["dv"], full["dv"][:, g0:g1])
        assert torch.equal(part["dsinks"], full["dsinks"][g0 * G:g1 * G])
    assert last_status(DEV) == 0
