"""The backward entry point that takes no scratch from the caller.

Some callers of the library cannot allocate device memory when they need a backward pass (all
memory already committed to their own pool, or an allocation's latency / implicit sync is not
acceptable where they run).  `b200attn_bwd_static_scratch` keeps its two scratch buffers in a
fixed array inside the library instead.  This test calls it through the C ABI twice in a row
-- the second call sees the first call's leftovers in the shared array -- and checks every
output bit-for-bit against the ordinary entry point, then checks the size limit is enforced.
It is collected last so that a run stopping at the first failure has run everything else.
"""
import ctypes

import pytest
import torch

from oracle import AttnCase, make_inputs
from oregon_gpt_oss_patching_b200 import _cabi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup(case, seed_shift=0):
    lib = _cabi.load()
    import dataclasses
    q, k, v, do, sinks = make_inputs(dataclasses.replace(case, seed=case.seed + seed_shift), dtype=torch.bfloat16, device=DEV)
    B, Hq, S, d = q.shape
    S_pad = _cabi.padded_len(S)
    t = {"q": q, "k": k, "v": v, "do": do, "sinks": sinks.float().contiguous(),
         "o": torch.empty(B, S, Hq, d, dtype=torch.bfloat16, device=DEV),
         "lse": torch.empty(B, Hq, S_pad, device=DEV), "status": torch.zeros(1, dtype=torch.int32, device=DEV)}
    p = _cabi.Params()
    p.B, p.Hq, p.Hkv, p.S, p.d, p.window, p.scale, p.device = B, Hq, k.shape[1], S, d, case.window, case.scale, 0
    p.stream, p.status, p.sinks = None, t["status"].data_ptr(), t["sinks"].data_ptr()
    p.q, p.k, p.v = (_cabi.tensor4(x, "bhsd") for x in (q, k, v))
    p.o, p.d_o, p.lse = _cabi.tensor4(t["o"], "bshd"), _cabi.tensor4(do, "bshd"), t["lse"].data_ptr()
    assert lib.b200attn_fwd(ctypes.byref(p)) == 0
    return lib, p, t


def _outputs(p, q, k, v, Hq):
    out = {"dq": torch.full_like(q, float("nan")), "dk": torch.full_like(k, float("nan")),
           "dv": torch.full_like(v, float("nan")), "dsinks": torch.full((Hq,), float("nan"), device=DEV)}
    p.dq, p.dk, p.dv = (_cabi.tensor4(out[x], "bhsd") for x in ("dq", "dk", "dv"))
    p.dsinks = out["dsinks"].data_ptr()
    return out


@pytest.mark.parametrize("window", [0, 128])
def test_static_scratch_backward_matches_the_allocating_one_twice_in_a_row(window):
    for call, (S, shift) in enumerate(((640, 0), (384, 1))):   # second call: other data, other size
        case = AttnCase("t", B=2, S=S, Hq=16, Hkv=2, window=window, seed=21)
        lib, p, t = _setup(case, shift)
        # ordinary entry point with caller-owned scratch
        want = _outputs(p, t["q"], t["k"], t["v"], 16)
        delta = torch.empty(_cabi.DELTA_PLANES, 2, 16, _cabi.padded_len(S), device=DEV)
        part = torch.empty(int(lib.b200attn_dsinks_scratch_floats(ctypes.byref(p))), device=DEV)
        p.delta, p.dsinks_partial = delta.data_ptr(), part.data_ptr()
        assert lib.b200attn_bwd(ctypes.byref(p)) == 0
        # entry point under test: no scratch passed at all
        got = _outputs(p, t["q"], t["k"], t["v"], 16)
        p.delta, p.dsinks_partial = None, None
        assert lib.b200attn_bwd_static_scratch(ctypes.byref(p)) == 0
        torch.cuda.synchronize()
        assert t["status"].item() == 0
        for key in want:
            assert not torch.isnan(got[key].float()).any(), (call, key)
            assert torch.equal(got[key], want[key]), (call, key)   # same kernels, same inputs: bit-identical


def test_static_scratch_rejects_problems_beyond_its_limit():
    lib = _cabi.load()
    p = _cabi.Params()
    p.B, p.Hq, p.Hkv, p.S, p.d, p.scale, p.device = 2, 64, 8, 16384, 64, 0.125, 0   # 2*64*16384 rows > 2^18
    assert lib.b200attn_bwd_static_scratch(ctypes.byref(p)) == -9
    assert b"B200ATTN_STATIC_MAX_ROWS" in lib.b200attn_strerror(-9)
