"""The C-ABI library without a GPU: it loads, exports every declared symbol, rejects bad arguments."""
import ctypes
import os
import re

import pytest
import torch

from oregon_gpt_oss_patching_b200 import _cabi, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _cabi.load()


def test_every_declared_symbol_is_exported(lib):
    declared = set()
    for name in ("b200attn.h", "b200moe.h"):
        header = open(os.path.join(ROOT, "include", name)).read()
        header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
        declared |= set(re.findall(r"\b(b200(?:attn|moe)_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_cabi.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_struct_mirror_matches(lib):
    assert lib.b200attn_sizeof_params() == ctypes.sizeof(_cabi.Params)
    assert lib.b200attn_version() == 1


def test_moe_struct_mirror_and_argument_validation(lib):
    assert lib.b200moe_sizeof_gemm_params() == ctypes.sizeof(_cabi.MoeGemmParams)
    assert lib.b200moe_grouped_gemm(None) == -1
    buf = torch.zeros(1 << 12, dtype=torch.bfloat16)
    off = torch.zeros(3, dtype=torch.int32)
    p = _cabi.MoeGemmParams(op=_cabi.MOE_ROWS_NN, num_groups=2, rows=256, N=64, K=64, offsets=off.data_ptr(),
                            a=buf.data_ptr(), b=buf.data_ptr(), d=buf.data_ptr(), device=0)
    p.rows = 200
    assert lib.b200moe_grouped_gemm(ctypes.byref(p)) == -2              # rows not a multiple of 128
    p.rows, p.N = 256, 60
    assert lib.b200moe_grouped_gemm(ctypes.byref(p)) == -4              # columns not a multiple of 8
    p.N, p.op = 64, 7
    assert lib.b200moe_grouped_gemm(ctypes.byref(p)) == -1              # unknown operation
    p.op, p.num_groups = _cabi.MOE_ROWS_NN, 1000
    assert lib.b200moe_grouped_gemm(ctypes.byref(p)) == -2              # too many groups
    assert lib.b200moe_gather_rows(None, None, None, None, 1, 8, 0, None) == -1
    assert lib.b200moe_glu(buf.data_ptr(), buf.data_ptr(), 4, 12, 0, None) == -4   # 12 columns: not a multiple of 8


def test_helpers(lib):
    assert lib.b200attn_padded_len(1) == 128 and lib.b200attn_padded_len(128) == 128
    assert lib.b200attn_padded_len(129) == 256 and _cabi.padded_len(16384) == 16384
    p = _cabi.Params()
    p.B, p.Hq, p.S = 2, 64, 300
    assert lib.b200attn_dsinks_scratch_floats(ctypes.byref(p)) == 64 * 2 * 3 * 9
    for code in range(0, -9, -1):
        assert b"unknown" not in lib.b200attn_strerror(code)
    assert b"unknown" in lib.b200attn_strerror(-99)


def test_argument_validation_needs_no_gpu(lib):
    assert lib.b200attn_fwd(None) == -1
    p = _cabi.Params()
    assert lib.b200attn_fwd(ctypes.byref(p)) == -1                      # sizes are zero
    p.B, p.Hq, p.Hkv, p.S, p.d, p.scale = 1, 8, 1, 128, 128, 0.125
    assert lib.b200attn_fwd(ctypes.byref(p)) == -3                      # head_dim
    p.d, p.Hkv = 64, 3
    assert lib.b200attn_fwd(ctypes.byref(p)) == -2                      # Hq % Hkv
    p.Hkv = 1
    assert lib.b200attn_fwd(ctypes.byref(p)) == -1                      # NULL pointers
    buf = torch.zeros(1 << 16, dtype=torch.bfloat16)
    f32 = torch.zeros(1 << 12, dtype=torch.float32)
    p.sinks, p.lse = f32.data_ptr(), f32.data_ptr()
    base = buf.data_ptr()
    for name in ("q", "k", "v", "o"):
        setattr(p, name, _cabi.Tensor4(base, 8 * 128 * 64, 128 * 64, 64))
    p.q = _cabi.Tensor4(base + 2, 8 * 128 * 64, 128 * 64, 64)
    assert lib.b200attn_fwd(ctypes.byref(p)) == -4                      # misaligned pointer
    p.q = _cabi.Tensor4(base, 8 * 128 * 64, 128 * 64, 60)
    assert lib.b200attn_fwd(ctypes.byref(p)) == -4                      # stride not % 8
    p.q = _cabi.Tensor4(base, 8 * 128 * 64, 128 * 64, 64)
    if not torch.cuda.is_available():
        assert lib.b200attn_fwd(ctypes.byref(p)) in (-5, -6)            # no sm_100 device


def test_python_wrapper_refuses_cpu_tensors():
    from oregon_gpt_oss_patching_b200 import attention
    q = torch.zeros(1, 8, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        attention(q, q[:, :1], q[:, :1], torch.zeros(8), 0.125, None, None)


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setenv("B200ATTN_LIB", "/nonexistent/libb200attn.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _cabi.load()


def test_seqlens_from_mask_forms():
    from oregon_gpt_oss_patching_b200.attention_kernel import seqlens_from_mask
    keep = torch.tensor([[1, 1, 1, 0], [1, 1, 1, 1]])
    assert seqlens_from_mask(keep, 2, 4).tolist() == [3, 4]
    assert seqlens_from_mask(keep.bool(), 2, 4).tolist() == [3, 4]
    neg = torch.finfo(torch.float32).min
    add = torch.zeros(2, 1, 4, 4)
    add[0, 0, :, 3] = neg
    add = add + torch.triu(torch.full((4, 4), neg), 1)
    assert seqlens_from_mask(add, 2, 4).tolist() == [3, 4]
    assert seqlens_from_mask(None, 2, 4) is None
    with pytest.raises(ValueError):
        seqlens_from_mask(torch.zeros(2, 5), 2, 4)


def test_delta_planes_constant_matches_the_header():
    import re
    from oregon_gpt_oss_patching_b200 import _cabi
    text = open(os.path.join(os.path.dirname(__file__), "..", "include", "b200attn.h")).read()
    assert int(re.search(r"#define B200ATTN_DELTA_PLANES (\d+)", text).group(1)) == _cabi.DELTA_PLANES
