"""ctypes binding of ``libb200attn.so`` (the C ABI declared in ``include/b200attn.h`` and ``include/b200moe.h``).

There is deliberately no fallback: if the library cannot be loaded, or a call returns an
error code, a ``RuntimeError`` is raised.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import build as _build

DELTA_PLANES = 6   # B200ATTN_DELTA_PLANES of include/b200attn.h: fp32-sized values per (b, h, padded row) in the delta scratch

EXPORTS = (
    "b200attn_version", "b200attn_sizeof_params", "b200attn_strerror", "b200attn_padded_len", "b200attn_dsinks_scratch_floats",
    "b200attn_fwd", "b200attn_bwd", "b200attn_bwd_preprocess", "b200attn_bwd_dsinks", "b200attn_bwd_dkdv",
    "b200attn_bwd_dq", "b200attn_bwd_dq_is_fused", "b200attn_bwd_static_scratch", "b200attn_umma_selftest",
    "b200attn_wait_selftest", "b200attn_rope",
    "b200moe_sizeof_gemm_params", "b200moe_grouped_gemm", "b200moe_gather_rows", "b200moe_combine_rows", "b200moe_row_dot",
    "b200moe_glu", "b200moe_glu_bwd", "b200moe_bias_grad", "b200moe_route",
)

ROW_TILE = 128
STATUS_WAIT_TIMEOUT = 1      # B200ATTN_STATUS_WAIT_TIMEOUT
STATUS_NONPREFIX_MASK = 2    # B200ATTN_STATUS_NONPREFIX_MASK


class Tensor4(ctypes.Structure):
    """``b200attn_tensor``: bf16 (batch, head, position, head_dim) view, element strides."""
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_h", ctypes.c_int64),
                ("stride_s", ctypes.c_int64)]


class Params(ctypes.Structure):
    """``b200attn_params`` -- field order and types mirror include/b200attn.h exactly."""
    _fields_ = [
        ("B", ctypes.c_int32), ("Hq", ctypes.c_int32), ("Hkv", ctypes.c_int32), ("S", ctypes.c_int32),
        ("d", ctypes.c_int32), ("window", ctypes.c_int32), ("scale", ctypes.c_float), ("device", ctypes.c_int32),
        ("stream", ctypes.c_void_p), ("status", ctypes.c_void_p), ("seqlens", ctypes.c_void_p),
        ("sinks", ctypes.c_void_p),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4), ("lse", ctypes.c_void_p),
        ("d_o", Tensor4), ("dq", Tensor4), ("dk", Tensor4), ("dv", Tensor4),
        ("delta", ctypes.c_void_p), ("dsinks", ctypes.c_void_p), ("dsinks_partial", ctypes.c_void_p),
    ]


MOE_ROW_ALIGN = 128          # B200MOE_ROW_ALIGN
MOE_ROWS_NN, MOE_ROWS_NT, MOE_INNER_TN = 0, 1, 2


class MoeGemmParams(ctypes.Structure):
    """``b200moe_gemm_params`` -- field order and types mirror include/b200moe.h exactly."""
    _fields_ = [
        ("op", ctypes.c_int32), ("num_groups", ctypes.c_int32), ("rows", ctypes.c_int32),
        ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32),
        ("offsets", ctypes.c_void_p), ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("bias", ctypes.c_void_p),
        ("d", ctypes.c_void_p), ("device", ctypes.c_int32), ("stream", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("glu_out", ctypes.c_void_p), ("max_ctas", ctypes.c_int32),
    ]


_lock = threading.Lock()
_lib = None


def lib_path() -> str:
    return os.environ.get("B200ATTN_LIB", _build.LIB_PATH)


def load() -> ctypes.CDLL:
    """Load (once) and return the library with prototypes set.  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} not found: the CUDA library has not been built "
                "(run `python -m oregon_gpt_oss_patching_b200.build`); there is no fallback path")
        lib = ctypes.CDLL(path)
        pp = ctypes.POINTER(Params)
        lib.b200attn_version.restype = ctypes.c_int
        lib.b200attn_version.argtypes = []
        lib.b200attn_sizeof_params.restype = ctypes.c_size_t
        lib.b200attn_sizeof_params.argtypes = []
        if lib.b200attn_sizeof_params() != ctypes.sizeof(Params):
            raise RuntimeError("b200attn_params layout mismatch between libb200attn.so and its Python mirror")
        lib.b200attn_strerror.restype = ctypes.c_char_p
        lib.b200attn_strerror.argtypes = [ctypes.c_int]
        lib.b200attn_padded_len.restype = ctypes.c_int64
        lib.b200attn_padded_len.argtypes = [ctypes.c_int64]
        lib.b200attn_dsinks_scratch_floats.restype = ctypes.c_int64
        lib.b200attn_dsinks_scratch_floats.argtypes = [pp]
        for name in ("b200attn_fwd", "b200attn_bwd", "b200attn_bwd_preprocess", "b200attn_bwd_dsinks",
                     "b200attn_bwd_dkdv", "b200attn_bwd_dq", "b200attn_bwd_dq_is_fused", "b200attn_bwd_static_scratch"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [pp]
        lib.b200attn_umma_selftest.restype = ctypes.c_int
        lib.b200attn_umma_selftest.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                               ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        lib.b200attn_wait_selftest.restype = ctypes.c_int
        lib.b200attn_wait_selftest.argtypes = [ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
        lib.b200attn_rope.restype = ctypes.c_int
        lib.b200attn_rope.argtypes = [ctypes.POINTER(Tensor4), ctypes.POINTER(Tensor4), vp, vp, i64, i64, i32, i32, i32, i32, i32, vp]
        lib.b200moe_sizeof_gemm_params.restype = ctypes.c_size_t
        lib.b200moe_sizeof_gemm_params.argtypes = []
        if lib.b200moe_sizeof_gemm_params() != ctypes.sizeof(MoeGemmParams):
            raise RuntimeError("b200moe_gemm_params layout mismatch between libb200attn.so and its Python mirror")
        lib.b200moe_grouped_gemm.restype = ctypes.c_int
        lib.b200moe_grouped_gemm.argtypes = [ctypes.POINTER(MoeGemmParams)]
        for name, args in (
            ("b200moe_gather_rows", [vp, vp, vp, vp, i32, i32, i32, vp]),
            ("b200moe_combine_rows", [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
            ("b200moe_row_dot", [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
            ("b200moe_glu", [vp, vp, i64, i32, i32, vp]),
            ("b200moe_glu_bwd", [vp, vp, vp, i64, i32, i32, vp]),
            ("b200moe_bias_grad", [vp, vp, vp, i32, i32, i32, vp]),
            ("b200moe_route", [vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, i32, vp]),
        ):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = args
        _lib = lib
    return _lib


def strerror(code: int) -> str:
    return load().b200attn_strerror(int(code)).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed: {strerror(code)} (code {code})")


def padded_len(S: int) -> int:
    return (int(S) + ROW_TILE - 1) // ROW_TILE * ROW_TILE


def tensor4(t, layout: str) -> Tensor4:
    """Describe a torch tensor as a (batch, head, position, head_dim) view.

    layout 'bhsd': dims are (B,H,S,d) as q/k/v arrive; 'bshd': dims are (B,S,H,d) as o/dO are.
    """
    st = t.stride()
    if st[3] != 1:
        raise RuntimeError("head_dim stride must be 1")
    if layout == "bhsd":
        return Tensor4(t.data_ptr(), st[0], st[1], st[2])
    if layout == "bshd":
        return Tensor4(t.data_ptr(), st[0], st[2], st[1])
    raise ValueError(layout)
