"""ctypes binding of the scalar C restatement ``oracle/attn_ref.c``.

TEST INFRASTRUCTURE ONLY -- see ``oracle/__init__.py``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "attn_ref.c")
_LIB = os.path.join(_HERE, "liboracle_attn.so")


def build(force: bool = False) -> str:
    """Compile ``attn_ref.c`` with gcc into ``oracle/liboracle_attn.so``."""
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(_SRC):
        subprocess.check_call(["gcc", "-O2", "-shared", "-fPIC", "-o", _LIB, _SRC, "-lm"])
    return _LIB


def _load():
    lib = ctypes.CDLL(build())
    fp = ctypes.POINTER(ctypes.c_float)
    ip = ctypes.POINTER(ctypes.c_int32)
    lib.oracle_attn_fwd_bwd.restype = ctypes.c_int
    lib.oracle_attn_fwd_bwd.argtypes = [fp, fp, fp, fp, fp, ip] + [ctypes.c_int] * 5 + \
        [ctypes.c_float, ctypes.c_int] + [fp] * 6
    return lib


def attention_fwd_bwd_c(q, k, v, sinks, do, scale, window=0, seqlens=None):
    """numpy in / numpy out.  q (B,Hq,S,d), k,v (B,Hkv,S,d), do (B,S,Hq,d), sinks (Hq,)."""
    lib = _load()
    q, k, v, sinks, do = (np.ascontiguousarray(np.asarray(t, dtype=np.float32))
                          for t in (q, k, v, sinks, do))
    B, Hq, S, d = q.shape
    Hkv = k.shape[1]
    out = {"o": np.empty((B, S, Hq, d), np.float32), "lse": np.empty((B, Hq, S), np.float32),
           "dq": np.empty_like(q), "dk": np.empty_like(k), "dv": np.empty_like(v),
           "dsinks": np.empty((Hq,), np.float32)}
    fp = ctypes.POINTER(ctypes.c_float)
    ptr = lambda a: a.ctypes.data_as(fp)
    if seqlens is not None:
        sl = np.ascontiguousarray(np.asarray(seqlens, dtype=np.int32))
        slp = sl.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
    else:
        slp = None
    rc = lib.oracle_attn_fwd_bwd(ptr(q), ptr(k), ptr(v), ptr(sinks), ptr(do), slp, B, Hq, Hkv, S, d,
                                 float(scale), int(window), ptr(out["o"]), ptr(out["lse"]),
                                 ptr(out["dq"]), ptr(out["dk"]), ptr(out["dv"]), ptr(out["dsinks"]))
    if rc != 0:
        raise RuntimeError(f"oracle_attn_fwd_bwd failed: {rc}")
    return out
