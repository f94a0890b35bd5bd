"""Loader and driver for the reference's own Triton attention as a GPU contender.

MEASUREMENT / TEST INFRASTRUCTURE ONLY: the shipped package never imports this file.  It
imports the UNMODIFIED reference module (``attention_kernel.py`` of the reference project:
``attention`` at :347, ``triton_flash_attention`` at :348-358) from, in this order,

  1. an explicit path (``--reference-path`` of bench.py, or ``$REFERENCE_PATH``),
  2. ``baseline/_ref`` (what ``baseline/install_ref.py`` installs; git-ignored),

and calls it through its stock public API on tensors the caller provides.  Nothing of this
repository's kernels is on that path.  When the module (or triton, or a GPU) is missing,
``load()`` returns ``(None, reason)`` and callers report "unavailable" -- never a guess.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from typing import Optional, Tuple

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEFAULT_DIR = os.path.join(ROOT, "baseline", "_ref")
_cache: dict = {}


def candidate_dirs(explicit: Optional[str] = None):
    out = []
    for p in (explicit, os.environ.get("REFERENCE_PATH"), DEFAULT_DIR):
        if p and p not in out:
            out.append(p)
    return out


def load(explicit: Optional[str] = None) -> Tuple[Optional[object], str]:
    """Import the reference's attention_kernel module.  Returns (module, where) or (None, why)."""
    key = explicit or ""
    if key in _cache:
        return _cache[key]
    try:
        import triton  # noqa: F401
    except Exception as e:  # pragma: no cover - triton is in the image
        _cache[key] = (None, f"triton cannot be imported: {e}")
        return _cache[key]
    reason = "no reference checkout found (looked in: " + ", ".join(candidate_dirs(explicit)) + ")"
    for d in candidate_dirs(explicit):
        path = os.path.join(d, "attention_kernel.py")
        if not os.path.exists(path):
            continue
        try:
            spec = importlib.util.spec_from_file_location("reference_attention_kernel", path)
            mod = importlib.util.module_from_spec(spec)
            sys.modules["reference_attention_kernel"] = mod
            spec.loader.exec_module(mod)
            _cache[key] = (mod, d)
            return _cache[key]
        except Exception as e:
            reason = f"importing {path} failed: {type(e).__name__}: {e}"
    _cache[key] = (None, reason)
    return _cache[key]


def fwd_bwd(mod, q, k, v, do, sinks, scale: float, window: int):
    """One forward+backward through the reference's ``attention`` (its autograd function).

    q (B,Hq,S,d), k/v (B,Hkv,S,d), do (B,S,Hq,d): bf16 CUDA tensors; sinks (Hq,) in the
    model dtype, as the attention module holds them.  ``window`` 0 means full causal (the
    reference takes ``None`` for that, attention_kernel.py:60-63).  Returns a dict like the
    test helpers' (o, dq, dk, dv, dsinks).
    """
    qq, kk, vv, ss = (t.detach().requires_grad_(True) for t in (q, k, v, sinks))
    o = mod.attention(qq, kk, vv, ss, scale, window if window else None, None)
    o.backward(do)
    return {"o": o.detach(), "dq": qq.grad, "dk": kk.grad, "dv": vv.grad, "dsinks": ss.grad}
