import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")
GOLDEN_CASES = ["full_s128", "full_s200_2kv", "swa64_s200", "swa128_s320", "pad_swa128", "pad_full"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _bits_to_f32(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(torch.float32)


def load_golden(name: str) -> dict:
    """Fixture -> dict with fp32 input tensors (bf16-representable), metadata and outputs."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    B, S, Hq, Hkv, d, window = (int(x) for x in z["meta"])
    g = {"name": name, "B": B, "S": S, "Hq": Hq, "Hkv": Hkv, "d": d, "window": window,
         "scale": 1.0 / d ** 0.5,
         "seqlens": [int(x) for x in z["seqlens"]] if bool(z["has_padding"]) else None}
    for key in ("q", "k", "v", "do", "sinks"):
        g[key] = _bits_to_f32(z[key + "_bits"])
    for key in z.files:
        if key.startswith(("hf_", "triton_")):
            g[key] = torch.from_numpy(z[key])
    return g


def valid_rows_view(t: torch.Tensor, kind: str, b: int, L: int) -> torch.Tensor:
    """Rows of sequence b that are inside its length. kind: 'bshd' (o, do) or 'bhsd' (q, dq)."""
    return t[b, :L] if kind == "bshd" else t[b, :, :L]


@pytest.fixture(params=GOLDEN_CASES)
def golden(request):
    return load_golden(request.param)
