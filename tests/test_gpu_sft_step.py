"""The fine-tuning step harness (`python -m oregon_gpt_oss_patching_b200.sft_step`) at a tiny size.

The reference is used by patching HF's GptOss attention and then training (sft.py:16-53); the
harness does one such step -- forward, backward through gradient checkpointing, SGD update -- on a
random-weight model of the gpt-oss layer layout (64 query heads, 8 KV heads, alternating
sliding-window / full layers).  Run as a child process exactly as a user would, patched and
un-patched: both must finish, report the attention they used, and agree on the loss of the same
seeded batch after the same number of updates.
"""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = ["--layers", "2", "--experts", "4", "--vocab", "512", "--seq", "512", "--steps", "2", "--warmup", "0"]


def _run(extra):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-m", "oregon_gpt_oss_patching_b200.sft_step", *TINY, *extra],
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, proc.stdout[-2000:]
    return json.loads(lines[0])


def test_one_fine_tuning_step_patched_and_unpatched_agree():
    patched = _run([])
    eager = _run(["--unpatched", "--moe", "hf_eager"])
    assert patched["attention"] == "b200" and eager["attention"] == "hf_eager"
    assert patched["moe"] == "b200" and eager["moe"] == "hf_eager"
    assert patched["kernel_status"] == 0
    for rec in (patched, eager):
        assert rec["n_gpus"] == 1 and rec["config"]["seq_len"] == 512 and rec["config"]["layers"] == 2
        assert rec["value"] > 0 and rec["loss"] == rec["loss"]          # finite
    # same weights (seeded), same batch, two SGD updates each: the losses differ by bf16 rounding in attention and the expert block only
    assert abs(patched["loss"] - eager["loss"]) < 2e-2 * abs(eager["loss"]), (patched["loss"], eager["loss"])
    # the patched step never materialises the S x S score matrix
    assert patched["peak_mem_gb"] <= eager["peak_mem_gb"] + 0.05
