"""CPU/fp32 oracle for the GPT-OSS attention forward/backward path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: the product path is the CUDA library behind the C ABI and it fails
loudly when that library is missing.  Only the test-suite, the smoke check and
the benchmark's CPU-baseline leg may import ``oracle``.

What it restates
----------------
The arithmetic of the reference's hot path lives in a third-party dependency,
``transformers`` (requirement ``transformers>=4.55.0`` in the reference's
``requirements.txt:4``; 5.5.0 is the version the restatement was checked
against): ``models/gpt_oss/modeling_gpt_oss.py:245-273``
(``eager_attention_forward``) with the masks of ``masking_utils.py:74-78``
(causal) and ``masking_utils.py:90-97`` (sliding-window overlay).  The
reference's own flash kernel (``attention_kernel.py:11-217``) computes the same
function blockwise.

Parity pin
----------
The reference ships no tests or golden vectors, so the pin is made from the
reference itself run on CPU: ``tests/golden/make_golden.py`` calls (1) the
unmodified ``transformers`` eager function in fp32 and (2) the reference's
Triton kernels under the Triton CPU interpreter (fp32), and stores their
outputs as fixtures in ``tests/golden``.  ``tests/test_oracle.py`` checks
every oracle implementation here against those fixtures.

The steps either side of attention
----------------------------------
``moe_fp32`` restates the expert block (``modeling_gpt_oss.py:76-114``) and is pinned by
``tests/golden/moe_*.npz`` (made by ``tests/golden/make_golden_moe.py`` from the unmodified module);
``rope_fp32`` restates the rotary embedding (``modeling_gpt_oss.py:226-242``) and is pinned against
the installed function itself in ``tests/test_rope_oracle.py``.  Both are imported by name
(``oracle.moe_fp32``, ``oracle.rope_fp32``), by the tests and the smoke check only.
"""
from .eager_fp32 import (  # noqa: F401
    AttnCase,
    CONFIGS,
    attention_fwd_bwd_blockwise,
    attention_fwd_bwd_dense,
    visible_mask,
    make_inputs,
    rel_err,
    visible_pairs,
    algorithmic_flops,
    algorithmic_bytes,
)
