#!/usr/bin/env python
"""Install the unmodified reference checkout into ``baseline/_ref`` (git-ignored).

    python baseline/install_ref.py [--reference /path/to/checkout]

The reference project ships no packaging metadata (no setup.py / pyproject.toml), so
``pip install <checkout>`` refuses it.  This recipe copies the checkout to a temporary
directory, adds a three-line ``pyproject.toml`` that names its two importable modules
(``attention_kernel`` and ``patching``) and lets pip install that copy with
``--no-index --no-build-isolation --no-deps --target baseline/_ref``.  The module sources land
byte-for-byte as they are upstream; nothing of this repository is on their import path.

The result is what the GPU contender arm of ``bench.py`` (``triton_reference``) and
``tests/test_gpu_vs_triton.py`` import.  When the checkout is absent the script says so and exits 0.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TARGET = os.path.join(ROOT, "baseline", "_ref")
MODULES = ("attention_kernel", "patching")

PYPROJECT = """[build-system]
requires = ["setuptools"]
build-backend = "setuptools.build_meta"

[project]
name = "oregon-gpt-oss-patching-reference"
version = "0"

[tool.setuptools]
py-modules = ["attention_kernel", "patching"]
"""


def install(reference: str, target: str = TARGET, quiet: bool = True) -> bool:
    """Returns True when ``target`` holds the reference modules afterwards."""
    if not all(os.path.exists(os.path.join(reference, m + ".py")) for m in MODULES):
        return False
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "reference")
        shutil.copytree(reference, src)
        os.chmod(src, 0o755)
        with open(os.path.join(src, "pyproject.toml"), "w") as f:
            f.write(PYPROJECT)
        if os.path.isdir(target):
            shutil.rmtree(target)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", target, src]
        subprocess.check_call(cmd, stdout=subprocess.DEVNULL if quiet else None)
    for m in MODULES:   # the installed files must be the upstream bytes
        with open(os.path.join(reference, m + ".py"), "rb") as a, open(os.path.join(target, m + ".py"), "rb") as b:
            if a.read() != b.read():
                raise RuntimeError(f"{m}.py in {target} differs from the checkout")
    return True


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("REFERENCE_PATH", "/root/reference"))
    args = ap.parse_args()
    if install(args.reference, quiet=False):
        print(f"reference installed into {TARGET}")
    else:
        print(f"no reference checkout at {args.reference}: nothing installed")


if __name__ == "__main__":
    main()
