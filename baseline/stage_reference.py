"""Stages the unmodified reference (shyampathak22/cinnamon) under ``baseline/_ref`` for side-by-side runs.

    python baseline/stage_reference.py [REFERENCE_ROOT]

The reference is pure Python + Triton (no build step, and its ``pyproject.toml`` names a build backend and a
package directory that do not exist), so "installing" it is a plain copy of ``src/*.py`` and ``tests/*.py``.
``baseline/_ref`` is ignored by git - nothing of the reference enters this repository's history - but it
travels with the working tree to a GPU machine, where

  * ``tests/test_reference_triton_gpu.py`` runs the reference's Triton kernels next to this library on the
    same inputs (bytes and scale bits of the quantisers, GEMM and grouped-GEMM results), runs the reference's own
    ``tests/test_kernels.py`` against the drop-in module and builds the reference's model on top of it;
  * ``bench.py`` times the reference's kernels as the ones to beat.

Nothing in the library imports from ``baseline/_ref``; when the directory is absent the tests skip with that
reason and the benchmark leaves the comparison entries out.

REFERENCE_ROOT defaults to ``$CINNAMON_REFERENCE``, then to ``reference_path`` of ``BASELINE.json``.
"""
from __future__ import annotations

import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def reference_root(arg: str | None = None) -> str | None:
    if arg:
        return arg
    if os.environ.get("CINNAMON_REFERENCE"):
        return os.environ["CINNAMON_REFERENCE"]
    try:
        with open(os.path.join(os.path.dirname(HERE), "BASELINE.json")) as f:
            return json.load(f).get("reference_path")
    except Exception:
        return None


def stage(root: str | None = None) -> str | None:
    """Copies the reference's Python sources; returns the destination, or None when there is no reference here."""
    root = reference_root(root)
    if not root or not os.path.isfile(os.path.join(root, "src", "kernels.py")):
        return None
    for sub in ("src", "tests"):
        dst = os.path.join(DEST, sub)
        os.makedirs(dst, exist_ok=True)
        for name in sorted(os.listdir(os.path.join(root, sub))):
            if name.endswith(".py"):
                shutil.copyfile(os.path.join(root, sub, name), os.path.join(dst, name))
                os.chmod(os.path.join(dst, name), 0o644)
    return DEST


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out if out else "no reference tree found: nothing staged")
