"""Binds this library's ``kernels`` module to the name the reference's model code imports.

The reference keeps flat modules on ``sys.path`` and its model code says ``from kernels import moe_grouped_gemm``
(src/layers.py:9), ``from kernels import sparse_attention`` (src/attention.py:6) and, in the trainers,
``from kernels import convert_to_fp8`` (src/train.py:697).  After ``install()`` those statements resolve to
``cinnamon_b200.kernels``; nothing else of the reference changes.

    import cinnamon_b200.dropin as dropin
    dropin.install()            # before the reference's model.py / layers.py / attention.py are imported
"""
from __future__ import annotations

import sys


def install(name: str = "kernels"):
    """Registers ``cinnamon_b200.kernels`` in ``sys.modules`` under ``name``; returns the module.  Raises if another
    module of that name was imported first (its importers already hold references to the other functions)."""
    from . import kernels
    other = sys.modules.get(name)
    if other is not None and other is not kernels:
        raise RuntimeError(f"a module named {name!r} is already imported from {getattr(other, '__file__', '?')}; "
                           "call cinnamon_b200.dropin.install() before importing the model code")
    sys.modules[name] = kernels
    return kernels
