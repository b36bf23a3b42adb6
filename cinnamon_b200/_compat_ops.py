"""A name that cinnamon's test-suite imports from ``kernels`` but that is not part of the FP8 path: the fused
lightning indexer (src/kernels.py:321-433, not called by the model).  It is provided as a plain torch op with
the reference's semantics; it is outside the scope of the hand-written kernels.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def lightning_indexer_fused(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """I[b, t, s] = sum_h relu(q[b, t, h] . k[b, s]) * w[b, t, h], fp16 result
    (reference src/kernels.py:392-433; operands are rounded to fp16 before the dot, :366-374)."""
    assert q.is_cuda and k.is_cuda, "Inputs must be on CUDA"
    scores = F.relu(torch.einsum("bthd,bsd->bths", q.half().float(), k.half().float()))
    return torch.einsum("bths,bth->bts", scores, w.float()).to(torch.float16)
