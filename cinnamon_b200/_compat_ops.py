"""Names that cinnamon's model code imports from ``kernels`` but that are not part of the
FP8 path: DSA sparse attention (src/kernels.py:913-1312) and the fused lightning indexer
(src/kernels.py:321-433).  They are provided as plain torch ops with the reference's
semantics so that ``from kernels import sparse_attention`` (src/attention.py:6) keeps
working; they are outside the scope of the hand-written kernels.
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


def _sparse_attention_impl(q, k, v, idx, scale):
    B, H, L, _ = q.shape
    K = idx.shape[-1]
    t = torch.arange(L, device=q.device).view(1, L, 1)
    valid = idx <= t                                                    # causal validity (:982)
    gidx = idx.clamp(0, L - 1).unsqueeze(1).expand(B, H, L, K)
    kf, vf = k.float(), v.float()
    kg = torch.gather(kf.unsqueeze(2).expand(B, H, L, L, kf.shape[-1]), 3,
                      gidx.unsqueeze(-1).expand(B, H, L, K, kf.shape[-1]))
    vg = torch.gather(vf.unsqueeze(2).expand(B, H, L, L, vf.shape[-1]), 3,
                      gidx.unsqueeze(-1).expand(B, H, L, K, vf.shape[-1]))
    scores = (q.float().unsqueeze(3) * kg).sum(-1) * scale
    scores = scores.masked_fill(~valid.unsqueeze(1), float("-inf"))
    has_valid = valid.any(-1).view(B, 1, L, 1)
    attn = torch.softmax(scores, dim=-1)
    attn = torch.where(has_valid, attn, torch.zeros_like(attn)).nan_to_num(0.0)
    out = (attn.unsqueeze(-1) * vg).sum(3)
    return out, attn


class SparseAttentionFunction(torch.autograd.Function):
    """Same call signature as the reference class (src/kernels.py:1176-1289); gradients come
    from differentiating the torch implementation."""

    @staticmethod
    def forward(ctx, q, k, v, idx, scale):
        with torch.enable_grad():
            qd, kd, vd = (t.detach().requires_grad_(True) for t in (q, k, v))
            out, attn = _sparse_attention_impl(qd, kd, vd, idx, scale)
        ctx.save_for_backward(qd, kd, vd, out)
        ctx.in_dtype = q.dtype
        return out.detach().to(q.dtype), attn.detach()

    @staticmethod
    def backward(ctx, grad_output, grad_attn_weights):
        qd, kd, vd, out = ctx.saved_tensors
        gq, gk, gv = torch.autograd.grad(out, (qd, kd, vd), grad_output.float())
        return gq.to(ctx.in_dtype), gk.to(ctx.in_dtype), gv.to(ctx.in_dtype), None, None


def sparse_attention(q, k, v, idx, scale=None):
    """Attention over K selected positions per query (reference src/kernels.py:1292-1312).
    q, k: [B, H, L, D_qk]; v: [B, H, L, D_v]; idx: [B, L, K].  Returns (output, attn_weights)."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return SparseAttentionFunction.apply(q, k, v, idx, scale)
