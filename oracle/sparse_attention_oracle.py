"""CPU restatement (float64) of cinnamon's sparse attention, forward and backward.

TEST INFRASTRUCTURE ONLY: imported by tests/ (and nothing that ships).  It follows the reference's Triton
kernels line by line in meaning, not in schedule:

  forward   src/kernels.py:913-1052   valid = idx <= t (:982); scores = scale * q.k over the gathered keys
            (:991), -inf where not valid (:992); lse = max + log(sum exp) with the "no valid key" rule
            max -> 0, sum -> 1 (:1009-1012); weights = exp(score - lse), 0 where not valid (:1031-1032);
            out = sum_j weights_j v[idx_j] (:1044)
  backward  src/kernels.py:1055-1186  delta = dO.O (:1122); p recomputed from lse (:1143-1144);
            dp = p (dO.v - delta) (:1152-1153); dq = scale * sum_j dp_j k_j (:1156); dk[idx_j] += scale dp_j q
            (:1161-1163); dv[idx_j] += p_j dO (:1165-1167); the gradient w.r.t. the returned weights is
            ignored (:1248)

Pinned by tests/golden/sparse_attention_vectors.npz: outputs of the reference's own kernels, executed by the
Triton CPU interpreter on seeded inputs (tests/golden/make_golden_sparse.py).
"""
from __future__ import annotations

import torch


def _gather(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """x [B, H, L, D], idx [B, L, K] (clamped) -> [B, H, L, K, D]"""
    B, H, L, D = x.shape
    return torch.stack([x[b][:, idx[b]] for b in range(B)])


def forward(q, k, v, idx, scale):
    """Returns (out [B,H,L,Dv], attn [B,H,L,K], lse [B,H,L]) in float64."""
    q, k, v = q.double(), k.double(), v.double()
    B, H, L, _ = q.shape
    t = torch.arange(L).view(1, L, 1)
    valid = (idx <= t) & (idx >= 0)                                           # [B, L, K]
    cl = idx.clamp(0, L - 1)
    kg, vg = _gather(k, cl), _gather(v, cl)
    scores = torch.einsum("bhld,bhlkd->bhlk", q, kg) * scale
    vm = valid.unsqueeze(1)
    scores = torch.where(vm, scores, torch.full_like(scores, float("-inf")))
    has = vm.any(-1, keepdim=True)
    mx = torch.where(has, scores.max(-1, keepdim=True).values, torch.zeros_like(scores[..., :1]))
    sm = torch.where(vm, (scores - mx).exp(), torch.zeros_like(scores)).sum(-1, keepdim=True)
    sm = torch.where(has, sm, torch.ones_like(sm))
    lse = mx + sm.log()
    attn = torch.where(vm, (scores - lse).exp(), torch.zeros_like(scores))
    out = torch.einsum("bhlk,bhlkd->bhld", attn, vg)
    return out, attn, lse.squeeze(-1)


def backward(q, k, v, idx, scale, grad_out):
    """Returns (dq, dk, dv) in float64 for the loss sum(out * grad_out)."""
    q, k, v, g = q.double(), k.double(), v.double(), grad_out.double()
    B, H, L, Dqk = q.shape
    out, attn, _ = forward(q, k, v, idx, scale)
    cl = idx.clamp(0, L - 1)
    kg, vg = _gather(k, cl), _gather(v, cl)
    delta = (g * out).sum(-1, keepdim=True)                                    # [B,H,L,1]
    dov = torch.einsum("bhld,bhlkd->bhlk", g, vg)
    dp = attn * (dov - delta)                                                  # zero where not valid (attn = 0)
    dq = torch.einsum("bhlk,bhlkd->bhld", dp, kg) * scale
    dk = torch.zeros_like(k)
    dv = torch.zeros_like(v)
    for b in range(B):
        flat = cl[b].reshape(-1)                                               # [L*K]
        dk_c = (dp[b].unsqueeze(-1) * q[b].unsqueeze(2) * scale).reshape(H, -1, Dqk)
        dv_c = (attn[b].unsqueeze(-1) * g[b].unsqueeze(2)).reshape(H, -1, v.shape[-1])
        dk[b].index_add_(1, flat, dk_c)
        dv[b].index_add_(1, flat, dv_c)
    return dq, dk, dv


def lightning_indexer(q, k, w):
    """Lightning indexer logits (src/kernels.py:321-433) in float64, rounded to fp16 at the end:
    I[b, t, s] = sum_h relu(fp16(q[b, t, h]) . fp16(k[b, s])) * w[b, t, h]  (:374, :377, :381)."""
    qh, kh = q.half().double(), k.half().double()
    dots = torch.einsum("bthd,bsd->bths", qh, kh).clamp(min=0.0)
    return torch.einsum("bths,bth->bts", dots, w.double())
