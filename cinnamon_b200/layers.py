"""The MoE block of the reference (``SwiGLU``, ``GroupedExperts``, ``MoE``; src/layers.py:15-179) on this library's
kernels, trainable, optionally with the routed experts sharded over a process group.

Same constructors, parameter and buffer names (``routed_experts.w12`` / ``.w3``, ``shared_experts.N.w1..w3``,
``router.weight``, ``expert_bias``) and the same ``(output, balance_loss)`` return as the reference, so a state dict
moves between the two (with one rank; with expert parallelism ``routed_experts`` holds this rank's slice).  What
differs is how the work is done:

  * routing after the router GEMM is three launches on the device (``kernels.moe_route``): no sort / bincount / cumsum
    chain and no ``.item()`` synchronisation (the reference reads ``expert_counts.max()`` back, src/layers.py:151);
  * the routed experts are two differentiable grouped GEMMs on e4m3 operands with a one-kernel SwiGLU between them
    (the reference's grouped GEMM has no backward, so its routed experts receive no gradient on a GPU);
  * gate multiply and scatter-add are one gather pass with the shared experts' output folded in;
  * with ``group`` the experts are sharded ``n_routed / world`` per rank and tokens travel to their experts and back,
    forward and backward (``moe.moe_forward_train``): by all-to-all collectives, or with ``exchange="p2p"`` (GPUs of
    one node) by peer stores over NVLink into symmetric memory.  Expert counts for the bias update are then
    summed over the ranks (the reference, which replicates every expert, keeps them rank-local).

On CPU tensors the block computes the same mathematics with torch (the reference's own fallback loop,
src/layers.py:76-87); the kernels need a GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from . import moe as _moe


class SwiGLU(nn.Module):
    """``w3(silu(w1 x) * w2 x)`` (src/layers.py:15-31); ``convert_to_fp8`` turns the three linears into FP8Linear."""

    def __init__(self, d_model: int, hidden_dim: int):
        super().__init__()
        self.w1 = nn.Linear(d_model, hidden_dim, bias=False)
        self.w2 = nn.Linear(d_model, hidden_dim, bias=False)
        self.w3 = nn.Linear(hidden_dim, d_model, bias=False)

    def forward(self, x):
        return self.w3(F.silu(self.w1(x)) * self.w2(x))


class GroupedExperts(nn.Module):
    """Stacked SwiGLU experts, ``w12`` (E, 2 * hidden, d) = [w1; w2] and ``w3`` (E, d, hidden), normal(0, 0.02)
    (src/layers.py:34-54)."""

    def __init__(self, n_experts: int, d_model: int, hidden_dim: int):
        super().__init__()
        self.n_experts, self.d_model, self.hidden_dim = n_experts, d_model, hidden_dim
        self.w12 = nn.Parameter(torch.empty(n_experts, 2 * hidden_dim, d_model))
        self.w3 = nn.Parameter(torch.empty(n_experts, d_model, hidden_dim))
        nn.init.normal_(self.w12, mean=0.0, std=0.02)
        nn.init.normal_(self.w3, mean=0.0, std=0.02)

    def forward(self, sorted_x, expert_starts, expert_ends, max_expert_tokens=None):
        """(rows, d) grouped by expert -> (rows, d) fp32 (src/layers.py:56-87).  ``max_expert_tokens`` is accepted
        for signature compatibility; nothing here depends on it."""
        if sorted_x.is_cuda:
            from . import kernels as K
            h12 = K.moe_grouped_gemm(sorted_x, self.w12, expert_starts, expert_ends, dtype=torch.bfloat16)
            h = K.swiglu(h12)
            return K.moe_grouped_gemm(h, self.w3, expert_starts, expert_ends, dtype=torch.bfloat16).float()
        out = torch.zeros(sorted_x.size(0), self.d_model, dtype=torch.float32, device=sorted_x.device)
        for i in range(self.n_experts):
            s, e = int(expert_starts[i]), int(expert_ends[i])
            if e > s:
                h1, h2 = F.linear(sorted_x[s:e].float(), self.w12[i].float()).chunk(2, dim=-1)
                piece = F.linear(F.silu(h1) * h2, self.w3[i].float())
                out = out.index_copy(0, torch.arange(s, e, device=out.device), piece)
        return out


class MoE(nn.Module):
    """Routed + shared experts (src/layers.py:89-179).  ``group``: process group over which the routed experts are
    sharded (None = all experts on this rank)."""

    def __init__(self, n_routed, n_shared, top_k, d_model, hidden_dim, expert_scale, gamma, balance_alpha=0.0, group=None,
                 exchange: str = "nccl"):
        super().__init__()
        assert exchange in ("nccl", "p2p"), "exchange: 'nccl' (all-to-all collectives) or 'p2p' (peer stores over NVLink)"
        self.exchange = exchange
        self._peer = None                # p2p.PeerBuffers, allocated (collectively) by the first sharded call on GPUs
        self._peer_tokens = 0
        world = dist.get_world_size(group) if group is not None else 1
        self.group = group
        self.sharded = world > 1
        if self.sharded:
            assert n_routed % world == 0, "the routed experts must divide evenly over the ranks"
        n_local = n_routed // world if self.sharded else n_routed
        self.routed_experts = GroupedExperts(n_local, d_model, hidden_dim // expert_scale)
        self.shared_experts = nn.ModuleList([SwiGLU(d_model, hidden_dim) for _ in range(n_shared)])
        self.router = nn.Linear(d_model, n_routed, bias=False)
        self.top_k, self.n_routed, self.d_model = top_k, n_routed, d_model
        self.gamma, self.balance_alpha = gamma, balance_alpha
        self.register_buffer("expert_bias", torch.zeros(n_routed))

    def _update_bias(self, expert_counts: torch.Tensor, total_selections: int):
        """Bias of over-used experts down by gamma, of under-used ones up, clamped to [-1, 1] (src/layers.py:111-116)."""
        expected = total_selections / self.n_routed
        step = torch.where(expert_counts.float() > expected, -self.gamma, self.gamma)
        self.expert_bias += step
        self.expert_bias.clamp_(-1, 1)

    def _balance_loss(self, scores, top_idx, batch, seq):
        """Sequence-wise balance loss (src/layers.py:167-177): per sequence, the fraction of selections each expert
        received (scaled by E / (k * L)) times its mean normalised score, summed over experts, averaged over
        sequences, times alpha."""
        sel = top_idx.reshape(batch, -1)
        counts = torch.zeros(batch, self.n_routed, device=scores.device, dtype=scores.dtype)
        counts.scatter_add_(1, sel, torch.ones_like(sel, dtype=scores.dtype))
        share = counts * (self.n_routed / (self.top_k * seq))
        normalised = scores / (scores.sum(dim=-1, keepdim=True) + 1e-9)
        return self.balance_alpha * (share * normalised.view(batch, seq, -1).mean(dim=1)).sum(dim=-1).mean()

    def _peer_buffers(self, n_tokens: int, d: int, device):
        """Receive buffers of the peer-store exchange, sized on the first call for the largest token count among the
        ranks (one all-reduce, that call only) and for fp32 rows, the widest that travel."""
        if self._peer is None:
            from . import p2p
            m = torch.tensor([n_tokens], dtype=torch.int64, device=device)
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.group)
            self._peer_tokens = int(m.item())
            home_rows = self._peer_tokens * self.top_k
            self._peer = p2p.PeerBuffers(self.group, device, home_rows * dist.get_world_size(self.group), home_rows, 4 * d, 1,
                                         n_experts=self.n_routed)
        if n_tokens > self._peer_tokens:
            raise ValueError(f"{n_tokens} tokens in this call, but the peer buffers were sized for {self._peer_tokens} per rank "
                             "by the first call")
        return self._peer

    def forward(self, x):
        batch, seq, d = x.shape
        shared_out = self.shared_experts[0](x) if len(self.shared_experts) == 1 else sum(e(x) for e in self.shared_experts)
        flat = x.reshape(-1, d)
        logits = self.router(flat)
        scores = torch.sigmoid(logits.float())
        if flat.is_cuda:
            from . import kernels as K
            r = K.moe_route(logits.detach().float(), self.expert_bias, self.top_k)
            routing = _moe.Routing(token_indices=r["token_indices"], sorted_scores=r["sorted_scores"],
                                   sorted_experts=r["sorted_experts"], counts=r["counts"], pair_pos=r["pair_pos"],
                                   pair_gate=r["pair_gate"])
            top_idx = r["top_experts"].long()
        else:
            routing = _moe.route_torch(logits.detach().float(), self.expert_bias, self.top_k, self.n_routed)
            top_idx = (scores.detach() + self.expert_bias).topk(self.top_k, dim=-1).indices
        # the gates once more, differentiably, in the order of routing.pair_pos (a token's pairs by ascending expert)
        chosen = top_idx.sort(dim=-1).values
        picked = scores.gather(-1, chosen)
        gates = picked / (picked.sum(dim=-1, keepdim=True) + 1e-9)
        experts = lambda rows, starts, ends: self.routed_experts(rows, starts, ends)          # noqa: E731
        peer = None
        if self.sharded and self.exchange == "p2p" and flat.is_cuda:
            peer = self._peer_buffers(flat.shape[0], d, flat.device)
        y = _moe.moe_forward_train(flat, routing, gates, experts, self.group if self.sharded else None,
                                   addend=shared_out.reshape(-1, d), peer=peer)
        if self.training:
            counts = routing.counts
            if self.sharded:
                counts = counts.clone()
                dist.all_reduce(counts, group=self.group)
                total = flat.shape[0] * self.top_k * dist.get_world_size(self.group)
            else:
                total = flat.shape[0] * self.top_k
            with torch.no_grad():
                self._update_bias(counts, total)
        balance_loss = None
        if self.balance_alpha > 0:
            balance_loss = self._balance_loss(scores, top_idx, batch, seq)
        return y.view(batch, seq, d), balance_loss
