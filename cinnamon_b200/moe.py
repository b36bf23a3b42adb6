"""Routed-expert MoE layer with FP8 grouped GEMMs and expert parallelism.

The reference replicates every expert on every rank (src/layers.py:89-179); its routed
path is: route -> sort pairs by expert -> gather tokens -> grouped SwiGLU (two grouped
GEMMs, src/layers.py:69-75) -> gate -> scatter-add.  This module keeps that arithmetic
and adds the partitioning the reference lacks:

  * experts are sharded contiguously, ``E / G`` per rank; every rank routes its own tokens;
  * dispatch: one all-to-all of e4m3 rows and one of their fp32 1x128 scales (tokens are
    quantised once, before the exchange, so 1 byte per element crosses NVLink);
  * each rank runs the two grouped GEMMs over the ragged per-expert ranges it received
    (offsets stay on the device; nothing is padded);
  * combine: one all-to-all of bf16 rows back to the owners, then the gate-weighted
    scatter-add of the reference (src/layers.py:157-160).

The exchange plan (who sends how many rows to whom, and the permutations on both sides)
is plain torch + ``torch.distributed`` and works on any backend, so it is tested with
gloo on CPU; the expert computation is a callable (the FP8 one needs a B200).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


# ---------------------------------------------------------------------------------------
# routing (src/layers.py:122-148)
# ---------------------------------------------------------------------------------------
@dataclass
class Routing:
    token_indices: torch.Tensor    # (T*k,) source token of each sorted pair
    sorted_scores: torch.Tensor    # (T*k,) normalised gate of each sorted pair
    sorted_experts: torch.Tensor   # (T*k,) global expert id, ascending
    counts: torch.Tensor           # (E,) pairs per expert
    pair_pos: torch.Tensor = None  # (T, k) sorted position of each of a token's pairs, ascending
    pair_gate: torch.Tensor = None  # (T, k) the gates in the same order


def router_logits(x: torch.Tensor, router_weight: torch.Tensor) -> torch.Tensor:
    """The reference's router is an ``nn.Linear`` under autocast (src/layers.py:122): a 16-bit GEMM for 16-bit
    activations, scores in fp32 afterwards."""
    if x.dtype in (torch.bfloat16, torch.float16):
        w = router_weight if router_weight.dtype == x.dtype else router_weight.to(x.dtype)
        return torch.nn.functional.linear(x, w).float()
    return torch.nn.functional.linear(x.float(), router_weight.float())


def route(x: torch.Tensor, router_weight: torch.Tensor, expert_bias: torch.Tensor, top_k: int) -> Routing:
    """Router of ``MoE.forward`` (src/layers.py:122-148): sigmoid scores, top-k on
    scores + bias, gates normalised over the selected experts, pairs sorted by expert.
    On a GPU everything after the router GEMM is three kernel launches (``kernels.moe_route``) with no host
    synchronisation; on the CPU (host-logic tests) it is the reference's chain of torch calls."""
    n_experts = router_weight.shape[0]
    logits = router_logits(x, router_weight)
    if logits.is_cuda:
        from . import kernels as K
        r = K.moe_route(logits, expert_bias, top_k)
        return Routing(token_indices=r["token_indices"], sorted_scores=r["sorted_scores"],
                       sorted_experts=r["sorted_experts"], counts=r["counts"], pair_pos=r["pair_pos"],
                       pair_gate=r["pair_gate"])
    return route_torch(logits, expert_bias, top_k, n_experts)


def route_torch(logits: torch.Tensor, expert_bias: torch.Tensor, top_k: int, n_experts: int) -> Routing:
    """The routing arithmetic as the reference writes it (src/layers.py:122-148), in torch."""
    scores = torch.sigmoid(logits)
    _, top_idx = (scores + expert_bias).topk(top_k, dim=-1)
    top_scores = scores.gather(-1, top_idx)
    top_scores = top_scores / (top_scores.sum(dim=-1, keepdim=True) + 1e-9)
    expanded = top_idx.reshape(-1)
    sorted_experts, order = expanded.sort(stable=True)
    # where each (token, slot) pair sits in the sorted order, per token in ascending position
    pos = torch.empty_like(order)
    pos[order] = torch.arange(order.numel(), device=order.device)
    pair_pos, perm = pos.view(-1, top_k).sort(dim=1)
    return Routing(token_indices=order // top_k, sorted_scores=top_scores.reshape(-1)[order],
                   sorted_experts=sorted_experts, counts=torch.bincount(expanded, minlength=n_experts),
                   pair_pos=pair_pos, pair_gate=top_scores.gather(1, perm))


def offsets_from_counts(counts: torch.Tensor):
    ends = counts.cumsum(0)
    return ends - counts, ends


# ---------------------------------------------------------------------------------------
# expert computation
# ---------------------------------------------------------------------------------------
class FP8Experts:
    """Stacked SwiGLU experts with cached e4m3 weights: w12 (E, 2*I, d), w3 (E, d, I)
    (the layout of ``GroupedExperts``, src/layers.py:47-50)."""

    def __init__(self, w12: torch.Tensor, w3: torch.Tensor):
        from . import kernels as K
        self.K = K
        self.n_experts, two_i, self.d_model = w12.shape
        self.hidden = two_i // 2
        self.requantize(w12, w3)

    def requantize(self, w12: torch.Tensor, w3: torch.Tensor) -> None:
        """Quantise the master weights in 128x128 blocks (once per optimiser step, not per call)."""
        self.w12_q, self.w12_s = self.K.quantize_expert_weights(w12)
        self.w3_q, self.w3_s = self.K.quantize_expert_weights(w3)

    def __call__(self, x_q: torch.Tensor, x_s: torch.Tensor, starts: torch.Tensor, ends: torch.Tensor,
                 out_dtype=torch.bfloat16, row_dst: torch.Tensor = None, n_rows_dev: torch.Tensor = None,
                 trace: Optional[list] = None, up_parts: Optional[list] = None) -> torch.Tensor:
        """x_q (R, d) e4m3 rows grouped by expert, x_s (R, d/128) -> (R, d) ``out_dtype``.
        Rows outside [starts[0], ends[-1]) are not written.  With ``row_dst`` (one byte address per row) the
        down-projection stores every output row there instead (possibly on a peer GPU) and nothing is returned.
        ``n_rows_dev``: device-side count of the leading rows of ``x_q`` that hold data (the rest of the buffer is
        capacity that no expert range covers).  ``up_parts``: ``[(e_lo, e_hi, before), ...]`` - the up-projection as
        one launch per range of experts, ``before()`` (a wait for that range's rows, say) enqueued ahead of each."""
        K = self.K
        if up_parts is None:
            h12 = K.fp8_grouped_gemm(x_q, x_s, self.w12_q, self.w12_s, starts, ends, out_dtype=torch.bfloat16)
            _mark(trace, "grouped GEMM up-projection")
        else:
            with torch.cuda.device(x_q.device):
                h12 = torch.empty((x_q.shape[0], 2 * self.hidden), dtype=torch.bfloat16, device=x_q.device)
            for lo, hi, before in up_parts:
                if before is not None:
                    before()
                    _mark(trace, f"wait for the rows of experts [{lo}, {hi})")
                K.fp8_grouped_gemm(x_q, x_s, self.w12_q[lo:hi], self.w12_s[lo:hi], starts[lo:hi], ends[lo:hi], out=h12)
                _mark(trace, f"grouped GEMM up-projection, experts [{lo}, {hi})")
        h_q, h_s = K.swiglu_quantize_rowwise(h12, n_rows_dev)
        _mark(trace, "SwiGLU + quantise")
        if row_dst is not None:
            K.fp8_grouped_gemm_scatter(h_q, h_s, self.w3_q, self.w3_s, starts, ends, row_dst, out_dtype=out_dtype)
            _mark(trace, "grouped GEMM down-projection (+ rows stored at their home ranks)")
            return None
        out = K.fp8_grouped_gemm(h_q, h_s, self.w3_q, self.w3_s, starts, ends, out_dtype=out_dtype)
        _mark(trace, "grouped GEMM down-projection")
        return out


class FP8SwiGLU:
    """A shared expert: the ``SwiGLU`` block (src/layers.py:15-32) after ``convert_to_fp8`` turned its three
    linears into FP8 ones, with the work the three separate layers repeat done once:

      * the weights are quantised when they change, not on every call;
      * w1 and w2 share their input, so x is quantised once and [w1; w2] is one GEMM of width 2 * hidden
        (the layout ``GroupedExperts`` uses for the routed experts, src/layers.py:47-49);
      * SiLU, the product and the quantisation of w3's input are one pass over that GEMM's output.

    ``round_scale`` is the power-of-two scale option of w1 / w2's input quantisation."""

    def __init__(self, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor, round_scale: bool = False):
        from . import kernels as K
        self.K = K
        self.round_scale = bool(round_scale)
        self.hidden, self.d_model = w1.shape
        self.requantize(w1, w2, w3)

    def requantize(self, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor) -> None:
        K = self.K
        w12 = torch.cat([w1, w2], dim=0)
        self.w12_q, self.w12_s = K.quantize_fp8_blockwise(w12 if w12.dtype in (torch.bfloat16, torch.float32, torch.float16)
                                                          else w12.float())
        self.w3_q, self.w3_s = K.quantize_fp8_blockwise(w3 if w3.dtype in (torch.bfloat16, torch.float32, torch.float16)
                                                        else w3.float())

    def __call__(self, x: torch.Tensor, x_q: torch.Tensor = None, x_s: torch.Tensor = None) -> torch.Tensor:
        """x (T, d) -> (T, d) bf16.  ``x_q, x_s``: an existing 1x128 quantisation of x to reuse."""
        K = self.K
        T = x.shape[0]
        if x_q is None:
            x_q, x_s = K.quantize_fp8_rowwise(x, 128, self.round_scale)
        h12 = K._gemm(x_q, x_s, self.w12_q, K._lib.B_NK, self.w12_s, self.w12_s.stride(1), self.w12_s.stride(0), T,
                      2 * self.hidden, self.d_model, torch.bfloat16)
        h_q, h_s = K.swiglu_quantize_rowwise(h12)
        return K._gemm(h_q, h_s, self.w3_q, K._lib.B_NK, self.w3_s, self.w3_s.stride(1), self.w3_s.stride(0), T,
                       self.d_model, self.hidden, torch.bfloat16)


# ---------------------------------------------------------------------------------------
# exchange plan
# ---------------------------------------------------------------------------------------
@dataclass
class DispatchPlan:
    send_splits: list              # rows this rank sends to each rank
    recv_splits: list              # rows this rank receives from each rank
    recv_counts: torch.Tensor      # (G, E_local) rows received from rank g for local expert e
    perm: torch.Tensor             # received order (by source rank, then expert) -> grouped by expert
    starts: torch.Tensor           # (E_local,) int64, device
    ends: torch.Tensor             # (E_local,) int64, device


def make_plan(counts: torch.Tensor, group=None, n_pairs: Optional[int] = None) -> DispatchPlan:
    """``counts``: (E,) pairs this rank routed to every global expert.  Exchanges the counts
    (one small all-to-all) and derives split sizes, the regrouping permutation and the
    per-expert row ranges on the receiving side.  With one rank nothing is exchanged or permuted, and when the
    caller passes the number of pairs (tokens x top_k) nothing is read back to the host either."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    n_experts = counts.numel()
    assert n_experts % world == 0, "experts must divide evenly over ranks"
    e_local = n_experts // world
    send_counts = counts.reshape(world, e_local).to(torch.int64).contiguous()
    if world == 1:
        ends = send_counts[0].cumsum(0)
        starts = ends - send_counts[0]
        n = int(n_pairs) if n_pairs is not None else int(ends[-1])
        return DispatchPlan([n], [n], send_counts, None, starts.contiguous(), ends.contiguous())
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    # the one host read-back of the layer: the collective wants its split sizes as Python ints
    splits = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).tolist()
    send_splits, recv_splits = splits[0], splits[1]
    # received rows arrive ordered by (source rank, local expert); regroup to (local expert, source rank)
    flat = recv_counts.reshape(-1)
    expert_of_segment = torch.arange(e_local, device=counts.device).repeat(world)
    row_expert = torch.repeat_interleave(expert_of_segment, flat, output_size=sum(recv_splits))
    perm = torch.sort(row_expert, stable=True).indices
    per_expert = recv_counts.sum(0)
    starts, ends = offsets_from_counts(per_expert)
    return DispatchPlan(send_splits, recv_splits, recv_counts, perm, starts.contiguous(), ends.contiguous())


def make_plans(counts_list, group=None):
    """Plans for several token chunks from ONE exchange of counts and ONE host read-back (several ranks).
    ``counts_list``: per chunk, the (E,) pairs this rank routed to every global expert."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return [make_plan(c, group) for c in counts_list]
    n_chunks = len(counts_list)
    n_experts = counts_list[0].numel()
    assert n_experts % world == 0, "experts must divide evenly over ranks"
    e_local = n_experts // world
    # (world, chunk, local expert): the slice for one destination rank is contiguous
    send_counts = torch.stack([c.reshape(world, e_local).to(torch.int64) for c in counts_list], dim=1).contiguous()
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    splits = torch.stack([send_counts.sum(2), recv_counts.sum(2)]).tolist()         # [2][world][chunk]
    plans = []
    expert_of_segment = torch.arange(e_local, device=send_counts.device).repeat(world)
    for c in range(n_chunks):
        send_splits = [splits[0][g][c] for g in range(world)]
        recv_splits = [splits[1][g][c] for g in range(world)]
        rc = recv_counts[:, c, :].contiguous()
        row_expert = torch.repeat_interleave(expert_of_segment, rc.reshape(-1), output_size=sum(recv_splits))
        perm = torch.sort(row_expert, stable=True).indices
        starts, ends = offsets_from_counts(rc.sum(0))
        plans.append(DispatchPlan(send_splits, recv_splits, rc, perm, starts.contiguous(), ends.contiguous()))
    return plans


def all_to_all_rows(rows: torch.Tensor, send_splits, recv_splits, group=None) -> torch.Tensor:
    """Variable-size all-to-all of the rows of a 2-D tensor (any dtype; e4m3 travels as bytes)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return rows
    view = rows.view(torch.uint8) if rows.dtype == torch.float8_e4m3fn else rows
    out = torch.empty((sum(recv_splits), view.shape[1]), dtype=view.dtype, device=view.device)
    dist.all_to_all_single(out, view.contiguous(), output_split_sizes=list(recv_splits),
                           input_split_sizes=list(send_splits), group=group)
    return out.view(rows.dtype) if rows.dtype == torch.float8_e4m3fn else out


# ---------------------------------------------------------------------------------------
# the layer
# ---------------------------------------------------------------------------------------
def moe_forward(x: torch.Tensor, routing: Routing, experts: Callable, quantize: Optional[Callable],
                group=None, addend: Optional[torch.Tensor] = None, before_combine: Optional[Callable] = None,
                trace: Optional[list] = None) -> torch.Tensor:
    """Routed part of ``MoE.forward`` for this rank's tokens ``x`` (T, d).

    ``experts(rows_q, rows_s, starts, ends)`` computes the expert SwiGLU for rows grouped by
    local expert; ``quantize(x) -> (q, s)`` is the row-wise quantiser (``None`` = rows travel
    unquantised and ``experts`` receives ``(rows, None, starts, ends)``: the CPU test path).
    ``addend`` (T, d), optional: the shared experts' output, folded into the combine pass
    (``shared_out + routed_out``, src/layers.py:179); ``before_combine`` is called right before that pass.
    (``moe_forward_p2p`` also takes a callable that produces it, called once the dispatch has been enqueued.)
    Returns the gate-weighted sum over each token's experts (plus ``addend``), fp32 (T, d).
    """
    T, d = x.shape
    plan = make_plan(routing.counts, group, n_pairs=routing.token_indices.numel())
    if quantize is not None:
        x_q, x_s = quantize(x)
        from . import kernels as K
        send_q, send_s = K.gather_quantized_rows(x_q, x_s, routing.token_indices)
        recv_q = all_to_all_rows(send_q, plan.send_splits, plan.recv_splits, group)
        recv_s = all_to_all_rows(send_s, plan.send_splits, plan.recv_splits, group)
        if len(plan.recv_splits) > 1:
            recv_q, recv_s = K.gather_quantized_rows(recv_q, recv_s, plan.perm)
        _mark(trace, "quantise + gather" + (" + all-to-all + regroup" if len(plan.recv_splits) > 1 else ""))
        out_rows = experts(recv_q, recv_s, plan.starts, plan.ends, trace=trace) if trace is not None else \
            experts(recv_q, recv_s, plan.starts, plan.ends)
    else:
        send = x.index_select(0, routing.token_indices)
        recv = all_to_all_rows(send, plan.send_splits, plan.recv_splits, group)
        if len(plan.recv_splits) > 1:
            recv = recv.index_select(0, plan.perm)
        out_rows = experts(recv, None, plan.starts, plan.ends)
    # back to arrival order, then home
    if len(plan.recv_splits) > 1:
        if out_rows.is_cuda:
            from . import kernels as K
            back = K.scatter_rows(out_rows, plan.perm)
        else:
            back = torch.empty_like(out_rows)
            back.index_copy_(0, plan.perm, out_rows)
        out_rows = all_to_all_rows(back, plan.recv_splits, plan.send_splits, group)
    if before_combine is not None:
        before_combine()                       # e.g. join the stream that produced ``addend``
    if out_rows.is_cuda:
        from . import kernels as K
        if len(plan.recv_splits) > 1:
            _mark(trace, "inverse permutation + all-to-all home")
        y = K.moe_combine(out_rows, routing.pair_pos, routing.pair_gate, addend)      # src/layers.py:157-160, fused
        _mark(trace, "combine (+ shared expert output)")
        return y
    weighted = out_rows.float() * routing.sorted_scores[:, None]                 # host-logic tests (CPU ranks)
    y = torch.zeros(T, d, dtype=torch.float32, device=x.device)
    y.index_add_(0, routing.token_indices, weighted)
    return y if addend is None else addend.float() + y


# ---------------------------------------------------------------------------------------
# the layer with gradients (training)
# ---------------------------------------------------------------------------------------
class _AllToAllRows(torch.autograd.Function):
    """Variable-size all-to-all of rows whose backward is the same exchange run the other way: what went from rank a
    to rank b as a row comes back from b to a as that row's gradient.  ``anchor`` is a scalar that requires grad on
    every rank: the backward is a collective, so it has to run on every rank, also on one whose ``rows`` happen not
    to require grad (a rank that received no row for its experts in this step)."""

    @staticmethod
    def forward(ctx, rows, send_splits, recv_splits, group, anchor):
        ctx.splits, ctx.group = (list(send_splits), list(recv_splits)), group
        return all_to_all_rows(rows, send_splits, recv_splits, group)

    @staticmethod
    def backward(ctx, grad):
        send, recv = ctx.splits
        return all_to_all_rows(grad.contiguous(), recv, send, ctx.group), None, None, None, None


def _peer_move(rows: torch.Tensor, to_experts: bool, tabs, peer, sorted_experts: torch.Tensor, n_out: int) -> torch.Tensor:
    """One direction of the peer-store exchange for rows of any element type (``cinnamon_b200/p2p.py``):
    ``to_experts``: my sorted pairs' rows -> their places in the expert-grouped buffers of the experts' ranks;
    otherwise: my expert-grouped rows -> their pairs' places on the ranks the tokens live on.  Barriers before (the
    buffers' previous contents are done with on every rank) and after (every row has landed); the result is copied
    out of the symmetric buffer, which the next exchange overwrites."""
    from . import kernels as K
    n, d = rows.shape
    row_bytes = d * rows.element_size()
    assert row_bytes <= peer.d and row_bytes % 16 == 0, "peer buffers were sized for narrower rows"
    as_bytes = rows.contiguous().view(torch.uint8).view(n, row_bytes)
    peer.barrier()
    if to_experts:
        if n:
            idx = torch.arange(n, dtype=torch.int64, device=rows.device)
            no_scale = torch.zeros((n, 1), dtype=torch.float32, device=rows.device)
            K.p2p_dispatch(as_bytes, no_scale, idx, sorted_experts, tabs.base_send, tabs.my_start, peer.peer_q, peer.peer_s,
                           peer.n_experts // peer.world, peer.world, peer.capacity_rows)
        peer.barrier()
        flat = peer.q
    else:
        if n:
            K.p2p_return(as_bytes, tabs.seg_start, tabs.home_base, peer.peer_home, peer.world, peer.home_rows)
        peer.barrier()
        flat = peer.home.view(torch.uint8)
    return flat[: n_out * row_bytes].clone().view(rows.dtype).view(n_out, d)


class _PeerRows(torch.autograd.Function):
    """``_peer_move`` whose backward is the move the other way with the same address tables: a row's gradient travels
    back along the row's path.  ``anchor``: see ``_AllToAllRows`` (the barriers involve every rank)."""

    @staticmethod
    def forward(ctx, rows, to_experts, tabs, peer, sorted_experts, n_out, anchor):
        ctx.args = (not to_experts, tabs, peer, sorted_experts, rows.shape[0])
        return _peer_move(rows, to_experts, tabs, peer, sorted_experts, n_out)

    @staticmethod
    def backward(ctx, grad):
        to_experts, tabs, peer, sorted_experts, n_out = ctx.args
        return _peer_move(grad, to_experts, tabs, peer, sorted_experts, n_out), None, None, None, None, None, None


def moe_forward_train(x: torch.Tensor, routing: Routing, gates: torch.Tensor, experts: Callable, group=None,
                      addend: Optional[torch.Tensor] = None, peer=None) -> torch.Tensor:
    """The routed part of ``MoE.forward`` (src/layers.py:137-160) built from differentiable pieces, with the experts
    sharded over ``group``: gather -> all-to-all -> regroup by expert -> ``experts(rows, starts, ends)`` -> inverse
    permutation -> all-to-all home -> gate-weighted sum (+ ``addend``).  In the backward the two exchanges run in
    reverse: the gradients of the returned rows are dispatched to the experts' ranks, and the gradients of the
    dispatched rows come home.  Rows travel in the activations' own type and are quantised where the experts run
    (row-wise quantisation commutes with the permutation, so the expert arithmetic is that of ``moe_forward``).

    ``gates`` (T, k): the normalised gates, differentiable, in the order of ``routing.pair_pos`` (ascending expert
    id per token).  ``experts`` must be differentiable.  ``group=None`` means every expert is on this rank (also
    inside a data-parallel job: nothing is exchanged).  Works on any backend (the CPU ranks of the tests pass a
    torch expert function).  ``peer`` (a ``p2p.PeerBuffers`` sized in bytes for the widest rows, GPUs of one node):
    both exchanges, forward and backward, are peer stores over NVLink instead of all-to-all collectives - the
    rows land expert-grouped, so the regrouping permutations go too.  Returns (T, d) fp32."""
    world = dist.get_world_size(group) if group is not None else 1
    if world > 1 and peer is not None and x.is_cuda:
        from . import p2p
        n_pairs = routing.token_indices.numel()
        assert n_pairs <= peer.home_rows, "peer buffers too small"
        t = peer.plan(routing.counts.to(torch.int64).contiguous())
        # the tables belong to `peer` and the next layer call overwrites them: the backward needs its own copy
        tabs = p2p.ExchangeTables(**{f: getattr(t, f).clone() for f in t.__dataclass_fields__})
        n_recv = int(tabs.total_rows)                      # host read-back: sizes the experts' input
        assert n_recv <= peer.capacity_rows, "peer buffers too small"
        rows = x.index_select(0, routing.token_indices)
        anchor = torch.zeros((), dtype=rows.dtype, device=rows.device, requires_grad=torch.is_grad_enabled())
        received = _PeerRows.apply(rows, True, tabs, peer, routing.sorted_experts, n_recv, anchor)
        out_rows = experts(received, tabs.starts, tabs.ends)
        out_rows = out_rows + (received.sum() * 0).to(out_rows.dtype)
        out_rows = _PeerRows.apply(out_rows, False, tabs, peer, routing.sorted_experts, n_pairs, anchor)
        from . import kernels as K
        return K.moe_combine_autograd(out_rows, routing.pair_pos, gates, addend)
    if world > 1:
        plan = make_plan(routing.counts, group, n_pairs=routing.token_indices.numel())
    else:
        starts, ends = offsets_from_counts(routing.counts.to(torch.int64))
        plan = DispatchPlan(None, None, None, None, starts.contiguous(), ends.contiguous())
    rows = x.index_select(0, routing.token_indices)
    if world > 1:
        # Both exchanges are collectives in the backward too.  The anchor makes their outputs part of the graph on
        # every rank, and the returned rows are tied to the received ones, so that a rank whose experts got no row
        # (and whose expert outputs therefore carry no gradient) still takes part in both reverse exchanges.
        anchor = torch.zeros((), dtype=rows.dtype, device=rows.device, requires_grad=torch.is_grad_enabled())
        received = _AllToAllRows.apply(rows, plan.send_splits, plan.recv_splits, group, anchor)
        rows = received.index_select(0, plan.perm)
    out_rows = experts(rows, plan.starts, plan.ends)
    if world > 1:
        back = torch.zeros_like(out_rows).index_copy(0, plan.perm, out_rows)
        back = back + (received.sum() * 0).to(back.dtype)
        out_rows = _AllToAllRows.apply(back, plan.recv_splits, plan.send_splits, group, anchor)
    if out_rows.is_cuda:
        from . import kernels as K
        return K.moe_combine_autograd(out_rows, routing.pair_pos, gates, addend)
    y = (out_rows.float()[routing.pair_pos] * gates.float().unsqueeze(-1)).sum(dim=1)
    return y if addend is None else addend.float() + y


def _mark(trace: Optional[list], name: str) -> None:
    """Phase timing for the benchmark: appends (name, CUDA event recorded on the current stream) when tracing."""
    if trace is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        trace.append((name, ev))


def moe_forward_p2p(x: torch.Tensor, routing: Routing, experts: Callable, quantize: Callable, buffers, group=None,
                    addend: Optional[torch.Tensor] = None, before_combine: Optional[Callable] = None,
                    fused_return: bool = False, trace: Optional[list] = None, up_splits: int = 1,
                    dispatch_sms: int = 0) -> torch.Tensor:
    """``moe_forward`` with the exchange done by peer stores over NVLink (``cinnamon_b200/p2p.py``) instead of
    all-to-all collectives: the routing counts of all ranks are exchanged (by the plan kernel itself with
    ``fused_return``, else by one small all-gather), then every quantised row is written
    straight to its place in the expert-grouped buffer of the rank that owns its expert, and every expert output
    straight to its pair's place on the rank its token lives on.  No gather, regrouping or inverse permutation
    passes, no send/receive kernels; three stream-ordered barriers order the phases.  One host read-back (the
    number of rows this rank received), none at all with ``fused_return``.  ``buffers``: a ``p2p.PeerBuffers``.  ``fused_return``: the expert
    down-projection stores its output rows straight to their home ranks from its epilogue (``experts`` must accept
    ``row_dst``), instead of a separate pass after the GEMM.  Same arithmetic per row as ``moe_forward``; returns
    fp32 (T, d).  ``up_splits`` (with ``fused_return``; 1, 2 or 4): the local experts are cut into that many ranges,
    each dispatched by a launch of its own with its own "landed" flags, and the up-projection runs range by range, so
    the experts of the first range are at work while the rows of the later ones still cross NVLink.
    ``dispatch_sms`` (with ``fused_return``): the dispatch stores come from that many SMs only and a callable
    ``addend`` (the shared expert) is enqueued BEFORE the dispatch, so that its GEMMs - which the caller caps to the
    other SMs - run beside the NVLink-bound stores instead of after them."""
    from . import kernels as K
    from . import p2p
    world, me = dist.get_world_size(group), dist.get_rank(group)
    n_experts = routing.counts.numel()
    e_local = n_experts // world
    n_pairs = routing.token_indices.numel()
    assert n_pairs <= buffers.home_rows, "peer buffers too small"
    if fused_return and buffers.n_experts == n_experts:
        # Thirteen launches per layer call, no collective, no host read-back:
        #   plan        counts to every rank, wait for all, address tables (also: every rank is done with the buffers)
        #   dispatch    rows straight into the owners' expert-grouped buffers; its last CTA flags "landed"
        #   row table   waits for the flags of all ranks, then the home address of every output row
        #   experts     up-projection, SwiGLU + quantise, down-projection storing every row at its home
        #   barrier     every expert output is home
        t = buffers.plan(routing.counts.to(torch.int64).contiguous())
        _mark(trace, "plan (counts to all ranks + tables)")
        x_q, x_s = quantize(x)
        _mark(trace, "quantise tokens")
        n_parts = max(1, min(int(up_splits), 4, e_local))
        cuts = [e_local * i // n_parts for i in range(n_parts + 1)]
        slot = lambda i: buffers.LANDED_SLOT + 16 * i                                      # noqa: E731
        if callable(addend) and dispatch_sms > 0:
            addend = addend()                           # the shared expert on its own stream and SMs, beside the dispatch
        for i in range(n_parts):
            K.p2p_dispatch_signal(x_q, x_s, routing.token_indices, routing.sorted_experts, t, buffers, cuts[i], cuts[i + 1],
                                  slot(i), n_sms=dispatch_sms)
        _mark(trace, "dispatch (peer stores)")
        if callable(addend):
            addend = addend()                           # the shared expert, on its own stream, from here on
        cap = buffers.capacity_rows
        recv_q = buffers.q.view(cap, buffers.d).view(x_q.dtype)
        recv_s = buffers.s.view(cap, buffers.n_scales)
        table = K.p2p_row_table_wait(t, buffers, cap, buffers.d * 2, slot(0))
        _mark(trace, "wait for the first rows + address table" if n_parts > 1 else "wait for all rows + address table")
        if n_parts == 1:
            experts(recv_q, recv_s, t.starts, t.ends, row_dst=table, n_rows_dev=t.total_rows, trace=trace)
        else:
            wait = lambda i: (lambda: K.p2p_row_table_wait(t, buffers, 0, buffers.d * 2, slot(i)))    # noqa: E731
            parts = [(cuts[i], cuts[i + 1], wait(i) if i else None) for i in range(n_parts)]
            experts(recv_q, recv_s, t.starts, t.ends, row_dst=table, n_rows_dev=t.total_rows, trace=trace, up_parts=parts)
        buffers.barrier()                               # every expert output is home
        _mark(trace, "barrier (outputs home)")
        home = buffers.home.view(buffers.home_rows, buffers.d)[:n_pairs]
        if before_combine is not None:
            before_combine()
        y = K.moe_combine(home, routing.pair_pos, routing.pair_gate, addend)
        _mark(trace, "combine (+ shared expert output)")
        return y
    if callable(addend):
        addend = addend()
    counts_all = torch.empty((world, n_experts), dtype=torch.int64, device=x.device)
    dist.all_gather_into_tensor(counts_all, routing.counts.to(torch.int64).contiguous(), group=group)
    t = p2p.exchange_tables(counts_all, me)
    x_q, x_s = quantize(x)
    buffers.barrier()                                   # every rank is done with the buffers' previous contents
    K.p2p_dispatch(x_q, x_s, routing.token_indices, routing.sorted_experts, t.base_send, t.my_start, buffers.peer_q,
                   buffers.peer_s, e_local, world, buffers.capacity_rows)
    buffers.barrier()                                   # every row has landed
    if fused_return:
        # The down-projection's epilogue stores every finished row straight to its home: the way home runs under
        # the GEMM.  Nothing here needs the number of received rows on the host: the GEMMs walk the device-side
        # expert ranges over the whole buffer, the SwiGLU pass and the address table take the count from the device.
        cap = buffers.capacity_rows
        recv_q = buffers.q.view(cap, buffers.d).view(x_q.dtype)
        recv_s = buffers.s.view(cap, buffers.n_scales)
        table = K.p2p_row_table(t.seg_start, t.home_base, buffers.peer_home, cap, buffers.d * 2, world, buffers.home_rows)
        experts(recv_q, recv_s, t.starts, t.ends, row_dst=table, n_rows_dev=t.total_rows.reshape(1))
    else:
        rows = int(t.total_rows)                        # host read-back: sizes the expert GEMMs' outputs
        assert rows <= buffers.capacity_rows, "peer buffers too small"
        recv_q = buffers.q.view(buffers.capacity_rows, buffers.d)[:rows].view(x_q.dtype)
        recv_s = buffers.s.view(buffers.capacity_rows, buffers.n_scales)[:rows]
        out_rows = experts(recv_q, recv_s, t.starts, t.ends)
        K.p2p_return(out_rows, t.seg_start, t.home_base, buffers.peer_home, world, buffers.home_rows)
    buffers.barrier()                                   # every expert output is home
    home = buffers.home.view(buffers.home_rows, buffers.d)[:n_pairs]
    if before_combine is not None:
        before_combine()
    return K.moe_combine(home, routing.pair_pos, routing.pair_gate, addend)


def moe_forward_pipelined(x: torch.Tensor, routings, experts: Callable, quantize: Callable, group=None,
                          addend: Optional[torch.Tensor] = None, before_combine: Optional[Callable] = None,
                          comm_sms: int = 16) -> torch.Tensor:
    """``moe_forward`` over token chunks with the exchanges of one chunk under the expert GEMMs of another.

    ``routings``: one ``Routing`` per chunk of ``x`` (chunks = ``torch.tensor_split(x, len(routings))``).  All
    chunks share one exchange of counts and one host read-back.  On a GPU the all-to-alls are enqueued on a
    second stream: while chunk c is in the experts, chunk c + 1 is being dispatched and chunk c - 1 is on its
    way home; the GEMMs leave ``comm_sms`` SMs to the send/receive kernels meanwhile.  The arithmetic per token
    is that of ``moe_forward``.  Returns fp32 (T, d)."""
    n = len(routings)
    chunks = torch.tensor_split(x, n)
    adds = torch.tensor_split(addend, n) if addend is not None else [None] * n
    plans = make_plans([r.counts for r in routings], group)
    cuda = x.is_cuda
    prev_limit = None
    if cuda:
        from . import kernels as K
        main = torch.cuda.current_stream(x.device)
        comm = _comm_stream(x.device)
        comm.wait_stream(main)
        if len(plans[0].recv_splits) > 1 and comm_sms > 0:
            # the GEMMs are persistent kernels that would hold every SM: leave a few to the send/receive kernels
            n_sm = torch.cuda.get_device_properties(x.device).multi_processor_count
            prev_limit = K.set_gemm_sm_limit(max(n_sm - comm_sms, n_sm // 2))
    keep = []                                   # every intermediate stays referenced until both streams are joined

    def on_comm(fn, after):
        """Run ``fn`` on the exchange stream once ``after`` (an event of the compute stream) has happened."""
        if not cuda:
            return fn(), None
        with torch.cuda.stream(comm):
            comm.wait_event(after)
            out = fn()
            done = torch.cuda.Event()
            done.record(comm)
        return out, done

    def mark():
        if not cuda:
            return None
        ev = torch.cuda.Event()
        ev.record(main)
        return ev

    # stage 1 for every chunk: quantise, gather, dispatch (the exchanges queue up behind one another on `comm`)
    dispatched = []
    for c in range(n):
        r, plan = routings[c], plans[c]
        if quantize is not None:
            x_q, x_s = quantize(chunks[c])
            send_q, send_s = K.gather_quantized_rows(x_q, x_s, r.token_indices)
            ev = mark()
            (recv_q, recv_s), done = on_comm(lambda sq=send_q, ss=send_s, p=plan: (
                all_to_all_rows(sq, p.send_splits, p.recv_splits, group),
                all_to_all_rows(ss, p.send_splits, p.recv_splits, group)), ev)
            keep += [x_q, x_s, send_q, send_s, recv_q, recv_s]
            dispatched.append((recv_q, recv_s, done))
        else:
            send = chunks[c].index_select(0, r.token_indices)
            recv, done = on_comm(lambda sd=send, p=plan: all_to_all_rows(sd, p.send_splits, p.recv_splits, group), mark())
            dispatched.append((recv, None, done))
    # stage 2 + 3: experts on the compute stream, the way home on the exchange stream
    returning = []
    for c in range(n):
        plan = plans[c]
        recv_q, recv_s, done = dispatched[c]
        if cuda:
            main.wait_event(done)
        if len(plan.recv_splits) > 1:
            if recv_s is not None:
                recv_q, recv_s = K.gather_quantized_rows(recv_q, recv_s, plan.perm)
            else:
                recv_q = recv_q.index_select(0, plan.perm)
        out_rows = experts(recv_q, recv_s, plan.starts, plan.ends)
        if len(plan.recv_splits) > 1:
            if cuda:
                back = K.scatter_rows(out_rows, plan.perm)
            else:
                back = torch.empty_like(out_rows)
                back.index_copy_(0, plan.perm, out_rows)
            home, done = on_comm(lambda b=back, p=plan: all_to_all_rows(b, p.recv_splits, p.send_splits, group), mark())
            keep += [recv_q, recv_s, out_rows, back, home]
        else:
            home, done = out_rows, mark()
        returning.append((home, done))
    if before_combine is not None:
        before_combine()
    ys = []
    for c in range(n):
        home, done = returning[c]
        r = routings[c]
        if cuda:
            main.wait_event(done)
            ys.append(K.moe_combine(home, r.pair_pos, r.pair_gate, adds[c]))
        else:
            y = torch.zeros(chunks[c].shape[0], x.shape[1], dtype=torch.float32, device=x.device)
            y.index_add_(0, r.token_indices, home.float() * r.sorted_scores[:, None])
            ys.append(y if adds[c] is None else adds[c].float() + y)
    if cuda:
        comm.wait_stream(main)                  # the exchange stream outlives none of the buffers it read
        main.wait_stream(comm)
        if prev_limit is not None:
            K.set_gemm_sm_limit(prev_limit)
    del keep
    return torch.cat(ys, dim=0)


_COMM_STREAMS = {}


def _comm_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index
    if key not in _COMM_STREAMS:
        _COMM_STREAMS[key] = torch.cuda.Stream(device)
    return _COMM_STREAMS[key]


class ExpertParallelMoE(torch.nn.Module):
    """Inference/forward module: router + FP8 routed experts sharded over ``group`` (+ an optional shared expert
    whose output is added in the combine pass, ``shared_out + routed_out``, src/layers.py:179).

    Holds this rank's slice of the expert weights: ``w12`` (E/G, 2*I, d), ``w3`` (E/G, d, I).
    """

    def __init__(self, router_weight: torch.Tensor, expert_bias: torch.Tensor, w12_local: torch.Tensor,
                 w3_local: torch.Tensor, top_k: int, group=None, shared: Optional[FP8SwiGLU] = None, n_chunks: int = 1,
                 exchange: str = "nccl", max_tokens_per_rank: Optional[int] = None, check_status_every: int = 0,
                 up_splits: int = 1, dispatch_sms: int = 0):
        """``max_tokens_per_rank`` (peer-store exchanges): the largest number of tokens any rank will ever bring to a
        call; it sizes the receive buffers, whose allocation is a collective, so it must be the same on every rank.
        When omitted the first call agrees on it (one all-reduce of the ranks' token counts, on the first call
        only); a later call with more tokens raises instead of re-allocating (a rank re-allocating on its own would
        leave the others waiting).  ``check_status_every``: read the device status word every so many calls (a host
        synchronisation) and raise when a bounded wait ran out or a row was dropped; 0 = never, the caller polls
        ``kernels.device_status()`` itself.  The output of a call that left a non-zero status is invalid.
        ``up_splits`` ("p2p-fused"; 1, 2 or 4): ranges of local experts that are dispatched and up-projected one
        after the other, the experts of one range at work while the rows of the next arrive.
        ``dispatch_sms`` ("p2p-fused" with a shared expert; 0 = off): the peer stores of the dispatch come from that
        many SMs and the shared expert's GEMMs run beside them on the other SMs, instead of after the dispatch."""
        super().__init__()
        self.up_splits = int(up_splits)
        self.dispatch_sms = int(dispatch_sms)
        self.max_tokens_per_rank = max_tokens_per_rank
        self.check_status_every = int(check_status_every)
        self._calls = 0
        self.trace = None                            # set to a list to collect (phase, CUDA event) pairs of a call
        assert exchange in ("nccl", "p2p", "p2p-fused"), \
            "exchange: 'nccl' (all-to-all collectives), 'p2p' (peer stores) or 'p2p-fused' (way home from the GEMM epilogue)"
        self.exchange = exchange
        self._peer_buffers = None
        from . import kernels as K
        self.K = K
        self.register_buffer("router_weight", router_weight)
        self.register_buffer("expert_bias", expert_bias)
        self._router_cache = (None, None)
        self.top_k = top_k
        self.group = group
        self.experts = FP8Experts(w12_local, w3_local)
        self.shared = shared
        self.n_chunks = max(1, int(n_chunks))      # several ranks: token chunks whose exchanges overlap the experts
        self._side = None

    def _router_as(self, dtype: torch.dtype) -> torch.Tensor:
        """The router weight in the activations' 16-bit type, converted when the weight changes, not per call."""
        w = self.router_weight
        if w.dtype == dtype or dtype not in (torch.bfloat16, torch.float16):
            return w
        key = (dtype, w._version, w.data_ptr())
        if self._router_cache[0] != key:
            self._router_cache = (key, w.to(dtype))
        return self._router_cache[1]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        flat = x.reshape(-1, x.shape[-1])
        router = self._router_as(flat.dtype)
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        sh, join = None, None
        if self.trace is not None and flat.is_cuda:
            _mark(self.trace, "start")
        else:
            self.trace = None
        launch_shared = None
        if self.shared is not None and world > 1 and flat.is_cuda:
            # The shared expert needs nothing from the exchange: it runs on a second stream and is joined before the
            # combine pass.  It is enqueued once the routing (and, with peer stores, the dispatch) has been: its GEMMs
            # take every SM, and launched first they would hold up the routing that every other rank waits for.
            cur = torch.cuda.current_stream(flat.device)
            if self._side is None:
                self._side = torch.cuda.Stream(flat.device)

            narrow = self.dispatch_sms if self.exchange == "p2p-fused" else 0

            def launch_shared():
                self._side.wait_stream(cur)
                prev = None
                if narrow > 0:
                    n_sm = torch.cuda.get_device_properties(flat.device).multi_processor_count
                    prev = self.K.set_gemm_sm_limit(max(n_sm - narrow, n_sm // 2))
                with torch.cuda.stream(self._side):
                    out = self.shared(flat)
                if prev is not None:
                    self.K.set_gemm_sm_limit(prev)
                out.record_stream(cur)
                return out
            join = lambda: cur.wait_stream(self._side)                    # noqa: E731
        elif self.shared is not None:
            sh = self.shared(flat)
            _mark(self.trace, "shared expert (on the main stream: one rank)")
        if world > 1 and self.exchange in ("p2p", "p2p-fused") and flat.is_cuda:
            from . import p2p
            r = route(flat, router, self.expert_bias, self.top_k)
            _mark(self.trace, "router GEMM + routing")
            T, d = flat.shape
            if self._peer_buffers is None:
                if self.max_tokens_per_rank is None:
                    # first call: the ranks agree on the largest token count among them (they all are in their first call)
                    m = torch.tensor([T], dtype=torch.int64, device=flat.device)
                    dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.group)
                    self.max_tokens_per_rank = int(m.item())
                home_rows = self.max_tokens_per_rank * self.top_k
                try:
                    # worst case: every pair of every rank routed to this rank's experts
                    self._peer_buffers = p2p.PeerBuffers(self.group, flat.device, home_rows * world, home_rows, d,
                                                         (d + 127) // 128, n_experts=self.router_weight.shape[0])
                except Exception as exc:                    # noqa: BLE001  (no symmetric memory here: the same on every rank)
                    import warnings
                    warnings.warn(f"symmetric memory is not available ({type(exc).__name__}: {exc}); "
                                  "the expert-parallel exchange uses all-to-all collectives instead")
                    self.exchange = "nccl"
                    return self.forward(x)
            if T > self.max_tokens_per_rank or d != self._peer_buffers.d:
                raise ValueError(f"{T} tokens of width {d} in this call, but the peer buffers were sized for at most "
                                 f"{self.max_tokens_per_rank} tokens of width {self._peer_buffers.d} per rank: construct the "
                                 "layer with max_tokens_per_rank set to the largest batch (the same value on every rank)")
            y = moe_forward_p2p(flat, r, self.experts, self.K.quantize_fp8_rowwise, self._peer_buffers, self.group,
                                addend=launch_shared if launch_shared is not None else sh,
                                before_combine=join, fused_return=self.exchange == "p2p-fused", trace=self.trace,
                                up_splits=self.up_splits,
                                dispatch_sms=self.dispatch_sms if launch_shared is not None else 0)
            self._calls += 1
            if self.check_status_every and self._calls % self.check_status_every == 0:
                status = self.K.device_status()
                if status:
                    raise RuntimeError(f"expert-parallel exchange: device status {status >> 8}/{status & 255} (a bounded wait "
                                       "ran out or a row fell outside a buffer); the outputs since the last check are invalid")
        elif world > 1 and self.n_chunks > 1 and flat.shape[0] >= self.n_chunks:
            routings = [route(c, router, self.expert_bias, self.top_k) for c in torch.tensor_split(flat, self.n_chunks)]
            if launch_shared is not None:
                sh = launch_shared()
            y = moe_forward_pipelined(flat, routings, self.experts, self.K.quantize_fp8_rowwise, self.group, addend=sh,
                                      before_combine=join)
        else:
            r = route(flat, router, self.expert_bias, self.top_k)
            _mark(self.trace, "router GEMM + routing")
            if launch_shared is not None:
                sh = launch_shared()
            y = moe_forward(flat, r, self.experts, self.K.quantize_fp8_rowwise, self.group, addend=sh, before_combine=join,
                            trace=self.trace)
        return y.reshape(x.shape)
