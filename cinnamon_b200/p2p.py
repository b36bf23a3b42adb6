"""Expert-parallel exchange by direct peer stores over NVLink, instead of all-to-all collectives.

Every rank keeps three buffers in symmetric memory (``torch.distributed._symmetric_memory``): where other
ranks drop the e4m3 rows and the scales of the tokens routed to its experts, and where they drop the expert
outputs of its own tokens on the way home.  With the routing counts of all ranks known everywhere (one small
all-gather), every row has a fixed address on its destination:

  dispatch  pair r of rank ``me`` (sorted by expert, expert e = its r-th sorted expert) lands on the rank that
            owns e, in that rank's expert-grouped order (expert-major, source-rank-minor): row
            ``start(e) + sum_{g < me} C[g][e] + (r - my_start[e])``
  return    row r' of the expert-grouped order on the expert's rank belongs to segment (e, g) and goes home to
            rank g at ``g_start[g][e] + (r' - seg_start[e][g])``: exactly the sorted-pair order the combine reads

so the gather, both dispatch all-to-alls and the regrouping collapse into one kernel that reads the quantised
tokens and writes peer memory, and the inverse permutation and the combine all-to-all into another.  The
reference keeps every expert on every rank (src/layers.py:89-179) and has no exchange at all; the arithmetic per
row is unchanged.

The address tables are plain tensor arithmetic on the (G, E) count matrix (`exchange_tables`), tested on the
CPU against a sort-based statement of the same exchange.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


def _excl_cumsum(t: torch.Tensor, dim: int) -> torch.Tensor:
    return t.cumsum(dim) - t


@dataclass
class ExchangeTables:
    base_send: torch.Tensor     # (E,)  destination row of my first pair of expert e, on the rank that owns e
    my_start: torch.Tensor      # (E,)  first position of expert e in my sorted pairs
    starts: torch.Tensor        # (E_local,) first row of my local experts in my expert-grouped buffer
    ends: torch.Tensor          # (E_local,)
    seg_start: torch.Tensor     # (E_local * G + 1,) first row of segment (local expert, source rank); last = total rows
    home_base: torch.Tensor     # (E_local * G,) row on the source rank where segment (local expert, source) starts
    total_rows: torch.Tensor    # () rows in my expert-grouped buffer


def exchange_tables(counts_all: torch.Tensor, me: int) -> ExchangeTables:
    """``counts_all``: (G, E) int64, pairs every rank routed to every global expert."""
    G, E = counts_all.shape
    e_local = E // G
    C = counts_all.to(torch.int64)
    per_expert = C.sum(0)                                                   # (E,)
    starts_all = _excl_cumsum(per_expert.view(G, e_local), 1).reshape(E)    # within the owning rank
    src_prefix = _excl_cumsum(C, 0)                                         # (G, E): rows of lower-ranked sources
    sorted_start = _excl_cumsum(C, 1)                                       # (G, E): position of e in g's sorted pairs
    lo, hi = me * e_local, (me + 1) * e_local
    starts = starts_all[lo:hi]
    ends = starts + per_expert[lo:hi]
    seg = (starts.view(e_local, 1) + src_prefix[:, lo:hi].t()).reshape(-1)  # (e_local * G,), expert-major
    total = per_expert[lo:hi].sum()
    return ExchangeTables(base_send=(starts_all + src_prefix[me]).contiguous(), my_start=sorted_start[me].contiguous(),
                          starts=starts.contiguous(), ends=ends.contiguous(),
                          seg_start=torch.cat([seg, total.view(1)]).contiguous(),
                          home_base=sorted_start[:, lo:hi].t().reshape(-1).contiguous(), total_rows=total)


class PeerBuffers:
    """The three receive buffers of one rank, allocated in symmetric memory and mapped into every rank of the
    group, plus the device arrays of peer base addresses that the kernels take.  Creating it is a collective."""

    # flag slots: [0, 64) the barrier, [64, 128) "my routing counts are in your matrix", [128, 192) "my rows have landed"
    PLAN_SLOT, LANDED_SLOT = 64, 128

    def __init__(self, group, device, capacity_rows: int, home_rows: int, d: int, n_scales: int, n_experts: int = 0):
        import os
        import torch.distributed as dist
        # The exchange uses plain peer stores only.  PyTorch would otherwise also bind the buffers to an NVLink
        # multicast object where the switch supports it; a rank that dies while bound to one can raise NVLink
        # faults on its peers' GPUs, so the binding is switched off (PyTorch's documented environment switch).
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.capacity_rows, self.home_rows, self.d, self.n_scales = int(capacity_rows), int(home_rows), int(d), int(n_scales)
        self.q = symm_mem.empty(self.capacity_rows * d, dtype=torch.uint8, device=device)
        self.s = symm_mem.empty(self.capacity_rows * n_scales, dtype=torch.float32, device=device)
        self.home = symm_mem.empty(self.home_rows * d, dtype=torch.bfloat16, device=device)
        self.flags = symm_mem.empty(256, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.n_experts = int(n_experts)
        # every rank's routing counts, one row per source rank (written by the ranks themselves, cinn_p2p_plan)
        self.counts = symm_mem.empty(max(1, self.world * self.n_experts), dtype=torch.int64, device=device)
        self.counts.zero_()
        self._handles = [symm_mem.rendezvous(t, self.group) for t in (self.q, self.s, self.home, self.flags, self.counts)]
        as_dev = lambda h: torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64, device=device)   # noqa: E731
        self.peer_q, self.peer_s, self.peer_home, self.peer_flags, self.peer_counts = (as_dev(h) for h in self._handles)
        self._epoch = 0
        self._call = 0                                  # layer calls so far: the epoch of the plan / landed flags
        self.done = torch.zeros(1, dtype=torch.int32, device=device)
        if self.n_experts:
            e_local = self.n_experts // self.world
            i64 = lambda n: torch.empty(n, dtype=torch.int64, device=device)                                 # noqa: E731
            self._tables = ExchangeTables(base_send=i64(self.n_experts), my_start=i64(self.n_experts), starts=i64(e_local),
                                          ends=i64(e_local), seg_start=i64(e_local * self.world + 1),
                                          home_base=i64(e_local * self.world), total_rows=i64(1))
        torch.cuda.synchronize(device)
        dist.barrier(self.group)                        # every rank's flags are zero before anyone signals

    def barrier(self) -> None:
        """Stream-ordered barrier over the ranks (``cinn_p2p_barrier``): bounded device-side wait on flags in
        symmetric memory, no host synchronisation, no collective."""
        import ctypes
        from . import _lib
        self._epoch += 1
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.flags.device).cuda_stream)
        with torch.cuda.device(self.flags.device):
            _lib.check(_lib.lib.cinn_p2p_barrier(ctypes.c_void_p(self.peer_flags.data_ptr()), self.rank, self.world,
                                                 self._epoch & 0x7FFFFFFF, stream), "cinn_p2p_barrier")

    def plan(self, counts: torch.Tensor) -> "ExchangeTables":
        """One launch (``cinn_p2p_plan``): this rank's routing counts go to every rank, the counts of all ranks are
        awaited (bounded), and the address tables of ``exchange_tables`` come out.  Starts a new layer call: the
        epoch it uses is the one ``dispatch_signal`` / ``row_table_wait`` of the same call use.  The tables are
        buffers owned by this object, overwritten by the next call."""
        import ctypes
        from . import _lib
        assert self.n_experts and counts.numel() == self.n_experts and counts.dtype == torch.int64 and counts.is_contiguous()
        self._call += 1
        t = self._tables
        p = lambda x: ctypes.c_void_p(x.data_ptr())                                                          # noqa: E731
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.flags.device).cuda_stream)
        with torch.cuda.device(self.flags.device):
            _lib.check(_lib.lib.cinn_p2p_plan(p(counts), p(self.peer_counts), p(self.peer_flags), self.rank, self.world,
                                              self.n_experts, self.PLAN_SLOT, self._call & 0x7FFFFFFF, p(t.base_send),
                                              p(t.my_start), p(t.starts), p(t.ends), p(t.seg_start), p(t.home_base),
                                              p(t.total_rows), stream), "cinn_p2p_plan")
        return t

    def fits(self, capacity_rows: int, home_rows: int, d: int, n_scales: int) -> bool:
        return (capacity_rows <= self.capacity_rows and home_rows <= self.home_rows and d == self.d
                and n_scales == self.n_scales)
