"""Address tables of the peer-store exchange (cinnamon_b200/p2p.py) against a sort-based statement of the same
exchange, for all ranks simulated in one process (no GPU, no process group)."""
import pytest
import torch

from cinnamon_b200 import p2p


@pytest.mark.parametrize("G,E,T,k,seed", [(2, 8, 37, 2, 0), (4, 16, 50, 3, 1), (8, 64, 129, 8, 2), (1, 4, 10, 2, 3)])
def test_dispatch_and_return_addresses(G, E, T, k, seed):
    g = torch.Generator().manual_seed(seed)
    e_local = E // G
    # per rank: experts of its T*k pairs, already sorted by expert (what routing produces), some experts empty
    sorted_experts = [torch.randint(0, E, (T * k,), generator=g).sort().values for _ in range(G)]
    for se in sorted_experts:
        se[se == 1] = 2
    sorted_experts = [se.sort().values for se in sorted_experts]
    counts = torch.stack([torch.bincount(se, minlength=E) for se in sorted_experts])
    tables = [p2p.exchange_tables(counts, me) for me in range(G)]
    # --- dispatch: every rank writes (source rank, pair index) into the owners' buffers
    recv = [torch.full((int(t.total_rows), 2), -1, dtype=torch.int64) for t in tables]
    for me in range(G):
        t = tables[me]
        r = torch.arange(T * k)
        e = sorted_experts[me]
        dst = t.base_send[e] + (r - t.my_start[e])
        owner = e // e_local
        for m in range(G):
            sel = owner == m
            assert dst[sel].numel() == 0 or int(dst[sel].max()) < recv[m].shape[0]
            recv[m][dst[sel], 0] = me
            recv[m][dst[sel], 1] = r[sel]
    for m in range(G):
        t = tables[m]
        assert (recv[m] >= 0).all()                                          # every row written exactly once
        # expert-grouped: rows [starts[e], ends[e]) hold expert e, sources ascending, pair order kept
        for el in range(e_local):
            rows = recv[m][int(t.starts[el]):int(t.ends[el])]
            src, pair = rows[:, 0], rows[:, 1]
            assert torch.equal(src, src.sort().values)
            for s in range(G):
                assert (sorted_experts[s][pair[src == s]] == m * e_local + el).all()
                assert torch.equal(pair[src == s], pair[src == s].sort().values)
        assert int(t.seg_start[-1]) == recv[m].shape[0]
    # --- return: every expert rank sends row r' home; it must land on the pair it came from
    for m in range(G):
        t = tables[m]
        R = int(t.total_rows)
        rp = torch.arange(R)
        seg = torch.searchsorted(t.seg_start[1:].contiguous(), rp, right=True)          # segment of every row
        src = seg % G
        home_row = t.home_base[seg] + (rp - t.seg_start[seg])
        assert torch.equal(src, recv[m][:, 0])
        assert torch.equal(home_row, recv[m][:, 1])
