"""Host-side logic of the expert-parallel MoE layer on CPU ranks (gloo, world_size 2):
the exchange plan, both all-to-alls and the permutations, with a plain torch expert
function standing in for the FP8 kernels; and a rank that leaves before the exchange."""
import datetime
import os
import socket
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cinnamon_b200 import moe

E, D, I, TOPK, T = 8, 64, 32, 2, 96


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _weights():
    g = torch.Generator().manual_seed(4)
    router = torch.randn(E, D, generator=g) * 0.02
    bias = torch.randn(E, generator=g)
    w12 = torch.randn(E, 2 * I, D, generator=g) * 0.1
    w3 = torch.randn(E, D, I, generator=g) * 0.1
    return router, bias, w12, w3


def _tokens(rank):
    return torch.randn(T, D, generator=torch.Generator().manual_seed(100 + rank))


def _plain_experts(w12, w3):
    """fp32 SwiGLU per expert over ragged row ranges (the reference's fallback loop, src/layers.py:76-87)."""
    def fn(rows, _scales, starts, ends):
        out = torch.zeros(rows.shape[0], w3.shape[1])
        for e in range(w12.shape[0]):
            s, t = int(starts[e]), int(ends[e])
            if t > s:
                h1, h2 = (rows[s:t] @ w12[e].t()).chunk(2, dim=-1)
                out[s:t] = (torch.nn.functional.silu(h1) * h2) @ w3[e].t()
        return out
    return fn


def _reference(rank):
    router, bias, w12, w3 = _weights()
    x = _tokens(rank)
    r = moe.route(x, router, bias, TOPK)
    return moe.moe_forward(x, r, _plain_experts(w12, w3), None)


def _worker(rank, world, port, q, leave_early):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
        router, bias, w12, w3 = _weights()
        lo, hi = rank * E // world, (rank + 1) * E // world
        x = _tokens(rank)
        r = moe.route(x, router, bias, TOPK)
        if leave_early and rank == 1:
            q.put((rank, "left", None))          # between steps, nothing in flight
            q.close()
            q.join_thread()
            os._exit(0)
        y = moe.moe_forward(x, r, _plain_experts(w12[lo:hi], w3[lo:hi]), None)
        plan = moe.make_plan(r.counts)
        # the same tokens in three chunks (uneven: 3 does not divide the token count) through the pipelined path
        routings = [moe.route(c, router, bias, TOPK) for c in torch.tensor_split(x, 3)]
        y_chunks = moe.moe_forward_pipelined(x, routings, _plain_experts(w12[lo:hi], w3[lo:hi]), None, addend=x.float())
        q.put((rank, "ok", (y, plan.recv_counts.clone(), r.counts.clone(), y_chunks - x.float())))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:                     # noqa: BLE001
        q.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()[-400:]}"))


def _run(world, leave_early):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, leave_early)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, status, payload = q.get(timeout=120)
        results[rank] = (status, payload)
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    return results


def test_plan_single_process():
    counts = torch.tensor([3, 0, 5, 1])
    plan = moe.make_plan(counts)
    assert plan.send_splits == [9] and plan.recv_splits == [9]
    assert plan.starts.tolist() == [0, 3, 3, 8] and plan.ends.tolist() == [3, 3, 8, 9]
    assert plan.perm is None                       # one rank: rows already arrive grouped by expert
    assert moe.make_plan(counts, n_pairs=9).send_splits == [9]      # no host read-back when the caller knows the total


def test_two_ranks_match_single_rank():
    res = _run(2, leave_early=False)
    for rank in range(2):
        status, payload = res[rank]
        assert status == "ok", payload
        y, recv_counts, counts, y_chunks = payload
        torch.testing.assert_close(y, _reference(rank), rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(y_chunks, _reference(rank), rtol=1e-5, atol=1e-5)
    # what rank r received from rank s for its experts is what s routed there
    for r in range(2):
        for s in range(2):
            sent = res[s][1][2].reshape(2, E // 2)[r]
            assert torch.equal(res[r][1][1][s], sent)


def test_rank_leaving_before_the_exchange_is_reported():
    res = _run(2, leave_early=True)
    assert res[1][0] == "left"
    status, payload = res[0]
    assert status == "error", "the surviving rank must fail, not hang or succeed"
    assert any(k in payload for k in ("Timed out", "timeout", "Connection", "closed", "peer", "reset", "Gloo")), payload
