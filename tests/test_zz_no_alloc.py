"""The routing entry point that brings its own scratch memory (``cinn_moe_route_static``).

Some hosts cannot give a library any device memory at call time: a serving process that handed the whole of
HBM to its own arena when it started, a job running at the memory limit, a latency-bound loop in which an
allocation (and the device-wide synchronisation it can imply) is not acceptable.  For them the library keeps a
fixed 2 MiB array inside its own image and routes with that; inputs and outputs still belong to the caller.

The test calls the entry point through the C ABI, twice in a row (the second call finds the first call's
leftovers in the shared array), and wants the very same bits as ``cinn_moe_route`` with a caller-provided
workspace: both run the same kernels, so the tolerance is zero.  It also checks that a problem too large for the
array is refused with a message instead of being run.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

OUTPUTS = (("top_experts", torch.int32, "Tk"), ("top_gates", torch.float32, "Tk"), ("token_indices", torch.int64, "N"),
           ("sorted_scores", torch.float32, "N"), ("sorted_experts", torch.int64, "N"), ("counts", torch.int64, "E"),
           ("pair_pos", torch.int64, "Tk"), ("pair_gate", torch.float32, "Tk"))


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _outputs(T, E, k, dev):
    shape = {"Tk": (T, k), "N": (T * k,), "E": (E,)}
    # filled with a pattern, so that a word the kernels fail to write shows up in the comparison
    return {name: torch.full(shape[kind], 123, dtype=dt, device=dev) for name, dt, kind in OUTPUTS}


def _route_static(L, logits, bias, k):
    T, E = logits.shape
    out = _outputs(T, E, k, logits.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.cinn_moe_route_static(_ptr(logits), _ptr(bias), T, E, k, *[_ptr(out[name]) for name, _, _ in OUTPUTS], stream)
    return rc, out


def _route_with_workspace(L, logits, bias, k):
    T, E = logits.shape
    out = _outputs(T, E, k, logits.device)
    ws = torch.empty(int(L.cinn_moe_route_workspace_ints(T, E)), dtype=torch.int32, device=logits.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.cinn_moe_route(_ptr(logits), _ptr(bias), T, E, k, _ptr(ws), *[_ptr(out[name]) for name, _, _ in OUTPUTS], stream)
    return rc, out


def test_route_without_allocation_matches_route_with_workspace():
    from cinnamon_b200 import _lib
    L = _lib.lib
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(4242)
    # two calls in a row on the shared array: a larger problem first, then a smaller one with other sizes
    for T, E, k in ((5000, 256, 8), (333, 64, 3)):
        logits = (torch.randn(T, E, generator=g) * 2.0).to(dev)
        bias = (torch.randn(E, generator=g) * 0.5).to(dev)
        rc, got = _route_static(L, logits, bias, k)
        assert rc == 0, _lib.last_error()
        rc, ref = _route_with_workspace(L, logits, bias, k)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        for name, _, _ in OUTPUTS:
            assert torch.equal(got[name], ref[name]), f"{name} differs for T={T} E={E} k={k}"
        assert int(got["counts"].sum()) == T * k


def test_route_without_allocation_refuses_what_does_not_fit():
    from cinnamon_b200 import _lib
    L = _lib.lib
    limit = int(L.cinn_moe_route_static_max_ints())
    assert limit == 1 << 19
    E, k = 1024, 2
    T = 128 * (limit // E) + 1                      # one CTA of tokens more than the array can serve
    assert int(L.cinn_moe_route_workspace_ints(T, E)) > limit
    # nothing is launched for a refused call, so no buffers are needed to see the refusal
    rc = L.cinn_moe_route_static(None, None, T, E, k, None, None, None, None, None, None, None, None, None)
    assert rc == _lib.ERR_INVALID
    assert "scratch" in _lib.last_error() and "cinn_moe_route" in _lib.last_error()
