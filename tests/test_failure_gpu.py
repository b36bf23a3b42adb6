"""Give-up paths of the device-side waits and range checks, made to happen on purpose - by conditions set up on
the host, never by a fault: a barrier flag that nobody sets (the wait limit shortened to about a millisecond), a
receive buffer that is too small, an address table that points nowhere.  Each kernel must return, leave its code in
the device status word, leave memory outside the valid range untouched, and leave the context usable: a GEMM run
afterwards still passes parity.  (The reference has no device-side waits; the status word replaces a hung GPU.)"""
import ctypes

import pytest
import torch

from _util import rel_fro
from oracle import fp8_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from cinnamon_b200 import kernels
    kernels.device_status()                      # start from a clean word
    yield kernels
    assert kernels.device_status() == 0


def _gemm_still_works(K):
    x, w, _ = O.make_linear_case(256, 512, 384, seed=31)
    xq, xs = O.quantize_rowwise(x, 128)
    wq, ws = O.quantize_blockwise(w.float(), 128, 128)
    ref = O.fp8_matmul_f64(xq, wq.t(), xs, ws.t())
    f8 = lambda t: t.cuda().view(torch.float8_e4m3fn)                                     # noqa: E731
    out = K.fp8_matmul_dsv3(f8(xq), f8(wq).t(), xs.cuda(), ws.cuda().t(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert rel_fro(out, ref) < 2e-5


def test_barrier_wait_runs_out(K):
    """Two "ranks" whose flag arrays are one local buffer: slot 1 is never written, so thread 1's wait cannot end."""
    lib = K._lib.lib
    prev = lib.cinn_set_wait_limit_cycles(2_000_000)                 # about a millisecond
    try:
        assert prev == 4_000_000_000
        flags = torch.zeros(64, dtype=torch.int32, device="cuda")
        peers = torch.tensor([flags.data_ptr(), flags.data_ptr()], dtype=torch.int64, device="cuda")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        K._lib.check(lib.cinn_p2p_barrier(ctypes.c_void_p(peers.data_ptr()), 0, 2, 1, stream), "cinn_p2p_barrier")
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 200.0, "the shortened wait limit was not honoured"
        assert int(flags[0]) == 1 and int(flags[1]) == 0
        assert K.device_status() == (5 << 8) | 3                     # read and reset
        assert K.device_status() == 0
        # with the flag set the same launch passes
        flags[1] = 2
        K._lib.check(lib.cinn_p2p_barrier(ctypes.c_void_p(peers.data_ptr()), 0, 2, 2, stream), "cinn_p2p_barrier")
        torch.cuda.synchronize()
        assert K.device_status() == 0
    finally:
        assert lib.cinn_set_wait_limit_cycles(0) == 2_000_000        # 0 restores the default
        assert lib.cinn_set_wait_limit_cycles(0) == 4_000_000_000
    _gemm_still_works(K)


def test_dispatch_into_a_buffer_that_is_too_small(K):
    """16 rows for a receive buffer of 8: the first 8 land, the others are dropped and reported (code 1); the
    canary behind the buffer is untouched."""
    T, d, cap = 16, 128, 8
    g = torch.Generator().manual_seed(2)
    xq, xs = K.quantize_fp8_rowwise(torch.randn(T, d, generator=g).bfloat16().cuda())
    token_indices = torch.arange(T, dtype=torch.int64, device="cuda")
    sorted_experts = torch.zeros(T, dtype=torch.int64, device="cuda")            # one expert, one rank
    base_send = torch.zeros(1, dtype=torch.int64, device="cuda")
    my_start = torch.zeros(1, dtype=torch.int64, device="cuda")
    recv_q = torch.full((cap + 4, d), 0xAB, dtype=torch.uint8, device="cuda")
    recv_s = torch.full((cap + 4, 1), -7.0, dtype=torch.float32, device="cuda")
    peer_q = torch.tensor([recv_q.data_ptr()], dtype=torch.int64, device="cuda")
    peer_s = torch.tensor([recv_s.data_ptr()], dtype=torch.int64, device="cuda")
    K.p2p_dispatch(xq, xs, token_indices, sorted_experts, base_send, my_start, peer_q, peer_s, 1, 1, cap)
    torch.cuda.synchronize()
    assert K.device_status() == (5 << 8) | 1
    assert torch.equal(recv_q[:cap], xq.view(torch.uint8)[:cap]) and torch.equal(recv_s[:cap], xs[:cap])
    assert torch.all(recv_q[cap:] == 0xAB) and torch.all(recv_s[cap:] == -7.0)
    _gemm_still_works(K)


def test_return_and_row_table_with_destinations_out_of_range(K):
    """Expert outputs whose home row lies past the home buffer: skipped and reported (codes 2 and 4)."""
    n, d, cap = 8, 64, 4
    rows = torch.randn(n, d, device="cuda").bfloat16()
    seg_start = torch.tensor([0, n], dtype=torch.int64, device="cuda")           # one segment
    home_base = torch.zeros(1, dtype=torch.int64, device="cuda")
    home = torch.full((cap + 2, d), 5.0, dtype=torch.bfloat16, device="cuda")
    peer_home = torch.tensor([home.data_ptr()], dtype=torch.int64, device="cuda")
    K.p2p_return(rows, seg_start, home_base, peer_home, 1, cap)
    torch.cuda.synchronize()
    assert K.device_status() == (5 << 8) | 2
    assert torch.equal(home[:cap], rows[:cap]) and torch.all(home[cap:] == 5.0)
    table = K.p2p_row_table(seg_start, home_base, peer_home, n, d * 2, 1, cap)
    torch.cuda.synchronize()
    assert K.device_status() == (5 << 8) | 4
    expect = [home.data_ptr() + i * d * 2 for i in range(cap)] + [0] * (n - cap)
    assert table.tolist() == expect
    _gemm_still_works(K)
