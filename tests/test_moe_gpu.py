"""MoE routed path on the GPU: fused SwiGLU quantiser, FP8 experts against the float64
oracle, and expert-parallel (2 GPUs, NCCL) against the single-GPU result."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from _util import bits_of, bytes_of, rel_fro
from oracle import fp8_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def K():
    from cinnamon_b200 import kernels
    kernels.set_div_mode("rn")
    yield kernels
    assert kernels.device_status() == 0
    kernels.set_div_mode("full")


def _oracle_swiglu(h12: torch.Tensor):
    h1, h2 = h12.float().chunk(2, dim=-1)
    return (torch.nn.functional.silu(h1) * h2).to(h12.dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("T,I", [(64, 256), (33, 200), (1, 2048)])
def test_swiglu_quantiser(K, dtype, T, I):
    g = torch.Generator().manual_seed(T + I)
    h12 = (torch.randn(T, 2 * I, generator=g) * 2).to(dtype)
    q, s = K.swiglu_quantize_rowwise(h12.cuda())
    # the same arithmetic with torch ops on the GPU (same expf), quantised by the oracle
    h_gpu = _oracle_swiglu(h12.cuda()).cpu()
    rq, rs = O.quantize_rowwise(h_gpu, 128)
    assert q.shape == (T, I) and s.shape == rs.shape
    frac_s = float((bits_of(s) != rs.numpy().view(np.uint32)).mean())
    frac_q = float((bytes_of(q) != rq.numpy()).mean())
    assert frac_s <= 0.02 and frac_q <= 0.02, (frac_s, frac_q)     # silu may differ in the last ulp before rounding
    # and against the CPU arithmetic within one e4m3 step of the tile scale
    h_cpu = _oracle_swiglu(h12)
    deq = O.dequantize_rowwise(torch.from_numpy(bytes_of(q)), s.cpu(), 128)
    tol = s.cpu().repeat_interleave(128, dim=1)[:, :I] * 32 + 1e-6          # half a step at the top binade
    assert torch.all((deq - h_cpu.float()).abs() <= tol)


def test_swiglu_quantiser_device_row_count(K):
    """Only the first n rows (a count that lives on the device) are converted; the rest of the buffer is left alone."""
    g = torch.Generator().manual_seed(19)
    h12 = (torch.randn(200, 512, generator=g) * 2).bfloat16().cuda()
    n = torch.tensor([77], dtype=torch.int64, device="cuda")
    q_all, s_all = K.swiglu_quantize_rowwise(h12)
    from cinnamon_b200 import _lib
    import ctypes
    q = torch.full((200, 256), 0x55, dtype=torch.uint8, device="cuda")
    s = torch.full((200, 2), -1.0, device="cuda")
    tag = {torch.bfloat16: _lib.BF16}[h12.dtype]
    mode = _lib.DIV_RN if K.get_div_mode() == "rn" else _lib.DIV_FULL
    rc = _lib.lib.cinn_swiglu_quant_rowwise_n(ctypes.c_void_p(h12.data_ptr()), tag, 200, 256, ctypes.c_void_p(n.data_ptr()),
                                              ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(s.data_ptr()), mode,
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _lib.last_error()
    assert torch.equal(q[:77], q_all.view(torch.uint8)[:77]) and torch.equal(s[:77], s_all[:77])
    assert torch.all(q[77:] == 0x55) and torch.all(s[77:] == -1.0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu_forward_backward(K, dtype):
    """The training-path SwiGLU kernels against torch's fp32 arithmetic (src/layers.py:71-74) and its autograd."""
    g = torch.Generator().manual_seed(31)
    h12 = (torch.randn(3, 50, 2 * 136, generator=g) * 2).to(dtype).cuda().requires_grad_(True)
    go = torch.randn(3, 50, 136, generator=g).to(dtype).cuda()
    h = K.swiglu(h12)
    h.backward(go)
    ref_in = h12.detach().float().requires_grad_(True)
    h1, h2 = ref_in.chunk(2, dim=-1)
    ref = torch.nn.functional.silu(h1) * h2
    ref.backward(go.float())
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    assert h.dtype == dtype and h12.grad.dtype == dtype
    torch.testing.assert_close(h.float(), ref, rtol=tol, atol=tol)
    torch.testing.assert_close(h12.grad.float(), ref_in.grad, rtol=tol, atol=tol)


def test_combine_kernel_matches_scatter_add(K):
    g = torch.Generator().manual_seed(8)
    T, k, d = 77, 4, 264
    rows = torch.randn(T * k + 5, d, generator=g).bfloat16()
    pos = torch.stack([torch.randperm(T * k, generator=g)[:k].sort().values for _ in range(T)])
    pos[3, 1] = -1                                                     # a skipped pair
    gates = torch.rand(T, k, generator=g)
    y = K.moe_combine(rows.cuda(), pos.cuda(), gates.cuda())
    ref = torch.zeros(T, d)
    for t in range(T):
        for j in range(k):
            if pos[t, j] >= 0:
                ref[t] += rows[pos[t, j]].float() * gates[t, j]
    assert torch.equal(y.cpu(), ref)                                   # same products, same order of sums
    # with the shared experts' output folded in: shared_out + routed_out (src/layers.py:179)
    for dt in (torch.bfloat16, torch.float32, torch.float16):
        shared = torch.randn(T, d, generator=g).to(dt)
        y2 = K.moe_combine(rows.cuda(), pos.cuda(), gates.cuda(), addend=shared.cuda())
        assert torch.equal(y2.cpu(), shared.float() + ref), dt


@pytest.mark.parametrize("T,E,k", [(1000, 256, 8), (128, 16, 2), (1, 8, 3), (777, 257, 5), (4096, 64, 6), (300, 1024, 32)])
def test_route_kernel_matches_torch(K, T, E, k):
    """Device routing (three launches) against the reference's chain of torch calls (src/layers.py:122-148) on
    the same logits: same experts, same stable order, gates to fp32 rounding."""
    from cinnamon_b200 import moe
    g = torch.Generator().manual_seed(T + E + k)
    logits = (torch.randn(T, E, generator=g) * 2.0).cuda()
    bias = (torch.randn(E, generator=g) * 0.5).cuda()
    got = K.moe_route(logits, bias, k)
    ref = moe.route_torch(logits, bias, k, E)
    assert torch.equal(got["counts"], ref.counts)
    assert torch.equal(got["sorted_experts"], ref.sorted_experts)
    assert torch.equal(got["token_indices"], ref.token_indices)
    assert torch.equal(got["pair_pos"], ref.pair_pos)
    torch.testing.assert_close(got["sorted_scores"], ref.sorted_scores, rtol=2e-6, atol=1e-8)
    torch.testing.assert_close(got["pair_gate"], ref.pair_gate, rtol=2e-6, atol=1e-8)
    sel = torch.sigmoid(logits) + bias
    assert torch.equal(got["top_experts"].long(), sel.topk(k, dim=-1).indices)
    torch.testing.assert_close(got["top_gates"].sum(1), torch.ones(T, device="cuda"), rtol=1e-5, atol=1e-6)
    # the same call again gives the same bits (no atomics decide an order)
    again = K.moe_route(logits, bias, k)
    for key in got:
        assert torch.equal(got[key], again[key]), key


def test_gather_quantized_rows(K):
    g = torch.Generator().manual_seed(5)
    q = torch.randint(0, 256, (300, 512), generator=g, dtype=torch.uint8).cuda().view(torch.float8_e4m3fn)
    s = torch.rand(300, 4, generator=g).cuda()
    idx = torch.randint(0, 300, (1000,), generator=g).cuda()
    out_q, out_s = K.gather_quantized_rows(q, s, idx)
    assert torch.equal(out_q.view(torch.uint8), q.view(torch.uint8)[idx]) and torch.equal(out_s, s[idx])
    out_q, out_s = K.gather_quantized_rows(q[:, :72].contiguous(), s[:, :1].contiguous(), idx)   # width not a multiple of 16
    assert torch.equal(out_q.view(torch.uint8), q.view(torch.uint8)[:, :72][idx]) and torch.equal(out_s, s[:, :1][idx])


def test_scatter_rows(K):
    g = torch.Generator().manual_seed(6)
    rows = torch.randn(500, 264, generator=g).bfloat16().cuda()              # 528-byte rows
    perm = torch.randperm(500, generator=g).cuda()
    assert torch.equal(K.scatter_rows(rows, perm), torch.empty_like(rows).index_copy_(0, perm, rows))
    odd = rows[:, :13].contiguous()                                          # 26-byte rows: the torch path
    assert torch.equal(K.scatter_rows(odd, perm), torch.empty_like(odd).index_copy_(0, perm, odd))


def test_route_ties_and_saturation(K):
    """Equal scores go to the lower expert id; saturated sigmoids (score exactly 1) and a NaN logit do not break
    the invariants (k distinct experts per token, counts add up, rows sorted by expert)."""
    T, E, k = 64, 40, 4
    logits = torch.zeros(T, E, device="cuda")
    logits[1] = 50.0                                  # every score saturates to 1.0: pure ties
    logits[2, 7] = float("nan")
    logits[3, :5] = torch.tensor([3.0, 3.0, 2.0, 3.0, 1.0], device="cuda")
    got = K.moe_route(logits, torch.zeros(E, device="cuda"), k)
    top = got["top_experts"].long()
    assert top[0].tolist() == [0, 1, 2, 3] and top[1].tolist() == [0, 1, 2, 3]
    assert 7 not in top[2].tolist() and top[3].tolist() == [0, 1, 3, 2]
    assert all(len(set(row)) == k for row in top.tolist())
    assert int(got["counts"].sum()) == T * k
    assert torch.equal(got["sorted_experts"], got["sorted_experts"].sort().values)
    assert torch.equal(torch.bincount(top.reshape(-1), minlength=E), got["counts"])


def test_route_empty(K):
    got = K.moe_route(torch.empty(0, 32, device="cuda"), torch.zeros(32, device="cuda"), 4)
    assert got["counts"].tolist() == [0] * 32 and got["token_indices"].numel() == 0


def _moe_case(E, d, I, T, top_k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, d, generator=g).bfloat16()
    router = torch.randn(E, d, generator=g) * 0.02
    bias = torch.randn(E, generator=g) * 0.3
    w12 = (torch.randn(E, 2 * I, d, generator=g) * 0.02).bfloat16()
    w3 = (torch.randn(E, d, I, generator=g) * 0.02).bfloat16()
    return x, router, bias, w12, w3


def _oracle_moe(x, routing, w12, w3):
    """float64 restatement: e4m3 tokens (1x128) x e4m3 weights (128x128) -> bf16 h12 -> SwiGLU -> bf16 ->
    e4m3 (1x128) x e4m3 weights -> bf16 rows -> gate-weighted sum (src/layers.py:69-75, 157-160)."""
    ti = routing.token_indices.cpu()
    counts = routing.counts.cpu()
    ends = counts.cumsum(0)
    starts = ends - counts
    rows = x[ti]
    h12 = O.grouped_gemm_fp8_f64(rows, w12, starts, ends).to(torch.bfloat16)
    h = _oracle_swiglu(h12)
    out = O.grouped_gemm_fp8_f64(h, w3, starts, ends).to(torch.bfloat16)
    y = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float64)
    y.index_add_(0, ti, out.double() * routing.sorted_scores.cpu().double()[:, None])
    return y


def test_fp8_moe_single_gpu(K):
    from cinnamon_b200 import moe
    E, d, I, T, k = 8, 512, 256, 300, 2
    x, router, bias, w12, w3 = _moe_case(E, d, I, T, k, seed=21)
    xc = x.cuda()
    r = moe.route(xc, router.cuda(), bias.cuda(), k)
    experts = moe.FP8Experts(w12.cuda(), w3.cuda())
    y = moe.moe_forward(xc, r, experts, K.quantize_fp8_rowwise)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    ref = _oracle_moe(x, r, w12, w3)
    err = rel_fro(y, ref)
    print(f"MoE routed path: rel-Fro {err:.3e}")
    assert err < 5e-3                       # two bf16 roundings (h12, rows) on top of the GEMM error
    layer = moe.ExpertParallelMoE(router.cuda(), bias.cuda(), w12.cuda(), w3.cuda(), k)
    y2 = layer(xc.view(3, 100, d))
    assert y2.shape == (3, 100, d) and rel_fro(y2.reshape(T, d), ref) < 5e-3


@pytest.mark.parametrize("rs", [False, True])
def test_shared_expert_and_combined_layer(K, rs):
    """FP8SwiGLU (w1|w2 as one GEMM, fused SiLU-product-quantise, w3) against the oracle's FP8 linears, and the
    layer output shared + routed from the one combine pass."""
    from cinnamon_b200 import moe
    E, d, I, T, k, H = 8, 512, 256, 300, 2, 384
    x, router, bias, w12, w3 = _moe_case(E, d, I, T, k, seed=23)
    g = torch.Generator().manual_seed(24)
    s1, s2, s3 = (torch.randn(H, d, generator=g) * 0.02, torch.randn(H, d, generator=g) * 0.02,
                  torch.randn(d, H, generator=g) * 0.02)
    shared = moe.FP8SwiGLU(s1.cuda(), s2.cuda(), s3.cuda(), round_scale=rs)
    got = shared(x.cuda())
    h12_ref, _ = O.fp8_linear_forward(x, torch.cat([s1, s2]), rs)
    h_ref = _oracle_swiglu(h12_ref.to(torch.bfloat16))
    sh_ref, _ = O.fp8_linear_forward(h_ref, s3, False)
    err = rel_fro(got.float(), sh_ref)
    print(f"shared expert: rel-Fro {err:.3e}")
    assert got.dtype == torch.bfloat16 and err < 5e-3
    layer = moe.ExpertParallelMoE(router.cuda(), bias.cuda(), w12.cuda(), w3.cuda(), k, shared=shared)
    y = layer(x.cuda())
    r = moe.route(x.cuda(), router.cuda(), bias.cuda(), k)
    routed = moe.moe_forward(x.cuda(), r, layer.experts, K.quantize_fp8_rowwise)
    assert torch.equal(y, got.float() + routed)                       # one pass, same sums
    assert K.device_status() == 0


EP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from cinnamon_b200 import kernels as K, moe
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
E, d, I, T, k = 16, 512, 256, 256, 2
g = torch.Generator().manual_seed(33)
router = (torch.randn(E, d, generator=g) * 0.02).cuda()
bias = (torch.randn(E, generator=g) * 0.3).cuda()
w12 = (torch.randn(E, 2 * I, d, generator=g) * 0.02).bfloat16().cuda()
w3 = (torch.randn(E, d, I, generator=g) * 0.02).bfloat16().cuda()
x = torch.randn(T, d, generator=torch.Generator().manual_seed(50 + rank)).bfloat16().cuda()
r = moe.route(x, router, bias, k)
lo, hi = rank * E // world, (rank + 1) * E // world
y_ep = moe.moe_forward(x, r, moe.FP8Experts(w12[lo:hi], w3[lo:hi]), K.quantize_fp8_rowwise)
# the whole layer: the shared expert runs on a second stream under the exchange
s1, s2, s3 = [(torch.randn(*shape, generator=g) * 0.02).cuda() for shape in ((384, d), (384, d), (d, 384))]
layer = moe.ExpertParallelMoE(router, bias, w12[lo:hi], w3[lo:hi], k, shared=moe.FP8SwiGLU(s1, s2, s3))
y_layer = [layer(x) for _ in range(3)][-1]
# and with the tokens in two chunks whose exchanges run under the other chunk's experts
layer2 = moe.ExpertParallelMoE(router, bias, w12[lo:hi], w3[lo:hi], k, shared=moe.FP8SwiGLU(s1, s2, s3), n_chunks=2)
y_chunked = [layer2(x) for _ in range(3)][-1]
# and with the exchange done by peer stores into symmetric memory (three calls: the buffers are reused)
layer3 = moe.ExpertParallelMoE(router, bias, w12[lo:hi], w3[lo:hi], k, shared=moe.FP8SwiGLU(s1, s2, s3), exchange="p2p")
y_p2p = [layer3(x) for _ in range(3)][-1]
# ... and with the way home written by the down-projection's epilogue
layer4 = moe.ExpertParallelMoE(router, bias, w12[lo:hi], w3[lo:hi], k, shared=moe.FP8SwiGLU(s1, s2, s3), exchange="p2p-fused")
y_fused = [layer4(x) for _ in range(3)][-1]
# ... and with the local experts dispatched and up-projected in two and in four ranges
layer5 = moe.ExpertParallelMoE(router, bias, w12[lo:hi], w3[lo:hi], k, shared=moe.FP8SwiGLU(s1, s2, s3), exchange="p2p-fused", up_splits=2)
y_split2 = [layer5(x) for _ in range(3)][-1]
layer6 = moe.ExpertParallelMoE(router, bias, w12[lo:hi], w3[lo:hi], k, shared=moe.FP8SwiGLU(s1, s2, s3), exchange="p2p-fused", up_splits=4)
y_split4 = [layer6(x) for _ in range(3)][-1]
# ... and with the dispatch stores coming from 24 SMs while the shared expert's GEMMs run on the others
layer7 = moe.ExpertParallelMoE(router, bias, w12[lo:hi], w3[lo:hi], k, shared=moe.FP8SwiGLU(s1, s2, s3), exchange="p2p-fused", dispatch_sms=24)
y_narrow = [layer7(x) for _ in range(3)][-1]
torch.cuda.synchronize()
torch.save({"y_ep": y_ep.cpu(), "y_layer": y_layer.cpu(), "y_chunked": y_chunked.cpu(), "y_p2p": y_p2p.cpu(), "y_fused": y_fused.cpu(), "x": x.cpu(),
            "y_split2": y_split2.cpu(), "y_split4": y_split4.cpu(), "y_narrow": y_narrow.cpu(),
            "status": K.device_status()},
           os.path.join(sys.argv[2], f"ep_{rank}.pt"))
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_matches_one_gpu(K, tmp_path, world):
    """Every exchange (all-to-all, chunked, peer stores, peer stores from the GEMM epilogue) on 2, 4 or 8 GPUs, one
    process each, against the one-GPU layer on the same tokens: bit-identical outputs."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this machine shows {torch.cuda.device_count()}")
    from cinnamon_b200 import moe
    script = tmp_path / "ep_worker.py"
    script.write_text(EP_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", CINN_DIV_MODE="rn")
    subprocess.check_call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT, str(tmp_path)],
                          env=env, timeout=300)
    E, d, I, T, k = 16, 512, 256, 256, 2
    g = torch.Generator().manual_seed(33)
    router = (torch.randn(E, d, generator=g) * 0.02).cuda()
    bias = (torch.randn(E, generator=g) * 0.3).cuda()
    w12 = (torch.randn(E, 2 * I, d, generator=g) * 0.02).bfloat16().cuda()
    w3 = (torch.randn(E, d, I, generator=g) * 0.02).bfloat16().cuda()
    experts = moe.FP8Experts(w12, w3)
    s1, s2, s3 = [(torch.randn(*shape, generator=g) * 0.02).cuda() for shape in ((384, d), (384, d), (d, 384))]
    shared = moe.FP8SwiGLU(s1, s2, s3)
    for rank in range(world):
        got = torch.load(tmp_path / f"ep_{rank}.pt")
        assert got["status"] == 0
        x = got["x"].cuda()
        r = moe.route(x, router, bias, k)
        y_one = moe.moe_forward(x, r, experts, K.quantize_fp8_rowwise)
        assert rel_fro(got["y_layer"], (shared(x).float() + y_one).cpu().double()) < 1e-6
        assert rel_fro(got["y_chunked"], (shared(x).float() + y_one).cpu().double()) < 1e-6
        assert torch.equal(got["y_p2p"], got["y_layer"])                  # same rows in the same order: same bits
        assert torch.equal(got["y_fused"], got["y_layer"])
        assert torch.equal(got["y_split2"], got["y_layer"]) and torch.equal(got["y_split4"], got["y_layer"])
        assert torch.equal(got["y_narrow"], got["y_layer"])
        # same e4m3 payloads and the same per-row arithmetic: only the fp32 summation order of a token's
        # experts could differ, and index_add_ keeps it
        assert rel_fro(got["y_ep"], y_one.cpu().double()) < 1e-6


def _fake_peers(t, n):
    return torch.tensor([t.data_ptr()] * n, dtype=torch.int64, device="cuda")


@pytest.mark.parametrize("G,me", [(1, 0), (2, 0), (2, 1), (4, 2), (8, 7)])
def test_plan_kernel_matches_exchange_tables(K, G, me):
    """cinn_p2p_plan for rank `me` of G, with the other ranks played by the host: their rows of the count matrix
    and their flags are filled in beforehand, all "peer" pointers name local memory.  The tables must equal the
    tensor-arithmetic statement (p2p.exchange_tables, itself checked against a sort-based exchange on the CPU)."""
    import ctypes
    from cinnamon_b200 import p2p
    E = 32
    g = torch.Generator().manual_seed(100 * G + me)
    counts_all = torch.randint(0, 50, (G, E), generator=g, dtype=torch.int64)
    counts_all[:, 3] = 0                                              # an expert nobody uses
    counts_all[me, 5] = 0
    ref = p2p.exchange_tables(counts_all, me)
    matrix = counts_all.clone().cuda()
    matrix[me] = -1                                                   # the kernel must write this row itself
    flags = torch.zeros(256, dtype=torch.int32, device="cuda")
    flags[64:64 + G] = 7                                              # every rank's counts "have arrived" (epoch 7)
    flags[64 + me] = 0
    e_local = E // G
    i64 = lambda n: torch.full((n,), -5, dtype=torch.int64, device="cuda")          # noqa: E731
    out = dict(base_send=i64(E), my_start=i64(E), starts=i64(e_local), ends=i64(e_local), seg_start=i64(e_local * G + 1),
               home_base=i64(e_local * G), total_rows=i64(1))
    p = lambda t: ctypes.c_void_p(t.data_ptr())                                       # noqa: E731
    mine = counts_all[me].contiguous().cuda()
    peer_matrix, peer_flags = _fake_peers(matrix, G), _fake_peers(flags, G)           # kept alive across the launch
    K._lib.check(K._lib.lib.cinn_p2p_plan(p(mine), p(peer_matrix), p(peer_flags), me, G, E, 64, 7,
                                          p(out["base_send"]), p(out["my_start"]), p(out["starts"]), p(out["ends"]),
                                          p(out["seg_start"]), p(out["home_base"]), p(out["total_rows"]),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "cinn_p2p_plan")
    torch.cuda.synchronize()
    assert K.device_status() == 0
    assert torch.equal(matrix.cpu(), counts_all) and int(flags[64 + me]) == 7
    for name, got in out.items():
        want = getattr(ref, name).reshape(-1)
        assert torch.equal(got.cpu(), want), name


def test_dispatch_signal_and_row_table_wait(K):
    """One rank: the dispatch's last CTA sets the "landed" flag, the row-table kernel waits for it; rows and table
    equal those of the plain kernels."""
    import ctypes
    T, d, E, k = 96, 256, 4, 2
    g = torch.Generator().manual_seed(8)
    xq, xs = K.quantize_fp8_rowwise(torch.randn(T, d, generator=g).bfloat16().cuda())
    r = K.moe_route(torch.randn(T, E, generator=g).cuda(), torch.zeros(E).cuda(), k)
    from cinnamon_b200 import p2p
    t = p2p.exchange_tables(r["counts"].view(1, E).cpu(), 0)
    t = p2p.ExchangeTables(**{f: getattr(t, f).cuda().reshape(-1) for f in t.__dataclass_fields__})
    n = T * k
    recv = [torch.zeros(n, d, dtype=torch.uint8, device="cuda") for _ in range(2)]
    recs = [torch.zeros(n, d // 128, device="cuda") for _ in range(2)]
    flags = torch.zeros(256, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = lambda x: ctypes.c_void_p(x.data_ptr())                                       # noqa: E731
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    home = torch.zeros(n, d, dtype=torch.bfloat16, device="cuda")
    table = torch.zeros(n, dtype=torch.int64, device="cuda")
    # the pointer arrays stay referenced until the launches that read them have run
    pq = [_fake_peers(recv[i], 1) for i in range(2)]
    ps = [_fake_peers(recs[i], 1) for i in range(2)]
    pf, ph = _fake_peers(flags, 1), _fake_peers(home, 1)
    K.p2p_dispatch(xq, xs, r["token_indices"], r["sorted_experts"], t.base_send, t.my_start, pq[0], ps[0], E, 1, n)
    K._lib.check(K._lib.lib.cinn_p2p_dispatch_signal(p(xq), p(xs), p(r["token_indices"]), p(r["sorted_experts"]), p(t.base_send),
                                                     p(t.my_start), p(pq[1]), p(ps[1]), n, T, d, d // 128, E, 1, n, p(pf), 0, 128,
                                                     3, p(done), 0, E, 0, st), "cinn_p2p_dispatch_signal")
    K._lib.check(K._lib.lib.cinn_p2p_row_table_wait(p(t.seg_start), p(t.home_base), p(ph), n, d * 2, E, 1, n, p(table), p(pf), 0,
                                                    128, 3, st), "cinn_p2p_row_table_wait")
    torch.cuda.synchronize()
    assert K.device_status() == 0 and int(flags[128]) == 3 and int(done) == 0
    assert torch.equal(recv[0], recv[1]) and torch.equal(recs[0], recs[1])
    assert torch.equal(table, K.p2p_row_table(t.seg_start, t.home_base, ph, n, d * 2, 1, n))


def test_dispatch_signal_by_expert_ranges(K):
    """The signalling dispatch called once per range of local experts (two destination ranks, stood in for by two
    local buffers; this rank is rank 1, so rank 0 is served first): together the calls write exactly the rows the
    plain dispatch writes, each sets its own flag slot, and a range outside the local experts is refused."""
    import ctypes
    from cinnamon_b200 import p2p
    T, d, E, k, G, me = 160, 256, 8, 2, 2, 1
    e_local = E // G
    g = torch.Generator().manual_seed(9)
    xq, xs = K.quantize_fp8_rowwise(torch.randn(T, d, generator=g).bfloat16().cuda())
    r = K.moe_route(torch.randn(T, E, generator=g).cuda(), torch.zeros(E).cuda(), k)
    counts_all = torch.zeros(G, E, dtype=torch.int64)
    counts_all[me] = r["counts"].cpu()
    t = p2p.exchange_tables(counts_all, me)
    t = p2p.ExchangeTables(**{f: getattr(t, f).cuda().reshape(-1) for f in t.__dataclass_fields__})
    n = T * k
    bufs = [[torch.zeros(n, d, dtype=torch.uint8, device="cuda") for _ in range(G)] for _ in range(2)]
    scs = [[torch.zeros(n, d // 128, device="cuda") for _ in range(G)] for _ in range(2)]
    flags = torch.zeros(256, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    ptrs = lambda ts: torch.tensor([x.data_ptr() for x in ts], dtype=torch.int64, device="cuda")   # noqa: E731
    pq, ps = [ptrs(bufs[i]) for i in range(2)], [ptrs(scs[i]) for i in range(2)]
    pf = ptrs([flags] * G)
    p = lambda x: ctypes.c_void_p(x.data_ptr())                                       # noqa: E731
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    K.p2p_dispatch(xq, xs, r["token_indices"], r["sorted_experts"], t.base_send, t.my_start, pq[0], ps[0], e_local, G, n)
    call = lambda lo, hi, slot: K._lib.lib.cinn_p2p_dispatch_signal(                               # noqa: E731
        p(xq), p(xs), p(r["token_indices"]), p(r["sorted_experts"]), p(t.base_send), p(t.my_start), p(pq[1]), p(ps[1]), n, T, d,
        d // 128, e_local, G, n, p(pf), me, slot, 5, p(done), lo, hi, sms, st)
    sms = 0
    K._lib.check(call(0, 1, 128), "range 0")
    torch.cuda.synchronize()
    assert int(flags[128 + me]) == 5 and int(flags[144 + me]) == 0
    covered = sum(int(r["counts"][rk * e_local]) for rk in range(G))
    written = sum(int((b != 0).any(dim=1).sum()) for b in bufs[1])
    assert 0 < written <= covered                                    # only the first local expert of every rank so far
    sms = 3                                                          # the second range from three SMs only
    K._lib.check(call(1, e_local, 144), "range 1")
    torch.cuda.synchronize()
    assert K.device_status() == 0 and int(flags[144 + me]) == 5 and int(done) == 0
    for i in range(G):
        assert torch.equal(bufs[0][i], bufs[1][i]) and torch.equal(scs[0][i], scs[1][i])
    assert call(2, 2, 160) != 0 and call(0, e_local + 1, 160) != 0   # empty / out-of-range expert ranges are refused
