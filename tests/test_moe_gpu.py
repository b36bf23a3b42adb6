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
torch.save({"y_ep": y_ep.cpu(), "x": x.cpu(), "status": K.device_status()}, os.path.join(sys.argv[2], f"ep_{rank}.pt"))
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_two_gpus_match_one(K, tmp_path):
    from cinnamon_b200 import moe
    script = tmp_path / "ep_worker.py"
    script.write_text(EP_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", CINN_DIV_MODE="rn")
    subprocess.check_call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT, str(tmp_path)],
                          env=env, timeout=300)
    E, d, I, T, k = 16, 512, 256, 256, 2
    g = torch.Generator().manual_seed(33)
    router = (torch.randn(E, d, generator=g) * 0.02).cuda()
    bias = (torch.randn(E, generator=g) * 0.3).cuda()
    w12 = (torch.randn(E, 2 * I, d, generator=g) * 0.02).bfloat16().cuda()
    w3 = (torch.randn(E, d, I, generator=g) * 0.02).bfloat16().cuda()
    experts = moe.FP8Experts(w12, w3)
    for rank in range(2):
        got = torch.load(tmp_path / f"ep_{rank}.pt")
        assert got["status"] == 0
        x = got["x"].cuda()
        r = moe.route(x, router, bias, k)
        y_one = moe.moe_forward(x, r, experts, K.quantize_fp8_rowwise)
        # same e4m3 payloads and the same per-row arithmetic: only the fp32 summation order of a token's
        # experts could differ, and index_add_ keeps it
        assert rel_fro(got["y_ep"], y_one.cpu().double()) < 1e-6
