"""The drop-in MoE block on the GPU: the combine pass's backward against autograd, the block against its own torch
path on the CPU (same weights; e4m3 noise only), and the expert-sharded block on 2 GPUs against the unsharded one
(forward, gradients, bias update)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def K():
    from cinnamon_b200 import kernels
    yield kernels
    assert kernels.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_combine_backward_matches_autograd(K, dtype):
    g = torch.Generator().manual_seed(4)
    T, k, d = 70, 3, 136
    rows = torch.randn(T * k + 5, d, generator=g).to(dtype).cuda().requires_grad_(True)
    perm = torch.randperm(T * k, generator=g)
    pos = perm.view(T, k).sort(dim=1).values.cuda()
    gates = torch.rand(T, k, generator=g).cuda().requires_grad_(True)
    addend = torch.randn(T, d, generator=g).bfloat16().cuda().requires_grad_(True)
    dy = torch.randn(T, d, generator=g).cuda()
    y = K.moe_combine_autograd(rows, pos, gates, addend)
    y.backward(dy)
    r2, g2, a2 = (t.detach().clone().requires_grad_(True) for t in (rows, gates, addend))
    y2 = (r2.float()[pos] * g2.unsqueeze(-1)).sum(1) + a2.float()
    y2.backward(dy)
    torch.testing.assert_close(y, y2, rtol=1e-5, atol=1e-5)
    tol = dict(rtol=1e-2, atol=1e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(rows.grad.float(), r2.grad.float(), **tol)
    torch.testing.assert_close(gates.grad, g2.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(addend.grad.float(), a2.grad.float(), rtol=1e-2, atol=1e-2)
    assert torch.all(rows.grad[T * k:] == 0)                  # rows no pair names


def test_moe_block_on_gpu_against_its_cpu_path(K):
    from cinnamon_b200 import layers
    torch.manual_seed(7)
    E, k, d, h = 8, 2, 256, 512
    cpu = layers.MoE(E, 1, k, d, h, 2, 0.001, 0.01)
    gpu = layers.MoE(E, 1, k, d, h, 2, 0.001, 0.01)
    gpu.load_state_dict(cpu.state_dict())
    gpu = K.convert_to_fp8(gpu.cuda())
    assert isinstance(gpu.shared_experts[0].w1, K.FP8Linear)
    x = torch.randn(3, 40, d)
    xc, xg = x.clone().requires_grad_(True), x.clone().cuda().requires_grad_(True)
    cpu.train(), gpu.train()
    yc, bc = cpu(xc)
    (yc.pow(2).mean() + bc).backward()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        yg, bg = gpu(xg)
    (yg.float().pow(2).mean() + bg).backward()
    torch.cuda.synchronize()
    rel = lambda a, b: float((a.detach().cpu().float() - b).norm() / b.norm())                    # noqa: E731
    assert rel(yg, yc.detach()) < 0.08 and abs(float(bg) - float(bc)) < 2e-3
    assert torch.equal(gpu.expert_bias.cpu(), cpu.expert_bias)
    assert rel(xg.grad, xc.grad) < 0.2
    for (n, pc), (_, pg) in zip(cpu.named_parameters(), gpu.named_parameters()):
        assert pg.grad is not None and torch.isfinite(pg.grad).all(), n
        assert rel(pg.grad, pc.grad) < 0.25, (n, rel(pg.grad, pc.grad))


EP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from cinnamon_b200 import kernels as K, layers
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
E, k, d, h = 8, 2, 256, 512
torch.manual_seed(3)
full = layers.MoE(E, 1, k, d, h, 2, 0.01, 0.02).cuda()
sharded = layers.MoE(E, 1, k, d, h, 2, 0.01, 0.02, group=dist.group.WORLD, exchange=sys.argv[3]).cuda()
el = E // world
with torch.no_grad():
    sharded.router.weight.copy_(full.router.weight)
    sharded.shared_experts.load_state_dict(full.shared_experts.state_dict())
    sharded.routed_experts.w12.copy_(full.routed_experts.w12[rank * el:(rank + 1) * el])
    sharded.routed_experts.w3.copy_(full.routed_experts.w3[rank * el:(rank + 1) * el])
xs = [torch.randn(2, 24 + 8 * r, d, generator=torch.Generator().manual_seed(40 + r)).cuda() for r in range(world)]
full.train(); sharded.train()
full.gamma = 0.0        # `full` is called once per rank's tokens: its bias must not move between the calls
x_full = [t.clone().requires_grad_(True) for t in xs]
outs = [full(t) for t in x_full]
sum(o.pow(2).sum() + b for o, b in outs).backward()
x = xs[rank].clone().requires_grad_(True)
y, bl = sharded(x)
(y.pow(2).sum() + bl).backward()
diffs = []
def close(a, b, tol=1e-3):
    err = float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))
    diffs.append(round(err, 6))
    return err < tol
ok = [torch.equal(y, outs[rank][0].detach()), close(x.grad, x_full[rank].grad)]
for a, b in ((sharded.router.weight, full.router.weight), (sharded.shared_experts[0].w1.weight, full.shared_experts[0].w1.weight)):
    ga = a.grad.clone(); dist.all_reduce(ga)
    ok.append(close(ga, b.grad))
gz = lambda p: p.grad if p.grad is not None else torch.zeros_like(p)
# the experts' weight gradients quantise dY and x in tiles that run along the rows of an expert; sharded, an expert's
# rows are the two ranks' tokens in one list, unsharded they arrive in two calls: same mathematics, different e4m3 tiles
ok.append(close(gz(sharded.routed_experts.w12), full.routed_experts.w12.grad[rank * el:(rank + 1) * el], 0.1))
ok.append(close(gz(sharded.routed_experts.w3), full.routed_experts.w3.grad[rank * el:(rank + 1) * el], 0.1))
# a second step through the same block (the exchange buffers and their flags are reused)
x2 = (xs[rank] * 0.5).clone().requires_grad_(True)
y2, bl2 = sharded(x2)
(y2.pow(2).sum() + bl2).backward()
ok.append(bool(torch.isfinite(y2).all()) and bool(torch.isfinite(x2.grad).all()) and float(x2.grad.abs().sum()) > 0)
torch.cuda.synchronize()
with open(os.path.join(sys.argv[2], f"ok_{rank}"), "w") as f:
    f.write(repr([bool(v) for v in ok]) + f" status {K.device_status()}" + (" " + repr(diffs) if not all(ok) else ""))
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.parametrize("exchange", ["nccl", "p2p"])
def test_sharded_moe_block_trains_like_the_unsharded_one_on_gpus(K, tmp_path, exchange):
    """Outputs and all gradients of the expert-sharded block on 2 GPUs against the unsharded block, with the rows
    exchanged by all-to-all collectives and by peer stores over NVLink (forward and backward)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "ep_train.py"
    script.write_text(EP_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    subprocess.check_call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT, str(tmp_path),
                           exchange],
                          timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    for rank in range(2):
        text = (tmp_path / f"ok_{rank}").read_text()
        assert text == "[True, True, True, True, True, True, True] status 0", f"rank {rank}: {text}"
