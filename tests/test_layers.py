"""The drop-in MoE block (cinnamon_b200/layers.py) on the CPU: against vectors recorded from the reference's own
``MoE`` (tests/golden/make_golden_moe.py: output, balance loss, bias update and every gradient), and - two gloo
ranks - the expert-sharded layer against the unsharded one, forward and backward (the exchange run in reverse)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASES = {
    "small": (8, 1, 2, 64, 128, 4, 0.001, 0.01),
    "two_shared_top3": (6, 2, 3, 32, 64, 2, 0.01, 0.05),
}


@pytest.mark.parametrize("name", list(CASES))
def test_moe_block_matches_reference_vectors(name):
    from cinnamon_b200 import layers
    g = np.load(os.path.join(ROOT, "tests", "golden", "moe_vectors.npz"))
    m = layers.MoE(*CASES[name])
    state = {k[len(name) + 7:]: torch.from_numpy(g[k]) for k in g.files if k.startswith(f"{name}/param/")}
    state["expert_bias"] = torch.from_numpy(g[f"{name}/bias_before"])
    m.load_state_dict(state)                                  # same names as the reference's block
    m.train()
    x = torch.from_numpy(g[f"{name}/x"]).requires_grad_(True)
    y, bl = m(x)
    (y.pow(2).mean() + bl).backward()
    torch.testing.assert_close(y, torch.from_numpy(g[f"{name}/y"]), rtol=1e-5, atol=1e-6)
    assert abs(float(bl) - float(g[f"{name}/balance_loss"])) < 1e-7
    assert torch.equal(m.expert_bias, torch.from_numpy(g[f"{name}/bias_after"]))
    torch.testing.assert_close(x.grad, torch.from_numpy(g[f"{name}/grad_x"]), rtol=1e-4, atol=1e-8)
    for pname, p in m.named_parameters():
        torch.testing.assert_close(p.grad, torch.from_numpy(g[f"{name}/grad/{pname}"]), rtol=1e-4, atol=1e-8, msg=pname)
    m.eval()
    bias = m.expert_bias.clone()
    m(x.detach())
    assert torch.equal(m.expert_bias, bias)                   # no bias update outside training


EP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from cinnamon_b200 import layers
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
E, k, d, h = 8, 2, 32, 64
torch.manual_seed(3)
full = layers.MoE(E, 1, k, d, h, 2, 0.01, 0.02)                     # identical on both ranks
with torch.no_grad():
    full.expert_bias.copy_(torch.linspace(-0.3, 0.3, E))
sharded = layers.MoE(E, 1, k, d, h, 2, 0.01, 0.02, group=dist.group.WORLD)
el = E // world
with torch.no_grad():
    sharded.router.weight.copy_(full.router.weight)
    sharded.expert_bias.copy_(full.expert_bias)
    sharded.shared_experts.load_state_dict(full.shared_experts.state_dict())
    sharded.routed_experts.w12.copy_(full.routed_experts.w12[rank * el:(rank + 1) * el])
    sharded.routed_experts.w3.copy_(full.routed_experts.w3[rank * el:(rank + 1) * el])
xs = [torch.randn(2, 5 + 3 * r, d, generator=torch.Generator().manual_seed(40 + r)) for r in range(world)]   # ragged: ranks differ
# the unsharded layer sees all tokens of all ranks as one batch of sequences; pad-free: run it per rank's tokens
res = {}
full.train(); sharded.train()
full.gamma = 0.0        # `full` is called once per rank's tokens: its bias must not move between the calls
x_full = [t.clone().requires_grad_(True) for t in xs]
outs = [full(t) for t in x_full]
# the bias update of `full` ran once per call; undo and apply the update for the global counts instead (what the
# sharded layer does): only outputs and gradients are compared, plus the sharded layer's bias against a manual update
loss_full = sum(o.pow(2).sum() + b for o, b in outs)
loss_full.backward()
x = xs[rank].clone().requires_grad_(True)
bias0 = sharded.expert_bias.clone()
y, bl = sharded(x)
(y.pow(2).sum() + bl).backward()
ok = torch.allclose(y, outs[rank][0].detach(), rtol=1e-5, atol=1e-6)
ok &= torch.allclose(x.grad, x_full[rank].grad, rtol=1e-4, atol=1e-7)
# router and shared experts: this rank's loss only covers its own tokens, so sum the gradients over the ranks
for a, b in ((sharded.router.weight, full.router.weight), (sharded.shared_experts[0].w1.weight, full.shared_experts[0].w1.weight)):
    ga = a.grad.clone(); dist.all_reduce(ga)
    ok &= torch.allclose(ga, b.grad, rtol=1e-4, atol=1e-7)
# the experts of this rank receive rows (and gradients) from both ranks: no reduction needed.  With this bias the
# experts of rank 0 receive no row at all: they get no gradient, and rank 0 must still take part in both reverse exchanges
g_or_zero = lambda p: p.grad if p.grad is not None else torch.zeros_like(p)
ok &= torch.allclose(g_or_zero(sharded.routed_experts.w12), full.routed_experts.w12.grad[rank * el:(rank + 1) * el], rtol=1e-4, atol=1e-7)
ok &= torch.allclose(g_or_zero(sharded.routed_experts.w3), full.routed_experts.w3.grad[rank * el:(rank + 1) * el], rtol=1e-4, atol=1e-7)
# bias update from the counts of all ranks
moved = (sharded.expert_bias - bias0).abs()
ok &= bool(torch.allclose(moved, torch.full_like(moved, 0.01)))
with open(os.path.join(sys.argv[2], f"ok_{rank}"), "w") as f:
    f.write("1" if ok else "0")
dist.destroy_process_group()
'''


def test_sharded_moe_block_trains_like_the_unsharded_one(tmp_path):
    script = tmp_path / "ep_train.py"
    script.write_text(EP_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    subprocess.check_call([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT, str(tmp_path)],
                          timeout=300, env=dict(os.environ, OMP_NUM_THREADS="2"))
    for rank in range(2):
        assert (tmp_path / f"ok_{rank}").read_text() == "1", f"rank {rank}: sharded and unsharded layers disagree"
