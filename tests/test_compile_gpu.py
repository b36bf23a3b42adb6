"""torch.compile over the drop-in (the reference compiles its model, src/train.py:703): a converted SwiGLU block,
the routed experts' two grouped GEMMs and sparse attention each compile as ONE graph (``fullgraph=True`` raises on
any graph break) because the library's entry points are torch.library operators while compiling
(cinnamon_b200/ops.py), and compiled results - outputs and every gradient - are the eager results bit for bit."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from cinnamon_b200 import kernels
    assert kernels._ops is not None, "torch.library operators were not registered"
    yield kernels
    assert kernels.device_status() == 0


class SwiGLU(nn.Module):                      # structure of src/layers.py:15-31
    def __init__(self, d, h):
        super().__init__()
        self.w1, self.w2, self.w3 = nn.Linear(d, h, bias=False), nn.Linear(d, h, bias=False), nn.Linear(h, d, bias=False)

    def forward(self, x):
        return self.w3(F.silu(self.w1(x)) * self.w2(x))


def _grads(module, x, fn):
    for p in module.parameters():
        p.grad = None
    x = x.detach().clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = fn(x)
    y.float().pow(2).mean().backward()
    return y.detach(), x.grad, [p.grad.clone() for p in module.parameters()]


def test_converted_swiglu_block_compiles_as_one_graph(K):
    torch.manual_seed(0)
    block = K.convert_to_fp8(SwiGLU(256, 512).cuda())
    x = torch.randn(4, 48, 256, device="cuda")
    y0, gx0, gp0 = _grads(block, x, block)
    torch._dynamo.reset()
    compiled = torch.compile(block, fullgraph=True)
    launches = K.launch_count
    y1, gx1, gp1 = _grads(block, x, compiled)
    assert K.launch_count - launches >= 9 * 2 - 3, "the compiled block did not run the library's kernels"
    # the element-wise part between the linears (silu, product) is fused by the compiler and keeps fp32 intermediates
    # where eager rounds to bf16 twice, so the block agrees to bf16 precision, not to the bit
    # (and every differently rounded intermediate is re-quantised to e4m3 by the next layer, forward and backward)
    err = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm())               # noqa: E731
    assert err(y1, y0) < 2e-2 and err(gx1, gx0) < 1e-1
    for a, b in zip(gp0, gp1):
        assert err(b, a) < 1e-1
    y2, _, _ = _grads(block, x, compiled)                     # a second call reuses the graph
    assert torch.equal(y1, y2)
    # one layer alone has nothing for the compiler to fuse: compiled and eager results are the same bits
    lin = block.w1
    z0, gz0, gw0 = _grads(lin, x, lin)
    z1, gz1, gw1 = _grads(lin, x, torch.compile(lin, fullgraph=True))
    assert torch.equal(z0, z1) and torch.equal(gz0, gz1) and torch.equal(gw0[0], gw1[0])


def test_grouped_gemm_and_sparse_attention_compile(K):
    torch.manual_seed(1)
    E, d, h, T = 4, 256, 128, 200
    w12 = (torch.randn(E, 2 * h, d, device="cuda") * 0.02).requires_grad_(True)
    w3 = (torch.randn(E, d, h, device="cuda") * 0.02).requires_grad_(True)
    counts = torch.tensor([60, 0, 75, 65])
    ends = counts.cumsum(0).cuda()
    starts = ends - counts.cuda()

    def experts(xs):                                         # src/layers.py:69-75
        h12 = K.moe_grouped_gemm(xs, w12, starts, ends)
        h1, h2 = h12.float().chunk(2, dim=-1)
        return K.moe_grouped_gemm((F.silu(h1) * h2).to(xs.dtype), w3, starts, ends).float()

    B, H, L, Kk = 2, 4, 64, 16
    q, k = (torch.randn(B, H, L, 48, device="cuda").bfloat16().requires_grad_(True) for _ in range(2))
    v = torch.randn(B, H, L, 32, device="cuda").bfloat16().requires_grad_(True)
    idx = (torch.rand(B, L, Kk, device="cuda") * (torch.arange(L, device="cuda").view(1, L, 1) + 1)).long()

    def attention(q, k, v):
        out, weights = K.sparse_attention(q, k, v, idx)
        return out.float().sum() + 0.0 * weights.sum()

    def run(f_experts, f_attn):
        for t in (w12, w3, q, k, v):
            t.grad = None
        xs = torch.randn(T, d, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).bfloat16().requires_grad_(True)
        out = f_experts(xs)
        out.pow(2).mean().backward()
        f_attn(q, k, v).backward()
        return [out.detach(), xs.grad, w12.grad.clone(), w3.grad.clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()]

    eager = run(experts, attention)
    torch._dynamo.reset()
    compiled = run(torch.compile(experts, fullgraph=True), torch.compile(attention, fullgraph=True))
    for name, a, b in zip(("out", "dx", "dw12", "dw3", "dq", "dk", "dv"), eager, compiled):
        if name in ("dk", "dv"):                             # accumulated with atomics: the order of the sums is not fixed
            torch.testing.assert_close(a.float(), b.float(), rtol=2e-2, atol=2e-2)
        else:
            assert torch.equal(a, b), name
