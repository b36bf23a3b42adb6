"""The drop-in module used the way cinnamon's model code uses src/kernels.py: convert_to_fp8 on a SwiGLU block
(src/layers.py:15-31), the routed experts calling moe_grouped_gemm twice with torch ops between
(src/layers.py:69-75), one forward + backward; and the reference's own grouped-GEMM test
(tests/test_kernels.py:131-155) on seeded inputs."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from cinnamon_b200 import kernels
    yield kernels
    assert kernels.device_status() == 0


class SwiGLU(nn.Module):                      # structure of src/layers.py:15-31
    def __init__(self, d, h):
        super().__init__()
        self.w1, self.w2, self.w3 = nn.Linear(d, h, bias=False), nn.Linear(d, h, bias=False), nn.Linear(h, d, bias=False)

    def forward(self, x):
        return self.w3(F.silu(self.w1(x)) * self.w2(x))


class Experts(nn.Module):                     # structure of src/layers.py:34-75
    def __init__(self, K, E, d, h):
        super().__init__()
        self.K = K
        self.w12 = nn.Parameter(torch.randn(E, 2 * h, d) * 0.02)
        self.w3 = nn.Parameter(torch.randn(E, d, h) * 0.02)

    def forward(self, sorted_x, starts, ends, use_kernel=True):
        if use_kernel:
            h12 = self.K.moe_grouped_gemm(sorted_x, self.w12, starts, ends)
            h1, h2 = h12.float().chunk(2, dim=-1)
            h = F.silu(h1) * h2
            return self.K.moe_grouped_gemm(h.to(sorted_x.dtype), self.w3, starts, ends).float()
        out = torch.zeros(sorted_x.size(0), self.w3.shape[1], device=sorted_x.device)
        for i in range(self.w12.shape[0]):                         # the reference's fallback loop (:76-87)
            s, e = int(starts[i]), int(ends[i])
            if e > s:
                h1, h2 = F.linear(sorted_x[s:e].float(), self.w12[i]).chunk(2, dim=-1)
                out[s:e] = F.linear(F.silu(h1) * h2, self.w3[i])
        return out


def test_reference_grouped_gemm_test_case(K):
    g = torch.Generator().manual_seed(12)
    E, d, h, T = 8, 512, 128, 256
    w = torch.randn(E, h, d, generator=g).bfloat16().cuda()
    x = torch.randn(T, d, generator=g).bfloat16().cuda()
    starts = torch.arange(0, T, T // E, device="cuda")[:E]
    ends = torch.cat([starts[1:], torch.tensor([T], device="cuda")])
    out = K.moe_grouped_gemm(x, w, starts, ends)
    assert out.shape == (T, h) and out.dtype == torch.float16
    ref = torch.zeros(T, h, device="cuda")
    for i in range(E):
        s, e = int(starts[i]), int(ends[i])
        ref[s:e] = F.linear(x[s:e].float(), w[i].float())
    rel = (ref - out.float()).abs() / (ref.abs() + 1e-6)
    # the reference asserts mean < 0.01 for its fp16 kernel; e4m3 operands carry about 4 % noise per element,
    # so the same statistic is bounded accordingly here
    assert rel.median().item() < 0.05 and (ref - out.float()).norm() / ref.norm() < 0.05


def test_swiglu_block_and_routed_experts_train(K):
    torch.manual_seed(3)
    d, h, E, T = 256, 512, 4, 192
    shared = SwiGLU(d, h).cuda()
    ref_shared = SwiGLU(d, h).cuda()
    ref_shared.load_state_dict(shared.state_dict())
    K.convert_to_fp8(shared)
    assert all(isinstance(m, K.FP8Linear) for m in (shared.w1, shared.w2, shared.w3))
    assert shared.w1.round_scale and shared.w2.round_scale and not shared.w3.round_scale
    experts = Experts(K, E, d, h // 4).cuda()
    x = torch.randn(T, d, device="cuda", requires_grad=True)
    counts = torch.tensor([50, 0, 77, 65])
    ends = counts.cumsum(0).cuda()
    starts = ends - counts.cuda()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = shared(x) + experts(x.bfloat16(), starts, ends)
    y.float().pow(2).mean().backward()
    for name, p in list(shared.named_parameters()) + list(experts.named_parameters()):
        assert p.grad is not None and torch.isfinite(p.grad).all(), name
        assert p.grad.abs().sum() > 0, name
    assert torch.all(experts.w12.grad[1] == 0)                      # the empty expert
    gx = x.grad.clone()
    # unquantised reference of the same block: FP8 noise only
    x2 = x.detach().clone().requires_grad_(True)
    y2 = ref_shared(x2) + experts(x2, starts, ends, use_kernel=False)
    y2.pow(2).mean().backward()
    assert (y.float() - y2).norm() / y2.norm() < 0.1
    assert (gx - x2.grad).norm() / x2.grad.norm() < 0.15
