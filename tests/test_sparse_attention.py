"""Sparse attention: the float64 oracle against the reference's own outputs (golden vectors made by running its
Triton kernels in the CPU interpreter), and the CUDA kernels against both."""
import os

import numpy as np
import pytest
import torch

from oracle import sparse_attention_oracle as SO

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = ["small", "ragged_dims", "causal_topk", "duplicates"]


@pytest.fixture(scope="module")
def vectors():
    return np.load(os.path.join(HERE, "golden", "sparse_attention_vectors.npz"))


def _case(vectors, name):
    t = {k: torch.from_numpy(vectors[f"{name}/{k}"]) for k in
         ("q", "k", "v", "idx", "out", "attn", "grad_out", "dq", "dk", "dv")}
    t["scale"] = float(vectors[f"{name}/scale"])
    return t


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_vectors(vectors, name):
    c = _case(vectors, name)
    out, attn, _ = SO.forward(c["q"], c["k"], c["v"], c["idx"], c["scale"])
    torch.testing.assert_close(out.float(), c["out"], rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(attn.float(), c["attn"], rtol=2e-5, atol=2e-7)
    dq, dk, dv = SO.backward(c["q"], c["k"], c["v"], c["idx"], c["scale"], c["grad_out"])
    torch.testing.assert_close(dq.float(), c["dq"], rtol=5e-5, atol=5e-6)
    torch.testing.assert_close(dk.float(), c["dk"], rtol=5e-5, atol=5e-6)
    torch.testing.assert_close(dv.float(), c["dv"], rtol=5e-5, atol=5e-6)


def test_oracle_backward_is_the_derivative():
    """The analytic backward against autograd through the float64 forward."""
    g = torch.Generator().manual_seed(9)
    q, k = (torch.randn(1, 2, 12, 8, generator=g, dtype=torch.float64).requires_grad_(True) for _ in range(2))
    v = torch.randn(1, 2, 12, 4, generator=g, dtype=torch.float64).requires_grad_(True)
    idx = torch.randint(0, 12, (1, 12, 5), generator=g)
    go = torch.randn(1, 2, 12, 4, generator=g, dtype=torch.float64)
    out, _, _ = SO.forward(q, k, v, idx, 0.3)
    ref = torch.autograd.grad(out, (q, k, v), go)
    got = SO.backward(q.detach(), k.detach(), v.detach(), idx, 0.3, go)
    for a, b in zip(got, ref):
        torch.testing.assert_close(a, b, rtol=1e-10, atol=1e-12)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_kernels_match_reference_vectors(vectors, name):
    from cinnamon_b200 import kernels as K
    c = _case(vectors, name)
    q, k, v = (c[n].cuda().requires_grad_(True) for n in ("q", "k", "v"))
    out, attn = K.sparse_attention(q, k, v, c["idx"].cuda(), c["scale"])
    assert out.dtype == torch.float32 and attn.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), c["out"], rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(attn.cpu(), c["attn"], rtol=2e-5, atol=2e-7)
    out.backward(c["grad_out"].cuda())
    torch.testing.assert_close(q.grad.cpu(), c["dq"], rtol=5e-5, atol=5e-6)
    torch.testing.assert_close(k.grad.cpu(), c["dk"], rtol=5e-5, atol=5e-6)
    torch.testing.assert_close(v.grad.cpu(), c["dv"], rtol=5e-5, atol=5e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(2, 4, 96, 32, 192, 64), (1, 3, 70, 128, 64, 64), (1, 2, 33, 7, 20, 6), (1, 1, 300, 40, 8, 136)])
def test_kernels_match_oracle(dtype, shape):
    """Model-like sizes (192-wide PoPE queries, 64-wide values), K larger than the sequence, odd sizes that take the
    scalar path; fp32 results against the float64 oracle on the same (already rounded) inputs."""
    from cinnamon_b200 import kernels as K
    B, H, L, Ks, Dqk, Dv = shape
    g = torch.Generator().manual_seed(sum(shape))
    q, k = (torch.randn(B, H, L, Dqk, generator=g).to(dtype) for _ in range(2))
    v = torch.randn(B, H, L, Dv, generator=g).to(dtype)
    idx = torch.randint(0, L, (B, L, Ks), generator=g)
    idx[:, :, 0] = torch.arange(L)                       # every query sees at least itself ...
    idx[0, 5, :] = L - 1                                 # ... except this one, which has no valid key at all
    go = torch.randn(B, H, L, Dv, generator=g).to(dtype)
    scale = Dqk ** -0.5
    ref_out, ref_attn, _ = SO.forward(q, k, v, idx, scale)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out, attn = K.sparse_attention(qc, kc, vc, idx.cuda(), scale)
    assert out.dtype == dtype and attn.shape == (B, H, L, Ks)
    tol = {torch.float32: 1e-5, torch.bfloat16: 8e-3, torch.float16: 1e-3}[dtype]       # rounding of the returned output
    torch.testing.assert_close(out.float().cpu().double(), ref_out, rtol=tol, atol=tol)
    torch.testing.assert_close(attn.cpu().double(), ref_attn, rtol=2e-5, atol=1e-7)
    assert torch.all(out[0, :, 5] == 0) and torch.all(attn[0, :, 5] == 0)
    out.backward(go.cuda())
    # the kernel differentiates with the fp32 output it saved; the oracle with its own float64 output
    ref = SO.backward(q, k, v, idx, scale, go)
    for name, got, want in zip(("dq", "dk", "dv"), (qc.grad, kc.grad, vc.grad), ref):
        assert got.dtype == dtype
        err = (got.float().cpu().double() - want).norm() / want.norm()
        assert err < {torch.float32: 2e-6, torch.bfloat16: 4e-3, torch.float16: 5e-4}[dtype], (name, float(err))


@pytest.mark.gpu
def test_edge_shapes():
    """No indices at all, indices outside the sequence, one query, a list much longer than the sequence."""
    from cinnamon_b200 import kernels as K
    g = torch.Generator().manual_seed(77)
    q, k, v = (torch.randn(1, 2, 9, 16, generator=g).cuda() for _ in range(3))
    out, attn = K.sparse_attention(q, k, v, torch.zeros(1, 9, 0, dtype=torch.int64, device="cuda"))
    assert attn.shape == (1, 2, 9, 0) and torch.all(out == 0)
    idx = torch.randint(-3, 14, (1, 9, 40), generator=g)                     # some below 0, some beyond L - 1
    ref_out, ref_attn, _ = SO.forward(q.cpu(), k.cpu(), v.cpu(), idx, 0.25)
    out, attn = K.sparse_attention(q, k, v, idx.cuda(), 0.25)
    torch.testing.assert_close(out.cpu().double(), ref_out, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(attn.cpu().double(), ref_attn, rtol=2e-5, atol=1e-7)
    q1, k1, v1 = (t[:, :, :1].contiguous() for t in (q, k, v))
    out, attn = K.sparse_attention(q1, k1, v1, torch.zeros(1, 1, 3, dtype=torch.int64, device="cuda"))
    torch.testing.assert_close(out, v1.expand_as(out))                       # the only key, listed three times
    torch.testing.assert_close(attn, torch.full_like(attn, 1.0 / 3.0))


@pytest.mark.gpu
def test_argument_checks():
    from cinnamon_b200 import kernels as K
    q = torch.randn(1, 1, 4, 8)
    with pytest.raises(AssertionError):
        K.sparse_attention(q, q, q, torch.zeros(1, 4, 2, dtype=torch.int64))


@pytest.mark.gpu
def test_backward_with_gradient_buffers_at_odd_addresses():
    """A C caller may hand in gradient buffers that start on a 4-byte boundary only (a slice of an arena): the
    kernel then must not use its 16- or 8-byte atomics.  Same result as with aligned buffers."""
    import ctypes
    from cinnamon_b200 import kernels as K
    lib = K._lib.lib
    g = torch.Generator().manual_seed(31)
    B, H, L, Kk, dqk, dv = 1, 2, 24, 6, 16, 8
    q, k = (torch.randn(B, H, L, dqk, generator=g).cuda() for _ in range(2))
    v = torch.randn(B, H, L, dv, generator=g).cuda()
    idx = (torch.rand(B, L, Kk, generator=g) * (torch.arange(L).view(1, L, 1) + 1)).long().cuda()
    go = torch.randn(B, H, L, dv, generator=g).cuda()
    out = torch.empty(B, H, L, dv, device="cuda")
    lse = torch.empty(B, H, L, device="cuda")
    attn = torch.empty(B, H, L, Kk, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())                                        # noqa: E731
    K._lib.check(lib.cinn_sparse_attn_fwd(p(q), p(k), p(v), 1, p(idx), p(out), p(lse), p(attn), B, H, L, Kk, dqk, dv, 0.25, st), "fwd")
    grads = []
    for shift in (0, 1):                                                                # 0: 16-byte aligned, 1: +4 bytes
        arena = torch.zeros(3 * B * H * L * dqk + 8, device="cuda")
        n_qk, n_v = B * H * L * dqk, B * H * L * dv
        gq, gk, gv = arena[shift:shift + n_qk], arena[shift + n_qk:shift + 2 * n_qk], arena[shift + 2 * n_qk:shift + 2 * n_qk + n_v]
        assert (gq.data_ptr() % 16 == 0) == (shift == 0)
        K._lib.check(lib.cinn_sparse_attn_bwd(p(go), 1, p(out), p(lse), p(q), p(k), p(v), 1, p(idx), p(gq), p(gk), p(gv), B, H, L,
                                              Kk, dqk, dv, 0.25, st), "bwd")
        torch.cuda.synchronize()
        grads.append([t.clone() for t in (gq, gk, gv)])
    for a, b in zip(*grads):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    assert K.device_status() == 0
