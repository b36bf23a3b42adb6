"""Lightning indexer: oracle against the reference kernel's outputs (Triton interpreter), CUDA kernel against both."""
import os

import numpy as np
import pytest
import torch

from oracle import sparse_attention_oracle as SO

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = ["model_like", "wide_head", "bf16_inputs", "narrow"]


@pytest.fixture(scope="module")
def vectors():
    return np.load(os.path.join(HERE, "golden", "indexer_vectors.npz"))


def _case(vectors, name):
    dt = torch.bfloat16 if int(vectors[f"{name}/bf16"]) else torch.float32
    q, k, w = (torch.from_numpy(vectors[f"{name}/{n}"]).to(dt) for n in ("q", "k", "w"))
    return q, k, w, torch.from_numpy(vectors[f"{name}/out"])


def _close_fp16(got, want64):
    """Within one fp16 rounding step of the float64 value (plus the fp32 accumulation noise near a tie)."""
    want = want64.float()
    tol = want.abs() * 2.0 ** -10 + 1e-4
    assert torch.all((got.float() - want).abs() <= tol), float(((got.float() - want).abs() - tol).max())


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_vectors(vectors, name):
    q, k, w, out = _case(vectors, name)
    _close_fp16(out, SO.lightning_indexer(q, k, w))


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_kernel_matches_reference_vectors(vectors, name):
    from cinnamon_b200 import kernels as K
    q, k, w, out = _case(vectors, name)
    got = K.lightning_indexer_fused(q.cuda(), k.cuda(), w.cuda())
    assert got.dtype == torch.float16 and got.shape == out.shape
    # same fp16-rounded operands, fp32 sums in another order: at most one fp16 step apart, nearly always equal
    assert torch.all((got.cpu().float() - out.float()).abs() <= out.float().abs() * 2.0 ** -10 + 1e-4)
    assert float((got.cpu() != out).float().mean()) < 0.02
    _close_fp16(got.cpu(), SO.lightning_indexer(q, k, w))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_kernel_views_and_sizes(dtype):
    """The model's call shape (B, L, 4 heads of 64) plus a strided view of the keys."""
    from cinnamon_b200 import kernels as K
    g = torch.Generator().manual_seed(12)
    q = torch.randn(2, 257, 4, 64, generator=g).to(dtype)
    kfull = torch.randn(2, 300, 128, generator=g).to(dtype)
    w = torch.rand(2, 257, 4, generator=g).to(dtype)
    k = kfull[:, :, 64:]                                                     # pitched rows
    got = K.lightning_indexer_fused(q.cuda(), kfull.cuda()[:, :, 64:], w.cuda())
    _close_fp16(got.cpu(), SO.lightning_indexer(q, k, w))
