"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import fp8_oracle as O


def bytes_of(q: torch.Tensor) -> np.ndarray:
    return q.detach().view(torch.uint8).cpu().numpy()


def bits_of(s: torch.Tensor) -> np.ndarray:
    return s.detach().float().cpu().numpy().view(np.uint32)


def assert_quant_equal(q_gpu, s_gpu, q_ref, s_ref, what=""):
    qg, sg = bytes_of(q_gpu), bits_of(s_gpu)
    qr, sr = q_ref.numpy(), s_ref.numpy().view(np.uint32)
    assert qg.shape == qr.shape and sg.shape == sr.shape, f"{what}: shape {qg.shape}/{sg.shape} vs {qr.shape}/{sr.shape}"
    ns = int((sg != sr).sum())
    nq = int((qg != qr).sum())
    assert ns == 0 and nq == 0, f"{what}: {ns} scale mismatches, {nq} byte mismatches of {qg.size}"


def ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    return np.abs(a_bits.astype(np.int64) - b_bits.astype(np.int64))


def rel_fro(a, ref):
    return O.rel_fro(a.detach().cpu(), ref)


def assert_bf16_close(got: torch.Tensor, ref64: torch.Tensor, what=""):
    """A bf16 result against the float64 result: each element within one bf16 rounding
    step (2^-8 relative) of the exact value, plus the fp32 accumulation error, which is
    relative to the size of the whole result, not of the element (matters next to zero)."""
    g = got.detach().cpu().double()
    r = ref64.double()
    tol = r.abs() * 2.0 ** -8 + 1e-5 * r.pow(2).mean().sqrt()
    bad = (g - r).abs() > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} elements off by more than a bf16 step"
