"""Generates tests/golden/sparse_attention_vectors.npz from the reference checkout.

Run in a container that has the reference tree ($CINNAMON_REFERENCE, else `reference_path` of BASELINE.json):

    python tests/golden/make_golden_sparse.py

The reference's sparse attention (src/kernels.py:913-1312) is Triton; the Triton CPU interpreter
(TRITON_INTERPRET=1) executes its forward and backward kernels on small seeded cases.  Recorded per case: the
inputs (they are tiny), output, attention weights and the three input gradients.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np
import torch

REF = os.environ.get("CINNAMON_REFERENCE")
if not REF:                          # else the checkout that BASELINE.json names
    import json
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "BASELINE.json")) as _f:
        REF = json.load(_f)["reference_path"]
sys.path.insert(0, os.path.join(REF, "src"))
import kernels as ref  # noqa: E402  (the reference's src/kernels.py)

# name, seed, B, H, L, K, D_qk, D_v, how the index lists are drawn
CASES = [
    ("small", 1, 1, 2, 24, 8, 16, 8, "random"),            # keys after the query are ignored; query 0 often has none
    ("ragged_dims", 2, 2, 1, 20, 12, 24, 12, "random"),    # K and the feature sizes are not powers of two
    ("causal_topk", 3, 1, 2, 40, 16, 32, 16, "prefix"),    # distinct indices out of 0..t, padded with later ones
    ("duplicates", 4, 1, 1, 16, 8, 8, 8, "dup"),           # the same key listed twice counts twice
]


def make_idx(kind, g, B, L, K):
    if kind == "random":
        return torch.randint(0, L, (B, L, K), generator=g)
    if kind == "dup":
        idx = torch.randint(0, L, (B, L, K), generator=g)
        idx[..., 1] = idx[..., 0]
        return idx
    idx = torch.empty(B, L, K, dtype=torch.int64)
    for b in range(B):
        for t in range(L):
            perm = torch.randperm(L, generator=g)
            early = perm[perm <= t][:K]
            late = perm[perm > t][:K - early.numel()]
            idx[b, t] = torch.cat([early, late])[:K] if early.numel() + late.numel() >= K else \
                torch.cat([early, late, early[:1].repeat(K - early.numel() - late.numel())])
    return idx


def main():
    out = {}
    for name, seed, B, H, L, K, Dqk, Dv, kind in CASES:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, H, L, Dqk, generator=g).requires_grad_(True)
        k = torch.randn(B, H, L, Dqk, generator=g).requires_grad_(True)
        v = torch.randn(B, H, L, Dv, generator=g).requires_grad_(True)
        idx = make_idx(kind, g, B, L, K)
        scale = Dqk ** -0.5
        o, aw = ref.SparseAttentionFunction.apply(q, k, v, idx, scale)
        go = torch.randn(o.shape, generator=g)
        o.backward(go)
        for key, val in (("q", q), ("k", k), ("v", v), ("idx", idx), ("out", o), ("attn", aw), ("grad_out", go),
                         ("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
            out[f"{name}/{key}"] = val.detach().numpy()
        out[f"{name}/scale"] = np.float64(scale)
        print(name, "ok", flush=True)
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "sparse_attention_vectors.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
