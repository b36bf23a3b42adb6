"""Generates tests/golden/indexer_vectors.npz from the reference checkout.

Run in a container that has the reference tree ($CINNAMON_REFERENCE, else `reference_path` of BASELINE.json):

    python tests/golden/make_golden_indexer.py

The reference's lightning indexer (src/kernels.py:321-433) is a Triton kernel; its Python wrapper asserts CUDA,
so the kernel is launched directly, with the wrapper's block sizes (:412-414), under the Triton CPU interpreter.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np
import torch
import triton

REF = os.environ.get("CINNAMON_REFERENCE")
if not REF:                          # else the checkout that BASELINE.json names
    import json
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "BASELINE.json")) as _f:
        REF = json.load(_f)["reference_path"]
sys.path.insert(0, os.path.join(REF, "src"))
import kernels as ref  # noqa: E402  (the reference's src/kernels.py)

# name, seed, B, Lq, Lk, H, d, dtype
CASES = [("model_like", 1, 2, 40, 70, 4, 64, torch.float32), ("wide_head", 2, 1, 33, 33, 2, 128, torch.float32),
         ("bf16_inputs", 3, 1, 48, 96, 4, 64, torch.bfloat16), ("narrow", 4, 1, 5, 7, 3, 16, torch.float32)]


def main():
    out = {}
    for name, seed, B, Lq, Lk, H, d, dtype in CASES:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, Lq, H, d, generator=g).to(dtype)
        k = torch.randn(B, Lk, d, generator=g).to(dtype)
        w = torch.rand(B, Lq, H, generator=g).to(dtype)
        o = torch.empty((B, Lq, Lk), dtype=torch.float16)
        grid = (B, triton.cdiv(Lq, 32), triton.cdiv(Lk, 32))
        ref.lightning_indexer_kernel[grid](q, k, w, o, B, Lq, Lk, d, *q.stride(), *k.stride(), *w.stride(), *o.stride(),
                                           BLOCK_Q=32, BLOCK_K=32, BLOCK_D=min(64, d), N_HEAD=H)
        for key, val in (("q", q), ("k", k), ("w", w)):
            out[f"{name}/{key}"] = val.float().numpy()
        out[f"{name}/out"] = o.numpy()
        out[f"{name}/bf16"] = np.int64(dtype == torch.bfloat16)
        print(name, "ok", flush=True)
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "indexer_vectors.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
