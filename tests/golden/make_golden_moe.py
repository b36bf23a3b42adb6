"""Generates tests/golden/moe_vectors.npz: the reference's own ``MoE`` block (src/layers.py:89-179) run on the CPU
(its fallback expert loop, :76-87) in training mode with the balance loss on, for seeded weights and inputs.

Run where the reference tree is present ($CINNAMON_REFERENCE, else `reference_path` of BASELINE.json):
    python tests/golden/make_golden_moe.py

Recorded per case: every parameter (so the test loads the very same weights), the input, the output, the balance
loss, the expert bias after the update, and the gradients of the input and of all parameters for the loss
``output.pow(2).mean() + balance_loss``.
"""
import os
import sys

import numpy as np
import torch

REF = os.environ.get("CINNAMON_REFERENCE")
if not REF:                          # else the checkout that BASELINE.json names
    import json
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "BASELINE.json")) as _f:
        REF = json.load(_f)["reference_path"]
sys.path.insert(0, os.path.join(REF, "src"))
import layers as ref_layers  # noqa: E402  (the reference's src/layers.py)

CASES = {
    # name: (n_routed, n_shared, top_k, d_model, hidden_dim, expert_scale, gamma, balance_alpha, batch, seq, seed)
    "small": (8, 1, 2, 64, 128, 4, 0.001, 0.01, 2, 16, 11),
    "two_shared_top3": (6, 2, 3, 32, 64, 2, 0.01, 0.05, 3, 8, 12),
}


def main():
    out = {}
    for name, (E, S, k, d, h, scale, gamma, alpha, B, L, seed) in CASES.items():
        torch.manual_seed(seed)
        m = ref_layers.MoE(E, S, k, d, h, scale, gamma, alpha)
        with torch.no_grad():
            m.expert_bias.copy_(torch.randn(E) * 0.2)
        m.train()
        x = torch.randn(B, L, d, requires_grad=True)
        bias_before = m.expert_bias.clone()
        y, bl = m(x)
        (y.pow(2).mean() + bl).backward()
        for pname, p in m.named_parameters():
            out[f"{name}/param/{pname}"] = p.detach().numpy().copy()
            out[f"{name}/grad/{pname}"] = p.grad.numpy().copy()
        out[f"{name}/bias_before"] = bias_before.numpy()
        out[f"{name}/bias_after"] = m.expert_bias.numpy().copy()
        out[f"{name}/x"] = x.detach().numpy().copy()
        out[f"{name}/y"] = y.detach().numpy().copy()
        out[f"{name}/balance_loss"] = np.float64(bl.item())
        out[f"{name}/grad_x"] = x.grad.numpy().copy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "moe_vectors.npz")
    np.savez_compressed(path, **out)
    print(path, len(out), "arrays")


if __name__ == "__main__":
    main()
