"""The reference's own model (staged under ``baseline/_ref/src``, see stage_reference.py) built on top of this
library's drop-in ``kernels`` module: what a user of the reference does after swapping ``src/kernels.py``.

``build_model`` constructs ``Cinnamon`` exactly as the reference's trainer does (src/train.py:650-683), runs
``convert_to_fp8`` (src/train.py:696-698) and moves it to the device; ``train_step`` is the reference's training
step (src/train.py:338-376: bf16 autocast, main + multi-token-prediction cross-entropy, auxiliary losses,
backward) followed by the optimiser step.  Used by the GPU test of the end-to-end configuration and by the
benchmark's end-to-end entry; nothing in the library imports this file.
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_SRC = os.path.join(HERE, "_ref", "src")

# the end-to-end benchmark configuration: fields that differ from the reference's ModelConfig defaults
CONFIG_5 = dict(d_model=512, n_layers=8, n_heads=8, d_cq=256, d_ckv=128, d_rope=64, n_routed=16, top_k=2, n_shared=1,
                hidden_dim=1024, mtp_depth=1, vocab_size=32000)


def available() -> bool:
    return os.path.isfile(os.path.join(REF_SRC, "model.py"))


def import_reference(own_kernels: bool = False):
    """Imports the reference's ``config`` and ``model`` modules with ``kernels`` bound to the drop-in - or, with
    ``own_kernels``, to the reference's own Triton ``src/kernels.py`` (the unmodified reference end to end; a process
    can hold only one of the two)."""
    if not available():
        raise RuntimeError("the reference is not staged: run baseline/stage_reference.py where the reference tree is present")
    root = os.path.dirname(HERE)
    if root not in sys.path:
        sys.path.insert(0, root)
    if own_kernels:
        sys.path.insert(0, REF_SRC)
        import kernels as K
        assert os.path.dirname(os.path.abspath(K.__file__)) == REF_SRC
    else:
        import cinnamon_b200.dropin as dropin
        K = dropin.install()
        if REF_SRC not in sys.path:
            sys.path.append(REF_SRC)        # appended: `kernels` is already bound, the rest resolves here
    import config as ref_config
    import model as ref_model
    import layers as ref_layers
    assert ref_layers.HAS_GROUPED_GEMM and ref_layers.moe_grouped_gemm is K.moe_grouped_gemm
    return ref_config, ref_model, K


def build_model(device, overrides: dict | None = None, fp8: bool = True, balance_alpha: float = 0.0,
                own_kernels: bool = False):
    ref_config, ref_model, K = import_reference(own_kernels)
    c = ref_config.ModelConfig()
    for k, v in dict(CONFIG_5, **(overrides or {})).items():
        assert hasattr(c, k), k
        setattr(c, k, v)
    model = ref_model.Cinnamon(c.d_model, c.n_layers, c.vocab_size, c.hidden_dim, c.n_heads, c.max_seq_len, c.d_ckv, c.d_cq,
                               c.d_head, c.d_v, c.d_rope, c.n_routed, c.n_shared, c.top_k, c.expert_scale, c.gamma,
                               balance_alpha, c.dsa_topk, c.local_window, c.n_indexer_heads, c.d_indexer_head, c.rms_eps,
                               c.rope_base, c.rope_type, c.mtp_depth, c.pope_delta_init, c.original_seq_len, c.rope_factor,
                               c.beta_fast, c.beta_slow, c.mscale, c.indexer_use_fp8, c.indexer_use_hadamard,
                               c.use_sparse_kernel)
    if fp8:
        model = K.convert_to_fp8(model)                       # src/train.py:696-698
    return model.to(device), c, K


def train_step(model, batch, optimizer=None, mtp_lambda: float = 0.3, dsa_kl_weight: float = 0.0, grad_clip: float = 1.0):
    """One training step as in src/train.py:338-376 (+ clip and optimiser step, :453-470).  ``batch``: (B, L + 1)
    token ids on the model's device.  Returns the loss tensor (not synchronised)."""
    import torch
    import torch.nn.functional as F
    x, y = batch[:, :-1], batch[:, 1:]
    with torch.autocast("cuda", dtype=torch.bfloat16):
        main_logits, mtp_logits, dsa_kl, moe_balance = model(x, dsa_warmup=False, compute_aux=True)
        main_loss = F.cross_entropy(main_logits.reshape(-1, main_logits.size(-1)), y.reshape(-1))
        mtp_losses = []
        for depth, logits in enumerate(mtp_logits, start=1):
            target = batch[:, depth + 1:]
            mtp_losses.append(F.cross_entropy(logits.reshape(-1, logits.size(-1)), target.reshape(-1)))
        mtp_loss = sum(mtp_losses) / len(mtp_losses) if mtp_losses else 0.0
        loss = main_loss + mtp_lambda * mtp_loss
        if dsa_kl is not None:
            loss = loss + dsa_kl_weight * dsa_kl
        if moe_balance is not None:
            loss = loss + moe_balance
    loss.backward()
    if optimizer is not None:
        torch.nn.utils.clip_grad_norm_([p for p in model.parameters() if p.grad is not None], grad_clip)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
    return loss.detach()


def _main():
    """``python baseline/reference_model.py [--own-kernels] [--steps N] [--batch B] [--seq L]``: times the training
    step on cuda:0 and prints one JSON line.  With ``--own-kernels`` the model runs on the reference's own Triton
    kernels: the unmodified reference, for a side-by-side figure on the same GPU."""
    import argparse
    import json
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--own-kernels", action="store_true")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=1024)
    a = ap.parse_args()
    torch.manual_seed(1005)
    model, cfg, _ = build_model("cuda", own_kernels=a.own_kernels)
    model.train()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.1)
    host = torch.randint(0, cfg.vocab_size, (a.batch, a.seq + 1), generator=torch.Generator().manual_seed(1005)).pin_memory()
    for _ in range(a.warmup):
        loss = train_step(model, host.to("cuda", non_blocking=True), optimizer=opt)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = train_step(model, host.to("cuda", non_blocking=True), optimizer=opt)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    print("RESULT " + json.dumps({"kernels": "reference (Triton)" if a.own_kernels else "cinnamon_b200", "ms_per_step": ms,
                                  "tokens_per_s": a.batch * a.seq / (ms * 1e-3), "loss": float(loss),
                                  "loss_is_finite": bool(torch.isfinite(loss))}))


if __name__ == "__main__":
    _main()
