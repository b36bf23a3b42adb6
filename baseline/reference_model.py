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


def import_reference():
    """Imports the reference's ``config`` and ``model`` modules with ``kernels`` bound to the drop-in."""
    if not available():
        raise RuntimeError("the reference is not staged: run baseline/stage_reference.py where the reference tree is present")
    root = os.path.dirname(HERE)
    if root not in sys.path:
        sys.path.insert(0, root)
    import cinnamon_b200.dropin as dropin
    K = dropin.install()
    if REF_SRC not in sys.path:
        sys.path.append(REF_SRC)            # appended: `kernels` is already bound, the rest resolves here
    import config as ref_config
    import model as ref_model
    import layers as ref_layers
    assert ref_layers.HAS_GROUPED_GEMM and ref_layers.moe_grouped_gemm is K.moe_grouped_gemm
    return ref_config, ref_model, K


def build_model(device, overrides: dict | None = None, fp8: bool = True, balance_alpha: float = 0.0):
    ref_config, ref_model, K = import_reference()
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
