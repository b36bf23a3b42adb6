"""The reference's own model on top of the drop-in: ``Cinnamon`` built with the fields of the end-to-end benchmark
configuration (d_model 512, 8 layers, 8 heads, MLA ranks 256 / 128, rope 64, 16 routed experts top-2 + 1 shared
expert of width 1024, multi-token prediction depth 1, vocabulary 32000), ``convert_to_fp8`` (src/train.py:696-698),
one training step as in src/train.py:338-376 under bf16 autocast.  The FP8 shared experts go through
``FP8Linear`` / ``FP8MatmulFunction``, the routed experts through ``moe_grouped_gemm`` (which, unlike the
reference's, is differentiable: routed expert weights must now receive gradients), attention through
``sparse_attention``.  Runs in a child process: the reference keeps flat module names (config, model, layers ...).
Skips when the reference is not staged beside the repository."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, sys
sys.path.insert(0, sys.argv[1])
import torch
from baseline import reference_model as RM
torch.manual_seed(5)
model, cfg, K = RM.build_model("cuda")
fp8 = sorted(n for n, m in model.named_modules() if isinstance(m, K.FP8Linear))
round_scale = sorted(n for n, m in model.named_modules() if isinstance(m, K.FP8Linear) and m.round_scale)
model.train()
opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
g = torch.Generator().manual_seed(1005)
batch = torch.randint(0, cfg.vocab_size, (2, 257), generator=g).cuda()
bias0 = model.transformer_layers[0].moe.expert_bias.clone()
loss1 = RM.train_step(model, batch, optimizer=None)
grads = {n: (p.grad is not None and bool(torch.isfinite(p.grad).all()), float(p.grad.abs().sum()) if p.grad is not None else 0.0)
         for n, p in model.named_parameters()}
opt.step(); opt.zero_grad(set_to_none=True)
loss2 = RM.train_step(model, batch, optimizer=opt)
loss3 = RM.train_step(model, batch, optimizer=opt)
torch.cuda.synchronize()
out = {"fp8": fp8, "round_scale": round_scale, "loss": [float(loss1), float(loss2), float(loss3)],
       "bad": [n for n, (ok, _) in grads.items() if not ok and "indexer" not in n],
       "routed_w12": grads["transformer_layers.0.moe.routed_experts.w12"][1],
       "routed_w3": grads["transformer_layers.3.moe.routed_experts.w3"][1],
       "shared_w1": grads["transformer_layers.0.moe.shared_experts.0.w1.weight"][1],
       "mtp_proj": grads["mtp_modules.0.proj.weight"][1],
       "router": grads["transformer_layers.0.moe.router.weight"][1],
       "bias_moved": bool((model.transformer_layers[0].moe.expert_bias != bias0).any()),
       "status": K.device_status(), "launches": K.launch_count}
print("RESULT " + json.dumps(out))
"""


def test_reference_model_trains_on_the_drop_in(tmp_path):
    if not os.path.isfile(os.path.join(ROOT, "baseline", "_ref", "src", "model.py")):
        pytest.skip("reference not staged (python baseline/stage_reference.py needs the reference tree)")
    script = tmp_path / "c5.py"
    script.write_text(CHILD)
    p = subprocess.run([sys.executable, str(script), ROOT], capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    line = [ln for ln in p.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    r = json.loads(line[len("RESULT "):])
    # convert_to_fp8's selection on this model: the shared expert's three linears per block (8 layers + the MTP
    # block) and the MTP projection; round_scale on w1 and w2 only (src/kernels.py:863-878)
    assert len(r["fp8"]) == 9 * 3 + 1 and "mtp_modules.0.proj" in r["fp8"], r["fp8"]
    assert len(r["round_scale"]) == 9 * 2 and all(n.endswith((".w1", ".w2")) for n in r["round_scale"])
    assert all(l == l and abs(l) < 1e4 for l in r["loss"]), r["loss"]               # finite
    assert r["loss"][2] < r["loss"][0], f"three steps on one batch did not lower the loss: {r['loss']}"
    assert not r["bad"], f"missing or non-finite gradients: {r['bad'][:8]}"
    for key in ("routed_w12", "routed_w3", "shared_w1", "mtp_proj", "router"):
        assert r[key] > 0.0, f"{key} received no gradient"
    assert r["bias_moved"] and r["status"] == 0 and r["launches"] > 100
