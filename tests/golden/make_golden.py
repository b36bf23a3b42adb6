"""Generates tests/golden/reference_vectors.npz from the reference checkout.

Run in a container that has the reference tree ($CINNAMON_REFERENCE, else the
`reference_path` of BASELINE.json):   python tests/golden/make_golden.py

What the reference can produce without a GPU:
  * scales of its two quantiser kernels (src/kernels.py:19-132) executed by the
    Triton CPU interpreter (TRITON_INTERPRET=1).  The interpreter's fp32->e4m3
    cast is not faithful, so its bytes are NOT recorded, only the scales;
  * outputs of its pure-torch dequantize_fp8_rowwise (src/kernels.py:262-281).
Inputs are regenerated in the tests from the recorded seeds; a digest of each
input is stored so a drift in the random generator is detected.
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


sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from cases import CASES, digest, gen_input  # noqa: E402


def run_rowwise(x, round_scale):
    M, N = x.shape
    nb = (N + 127) // 128
    q = torch.empty((M, N), dtype=torch.float8_e4m3fn)
    s = torch.empty((M, nb), dtype=torch.float32)
    ref.quantize_fp8_rowwise_kernel[(M, nb)](
        x, q, s, M, N, x.stride(0), x.stride(1), q.stride(0), q.stride(1),
        BLOCK_SIZE=128, ROUND_SCALE=round_scale, FP8_MAX=448.0)
    return s


def run_blockwise(x, round_scale):
    M, N = x.shape
    mb, nb = (M + 127) // 128, (N + 127) // 128
    q = torch.empty((M, N), dtype=torch.float8_e4m3fn)
    s = torch.empty((mb, nb), dtype=torch.float32)
    ref.quantize_fp8_blockwise_kernel[(mb, nb)](
        x, q, s, M, N, x.stride(0), x.stride(1), q.stride(0), q.stride(1),
        BLOCK_M=128, BLOCK_N=128, ROUND_SCALE=round_scale, FP8_MAX=448.0)
    return s


def main():
    out = {}
    names = []
    for name, seed, M, N, dtype, std, special in CASES:
        x = gen_input(seed, M, N, dtype, std, special)
        names.append(name)
        out[f"{name}/digest"] = np.frombuffer(bytes.fromhex(digest(x)), dtype=np.uint8)
        for rs in (False, True):
            out[f"{name}/row_scales_rs{int(rs)}"] = run_rowwise(x, rs).numpy()
            out[f"{name}/block_scales_rs{int(rs)}"] = run_blockwise(x, rs).numpy()
        print(name, "ok", flush=True)
    # dequantize_fp8_rowwise: random codes (NaN codes excluded) x random positive scales
    g = torch.Generator().manual_seed(2001)
    for tag, (M, N) in {"deq_a": (37, 512), "deq_ragged": (9, 200)}.items():
        codes = torch.randint(0, 256, (M, N), generator=g, dtype=torch.int32).to(torch.uint8)
        codes[(codes & 0x7F) == 0x7F] = 0x3A
        nb = (N + 127) // 128
        scales = torch.rand(M, nb, generator=g) * 0.01 + 1e-6
        y = ref.dequantize_fp8_rowwise(codes.view(torch.float8_e4m3fn), scales, 128)
        out[f"{tag}/codes"] = codes.numpy()
        out[f"{tag}/scales"] = scales.numpy()
        out[f"{tag}/out"] = y.numpy()
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "reference_vectors.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
