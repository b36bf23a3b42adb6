"""Seeded inputs shared by make_golden.py (which records what the reference
produces for them) and by the tests (which regenerate them and compare)."""
import hashlib

import torch


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def gen_input(seed, M, N, dtype, std, special):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, N, generator=g) * std)
    if special == "outliers":          # the reference's own outlier test, tests/test_kernels.py:67-69
        x[0, 0] = 1000.0
        x[M // 2, N // 2] = -500.0
    elif special == "zero_tile":
        x[:, :128] = 0.0
    elif special == "pow2_amax":       # amax exactly 448 * 2^k in some tiles
        for r in range(min(M, 12)):
            x[r, 5] = 448.0 * 2.0 ** (r - 6)
    return x.to(dtype)


CASES = [
    # name, seed, M, N, dtype, std, special
    ("c1_x_bf16", 1001, 64, 512, torch.bfloat16, 1.0, None),
    ("c1_w_bf16", 1002, 256, 512, torch.bfloat16, 0.02, None),
    ("fp32_act", 1003, 48, 384, torch.float32, 1.0, None),
    ("ragged_n", 1004, 40, 576 + 64, torch.float32, 1.0, None),     # N not a multiple of 128
    ("narrow_n", 1005, 33, 64, torch.bfloat16, 1.0, None),          # N < 128 (indexer call, src/attention.py:293)
    ("outliers", 1006, 256, 512, torch.bfloat16, 1.0, "outliers"),
    ("zero_tile", 1007, 16, 256, torch.bfloat16, 1.0, "zero_tile"),
    ("pow2_amax", 1008, 16, 256, torch.float32, 0.01, "pow2_amax"),
    ("ragged_m", 1009, 130, 200, torch.float32, 0.02, None),        # both dims ragged (block-wise)
]
