"""The CPU checker against everything that pins it (no GPU needed)."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from cases import CASES, digest, gen_input
from oracle import fp8_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cref():
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_build", "libquant_ref.so"))
    return lib


def _c_quant(lib, fn, x32, round_scale, block):
    M, N = x32.shape
    x32 = np.ascontiguousarray(x32, dtype=np.float32)
    q = np.empty((M, N), dtype=np.uint8)
    nb = (N + 127) // 128
    s = np.empty(((M + 127) // 128 if block else M, nb), dtype=np.float32)
    getattr(lib, fn)(x32.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(M), ctypes.c_int64(N),
                     ctypes.c_int64(N), q.ctypes.data_as(ctypes.c_void_p),
                     s.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(int(round_scale)))
    return q, s


def test_e4m3_decode_matches_torch():
    codes = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    t = codes.view(torch.float8_e4m3fn).float().numpy()
    mine = O.e4m3_decode(codes.numpy())
    assert np.array_equal(np.isnan(t), np.isnan(mine))
    ok = ~np.isnan(t)
    assert np.array_equal(t[ok], mine[ok])


def test_e4m3_encode_every_bf16_value_and_midpoints(cref):
    # every bf16 bit pattern, widened to fp32, clamped as the quantiser does
    bits = (np.arange(65536, dtype=np.uint32) << 16)
    v = bits.view(np.float32)
    finite = np.isfinite(v)
    v = np.clip(v[finite], -448.0, 448.0)
    tab = O.e4m3_decode_table()
    pos = np.sort(tab[:0x7F].astype(np.float64))
    mids = ((pos[1:] + pos[:-1]) / 2).astype(np.float32)          # exact ties
    near = np.concatenate([np.nextafter(mids, np.float32(0)), mids, np.nextafter(mids, np.float32(1e9))])
    rng = np.random.default_rng(7)
    rnd = (rng.standard_normal(2_000_000) * np.exp(rng.uniform(-12, 6.2, 2_000_000))).astype(np.float32)
    rnd = np.clip(rnd, -448, 448)
    allv = np.concatenate([v, near, -near, rnd, np.float32([0.0, -0.0, 448, -448, 2 ** -9, 2 ** -10, 3 * 2 ** -10])])
    mine = O.e4m3_encode_bits(allv)
    ref = O.e4m3_encode_torch(torch.from_numpy(allv)).numpy()
    assert np.array_equal(mine, ref)
    out = np.empty(allv.shape, dtype=np.uint8)
    cref.oracle_e4m3_encode(allv.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p),
                            ctypes.c_int64(allv.size))
    assert np.array_equal(out, mine)


def test_e4m3_encode_saturates_and_nan():
    v = np.float32([1e9, -1e9, np.inf, -np.inf, np.nan, 464.0, 479.9])
    assert O.e4m3_encode_bits(v).tolist() == [0x7E, 0xFE, 0x7E, 0xFE, 0x7F, 0x7E, 0x7E]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_scales_match_reference_kernels(case, golden):
    """Scales from the reference's Triton kernels (run by the Triton CPU
    interpreter when the fixture was made) equal the restatement's, bit for bit."""
    name, seed, M, N, dtype, std, special = case
    x = gen_input(seed, M, N, dtype, std, special)
    assert bytes.fromhex(digest(x)) == golden[f"{name}/digest"].tobytes(), "seeded input drifted"
    for rs in (False, True):
        _, s_row = O.quantize_rowwise(x, 128, rs)
        _, s_blk = O.quantize_blockwise(x, 128, 128, rs)
        assert np.array_equal(s_row.numpy().view(np.uint32), golden[f"{name}/row_scales_rs{int(rs)}"].view(np.uint32))
        assert np.array_equal(s_blk.numpy().view(np.uint32), golden[f"{name}/block_scales_rs{int(rs)}"].view(np.uint32))


@pytest.mark.parametrize("tag", ["deq_a", "deq_ragged"])
def test_dequant_rowwise_matches_reference_torch(tag, golden):
    codes = torch.from_numpy(golden[f"{tag}/codes"])
    scales = torch.from_numpy(golden[f"{tag}/scales"])
    y = O.dequantize_rowwise(codes, scales, 128)
    assert np.array_equal(y.numpy().view(np.uint32), golden[f"{tag}/out"].view(np.uint32))


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_python_and_c_restatements_agree(case, cref):
    name, seed, M, N, dtype, std, special = case
    x = gen_input(seed, M, N, dtype, std, special)
    for rs in (False, True):
        for enc in ("torch", "bits"):
            q, s = O.quantize_rowwise(x, 128, rs, encoder=enc)
            qc, sc = _c_quant(cref, "oracle_quant_rowwise_f32", x.float().numpy(), rs, False)
            assert np.array_equal(q.numpy(), qc) and np.array_equal(s.numpy().view(np.uint32), sc.view(np.uint32))
            q, s = O.quantize_blockwise(x, 128, 128, rs, encoder=enc)
            qc, sc = _c_quant(cref, "oracle_quant_blockwise_f32", x.float().numpy(), rs, True)
            assert np.array_equal(q.numpy(), qc) and np.array_equal(s.numpy().view(np.uint32), sc.view(np.uint32))


def test_round_scale_is_power_of_two_and_covers_amax():
    x = gen_input(5, 64, 512, torch.bfloat16, 3.0, None)
    q, s = O.quantize_rowwise(x, 128, True)
    m, e = torch.frexp(s)
    assert torch.all(m == 0.5)
    amax = x.float().reshape(64, 4, 128).abs().amax(-1).clamp_min(1e-4)
    assert torch.all(s * 448.0 >= amax) and torch.all(s * 224.0 < amax * (1 + 1e-6))


def test_roundtrip_error_like_reference_test():
    # tests/test_kernels.py:50-60 of the reference: mean relative error < 0.1
    x = gen_input(11, 256, 512, torch.bfloat16, 1.0, None)
    q, s = O.quantize_rowwise(x, 128)
    y = O.dequantize_rowwise(q, s)
    rel = (x.float() - y).abs() / (x.float().abs() + 1e-6)
    assert rel.mean().item() < 0.1


def test_nan_and_inf_follow_ptx_min_max():
    x = torch.zeros(1, 128)
    x[0, 3] = float("nan")
    x[0, 4] = 2.0
    q, s = O.quantize_rowwise(x, 128)
    assert s[0, 0].item() == np.float32(2.0) / np.float32(448.0)
    assert q[0, 3].item() == 0xFE and q[0, 4].item() == 0x7E


def test_linear_fwd_bwd_shapes_and_fp8_noise():
    x, w, dy = O.make_linear_case(256, 512, 384, seed=3)
    out, saved = O.fp8_linear_forward(x, w, False)
    gx, gw = O.fp8_linear_backward(dy, saved, False)
    assert out.shape == (256, 384) and gx.shape == (256, 512) and gw.shape == (384, 512)
    exact = x.double() @ w.double().t()
    assert 5e-3 < O.rel_fro(out, exact) < 8e-2      # fp8 quantisation noise, not a bug
    assert O.rel_fro(gx, dy.double() @ w.double()) < 8e-2
    assert O.rel_fro(gw, dy.double().t() @ x.double()) < 8e-2


def test_grouped_oracles_agree_up_to_fp8_noise():
    g = torch.Generator().manual_seed(9)
    E, d_in, d_out = 4, 256, 128
    x = torch.randn(300, d_in, generator=g).bfloat16()
    w = (torch.randn(E, d_out, d_in, generator=g) * 0.02).bfloat16()
    starts = torch.tensor([0, 0, 130, 131])
    ends = torch.tensor([0, 130, 131, 300])
    a = O.grouped_gemm_f64(x, w, starts, ends)
    b = O.grouped_gemm_fp8_f64(x, w, starts, ends)
    assert O.rel_fro(b, a) < 8e-2
