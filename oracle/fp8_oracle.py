"""CPU restatement of cinnamon's FP8 training path.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA kernels are compared with.  Nothing in the
shipped package imports it; only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may.

Every function names the reference lines (``src/kernels.py`` in
shyampathak22/cinnamon) whose arithmetic it restates.  The reference itself
cannot run on a CPU: its wrappers ``assert x.is_cuda`` (src/kernels.py:194,
237, 296), so the CPU branches of ``FP8MatmulFunction`` are unreachable.  What
is restated here is the arithmetic of the Triton kernels:

  * amax over the tile, masked elements count as 0     (src/kernels.py:48-51, 109-112)
  * amax = max(amax, 1e-4) in fp32                      (:53, :114)
  * scale = amax / 448                                  (:57, :118)
    or 2**ceil(log2(amax / 448)) with ``round_scale``   (:55, :116)
  * q = clamp(x / scale, -448, 448) -> e4m3, RNE        (:60-62, :121-123)

Division flavour.  On a GPU Triton lowers both fp32 divisions to the PTX
instruction ``div.full.f32`` (an approximate division, <= 2 ulp).  A CPU has
no such instruction, so this restatement divides in IEEE round-to-nearest; the
CUDA library offers both flavours (``div_mode="rn"`` is the one that must be
bit-identical to this file, ``div_mode="full"`` is the one that matches the
Triton kernels on the same GPU).

Parity pin.  The reference's tests hold no golden vectors for this path (they
check shapes and loose tolerances on unseeded inputs only), and the reference
cannot be executed here, so the pins are: (1) scales produced by the
reference's own kernels under the Triton CPU interpreter (fixtures in
tests/golden, made by tests/golden/make_golden.py); (2) the reference's
pure-torch ``dequantize_fp8_rowwise`` (src/kernels.py:262-281) imported and run
on seeded inputs (same fixtures); (3) torch's own CPU e4m3 cast, compared with
the independent bit-level encoder below over every bf16 value and a dense fp32
sweep.  Bytes produced by the reference on a B200 are NOT pinned: parity of the
``full`` division flavour is unpinned.
"""
from __future__ import annotations

import numpy as np
import torch

FP8_MAX = 448.0          # src/kernels.py:16
AMAX_FLOOR = 1e-4        # src/kernels.py:53,114 (applied in fp32: 0x38D1B717)


# ----------------------------------------------------------------------------
# e4m3 (float8_e4m3fn) encode / decode, written from the format definition:
# 1 sign, 4 exponent (bias 7), 3 mantissa bits; no infinities; 0x7F/0xFF = NaN;
# largest finite 0x7E = 448; subnormals are multiples of 2**-9.
# ----------------------------------------------------------------------------
def e4m3_decode_table() -> np.ndarray:
    """All 256 codes as float32 (NaN for 0x7F / 0xFF)."""
    codes = np.arange(256, dtype=np.uint32)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    e = (codes >> 3) & 0xF
    m = codes & 0x7
    val = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2(e.astype(np.float64) - 7))
    val = np.where((codes & 0x7F) == 0x7F, np.nan, val)
    return (sign * val).astype(np.float32)


_DECODE = e4m3_decode_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    return _DECODE[np.asarray(codes, dtype=np.uint8)]


def e4m3_encode_bits(v: np.ndarray) -> np.ndarray:
    """fp32 -> e4m3 code, round-to-nearest-even, saturating to +-448.

    Semantics of ``cvt.rn.satfinite.e4m3x2.f32`` (what ``.to(tl.float8e4nv)``
    becomes, src/kernels.py:62,123): finite values beyond 448 saturate, NaN
    gives 0x7F.  Works on the raw bit pattern so it does not depend on any
    library's fp8 support.
    """
    v = np.ascontiguousarray(v, dtype=np.float32)
    bits = v.view(np.uint32)
    sign = ((bits >> 24) & 0x80).astype(np.uint8)
    mag = bits & 0x7FFFFFFF
    a = mag.view(np.float32)
    out = np.empty(v.shape, dtype=np.uint8)

    nan = mag > 0x7F800000
    big = (a >= 448.0) & ~nan                       # saturate (also +-inf)
    sub = a < 2.0 ** -6                              # below the smallest normal
    # normal range: round the 23-bit mantissa to 3 bits, ties to even
    lsb = (mag >> 20) & 1
    r = mag + 0x7FFFF + lsb
    r &= ~np.uint32(0xFFFFF)
    exp = (r >> 23).astype(np.int32) - 127 + 7
    man = (r >> 20) & 0x7
    code = ((exp << 3) | man.astype(np.int32))
    code = np.minimum(code, 0x7E).astype(np.uint8)
    # subnormal range: units of 2**-9, rint is ties-to-even; 8 -> 0x08 = 2**-6
    subcode = np.rint(np.where(sub, a, 0).astype(np.float64) * 512.0).astype(np.uint8)
    out[...] = code
    out[sub] = subcode[sub]
    out[big] = 0x7E
    out |= sign
    out[nan] = 0x7F
    return out


def e4m3_encode_torch(v: torch.Tensor) -> torch.Tensor:
    """torch's CPU cast (RNE); equal to e4m3_encode_bits for |v| <= 448."""
    return v.to(torch.float8_e4m3fn).view(torch.uint8)


# ----------------------------------------------------------------------------
# scale arithmetic
# ----------------------------------------------------------------------------
def _scale_from_amax(amax: torch.Tensor, round_scale: bool) -> torch.Tensor:
    """fp32 amax -> fp32 scale (src/kernels.py:53-57, 114-118).

    ``round_scale``: 2**ceil(log2(amax/448)).  The reference evaluates log2 in
    fp32 (CUDA's log2f), rounds up to an integer and feeds ``ex2``.  Its log2f
    is accurate to an ulp, and next to an integer result the only rounding
    that matters is the final one to fp32, so the restatement evaluates log2
    in float64 and rounds once to fp32 before the ceil.
    """
    amax = torch.clamp(amax.float(), min=AMAX_FLOOR)
    s = amax / torch.tensor(FP8_MAX, dtype=torch.float32)
    if round_scale:
        lg = torch.log2(s.double()).float()
        e = torch.ceil(lg)
        s = torch.ldexp(torch.ones_like(s), e.to(torch.int32))
    return s


def _quantize_values(x32: torch.Tensor, scale: torch.Tensor, encoder: str) -> torch.Tensor:
    """x / scale, clamp to +-448, e4m3 RNE (src/kernels.py:60-62, 121-123).

    The clamp is PTX ``max`` then ``min``, which drop a NaN operand, so a NaN
    input becomes -448 (max(NaN, -448) = -448); restated with fmax/fmin.
    """
    y = x32 / scale
    lo = torch.full((), -FP8_MAX, dtype=torch.float32)
    hi = torch.full((), FP8_MAX, dtype=torch.float32)
    y = torch.fmin(torch.fmax(y, lo), hi)
    if encoder == "bits":
        return torch.from_numpy(e4m3_encode_bits(y.numpy()))
    return e4m3_encode_torch(y)


def _nan_dropping_amax(t: torch.Tensor, dim) -> torch.Tensor:
    # tl.max lowers to max.f32 / redux.sync.max.f32, which ignore NaN operands.
    return torch.nan_to_num(t.abs(), nan=0.0, posinf=float("inf")).amax(dim=dim)


def quantize_rowwise(x: torch.Tensor, block_size: int = 128, round_scale: bool = False,
                     encoder: str = "torch"):
    """1 x block_size tiles along the last dim (src/kernels.py:19-71, 178-216).

    Returns (codes uint8 [M, N], scales fp32 [M, ceil(N / block_size)]).
    """
    assert x.ndim == 2
    M, N = x.shape
    nb = (N + block_size - 1) // block_size
    x32 = x.detach().float()
    pad = nb * block_size - N
    xp = torch.nn.functional.pad(x32, (0, pad)) if pad else x32      # masked loads read 0.0 (:48)
    tiles = xp.reshape(M, nb, block_size)
    scale = _scale_from_amax(_nan_dropping_amax(tiles, -1), round_scale)   # (M, nb)
    q = _quantize_values(tiles, scale[:, :, None], encoder).reshape(M, nb * block_size)
    return q[:, :N].contiguous(), scale.contiguous()


def quantize_blockwise(x: torch.Tensor, block_m: int = 128, block_n: int = 128,
                       round_scale: bool = False, encoder: str = "torch"):
    """block_m x block_n tiles (src/kernels.py:74-132, 219-259).

    Returns (codes uint8 [M, N], scales fp32 [ceil(M/block_m), ceil(N/block_n)]).
    """
    assert x.ndim == 2
    M, N = x.shape
    mb = (M + block_m - 1) // block_m
    nb = (N + block_n - 1) // block_n
    x32 = x.detach().float()
    xp = torch.nn.functional.pad(x32, (0, nb * block_n - N, 0, mb * block_m - M))
    tiles = xp.reshape(mb, block_m, nb, block_n)
    scale = _scale_from_amax(_nan_dropping_amax(tiles, (1, 3)), round_scale)   # (mb, nb)
    q = _quantize_values(tiles, scale[:, None, :, None], encoder)
    q = q.reshape(mb * block_m, nb * block_n)
    return q[:M, :N].contiguous(), scale.contiguous()


def decode(codes: torch.Tensor) -> torch.Tensor:
    """uint8 e4m3 codes -> fp32 values (exact)."""
    return torch.from_numpy(_DECODE)[codes.long()]


def dequantize_rowwise(q: torch.Tensor, scales: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    """codes * per-tile scale in fp32 (src/kernels.py:262-281)."""
    M, N = q.shape
    nb = scales.shape[1]
    v = decode(q)
    s = scales.float().repeat_interleave(block_size, dim=1)[:, :N]
    return v * s


def dequantize_block(q: torch.Tensor, scales: torch.Tensor, block_m: int = 128, block_n: int = 128,
                     out_dtype=torch.bfloat16) -> torch.Tensor:
    """codes * per-block scale in fp32, rounded to bf16 (src/kernels.py:135-173, 284-314).

    ``scales`` is used flattened with row pitch ceil(N/block_n) (:164-166, :306).
    """
    M, N = q.shape
    mb = (M + block_m - 1) // block_m
    nb = (N + block_n - 1) // block_n
    s = scales.float().reshape(-1)[: mb * nb].reshape(mb, nb)
    s = s.repeat_interleave(block_m, dim=0)[:M].repeat_interleave(block_n, dim=1)[:, :N]
    return (decode(q) * s).to(out_dtype)


# ----------------------------------------------------------------------------
# GEMM oracle: float64 dequantise -> matmul (the tolerance reference)
# ----------------------------------------------------------------------------
def _expand_rows(scales: torch.Tensor, n: int, block: int = 128) -> torch.Tensor:
    return scales.double().repeat_interleave(block, dim=1)[:, :n]


def fp8_matmul_f64(a_q, b_q, a_scales, b_scales) -> torch.Tensor:
    """C = sum_kb (A_kb * sA[:, kb]) @ (B_kb * sB[kb, nb]) in float64.

    Operand meaning as ``fp8_matmul_dsv3`` (src/kernels.py:618-664, 667-702):
    a_q (M, K) codes with scales (M, ceil(K/128)); b_q (K, N) codes with
    scales (ceil(K/128), ceil(N/128)).
    """
    M, K = a_q.shape
    K2, N = b_q.shape
    assert K == K2
    a = decode(a_q).double() * _expand_rows(a_scales, K)
    sb = b_scales.double().repeat_interleave(128, dim=0)[:K].repeat_interleave(128, dim=1)[:, :N]
    b = decode(b_q).double() * sb
    return a @ b


def fp8_linear_forward(x: torch.Tensor, weight: torch.Tensor, round_scale: bool):
    """FP8MatmulFunction.forward (src/kernels.py:739-761) up to the fp64 product.

    Returns (out_f64 [M, N], saved) where saved = (x_q, x_s, w_q, w_s) as the
    reference saves them for backward (:758).
    """
    x_flat = x.reshape(-1, x.shape[-1])
    x_q, x_s = quantize_rowwise(x_flat, 128, round_scale)                 # :746
    w_q, w_s = quantize_blockwise(weight.float(), 128, 128)               # :747
    out = fp8_matmul_f64(x_q, w_q.t(), x_s, w_s.t())                      # :748-752
    return out, (x_q, x_s, w_q, w_s)


def fp8_linear_backward(grad_output: torch.Tensor, saved, round_scale: bool):
    """FP8MatmulFunction.backward, CUDA branch (src/kernels.py:763-794).

    dgrad: rowwise(dy) @ W (W's 128x128 scales used untransposed)  (:771-774)
    wgrad: rowwise(dy^T) @ blockwise(dequant_rowwise(x_q))          (:781-788)
    Returns (grad_x_f64 [M, K], grad_w_f64 [N, K]).
    """
    x_q, x_s, w_q, w_s = saved
    g = grad_output.reshape(-1, grad_output.shape[-1])
    g_q, g_s = quantize_rowwise(g, 128, round_scale)
    grad_x = fp8_matmul_f64(g_q, w_q, g_s, w_s)
    gt_q, gt_s = quantize_rowwise(g.t().contiguous(), 128, round_scale)
    x_deq = dequantize_rowwise(x_q, x_s, 128)
    xb_q, xb_s = quantize_blockwise(x_deq, 128, 128, round_scale=False)
    grad_w = fp8_matmul_f64(gt_q, xb_q, gt_s, xb_s)
    return grad_x, grad_w


def requantize_row_to_block(x_q: torch.Tensor, x_s: torch.Tensor):
    """The wgrad re-quantisation of x (src/kernels.py:784-787) on its own."""
    return quantize_blockwise(dequantize_rowwise(x_q, x_s, 128), 128, 128, round_scale=False)


# ----------------------------------------------------------------------------
# grouped GEMM
# ----------------------------------------------------------------------------
def grouped_gemm_f64(sorted_x: torch.Tensor, weights: torch.Tensor, starts, ends) -> torch.Tensor:
    """Unquantised per-expert product in float64 (src/kernels.py:466-523).

    C[s_e:e_e] = A[s_e:e_e] @ W_e^T.  Rows outside every expert's range stay 0
    (the reference leaves them uninitialised, :550).
    """
    T = sorted_x.shape[0]
    E, d_out, d_in = weights.shape
    out = torch.zeros(T, d_out, dtype=torch.float64)
    for e in range(E):
        s, t = int(starts[e]), int(ends[e])
        if t > s:
            out[s:t] = sorted_x[s:t].double() @ weights[e].double().t()
    return out


def grouped_gemm_fp8_f64(sorted_x: torch.Tensor, weights: torch.Tensor, starts, ends,
                         round_scale: bool = False) -> torch.Tensor:
    """FP8 block-scaled per-expert product in float64.

    Tokens are quantised in 1x128 tiles, each expert's (d_out, d_in) matrix in
    128x128 blocks, exactly as the dense path does (src/kernels.py:746-752);
    the product is the float64 dequantise -> matmul of those operands.
    """
    T = sorted_x.shape[0]
    E, d_out, d_in = weights.shape
    x_q, x_s = quantize_rowwise(sorted_x, 128, round_scale)
    out = torch.zeros(T, d_out, dtype=torch.float64)
    for e in range(E):
        s, t = int(starts[e]), int(ends[e])
        if t > s:
            w_q, w_s = quantize_blockwise(weights[e].float(), 128, 128)
            out[s:t] = fp8_matmul_f64(x_q[s:t], w_q.t(), x_s[s:t], w_s.t())
    return out


def grouped_gemm_fp8_backward_f64(sorted_x: torch.Tensor, weights: torch.Tensor, starts, ends, grad_out: torch.Tensor):
    """Backward of the FP8 grouped GEMM, expert by expert with the arithmetic of
    FP8MatmulFunction.backward (src/kernels.py:763-794); the reference itself defines no
    backward for its grouped GEMM.  Returns (dX float64 [T, d_in], dW float64 [E, d_out, d_in])."""
    T, d_in = sorted_x.shape
    E, d_out, _ = weights.shape
    x_q, x_s = quantize_rowwise(sorted_x, 128, False)
    dx = torch.zeros(T, d_in, dtype=torch.float64)
    dw = torch.zeros(E, d_out, d_in, dtype=torch.float64)
    for e in range(E):
        s, t = int(starts[e]), int(ends[e])
        if t <= s:
            continue
        w_q, w_s = quantize_blockwise(weights[e].float(), 128, 128)
        gx, gw = fp8_linear_backward(grad_out[s:t], (x_q[s:t], x_s[s:t], w_q, w_s), False)
        dx[s:t] = gx
        dw[e] = gw
    return dx, dw


# ----------------------------------------------------------------------------
# MoE routing (src/layers.py:118-160), used by the expert-parallel tests
# ----------------------------------------------------------------------------
def moe_route(x: torch.Tensor, router_w: torch.Tensor, expert_bias: torch.Tensor, top_k: int):
    """Router of MoE.forward: sigmoid scores, biased top-k, normalised gates,
    stable sort by expert (src/layers.py:122-148).

    Returns dict(token_indices, sorted_scores, starts, ends, counts).
    """
    scores = torch.sigmoid(x.float() @ router_w.float().t())
    _, top_idx = (scores + expert_bias).topk(top_k, dim=-1)
    top_scores = scores.gather(-1, top_idx)
    top_scores = top_scores / (top_scores.sum(dim=-1, keepdim=True) + 1e-9)
    expanded_idx = top_idx.reshape(-1)
    sorted_idx, order = expanded_idx.sort(stable=True)
    token_indices = order // top_k
    counts = torch.bincount(sorted_idx, minlength=router_w.shape[0])
    ends = counts.cumsum(0)
    starts = torch.cat([torch.zeros(1, dtype=torch.long), ends[:-1]])
    return dict(token_indices=token_indices, sorted_scores=top_scores.reshape(-1)[order],
                starts=starts, ends=ends, counts=counts)


def rel_fro(a: torch.Tensor, ref: torch.Tensor) -> float:
    """||a - ref||_F / ||ref||_F in float64."""
    a = a.double()
    ref = ref.double()
    return float((a - ref).norm() / ref.norm().clamp_min(1e-300))


# ----------------------------------------------------------------------------
# seeded workloads (shapes, sizes and value distributions of the benchmark
# configurations; generated on the CPU so checker and GPU see identical bits)
# ----------------------------------------------------------------------------
def make_linear_case(M: int, K: int, N: int, seed: int, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    dy = torch.randn(M, N, generator=g).to(dtype)
    return x, w, dy
