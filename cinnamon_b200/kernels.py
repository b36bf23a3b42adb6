"""Drop-in replacement for cinnamon's ``src/kernels.py`` on B200.

Same module-level names, argument meaning, return conventions and error
behaviour as the reference file (shyampathak22/cinnamon, src/kernels.py); the
GPU work is done by hand-written sm_100a kernels reached through the C ABI of
``libcinnamon_b200.so`` (include/cinnamon_b200.h).  There is no Triton import,
no backend dispatch and no CPU path: a CPU tensor raises ``AssertionError``
exactly where the reference asserts ``x.is_cuda``.

Differences a caller can observe, all deliberate:
  * ``FP8MatmulFunction`` feeds the GEMM the weight as stored, (N, K), instead of
    materialising ``w_fp8.t().contiguous()`` (reference :748-749); the weight
    gradient quantises ``dy`` along tokens straight from ``dy`` (no
    ``.t().contiguous()`` copy, reference :781-783) and re-quantises ``x`` in one
    fused pass (no fp32 temporary, reference :784-787).  Values are unchanged.
  * ``moe_grouped_gemm`` multiplies e4m3 operands with 1x128 / 128x128 scales (the
    reference multiplies in fp16); it still returns fp16 and accepts ``dtype=``.
  * the fp32 division flavour of the quantisers is selectable: ``"full"`` is the PTX
    ``div.full.f32`` Triton emits for the reference on a GPU (default), ``"rn"`` is
    IEEE division (what a CPU computes).  ``CINN_DIV_MODE`` or ``set_div_mode``.
"""
from __future__ import annotations

import ctypes
import os
import weakref

import torch

from . import _lib
from .sparse_attention import SparseAttentionFunction, sparse_attention  # noqa: F401

_L = _lib.lib
FP8_E4M3_MAX = 448.0

_DTYPE_TAG = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32, torch.float16: _lib.F16}
_DIV_MODE = {"full": _lib.DIV_FULL, "rn": _lib.DIV_RN}[os.environ.get("CINN_DIV_MODE", "full")]

# FP8MatmulFunction hands the dgrad / wgrad GEMMs operands with the reduction axis innermost (a transposed copy of
# the quantised weight and of the block-quantised activations, both written by the quantiser passes themselves).
# CINN_KMAJOR_BACKWARD=0 keeps the stored layouts and lets the GEMM read them (reduction, output).
_KMAJOR_BACKWARD = os.environ.get("CINN_KMAJOR_BACKWARD", "1") != "0"

# Arithmetic of the drop-in ``moe_grouped_gemm``: "fp8" = e4m3 operands with 1x128 / 128x128 scales (default: what this
# library is for), "16bit" = fp16 operands and fp32 accumulation, the reference kernel's own arithmetic
# (src/kernels.py:515-523).  CINN_MOE_GROUPED or ``set_moe_grouped_precision``.
_MOE_GROUPED_PRECISION = os.environ.get("CINN_MOE_GROUPED", "fp8")
assert _MOE_GROUPED_PRECISION in ("fp8", "16bit"), "CINN_MOE_GROUPED must be fp8 or 16bit"

# number of kernels of this library launched since import (the benchmark reports it)
launch_count = 0
# when set to a list, every GEMM launch appends a (start, end) pair of CUDA events to it
gemm_events = None


def set_div_mode(mode: str) -> None:
    """``"full"`` (div.full.f32, matches the reference's Triton kernels on a GPU) or
    ``"rn"`` (IEEE division, matches a CPU restatement)."""
    global _DIV_MODE
    _DIV_MODE = {"full": _lib.DIV_FULL, "rn": _lib.DIV_RN}[mode]


def set_moe_grouped_precision(mode: str) -> str:
    """``"fp8"`` or ``"16bit"`` for the drop-in ``moe_grouped_gemm`` (see ``_MOE_GROUPED_PRECISION``); returns the
    previous setting."""
    global _MOE_GROUPED_PRECISION
    assert mode in ("fp8", "16bit"), "precision must be 'fp8' or '16bit'"
    prev, _MOE_GROUPED_PRECISION = _MOE_GROUPED_PRECISION, mode
    return prev


def get_div_mode() -> str:
    return "full" if _DIV_MODE == _lib.DIV_FULL else "rn"


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


def device_status(reset: bool = True) -> int:
    """Device-side status word (0 = no kernel gave up on a bounded wait). Synchronises."""
    out = ctypes.c_int(0)
    _lib.check(_L.cinn_device_status(ctypes.byref(out), int(reset)), "cinn_device_status")
    return out.value


def selfcheck_division(device=None) -> int:
    """Number of (x, scale) pairs for which ``x * rcp.approx(scale)`` (what the ``full`` flavour computes, one
    reciprocal per scale) differs in bits from ``div.full.f32(x, scale)`` (what Triton emits for the reference's
    ``x / scale``, src/kernels.py:60, :121), over every positive bf16/fp16 amax, both scale kinds, every 16-bit
    x and 65536 fp32 patterns per scale.  0 on a GPU where the hoisting is exact."""
    n = ctypes.c_ulonglong(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(_L.cinn_selfcheck_division(ctypes.byref(n), stream), "cinn_selfcheck_division")
    _count(2)
    return int(n.value)


def _as_quant_input(x: torch.Tensor) -> torch.Tensor:
    if x.dtype not in _DTYPE_TAG:
        x = x.float()
    if x.stride(0) < 0 or x.stride(1) < 0:
        x = x.contiguous()
    return x


# -----------------------------------------------------------------------------
# quantisers (reference: src/kernels.py:178-314)
# -----------------------------------------------------------------------------
def quantize_fp8_rowwise(x: torch.Tensor, block_size: int = 128, round_scale: bool = False):
    """Row-wise 1 x block_size quantisation (reference src/kernels.py:178-216).

    Returns ``(x_fp8 [M, N] float8_e4m3fn, scales [M, ceil(N/block_size)] fp32)``,
    both freshly allocated and contiguous.  ``x`` may have any strides; a transposed
    view is read in place."""
    assert x.is_cuda, "Input must be on CUDA"
    assert x.ndim == 2, "Input must be 2D for now"
    x = _as_quant_input(x)
    M, N = x.shape
    nb = (N + block_size - 1) // block_size
    with torch.cuda.device(x.device):
        q = torch.empty((M, N), dtype=torch.float8_e4m3fn, device=x.device)
        s = torch.empty((M, nb), dtype=torch.float32, device=x.device)
        _lib.check(_L.cinn_quant_rowwise(_ptr(x), _DTYPE_TAG[x.dtype], M, N, x.stride(0), x.stride(1), _ptr(q),
                                         _ptr(s), block_size, int(bool(round_scale)), _DIV_MODE, _stream(x)),
                   "cinn_quant_rowwise")
    _count()
    return q, s


def quantize_fp8_rowwise_dual(x: torch.Tensor, round_scale: bool = False):
    """``quantize_fp8_rowwise(x)`` and ``quantize_fp8_rowwise(x.t())`` (1 x 128 tiles) from one pass over
    ``x``: the two quantisations of the output gradient in ``FP8MatmulFunction.backward`` (reference
    src/kernels.py:771 and :781-783).  Returns ``(q_row, s_row, q_col, s_col)`` with ``q_row`` (M, N),
    ``q_col`` (N, M); bit-identical to the two separate calls."""
    assert x.is_cuda, "Input must be on CUDA"
    assert x.ndim == 2, "Input must be 2D for now"
    x = _as_quant_input(x)
    if x.stride(1) != 1:
        x = x.contiguous()
    M, N = x.shape
    with torch.cuda.device(x.device):
        q_row = torch.empty((M, N), dtype=torch.float8_e4m3fn, device=x.device)
        s_row = torch.empty((M, (N + 127) // 128), dtype=torch.float32, device=x.device)
        q_col = torch.empty((N, M), dtype=torch.float8_e4m3fn, device=x.device)
        s_col = torch.empty((N, (M + 127) // 128), dtype=torch.float32, device=x.device)
        _lib.check(_L.cinn_quant_rowwise_dual(_ptr(x), _DTYPE_TAG[x.dtype], M, N, x.stride(0), _ptr(q_row), _ptr(s_row),
                                              _ptr(q_col), _ptr(s_col), int(bool(round_scale)), _DIV_MODE, _stream(x)),
                   "cinn_quant_rowwise_dual")
    _count()
    return q_row, s_row, q_col, s_col


def quantize_fp8_rowwise_with_block(x: torch.Tensor, round_scale: bool = False, transpose_block: bool = False):
    """``quantize_fp8_rowwise(x)`` together with ``quantize_fp8_blockwise(dequantize_fp8_rowwise(q, s))`` of its result
    (what ``FP8MatmulFunction`` computes in its forward, reference src/kernels.py:746, and on the saved activations in
    its backward, :784-787) from one pass over ``x``.  Returns ``(q_row, s_row, q_block, s_block)``; bit-identical to
    the separate calls.  The row length must be a multiple of 16.  ``transpose_block``: ``q_block`` comes out as
    (N, M) - the bytes of the block copy transposed, tokens contiguous (M a multiple of 16) - which is how the
    weight-gradient GEMM reads it K-major."""
    assert x.is_cuda, "Input must be on CUDA"
    assert x.ndim == 2, "Input must be 2D for now"
    x = _as_quant_input(x)
    if x.stride(1) != 1:
        x = x.contiguous()
    M, N = x.shape
    nb = (N + 127) // 128
    with torch.cuda.device(x.device):
        q_row = torch.empty((M, N), dtype=torch.float8_e4m3fn, device=x.device)
        s_row = torch.empty((M, nb), dtype=torch.float32, device=x.device)
        q_blk = torch.empty((N, M) if transpose_block else (M, N), dtype=torch.float8_e4m3fn, device=x.device)
        s_blk = torch.empty(((M + 127) // 128, nb), dtype=torch.float32, device=x.device)
        fn = _L.cinn_quant_rowwise_with_block_t if transpose_block else _L.cinn_quant_rowwise_with_block
        _lib.check(fn(_ptr(x), _DTYPE_TAG[x.dtype], M, N, x.stride(0), _ptr(q_row), _ptr(s_row),
                      _ptr(q_blk), _ptr(s_blk), int(bool(round_scale)), _DIV_MODE, _stream(x)),
                   "cinn_quant_rowwise_with_block")
    _count()
    return q_row, s_row, q_blk, s_blk


def quantize_fp8_blockwise(x: torch.Tensor, block_m: int = 128, block_n: int = 128, round_scale: bool = False):
    """Block-wise block_m x block_n quantisation (reference src/kernels.py:219-259).

    Returns ``(x_fp8 [M, N], scales [ceil(M/block_m), ceil(N/block_n)])``."""
    assert x.is_cuda, "Input must be on CUDA"
    assert x.ndim == 2, "Input must be 2D"
    x = _as_quant_input(x)
    M, N = x.shape
    mb, nb = (M + block_m - 1) // block_m, (N + block_n - 1) // block_n
    with torch.cuda.device(x.device):
        q = torch.empty((M, N), dtype=torch.float8_e4m3fn, device=x.device)
        s = torch.empty((mb, nb), dtype=torch.float32, device=x.device)
        _lib.check(_L.cinn_quant_blockwise(_ptr(x), _DTYPE_TAG[x.dtype], M, N, x.stride(0), x.stride(1), _ptr(q),
                                           _ptr(s), block_m, block_n, int(bool(round_scale)), _DIV_MODE, _stream(x)),
                   "cinn_quant_blockwise")
    _count()
    return q, s


def quantize_fp8_blockwise_t(x: torch.Tensor, round_scale: bool = False):
    """``quantize_fp8_blockwise(x)`` (128 x 128 blocks) that also returns the byte-transposed copy of the quantised
    matrix, from one pass over ``x``: ``(x_fp8 [M, N], scales, x_fp8_t [N, M])``.  The scales serve both copies
    (``scales.t()`` indexes the transposed one).  Replaces the reference's quantise + ``.t().contiguous()``
    (src/kernels.py:747-748).  M and N must be multiples of 4."""
    assert x.is_cuda, "Input must be on CUDA"
    assert x.ndim == 2, "Input must be 2D"
    x = _as_quant_input(x)
    if x.stride(1) != 1:
        x = x.contiguous()
    M, N = x.shape
    with torch.cuda.device(x.device):
        q = torch.empty((M, N), dtype=torch.float8_e4m3fn, device=x.device)
        q_t = torch.empty((N, M), dtype=torch.float8_e4m3fn, device=x.device)
        s = torch.empty(((M + 127) // 128, (N + 127) // 128), dtype=torch.float32, device=x.device)
        _lib.check(_L.cinn_quant_blockwise_t(_ptr(x), _DTYPE_TAG[x.dtype], M, N, x.stride(0), _ptr(q), _ptr(q_t), _ptr(s),
                                             int(bool(round_scale)), _DIV_MODE, _stream(x)), "cinn_quant_blockwise_t")
    _count()
    return q, s, q_t


def _dequant(x_fp8, scales, block_m, block_n, out_dtype):
    M, N = x_fp8.shape
    x_fp8 = x_fp8.contiguous()
    scales = scales.contiguous().float()
    with torch.cuda.device(x_fp8.device):
        out = torch.empty((M, N), dtype=out_dtype, device=x_fp8.device)
        _lib.check(_L.cinn_dequant(_ptr(x_fp8), _ptr(scales), _ptr(out), _DTYPE_TAG[out_dtype], M, N, block_m, block_n,
                                   _stream(x_fp8)), "cinn_dequant")
    _count()
    return out


def dequantize_fp8_rowwise(x_fp8: torch.Tensor, scales: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    """fp32 = e4m3 * per-tile scale (reference src/kernels.py:262-281, pure torch there)."""
    assert x_fp8.is_cuda, "Input must be on CUDA"
    return _dequant(x_fp8, scales, 1, block_size, torch.float32)


def dequantize_fp8(x_fp8: torch.Tensor, scales: torch.Tensor, block_m: int = 128, block_n: int = 128) -> torch.Tensor:
    """bf16 = e4m3 * per-block scale (reference src/kernels.py:284-314).  ``scales`` is
    used flattened with row pitch ceil(N/block_n), so ``block_m=1`` de-quantises
    row-wise scales as the reference's round-trip test does (tests/test_kernels.py:57)."""
    assert x_fp8.is_cuda, "Input must be on CUDA"
    return _dequant(x_fp8, scales.flatten(), block_m, block_n, torch.bfloat16)


def requantize_rowwise_to_blockwise(x_fp8: torch.Tensor, x_scale: torch.Tensor, transpose_out: bool = False):
    """Fused ``quantize_fp8_blockwise(dequantize_fp8_rowwise(x_fp8, x_scale))`` (reference
    src/kernels.py:784-787) without the fp32 temporary.  Returns block-scaled bytes
    (M, K) - or (K, M) with ``transpose_out`` - and scales (ceil(M/128), ceil(K/128))."""
    assert x_fp8.is_cuda, "Input must be on CUDA"
    M, K = x_fp8.shape
    x_fp8 = x_fp8.contiguous()
    x_scale = x_scale.contiguous()
    with torch.cuda.device(x_fp8.device):
        out = torch.empty((K, M) if transpose_out else (M, K), dtype=torch.float8_e4m3fn, device=x_fp8.device)
        s = torch.empty(((M + 127) // 128, (K + 127) // 128), dtype=torch.float32, device=x_fp8.device)
        _lib.check(_L.cinn_requant_row_to_block(_ptr(x_fp8), _ptr(x_scale), M, K, _ptr(out), _ptr(s),
                                                int(transpose_out), _DIV_MODE, _stream(x_fp8)),
                   "cinn_requant_row_to_block")
    _count()
    return out, s


def transpose_fp8(x_fp8: torch.Tensor) -> torch.Tensor:
    """``x_fp8.t().contiguous()`` of a 2-D e4m3 (or uint8) tensor as one byte-transposing pass (the reference makes
    such copies with torch, src/kernels.py:748).  Block scales of a 128x128-quantised matrix are those of its
    transpose with the two indices swapped, so a transposed weight needs no second quantisation."""
    assert x_fp8.is_cuda and x_fp8.ndim == 2 and x_fp8.element_size() == 1
    if x_fp8.stride(1) != 1:
        x_fp8 = x_fp8.contiguous()
    R, C = x_fp8.shape
    with torch.cuda.device(x_fp8.device):
        out = torch.empty((C, R), dtype=x_fp8.dtype, device=x_fp8.device)
        _lib.check(_L.cinn_transpose_bytes(_ptr(x_fp8), x_fp8.stride(0), _ptr(out), R, C, _stream(x_fp8)),
                   "cinn_transpose_bytes")
    _count()
    return out


# -----------------------------------------------------------------------------
# GEMM (reference: src/kernels.py:667-702)
# -----------------------------------------------------------------------------
def _gemm(a, a_scales, b, b_layout, sb, sb_stride_k, sb_stride_n, M, N, K, out_dtype, bf16_rounded=False, out=None):
    """``bf16_rounded`` (fp32 output only): store the result rounded to bf16, i.e. exactly what a
    bf16 result cast to fp32 would hold.  ``out``: a contiguous (M, N) tensor of ``out_dtype`` to write into."""
    with torch.cuda.device(a.device):
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        else:
            assert out.shape == (M, N) and out.dtype == out_dtype and out.is_contiguous()
        tag = _lib.F32_BF16 if (bf16_rounded and out_dtype == torch.float32) else _DTYPE_TAG[out_dtype]
        ev = None
        if gemm_events is not None:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        _lib.check(_L.cinn_fp8_gemm(_ptr(a), _ptr(a_scales), a_scales.stride(0), _ptr(b), _ptr(sb), sb_stride_k,
                                    sb_stride_n, _ptr(out), M, N, K, b_layout, tag, _stream(a)),
                   "cinn_fp8_gemm")
        if ev is not None:
            ev[1].record()
            gemm_events.append(ev)
    _count()
    return out


def fp8_matmul_dsv3(a: torch.Tensor, b: torch.Tensor, a_scales: torch.Tensor, b_scales: torch.Tensor,
                    out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """C = A @ B with DeepSeek-V3 scaling (reference src/kernels.py:667-702).

    a: (M, K) e4m3; b: (K, N) e4m3 with any strides (a ``.t()`` view of an (N, K)
    weight is consumed in place); a_scales: (M, ceil(K/128)); b_scales:
    (ceil(K/128), ceil(N/128)).  fp32 accumulation, bf16 result (``out_dtype`` may
    ask for fp32)."""
    assert a.is_cuda and b.is_cuda, "Inputs must be on CUDA"
    M, K = a.shape
    K2, N = b.shape
    assert K == K2, f"Dimension mismatch: {K} vs {K2}"
    if a.stride(1) != 1 or a.stride(0) != K:
        a = a.contiguous()
    if a_scales.stride(1) != 1:
        a_scales = a_scales.contiguous()
    if b.stride(0) == 1 and b.stride(1) == K:          # (N, K) storage seen through .t()
        layout = _lib.B_NK
    elif b.stride(1) == 1 and b.stride(0) == N:
        layout = _lib.B_KN
    else:
        b = b.contiguous()
        layout = _lib.B_KN
    return _gemm(a, a_scales.float(), b, layout, b_scales, b_scales.stride(0), b_scales.stride(1), M, N, K, out_dtype)


def _fp8_quantize_tensor(x: torch.Tensor):
    """Per-tensor quantisation helper kept for name compatibility (reference :705-713, unused there)."""
    abs_max = x.abs().max().clamp(min=1e-12)
    scale = abs_max / 448.0
    x_fp8 = (x / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    return x_fp8, scale.float().reshape(1).to(x.device)


def _pad_to_multiple(x: torch.Tensor, multiple: int = 16):
    """Reference :716-723 (unused there)."""
    M, K = x.shape
    pad_m = (multiple - M % multiple) % multiple
    pad_k = (multiple - K % multiple) % multiple
    if pad_m > 0 or pad_k > 0:
        x = torch.nn.functional.pad(x, (0, pad_k, 0, pad_m))
    return x, (M, K)


def _unpad(x: torch.Tensor, orig_shape):
    """Reference :726-728 (unused there)."""
    return x[:orig_shape[0], :orig_shape[1]]


class FP8MatmulFunction(torch.autograd.Function):
    """DeepSeek-V3 style FP8 matmul (reference src/kernels.py:731-794):
    activations / gradients 1x128, weights 128x128, e4m3 everywhere."""

    @staticmethod
    def forward(ctx, x, weight, round_scale, weight_fp8=None):
        """``weight_fp8``: optional ``(w_fp8, w_scale)`` or ``(w_fp8, w_scale, w_fp8_t)`` of this very weight
        (``quantize_fp8_blockwise``, ``transpose_fp8``), for callers that quantise a weight once per optimiser step
        instead of once per call; the reference's three-argument call re-quantises every time (:747)."""
        assert x.is_cuda, "Input must be on CUDA"
        x_shape = x.shape
        x_flat = x.reshape(-1, x_shape[-1])
        M, K = x_flat.shape
        N = weight.shape[0]
        # :746; when the weight will want a gradient, the block re-quantisation of the saved activations that the
        # backward needs (:784-787) comes out of the same pass over x and is what gets saved
        want_wgrad = ctx.needs_input_grad[1] and K % 16 == 0
        # the block copy is written with the token axis contiguous: the weight gradient reduces over tokens, and both
        # of its operands are then K-major like the forward's (tensor-core operand reads are fastest that way)
        x_blk_t = want_wgrad and M % 16 == 0 and _KMAJOR_BACKWARD
        if want_wgrad:
            x_fp8, x_scale, x_blk, x_blk_scale = quantize_fp8_rowwise_with_block(x_flat, round_scale=round_scale,
                                                                                 transpose_block=x_blk_t)
        else:
            x_fp8, x_scale = quantize_fp8_rowwise(x_flat, block_size=128, round_scale=round_scale)
        ctx.w_fp8_t = None
        if weight_fp8 is not None:
            w_fp8, w_scale = weight_fp8[0], weight_fp8[1]
            ctx.w_fp8_t = weight_fp8[2] if len(weight_fp8) > 2 else None
        else:
            w_in = weight.float() if weight.dtype not in _DTYPE_TAG else weight
            if (_KMAJOR_BACKWARD and ctx.needs_input_grad[0] and N % 16 == 0 and K % 4 == 0 and w_in.stride(1) == 1
                    and w_in.stride(0) % 4 == 0):
                # the input gradient multiplies by the weight with N as the reduction axis: the byte-transposed
                # copy it reads comes out of the same pass (:747-748)
                w_fp8, w_scale, ctx.w_fp8_t = quantize_fp8_blockwise_t(w_in)
            else:
                w_fp8, w_scale = quantize_fp8_blockwise(w_in, block_m=128, block_n=128)              # :747
        ctx.n_inputs = 3 if weight_fp8 is None else 4
        # :748-752 without the transposed copies: B stays (N, K); sB[kb, nb] = w_scale[nb, kb]
        out = _gemm(x_fp8, x_scale, w_fp8, _lib.B_NK, w_scale, w_scale.stride(1), w_scale.stride(0), M, N, K,
                    torch.bfloat16)
        if want_wgrad:
            ctx.save_for_backward(x_blk, x_blk_scale, w_fp8, w_scale)
        else:
            ctx.save_for_backward(x_fp8, x_scale, w_fp8, w_scale)
        ctx.x_is_block = want_wgrad
        ctx.x_is_block_t = x_blk_t
        ctx.x_shape = x_shape
        ctx.round_scale = round_scale
        ctx.weight_dtype = weight.dtype
        return out.reshape(*x_shape[:-1], -1)

    @staticmethod
    def backward(ctx, grad_output):
        x_fp8, x_scale, w_fp8, w_scale = ctx.saved_tensors
        x_shape = ctx.x_shape
        round_scale = ctx.round_scale
        N, K = w_fp8.shape
        grad_flat = grad_output.reshape(-1, grad_output.shape[-1])
        if grad_flat.stride(1) != 1:
            grad_flat = grad_flat.contiguous()
        M = grad_flat.shape[0]
        # The token axis is the reduction axis of the weight gradient; the GEMM wants it in multiples
        # of 16, so a ragged token count is padded with zero rows (they change neither an amax nor a sum).
        Mp = (M + 15) // 16 * 16
        if Mp != M:                                        # (never with a transposed block copy: that needs M % 16 == 0)
            grad_flat = torch.nn.functional.pad(grad_flat, (0, 0, 0, Mp - M))
            x_fp8 = torch.nn.functional.pad(x_fp8.view(torch.uint8), (0, 0, 0, Mp - M)).view(torch.float8_e4m3fn)
            if not ctx.x_is_block:                         # block scales: zero rows stay inside the last row block
                x_scale = torch.nn.functional.pad(x_scale, (0, 0, 0, Mp - M), value=1.0)
        # dy quantised along features for dgrad (:771) and along tokens for wgrad (:781-783), one pass over dy
        grad_fp8, grad_scale, grad_fp8_t, grad_scale_t = quantize_fp8_rowwise_dual(grad_flat, round_scale=round_scale)
        # dgrad (:771-774): dy (M, N) @ W (N, K).  W is the B operand with the reduction axis N; a byte-transposed
        # copy (K, N) puts that axis innermost (the block scales are shared, indices swapped), otherwise the stored
        # bytes are read (reduction, output)
        if N % 16 == 0 and (_KMAJOR_BACKWARD or ctx.w_fp8_t is not None):
            w_t = ctx.w_fp8_t if ctx.w_fp8_t is not None else transpose_fp8(w_fp8)
            grad_x = _gemm(grad_fp8, grad_scale, w_t, _lib.B_NK, w_scale, w_scale.stride(0), w_scale.stride(1), M, K, N,
                           torch.bfloat16)
        else:
            grad_x = _gemm(grad_fp8, grad_scale, w_fp8, _lib.B_KN, w_scale, w_scale.stride(0), w_scale.stride(1), M, K, N,
                           torch.bfloat16)
        # wgrad (:781-788): x re-quantised in 128x128 blocks
        if ctx.x_is_block:
            x_fp8_block, x_scale_block = x_fp8, x_scale            # made by the forward's pass over x
        else:
            x_fp8_block, x_scale_block = requantize_rowwise_to_blockwise(x_fp8, x_scale)
        # the reference returns a bf16 grad_weight which autograd then casts to the fp32 master
        # weight's dtype (:788, :794); the GEMM writes those same values as fp32 directly
        ctx_w_fp32 = ctx.weight_dtype == torch.float32
        grad_weight = _gemm(grad_fp8_t, grad_scale_t, x_fp8_block, _lib.B_NK if ctx.x_is_block_t else _lib.B_KN,
                            x_scale_block, x_scale_block.stride(0), x_scale_block.stride(1), N, K, Mp,
                            torch.float32 if ctx_w_fp32 else torch.bfloat16, bf16_rounded=True)
        return (grad_x.reshape(x_shape), grad_weight, None) + (None,) * (ctx.n_inputs - 3)


class FP8Linear(torch.nn.Module):
    """FP8 Linear layer (reference src/kernels.py:797-840): fp32 master weight,
    bias added after the matmul, ``round_scale`` applied to activations and gradients."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, round_scale: bool = False,
                 cache_quantized_weight: bool = False):
        """``cache_quantized_weight`` (not in the reference, off by default): keep the e4m3 copy of the weight until
        the weight changes (an in-place optimiser update bumps its version), so the micro-steps of a gradient
        accumulation quantise it once instead of once each.  An update made through ``weight.data`` leaves the
        version counter untouched: call ``invalidate_weight_cache(model)`` after one."""
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.round_scale = round_scale
        self.cache_quantized_weight = cache_quantized_weight
        self._w_cache = (None, None)
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features))
        torch.nn.init.normal_(self.weight, mean=0.0, std=0.02)
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda and self.cache_quantized_weight:
            w = self.weight
            key = (w._version, w.data_ptr(), w.dtype)
            if self._w_cache[0] != key:
                with torch.no_grad():
                    wf = w.float() if w.dtype not in _DTYPE_TAG else w
                    # the input gradient reads the weight transposed; cached with it when that copy can be made
                    if w.shape[0] % 16 == 0 and w.shape[1] % 4 == 0:
                        q, s, q_t = quantize_fp8_blockwise_t(wf)
                        self._w_cache = (key, (q, s, q_t))
                    else:
                        self._w_cache = (key, quantize_fp8_blockwise(wf, 128, 128))
            out = FP8MatmulFunction.apply(x, w, self.round_scale, self._w_cache[1])
        elif x.is_cuda and _ops is not None and torch.compiler.is_compiling():
            out = _ops.fp8_linear(x, self.weight, self.round_scale)       # one opaque graph node under torch.compile
        elif x.is_cuda:
            out = FP8MatmulFunction.apply(x, self.weight, self.round_scale)
        else:
            # the reference does the same: an unquantised linear on CPU tensors (:823-824)
            out = torch.nn.functional.linear(x, self.weight, None)
        if self.bias is not None:
            out = out + self.bias
        return out

    @classmethod
    def from_linear(cls, linear: torch.nn.Linear, round_scale: bool = False) -> "FP8Linear":
        fp8_linear = cls(linear.in_features, linear.out_features, bias=linear.bias is not None,
                         round_scale=round_scale)
        fp8_linear.weight = torch.nn.Parameter(linear.weight.data.clone())
        if linear.bias is not None:
            fp8_linear.bias = torch.nn.Parameter(linear.bias.data.clone())
        return fp8_linear


def convert_to_fp8(model: torch.nn.Module, exclude_names: list = None) -> torch.nn.Module:
    """Swap eligible ``nn.Linear`` modules for ``FP8Linear`` in place (reference
    src/kernels.py:843-905): names containing embedding / lm_head / router / norm /
    attn / indexer are kept, as is any layer with a dimension below 128; ``round_scale``
    is switched on for names containing w_out, w1 or w2."""
    default_exclude = ["embedding", "lm_head", "router", "norm", "attn", "indexer"]
    exclude_names = (exclude_names or []) + default_exclude
    round_scale_names = ["w_out", "w1", "w2"]
    for name, module in list(model.named_modules()):
        if not isinstance(module, torch.nn.Linear):
            continue
        if any(excl in name for excl in exclude_names):
            continue
        if module.in_features < 128 or module.out_features < 128:
            print(f"[FP8] Auto-excluding {name}: shape ({module.out_features}, {module.in_features}) < 128")
            continue
        parts = name.rsplit(".", 1)
        if len(parts) == 2:
            parent = model.get_submodule(parts[0])
            attr_name = parts[1]
        else:
            parent, attr_name = model, name
        round_scale = any(key in name for key in round_scale_names)
        setattr(parent, attr_name, FP8Linear.from_linear(module, round_scale=round_scale))
    return model


# -----------------------------------------------------------------------------
# MoE grouped GEMM (reference: src/kernels.py:526-581)
# -----------------------------------------------------------------------------
def quantize_expert_weights(weights: torch.Tensor):
    """(E, d_out, d_in) -> e4m3 bytes of the same shape + scales (E, ceil(d_out/128), ceil(d_in/128)).
    Each expert's matrix is quantised in 128x128 blocks like a dense weight (reference :747)."""
    assert weights.is_cuda and weights.ndim == 3
    E, d_out, d_in = weights.shape
    w = weights if weights.dtype in _DTYPE_TAG else weights.float()
    w = w.contiguous()
    nob, nkb = (d_out + 127) // 128, (d_in + 127) // 128
    if d_out % 128 == 0:
        q, s = quantize_fp8_blockwise(w.view(E * d_out, d_in))
        return q.view(E, d_out, d_in), s.view(E, nob, nkb)
    q = torch.empty((E, d_out, d_in), dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((E, nob, nkb), dtype=torch.float32, device=w.device)
    for e in range(E):
        qe, se = quantize_fp8_blockwise(w[e])
        q[e], s[e] = qe, se
    return q, s


# e4m3 copies of expert weight stacks, kept while the weight tensor lives and until it changes
_EXPERT_WEIGHT_CACHE = {}           # id(weight tensor) -> (key, e4m3 bytes, scales); entries leave with their tensor


def cached_expert_weights(weights: torch.Tensor):
    """``quantize_expert_weights(weights)``, remembered per weight tensor until the tensor changes: the key is the
    tensor's version counter (every in-place update through the tensor itself bumps it: optimiser steps,
    ``load_state_dict``, DDP's parameter broadcast), its storage address and dtype.  At the MoE benchmark's size a
    call would otherwise re-read and re-quantise 22.5 GB of expert weights.  An update made through ``weights.data``
    does not bump the counter: call ``invalidate_weight_cache()`` after such an update."""
    key = (weights._version, weights.data_ptr(), weights.dtype, tuple(weights.shape))
    ident = id(weights)
    hit = _EXPERT_WEIGHT_CACHE.get(ident)
    if hit is not None and hit[0] == key:
        return hit[1], hit[2]
    with torch.no_grad():
        q, s = quantize_expert_weights(weights.detach())
    if hit is None:
        weakref.finalize(weights, _EXPERT_WEIGHT_CACHE.pop, ident, None)
    _EXPERT_WEIGHT_CACHE[ident] = (key, q, s)
    return q, s


def invalidate_weight_cache(module: torch.nn.Module = None) -> None:
    """Drops every cached e4m3 weight copy (expert stacks of ``moe_grouped_gemm``; with ``module`` also the caches of
    its ``FP8Linear(cache_quantized_weight=True)`` layers).  Needed only after weights were changed behind autograd's
    back (``p.data.copy_(...)``, ``p.data.add_(...)``), which leaves the version counter untouched."""
    _EXPERT_WEIGHT_CACHE.clear()
    if module is not None:
        for m in module.modules():
            if isinstance(m, FP8Linear):
                m._w_cache = (None, None)


def fp8_grouped_gemm(x_fp8, x_scale, w_fp8, w_scale, expert_starts, expert_ends, out_dtype=torch.float16,
                     out: torch.Tensor = None):
    """Grouped GEMM on already-quantised operands.  Rows outside every expert's range are
    left as allocated (the reference leaves them uninitialised too, :550)."""
    T, d_in = x_fp8.shape
    E, d_out, _ = w_fp8.shape
    starts = expert_starts.to(torch.int64).contiguous()
    ends = expert_ends.to(torch.int64).contiguous()
    with torch.cuda.device(x_fp8.device):
        if out is None:
            out = torch.empty((T, d_out), dtype=out_dtype, device=x_fp8.device)
        _lib.check(_L.cinn_fp8_grouped_gemm(_ptr(x_fp8), _ptr(x_scale), _ptr(w_fp8), _ptr(w_scale), _ptr(starts),
                                            _ptr(ends), E, T, d_in, d_out, _ptr(out), _DTYPE_TAG[out.dtype],
                                            _stream(x_fp8)), "cinn_fp8_grouped_gemm")
    _count()
    return out


def fp8_grouped_gemm_scatter(x_fp8, x_scale, w_fp8, w_scale, expert_starts, expert_ends, row_dst: torch.Tensor,
                             out_dtype=torch.bfloat16) -> None:
    """The grouped GEMM with every finished output row stored at the byte address ``row_dst[r]`` (int64 device
    tensor, one entry per row, 0 = drop), which may lie in a peer GPU's memory (``cinn_fp8_grouped_gemm_scatter``)."""
    T, d_in = x_fp8.shape
    E, d_out, _ = w_fp8.shape
    assert row_dst.dtype == torch.int64 and row_dst.numel() == T, "row_dst: one int64 byte address per row"
    starts = expert_starts.to(torch.int64).contiguous()
    ends = expert_ends.to(torch.int64).contiguous()
    with torch.cuda.device(x_fp8.device):
        _lib.check(_L.cinn_fp8_grouped_gemm_scatter(_ptr(x_fp8), _ptr(x_scale), _ptr(w_fp8), _ptr(w_scale), _ptr(starts),
                                                    _ptr(ends), E, T, d_in, d_out, _ptr(row_dst), _DTYPE_TAG[out_dtype],
                                                    _stream(x_fp8)), "cinn_fp8_grouped_gemm_scatter")
    _count()


def p2p_row_table(seg_start, home_base, peer_home, n_rows: int, row_bytes: int, n_ranks: int, capacity_rows: int) -> torch.Tensor:
    """Byte address, on the rank it goes home to, of every row of this rank's expert-grouped outputs
    (``cinn_p2p_row_table``): the ``row_dst`` of ``fp8_grouped_gemm_scatter``."""
    with torch.cuda.device(seg_start.device):
        table = torch.empty(max(n_rows, 1), dtype=torch.int64, device=seg_start.device)[:n_rows]
        _lib.check(_L.cinn_p2p_row_table(_ptr(seg_start), _ptr(home_base), _ptr(peer_home), n_rows, row_bytes,
                                         home_base.numel(), n_ranks, capacity_rows, _ptr(table), _stream(seg_start)),
                   "cinn_p2p_row_table")
    _count()
    return table


def swiglu_quantize_rowwise(h12: torch.Tensor, n_rows_dev: torch.Tensor = None):
    """``h = (silu(h1) * h2).to(h12.dtype)`` with ``h1, h2 = h12.float().chunk(2, -1)`` (reference
    src/layers.py:72-74), quantised row-wise in 1x128 tiles, in one pass.
    Returns ``(h_fp8 [T, I], scales [T, ceil(I/128)])``.  ``n_rows_dev`` (int64 device scalar, optional): only
    that many leading rows hold data; the others are neither read nor written."""
    assert h12.is_cuda and h12.ndim == 2 and h12.shape[1] % 2 == 0
    h12 = h12.contiguous()
    T, I2 = h12.shape
    I = I2 // 2
    with torch.cuda.device(h12.device):
        q = torch.empty((T, I), dtype=torch.float8_e4m3fn, device=h12.device)
        s = torch.empty((T, (I + 127) // 128), dtype=torch.float32, device=h12.device)
        if n_rows_dev is None:
            _lib.check(_L.cinn_swiglu_quant_rowwise(_ptr(h12), _DTYPE_TAG[h12.dtype], T, I, _ptr(q), _ptr(s), _DIV_MODE,
                                                    _stream(h12)), "cinn_swiglu_quant_rowwise")
        else:
            assert n_rows_dev.dtype == torch.int64 and n_rows_dev.is_cuda
            _lib.check(_L.cinn_swiglu_quant_rowwise_n(_ptr(h12), _DTYPE_TAG[h12.dtype], T, I, _ptr(n_rows_dev), _ptr(q),
                                                      _ptr(s), _DIV_MODE, _stream(h12)), "cinn_swiglu_quant_rowwise_n")
    _count()
    return q, s


class SwiGLUFunction(torch.autograd.Function):
    """``h = (silu(h1) * h2).to(h12.dtype)`` with ``h1, h2 = h12.float().chunk(2, -1)`` (the step between the two
    expert GEMMs, reference src/layers.py:71-74) with its backward, one kernel each: the training-path sibling of
    ``swiglu_quantize_rowwise``."""

    @staticmethod
    def forward(ctx, h12):
        assert h12.is_cuda and h12.shape[-1] % 2 == 0, "Input must be on CUDA with an even last dimension"
        shape = h12.shape
        flat = h12.reshape(-1, shape[-1])
        flat = flat.contiguous() if flat.dtype in _DTYPE_TAG else flat.float().contiguous()
        T, I = flat.shape[0], flat.shape[1] // 2
        with torch.cuda.device(flat.device):
            h = torch.empty((T, I), dtype=flat.dtype, device=flat.device)
            _lib.check(_L.cinn_swiglu(_ptr(flat), _ptr(h), _DTYPE_TAG[flat.dtype], T, I, _stream(flat)), "cinn_swiglu")
        _count()
        ctx.save_for_backward(flat)
        ctx.shape, ctx.in_dtype = shape, h12.dtype
        return h.reshape(*shape[:-1], I).to(h12.dtype)

    @staticmethod
    def backward(ctx, grad_h):
        (flat,) = ctx.saved_tensors
        T, I = flat.shape[0], flat.shape[1] // 2
        g = grad_h.reshape(T, I).to(flat.dtype).contiguous()
        with torch.cuda.device(flat.device):
            grad = torch.empty_like(flat)
            _lib.check(_L.cinn_swiglu_backward(_ptr(flat), _ptr(g), _ptr(grad), _DTYPE_TAG[flat.dtype], T, I, _stream(flat)),
                       "cinn_swiglu_backward")
        _count()
        return grad.reshape(ctx.shape).to(ctx.in_dtype)


def swiglu(h12: torch.Tensor) -> torch.Tensor:
    """Differentiable ``silu(h12[..., :I]) * h12[..., I:]`` (reference src/layers.py:71-74) on the CUDA kernels."""
    return SwiGLUFunction.apply(h12)


def moe_combine(rows: torch.Tensor, pos: torch.Tensor, gates: torch.Tensor, addend: torch.Tensor = None) -> torch.Tensor:
    """``y[t] = sum_j gates[t, j] * rows[pos[t, j]]`` in fp32: the gate multiply + scatter-add of
    ``MoE.forward`` (reference src/layers.py:157-160) as one gather pass without atomics.
    rows (R, d) bf16/fp16/fp32, pos (T, k) int64 (negative = skip), gates (T, k) fp32.
    ``addend`` (T, d), optional: the shared experts' output, added to the routed sum in the same pass
    (``shared_out + routed_out``, src/layers.py:179)."""
    assert rows.is_cuda and pos.is_cuda and gates.is_cuda, "Inputs must be on CUDA"
    T, k = pos.shape
    rows = rows.contiguous()
    pos = pos.to(torch.int64).contiguous()
    gates = gates.float().contiguous()
    d = rows.shape[1]
    with torch.cuda.device(rows.device):
        y = torch.empty((T, d), dtype=torch.float32, device=rows.device)
        if addend is None:
            _lib.check(_L.cinn_moe_combine(_ptr(rows), _DTYPE_TAG[rows.dtype], _ptr(pos), _ptr(gates), _ptr(y), T,
                                           rows.shape[0], k, d, _stream(rows)), "cinn_moe_combine")
        else:
            assert addend.shape == (T, d), f"addend must be ({T}, {d})"
            if addend.dtype not in _DTYPE_TAG:
                addend = addend.float()
            addend = addend.contiguous()
            _lib.check(_L.cinn_moe_combine_add(_ptr(rows), _DTYPE_TAG[rows.dtype], _ptr(pos), _ptr(gates), _ptr(addend),
                                               _DTYPE_TAG[addend.dtype], _ptr(y), T, rows.shape[0], k, d, _stream(rows)),
                       "cinn_moe_combine_add")
    _count()
    return y


class MoECombineFunction(torch.autograd.Function):
    """``moe_combine`` with its backward (one kernel each): gradients for the expert outputs, the gates and the
    addend.  The reference's gate multiply + ``scatter_add_`` (src/layers.py:157-160) is differentiated by autograd;
    this is the same derivative for the fused gather pass."""

    @staticmethod
    def forward(ctx, rows, pos, gates, addend):
        y = moe_combine(rows.detach(), pos, gates.detach(), None if addend is None else addend.detach())
        ctx.save_for_backward(rows, pos, gates)
        ctx.addend_dtype = None if addend is None else addend.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        rows, pos, gates = ctx.saved_tensors
        T, k = pos.shape
        dy = dy.float().contiguous()
        rows_c = rows.contiguous()
        pos_c, gates_c = pos.to(torch.int64).contiguous(), gates.float().contiguous()
        with torch.cuda.device(rows.device):
            d_rows = torch.zeros_like(rows_c)
            d_gates = torch.empty((T, k), dtype=torch.float32, device=rows.device)
            _lib.check(_L.cinn_moe_combine_backward(_ptr(rows_c), _DTYPE_TAG[rows_c.dtype], _ptr(pos_c), _ptr(gates_c), _ptr(dy),
                                                    _ptr(d_rows), _ptr(d_gates), T, rows_c.shape[0], k, rows_c.shape[1],
                                                    _stream(rows_c)), "cinn_moe_combine_backward")
        _count()
        d_add = None if ctx.addend_dtype is None else dy.to(ctx.addend_dtype)
        return d_rows, None, d_gates.to(gates.dtype), d_add


def moe_combine_autograd(rows, pos, gates, addend=None):
    """Differentiable ``moe_combine`` (gradients reach ``rows``, ``gates`` and ``addend``)."""
    return MoECombineFunction.apply(rows, pos, gates, addend)


def lightning_indexer_fused(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Lightning indexer logits (reference src/kernels.py:392-433):
    ``I[b, t, s] = sum_h relu(q[b, t, h] . k[b, s]) * w[b, t, h]``, dot-product operands rounded to fp16,
    fp32 accumulation, fp16 result.  q (B, Lq, H, d), k (B, Lk, d), w (B, Lq, H), any strides."""
    assert q.is_cuda and k.is_cuda, "Inputs must be on CUDA"
    B, Lq, H, d = q.shape
    Lk = k.shape[1]
    work = q.dtype if q.dtype in _DTYPE_TAG else torch.float32
    q, k, w = q.to(work), k.to(work), w.to(work)
    with torch.cuda.device(q.device):
        out = torch.empty((B, Lq, Lk), dtype=torch.float16, device=q.device)
        sq = (ctypes.c_int64 * 4)(*q.stride())
        sk = (ctypes.c_int64 * 3)(*k.stride())
        sw = (ctypes.c_int64 * 3)(*w.stride())
        _lib.check(_L.cinn_lightning_indexer(_ptr(q), _ptr(k), _ptr(w), _DTYPE_TAG[work], _ptr(out), B, Lq, Lk, H, d,
                                             sq, sk, sw, _stream(q)), "cinn_lightning_indexer")
    _count()
    return out


def gather_quantized_rows(x_fp8: torch.Tensor, x_scale: torch.Tensor, idx: torch.Tensor):
    """``(x_fp8[idx], x_scale[idx])`` in one pass: the dispatch gather of ``MoE.forward``
    (reference src/layers.py:140) on tokens quantised once before the gather."""
    assert x_fp8.is_cuda and x_scale.is_cuda and idx.is_cuda, "Inputs must be on CUDA"
    n_src, d = x_fp8.shape
    x_fp8, x_scale = x_fp8.contiguous(), x_scale.float().contiguous()
    idx = idx.to(torch.int64).contiguous()
    n_out, ns = idx.numel(), x_scale.shape[1]
    if d % 16 != 0:
        return x_fp8.view(torch.uint8).index_select(0, idx).view(x_fp8.dtype), x_scale.index_select(0, idx)
    with torch.cuda.device(x_fp8.device):
        out_q = torch.empty((n_out, d), dtype=x_fp8.dtype, device=x_fp8.device)
        out_s = torch.empty((n_out, ns), dtype=torch.float32, device=x_fp8.device)
        _lib.check(_L.cinn_gather_rows(_ptr(x_fp8), _ptr(x_scale), _ptr(idx), _ptr(out_q), _ptr(out_s), n_out, n_src, d, ns,
                                       _stream(x_fp8)), "cinn_gather_rows")
    _count()
    return out_q, out_s


def set_gemm_sm_limit(n_sms: int) -> int:
    """Caps the SMs the persistent GEMM kernels occupy (0 = all); returns the previous cap."""
    return int(_L.cinn_set_gemm_sm_limit(int(n_sms)))


def scatter_rows(rows: torch.Tensor, idx: torch.Tensor, n_out: int = None) -> torch.Tensor:
    """``out[idx[r]] = rows[r]`` (``out.index_copy_(0, idx, rows)`` into a fresh tensor) with 16-byte vectors."""
    assert rows.is_cuda and idx.is_cuda, "Inputs must be on CUDA"
    rows = rows.contiguous()
    n, d = rows.shape
    n_out = n if n_out is None else int(n_out)
    row_bytes = d * rows.element_size()
    if row_bytes % 16 != 0:
        out = torch.empty((n_out, d), dtype=rows.dtype, device=rows.device)
        return out.index_copy_(0, idx, rows)
    idx = idx.to(torch.int64).contiguous()
    with torch.cuda.device(rows.device):
        out = torch.empty((n_out, d), dtype=rows.dtype, device=rows.device)
        _lib.check(_L.cinn_scatter_rows(_ptr(rows), _ptr(idx), _ptr(out), n, n_out, row_bytes, _stream(rows)),
                   "cinn_scatter_rows")
    _count()
    return out


def p2p_dispatch(x_fp8, x_scale, token_indices, sorted_experts, base_send, my_start, peer_q, peer_s, experts_per_rank: int,
                 n_ranks: int, capacity_rows: int) -> None:
    """Writes the quantised rows of this rank's sorted (token, expert) pairs straight into the receive buffers of
    the ranks that own the experts (``cinn_p2p_dispatch``; tables from ``p2p.exchange_tables``)."""
    assert x_fp8.is_cuda, "Inputs must be on CUDA"
    n_tokens, d = x_fp8.shape
    x_fp8, x_scale = x_fp8.contiguous(), x_scale.float().contiguous()
    with torch.cuda.device(x_fp8.device):
        _lib.check(_L.cinn_p2p_dispatch(_ptr(x_fp8), _ptr(x_scale), _ptr(token_indices), _ptr(sorted_experts), _ptr(base_send),
                                        _ptr(my_start), _ptr(peer_q), _ptr(peer_s), token_indices.numel(), n_tokens, d,
                                        x_scale.shape[1], experts_per_rank, n_ranks, capacity_rows, _stream(x_fp8)),
                   "cinn_p2p_dispatch")
    _count()


def p2p_dispatch_signal(x_fp8, x_scale, token_indices, sorted_experts, tables, buffers, e_lo: int = 0, e_hi: int = None,
                        flag_slot: int = None, n_sms: int = 0) -> None:
    """``p2p_dispatch`` for the pairs of the local experts ``[e_lo, e_hi)`` of every rank (default: all), whose last
    CTA flags "these rows have landed" to every rank under ``flag_slot`` (``cinn_p2p_dispatch_signal``);
    ``tables``: what ``buffers.plan`` returned for this layer call, ``buffers``: a ``p2p.PeerBuffers``; ``n_sms`` > 0:
    the stores come from that many SMs only (the rest stay free for a GEMM on another stream)."""
    assert x_fp8.is_cuda, "Inputs must be on CUDA"
    n_tokens, d = x_fp8.shape
    x_fp8, x_scale = x_fp8.contiguous(), x_scale.float().contiguous()
    b = buffers
    e_local = b.n_experts // b.world
    with torch.cuda.device(x_fp8.device):
        _lib.check(_L.cinn_p2p_dispatch_signal(_ptr(x_fp8), _ptr(x_scale), _ptr(token_indices), _ptr(sorted_experts),
                                               _ptr(tables.base_send), _ptr(tables.my_start), _ptr(b.peer_q), _ptr(b.peer_s),
                                               token_indices.numel(), n_tokens, d, x_scale.shape[1], e_local,
                                               b.world, b.capacity_rows, _ptr(b.peer_flags), b.rank,
                                               b.LANDED_SLOT if flag_slot is None else flag_slot,
                                               b._call & 0x7FFFFFFF, _ptr(b.done), e_lo, e_local if e_hi is None else e_hi,
                                               int(n_sms), _stream(x_fp8)), "cinn_p2p_dispatch_signal")
    _count()


def p2p_row_table_wait(tables, buffers, n_rows: int, row_bytes: int, flag_slot: int = None) -> torch.Tensor:
    """``p2p_row_table`` that first waits for the "landed" flags of all ranks under ``flag_slot``
    (``cinn_p2p_row_table_wait``); with ``n_rows = 0`` it only waits."""
    b = buffers
    dev = b.flags.device
    with torch.cuda.device(dev):
        table = torch.empty(max(n_rows, 1), dtype=torch.int64, device=dev)[:n_rows]
        _lib.check(_L.cinn_p2p_row_table_wait(_ptr(tables.seg_start), _ptr(tables.home_base), _ptr(b.peer_home), n_rows,
                                              row_bytes, tables.home_base.numel(), b.world, b.home_rows, _ptr(table),
                                              _ptr(b.peer_flags), b.rank, b.LANDED_SLOT if flag_slot is None else flag_slot,
                                              b._call & 0x7FFFFFFF,
                                              ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)),
                   "cinn_p2p_row_table_wait")
    _count()
    return table


def p2p_return(rows, seg_start, home_base, peer_home, n_ranks: int, capacity_rows: int) -> None:
    """Writes this rank's expert outputs straight into the home buffers of the ranks the tokens live on
    (``cinn_p2p_return``)."""
    assert rows.is_cuda, "Inputs must be on CUDA"
    rows = rows.contiguous()
    with torch.cuda.device(rows.device):
        _lib.check(_L.cinn_p2p_return(_ptr(rows), _ptr(seg_start), _ptr(home_base), _ptr(peer_home), rows.shape[0],
                                      rows.shape[1] * rows.element_size(), home_base.numel(), n_ranks, capacity_rows,
                                      _stream(rows)), "cinn_p2p_return")
    _count()


def moe_route(logits: torch.Tensor, bias: torch.Tensor, top_k: int):
    """Routing of ``MoE.forward`` (reference src/layers.py:122-148) from the router's fp32 logits, on the
    device and without a host synchronisation: sigmoid scores, top-k of score + bias, normalised gates, and the
    (token, expert) pairs in the order of a stable sort by expert.  Returns a dict of tensors:
    ``top_experts`` (T, k) int32, ``top_gates`` (T, k), ``token_indices`` / ``sorted_scores`` /
    ``sorted_experts`` (T*k), ``counts`` (E) int64, ``pair_pos`` / ``pair_gate`` (T, k)."""
    assert logits.is_cuda and bias.is_cuda, "Inputs must be on CUDA"
    assert logits.ndim == 2, "logits must be (tokens, experts)"
    logits = logits.float().contiguous()
    bias = bias.float().contiguous()
    T, E = logits.shape
    dev = logits.device
    with torch.cuda.device(dev):
        ws = torch.empty(max(1, int(_L.cinn_moe_route_workspace_ints(T, E))), dtype=torch.int32, device=dev)
        out = {
            "top_experts": torch.empty((T, top_k), dtype=torch.int32, device=dev),
            "top_gates": torch.empty((T, top_k), dtype=torch.float32, device=dev),
            "token_indices": torch.empty(T * top_k, dtype=torch.int64, device=dev),
            "sorted_scores": torch.empty(T * top_k, dtype=torch.float32, device=dev),
            "sorted_experts": torch.empty(T * top_k, dtype=torch.int64, device=dev),
            "counts": torch.empty(E, dtype=torch.int64, device=dev),
            "pair_pos": torch.empty((T, top_k), dtype=torch.int64, device=dev),
            "pair_gate": torch.empty((T, top_k), dtype=torch.float32, device=dev),
        }
        _lib.check(_L.cinn_moe_route(_ptr(logits), _ptr(bias), T, E, top_k, _ptr(ws), _ptr(out["top_experts"]),
                                     _ptr(out["top_gates"]), _ptr(out["token_indices"]), _ptr(out["sorted_scores"]),
                                     _ptr(out["sorted_experts"]), _ptr(out["counts"]), _ptr(out["pair_pos"]),
                                     _ptr(out["pair_gate"]), _stream(logits)), "cinn_moe_route")
    _count(3)
    return out


def fp8_grouped_gemm_dgrad(dy_fp8, dy_scale, w_fp8, w_scale, expert_starts, expert_ends, out_dtype=torch.bfloat16):
    """``dX[starts[e]:ends[e]] = dY[starts[e]:ends[e]] @ W[e]`` on quantised operands (one launch, ragged ranges)."""
    T, d_out = dy_fp8.shape
    E, _, d_in = w_fp8.shape
    starts = expert_starts.to(torch.int64).contiguous()
    ends = expert_ends.to(torch.int64).contiguous()
    with torch.cuda.device(dy_fp8.device):
        dx = torch.empty((T, d_in), dtype=out_dtype, device=dy_fp8.device)
        # rows of no expert get no gradient: cleared by a pass that touches only those rows
        _lib.check(_L.cinn_zero_rows_outside(_ptr(dx), T, d_in * dx.element_size(), _ptr(starts), _ptr(ends), E,
                                             _stream(dy_fp8)), "cinn_zero_rows_outside")
        _lib.check(_L.cinn_fp8_grouped_gemm_dgrad(_ptr(dy_fp8), _ptr(dy_scale), _ptr(w_fp8), _ptr(w_scale), _ptr(starts),
                                                  _ptr(ends), E, T, d_in, d_out, _ptr(dx), _DTYPE_TAG[out_dtype],
                                                  _stream(dy_fp8)), "cinn_fp8_grouped_gemm_dgrad")
    _count(2)
    return dx


def fp8_grouped_wgrad(grad_out: torch.Tensor, x_fp8: torch.Tensor, x_scale: torch.Tensor, expert_starts, expert_ends,
                      n_experts: int, d_in: int, d_out: int, w_dtype=torch.float32, fused: bool = None,
                      with_row_quant: bool = False):
    """``dW[e] = rowwise(dY[e rows]^T) @ blockwise(dequant_rowwise(x_q[e rows]))`` for every expert: the weight
    gradient of ``FP8MatmulFunction.backward`` (reference src/kernels.py:780-788) expert by expert.  With ``d_in`` and
    ``d_out`` multiples of 256: four launches for all experts (segments padded to whole tiles on the device, dY^T
    and x quantised per segment, one grouped-K GEMM), no host read-back.  Otherwise the row ranges are read back
    once and three launches per non-empty expert are enqueued by one library call.  Returns (E, d_out, d_in) of
    ``w_dtype`` (fp32 holds bf16-rounded values, as a bf16 result cast to the master weight's type would).
    ``with_row_quant``: also return the row-wise quantisation of ``grad_out`` (e4m3 bytes and scales; defined for the
    rows inside expert ranges) as ``(grad_w, dy_fp8, dy_scale)`` - on the four-launch path with 2-byte gradients it
    comes out of the pass that quantises dY^T, so dY is read once for the input and the weight gradient."""
    g = grad_out if grad_out.is_contiguous() else grad_out.contiguous()
    if g.dtype not in _DTYPE_TAG:
        g = g.float()
    x_fp8, x_scale = x_fp8.contiguous(), x_scale.float().contiguous()
    T = g.shape[0]
    out_tag = _lib.F32_BF16 if w_dtype == torch.float32 else _lib.BF16
    can_fuse = d_in % 256 == 0 and d_out % 256 == 0 and 1 <= n_experts <= 1024 and T > 0
    assert not fused or can_fuse, "the one-launch weight gradient needs d_in and d_out multiples of 256"
    if can_fuse and fused is not False:
        # all experts in four launches, row ranges read on the device: no host read-back
        starts = expert_starts.to(torch.int64).contiguous()
        ends = expert_ends.to(torch.int64).contiguous()
        need = int(_L.cinn_fp8_grouped_wgrad_fused_scratch_bytes(T, n_experts, d_in, d_out))
        one_pass = with_row_quant and g.dtype in (torch.bfloat16, torch.float16)
        with torch.cuda.device(g.device):
            scratch = torch.empty(need, dtype=torch.uint8, device=g.device)
            grad_w = torch.empty((n_experts, d_out, d_in), dtype=w_dtype, device=g.device)
            g_q = torch.empty((T, d_out), dtype=torch.float8_e4m3fn, device=g.device) if one_pass else None
            g_s = torch.empty((T, d_out // 128), dtype=torch.float32, device=g.device) if one_pass else None
            _lib.check(_L.cinn_fp8_grouped_wgrad_fused(_ptr(g), _DTYPE_TAG[g.dtype], _ptr(x_fp8), _ptr(x_scale), _ptr(starts),
                                                       _ptr(ends), n_experts, T, d_in, d_out, _ptr(scratch), need, _ptr(grad_w),
                                                       out_tag, _DIV_MODE, _ptr(g_q) if one_pass else None,
                                                       _ptr(g_s) if one_pass else None, _stream(g)),
                       "cinn_fp8_grouped_wgrad_fused")
        _count(4)
        if with_row_quant:
            return (grad_w, g_q, g_s) if one_pass else (grad_w, *quantize_fp8_rowwise(g, block_size=128))
        return grad_w
    bounds = torch.stack([expert_starts.to(torch.int64), expert_ends.to(torch.int64)]).cpu()     # one host read-back
    starts_h, ends_h = bounds[0].contiguous(), bounds[1].contiguous()
    max_rows = int((ends_h.clamp(max=T) - starts_h.clamp(min=0)).clamp(min=0).max()) if n_experts > 0 else 0
    need = int(_L.cinn_fp8_grouped_wgrad_scratch_bytes(max_rows, d_in, d_out))
    with torch.cuda.device(g.device):
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=g.device)
        grad_w = torch.empty((n_experts, d_out, d_in), dtype=w_dtype, device=g.device)
        _lib.check(_L.cinn_fp8_grouped_wgrad(_ptr(g), _DTYPE_TAG[g.dtype], _ptr(x_fp8), _ptr(x_scale),
                                             ctypes.c_void_p(starts_h.data_ptr()), ctypes.c_void_p(ends_h.data_ptr()), n_experts,
                                             T, d_in, d_out, _ptr(scratch), scratch.numel(), _ptr(grad_w), out_tag, _DIV_MODE,
                                             _stream(g)), "cinn_fp8_grouped_wgrad")
    _count(3 * n_experts)
    if with_row_quant:
        return (grad_w, *quantize_fp8_rowwise(g, block_size=128))
    return grad_w


_EXPERT_WEIGHT_CACHE_16 = {}        # id(weight tensor) -> (key, fp16 copy)


def _expert_weights_fp16(weights: torch.Tensor) -> torch.Tensor:
    """The expert stack as fp16 (the reference casts every operand tile to fp16 in its kernel, src/kernels.py:515),
    converted when the tensor changes, not per call (same key and caveat as ``cached_expert_weights``)."""
    if weights.dtype == torch.float16 and weights.is_contiguous():
        return weights.detach()
    key = (weights._version, weights.data_ptr(), weights.dtype, tuple(weights.shape))
    ident = id(weights)
    hit = _EXPERT_WEIGHT_CACHE_16.get(ident)
    if hit is not None and hit[0] == key:
        return hit[1]
    w16 = weights.detach().to(torch.float16).contiguous()
    if hit is None:
        weakref.finalize(weights, _EXPERT_WEIGHT_CACHE_16.pop, ident, None)
    _EXPERT_WEIGHT_CACHE_16[ident] = (key, w16)
    return w16


def grouped_gemm_16bit(sorted_x: torch.Tensor, weights: torch.Tensor, expert_starts, expert_ends,
                       out_dtype=torch.float16, out: torch.Tensor = None) -> torch.Tensor:
    """``out[starts[e]:ends[e]] = sorted_x[starts[e]:ends[e]] @ weights[e].T`` on 16-bit operands (both bf16 or both
    fp16), fp32 accumulation (``cinn_grouped_gemm_16bit``): the arithmetic of the reference's kernel
    (src/kernels.py:466-523).  Rows outside every range are left as allocated."""
    assert sorted_x.is_cuda and weights.is_cuda, "Inputs must be on CUDA"
    assert sorted_x.dtype == weights.dtype and sorted_x.dtype in (torch.bfloat16, torch.float16), "operands: both bf16 or both fp16"
    x, w = sorted_x.contiguous(), weights.contiguous()
    T, d_in = x.shape
    E, d_out, _ = w.shape
    starts = expert_starts.to(torch.int64).contiguous()
    ends = expert_ends.to(torch.int64).contiguous()
    with torch.cuda.device(x.device):
        if out is None:
            out = torch.empty((T, d_out), dtype=out_dtype, device=x.device)
        _lib.check(_L.cinn_grouped_gemm_16bit(_ptr(x), _ptr(w), _DTYPE_TAG[x.dtype], _ptr(starts), _ptr(ends), E, T, d_in, d_out,
                                              _ptr(out), _DTYPE_TAG[out.dtype], _stream(x)), "cinn_grouped_gemm_16bit")
    _count()
    return out


class MoEGroupedGemm16Function(torch.autograd.Function):
    """``moe_grouped_gemm`` with the forward in the reference's precision (fp16 operands, fp32 accumulation).  The
    reference has no backward for it; here the gradients come from the same e4m3 kernels as in the default mode
    (``MoEGroupedGemmFunction``), fed with the saved 16-bit rows."""

    @staticmethod
    def forward(ctx, sorted_x, weights, expert_starts, expert_ends, out_dtype):
        x16 = sorted_x.detach().to(torch.float16)
        out = grouped_gemm_16bit(x16, _expert_weights_fp16(weights), expert_starts, expert_ends, out_dtype)
        ctx.save_for_backward(x16, weights, expert_starts, expert_ends)
        ctx.x_dtype, ctx.w_dtype = sorted_x.dtype, weights.dtype
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x16, weights, starts, ends = ctx.saved_tensors
        x_fp8, x_scale = quantize_fp8_rowwise(x16, block_size=128)
        w_fp8, w_scale = cached_expert_weights(weights)
        inner = _Saved((x_fp8, x_scale, w_fp8, w_scale, starts, ends), ctx.x_dtype, ctx.w_dtype)
        return MoEGroupedGemmFunction.backward(inner, grad_out)


class _Saved:
    """What ``MoEGroupedGemmFunction.backward`` reads from its context."""

    def __init__(self, saved_tensors, x_dtype, w_dtype):
        self.saved_tensors, self.x_dtype, self.w_dtype = saved_tensors, x_dtype, w_dtype


class MoEGroupedGemmFunction(torch.autograd.Function):
    """Differentiable grouped GEMM.  The reference's ``moe_grouped_gemm`` is a plain function (src/kernels.py:526-581),
    so on CUDA no gradient reaches the routed experts there; this function gives the grouped GEMM the backward of
    ``FP8MatmulFunction`` (src/kernels.py:763-794) expert by expert:

      dX[e rows] = rowwise(dY[e rows]) @ W_q[e]                                 one grouped launch
      dW[e]      = rowwise(dY[e rows]^T) @ blockwise(dequant_rowwise(x_q[e rows]))   per non-empty expert

    The weight gradient walks the experts on the host (their row counts are read back once per backward)."""

    @staticmethod
    def forward(ctx, sorted_x, weights, expert_starts, expert_ends, out_dtype):
        x = sorted_x if sorted_x.stride(-1) == 1 else sorted_x.contiguous()
        x_fp8, x_scale = quantize_fp8_rowwise(x, block_size=128)
        w_fp8, w_scale = cached_expert_weights(weights)
        out = fp8_grouped_gemm(x_fp8, x_scale, w_fp8, w_scale, expert_starts, expert_ends, out_dtype=out_dtype)
        ctx.save_for_backward(x_fp8, x_scale, w_fp8, w_scale, expert_starts, expert_ends)
        ctx.x_dtype, ctx.w_dtype = sorted_x.dtype, weights.dtype
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x_fp8, x_scale, w_fp8, w_scale, starts, ends = ctx.saved_tensors
        E, d_out, d_in = w_fp8.shape
        g = grad_out if grad_out.is_contiguous() else grad_out.contiguous()
        dx_dtype = ctx.x_dtype if ctx.x_dtype in _DTYPE_TAG else torch.float32
        w_dtype = ctx.w_dtype if ctx.w_dtype in (torch.float32, torch.bfloat16) else torch.float32
        # the weight gradient first: its pass over dY also yields the row-wise quantisation the input gradient reads
        grad_w, g_fp8, g_scale = fp8_grouped_wgrad(g, x_fp8, x_scale, starts, ends, E, d_in, d_out, w_dtype, with_row_quant=True)
        grad_x = fp8_grouped_gemm_dgrad(g_fp8, g_scale, w_fp8, w_scale, starts, ends, out_dtype=dx_dtype)
        return grad_x.to(ctx.x_dtype), grad_w.to(ctx.w_dtype), None, None, None


def moe_grouped_gemm(sorted_x: torch.Tensor, weights: torch.Tensor, expert_starts: torch.Tensor,
                     expert_ends: torch.Tensor, max_expert_tokens: int = None,
                     dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Grouped GEMM for MoE (reference src/kernels.py:526-581): for each expert e,
    ``out[starts[e]:ends[e]] = sorted_x[starts[e]:ends[e]] @ weights[e].T``.

    ``expert_starts`` / ``expert_ends`` are read on the device; ``max_expert_tokens`` is
    accepted for signature compatibility and ignored (no grid depends on it, so the
    caller's ``.item()`` synchronisation is unnecessary).  By default tokens and weights are quantised
    to e4m3 on the fly (the weights once per weight update, ``cached_expert_weights``); with
    ``set_moe_grouped_precision("16bit")`` / ``CINN_MOE_GROUPED=16bit`` the product runs on fp16 operands
    with fp32 accumulation, the reference kernel's own arithmetic.  Returns fp16 like the reference unless
    ``dtype`` says otherwise.  Unlike the reference it is differentiable (``MoEGroupedGemmFunction``)."""
    assert sorted_x.is_cuda and weights.is_cuda, "Inputs must be on CUDA"
    if _MOE_GROUPED_PRECISION == "16bit" and sorted_x.shape[1] % 8 == 0:
        if torch.is_grad_enabled() and (sorted_x.requires_grad or weights.requires_grad):
            return MoEGroupedGemm16Function.apply(sorted_x, weights, expert_starts, expert_ends, dtype)
        return grouped_gemm_16bit(sorted_x.to(torch.float16), _expert_weights_fp16(weights), expert_starts, expert_ends, dtype)
    if _ops is not None and torch.compiler.is_compiling():
        return _ops.grouped_gemm(sorted_x, weights, expert_starts, expert_ends, dtype)
    if torch.is_grad_enabled() and (sorted_x.requires_grad or weights.requires_grad):
        return MoEGroupedGemmFunction.apply(sorted_x, weights, expert_starts, expert_ends, dtype)
    x = sorted_x if sorted_x.stride(-1) == 1 else sorted_x.contiguous()
    x_fp8, x_scale = quantize_fp8_rowwise(x, block_size=128)
    w_fp8, w_scale = cached_expert_weights(weights)
    return fp8_grouped_gemm(x_fp8, x_scale, w_fp8, w_scale, expert_starts, expert_ends, out_dtype=dtype)


# -----------------------------------------------------------------------------
# torch.compile: the differentiable entry points as torch.library operators (cinnamon_b200/ops.py)
# -----------------------------------------------------------------------------
try:
    from . import ops as _ops
except Exception as _exc:                                   # noqa: BLE001  (an older torch without torch.library.custom_op)
    import warnings
    warnings.warn(f"cinnamon_b200: torch.library operators were not registered ({type(_exc).__name__}: {_exc}); "
                  "torch.compile will break the graph at every call into the library")
    _ops = None

_sparse_attention_eager = sparse_attention


def sparse_attention(q, k, v, idx, scale=None):             # noqa: F811
    """Attention over the K selected positions of every query (reference src/kernels.py:1292-1312).
    q, k: [B, H, L, D_qk]; v: [B, H, L, D_v]; idx: [B, L, K] int64.  Returns ``(output, attn_weights)``.
    Under ``torch.compile`` the call is one opaque graph node (``cinnamon_b200::sparse_attn_fwd``)."""
    if _ops is not None and torch.compiler.is_compiling():
        return _ops.sparse_attention(q, k, v, idx, q.shape[-1] ** -0.5 if scale is None else scale)
    return _sparse_attention_eager(q, k, v, idx, scale)
