"""``torch.library`` custom operators over the library's kernels, so that ``torch.compile`` can hold them.

The reference compiles its model (``torch.compile(model)``, src/train.py:703) and its Triton kernels are traced as
part of the graph.  This library's kernels are reached through ctypes, which a tracing compiler cannot look into: an
``autograd.Function`` whose forward calls ctypes makes dynamo break the graph at every FP8 layer.  The operators
below wrap forward and backward of the three differentiable entry points as opaque nodes with shape functions
(``register_fake``) and autograd formulas (``register_autograd``):

  cinnamon_b200::fp8_linear_fwd / fp8_linear_bwd      FP8MatmulFunction   (src/kernels.py:731-794)
  cinnamon_b200::grouped_gemm_fwd / grouped_gemm_bwd  moe_grouped_gemm    (src/kernels.py:526-581; differentiable here)
  cinnamon_b200::sparse_attn_fwd / sparse_attn_bwd    SparseAttentionFunction (src/kernels.py:1189-1289)

Each operator body runs the very code of the eager ``autograd.Function`` (its ``forward`` / ``backward`` static
methods, handed a stand-in context), so compiled and eager results are the same bits.  ``FP8Linear.forward``,
``moe_grouped_gemm`` and ``sparse_attention`` switch to the operators while ``torch.compiler.is_compiling()``; in
eager mode they keep calling the autograd functions directly, as the reference does.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
from torch import Tensor

from . import kernels as K
from . import sparse_attention as SA

_DTYPES = [torch.bfloat16, torch.float32, torch.float16, torch.float64]
F8 = torch.float8_e4m3fn


def _tag(dtype: torch.dtype) -> int:
    return _DTYPES.index(dtype)


class _Ctx:
    """Stand-in for the autograd context when an autograd function's static methods are run as plain code."""

    def __init__(self, needs_input_grad=()):
        self.needs_input_grad = tuple(needs_input_grad)
        self.saved_tensors = ()

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors

    def mark_non_differentiable(self, *tensors):
        pass


def _nb(n: int) -> int:
    return (n + 127) // 128


# ---------------------------------------------------------------------------------------------------------------
# FP8 linear
# ---------------------------------------------------------------------------------------------------------------
def _linear_layout(x_shape, w_shape, w_stride, w_dtype, need_dgrad: bool, need_wgrad: bool):
    """Which copies FP8MatmulFunction.forward makes for these shapes (it decides from shapes and flags alone)."""
    Kd = x_shape[-1]
    M = 1
    for s in x_shape[:-1]:
        M *= s
    N = w_shape[0]
    want_wgrad = need_wgrad and Kd % 16 == 0
    x_blk_t = want_wgrad and M % 16 == 0 and K._KMAJOR_BACKWARD
    w_contig = (w_stride[1] == 1 and w_stride[0] % 4 == 0) or w_dtype not in K._DTYPE_TAG
    w_t = K._KMAJOR_BACKWARD and need_dgrad and N % 16 == 0 and Kd % 4 == 0 and w_contig
    return M, Kd, N, want_wgrad, x_blk_t, w_t


@torch.library.custom_op("cinnamon_b200::fp8_linear_fwd", mutates_args=(), device_types="cuda")
def fp8_linear_fwd(x: Tensor, weight: Tensor, round_scale: bool, need_dgrad: bool,
                   need_wgrad: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    ctx = _Ctx((need_dgrad, need_wgrad, False))
    out = K.FP8MatmulFunction.forward(ctx, x, weight, round_scale)
    x_saved, x_scale, w_fp8, w_scale = ctx.saved_tensors
    w_t = ctx.w_fp8_t if ctx.w_fp8_t is not None else torch.empty(0, dtype=F8, device=x.device)
    return out, x_saved, x_scale, w_fp8, w_scale, w_t


@fp8_linear_fwd.register_fake
def _(x, weight, round_scale, need_dgrad, need_wgrad):
    M, Kd, N, want_wgrad, x_blk_t, w_t = _linear_layout(x.shape, weight.shape, weight.stride(), weight.dtype, need_dgrad, need_wgrad)
    e = lambda shape, dt: torch.empty(shape, dtype=dt, device=x.device)                         # noqa: E731
    return (e(tuple(x.shape[:-1]) + (N,), torch.bfloat16), e((Kd, M) if x_blk_t else (M, Kd), F8),
            e((_nb(M) if want_wgrad else M, _nb(Kd)), torch.float32), e((N, Kd), F8), e((_nb(N), _nb(Kd)), torch.float32),
            e((Kd, N) if w_t else (0,), F8))


@torch.library.custom_op("cinnamon_b200::fp8_linear_bwd", mutates_args=(), device_types="cuda")
def fp8_linear_bwd(grad_out: Tensor, x_saved: Tensor, x_scale: Tensor, w_fp8: Tensor, w_scale: Tensor, w_fp8_t: Tensor,
                   x_shape: List[int], round_scale: bool, x_is_block: bool, x_is_block_t: bool,
                   weight_dtype: int) -> Tuple[Tensor, Tensor]:
    ctx = _Ctx((True, True, False))
    ctx.saved_tensors = (x_saved, x_scale, w_fp8, w_scale)
    ctx.x_shape, ctx.round_scale, ctx.n_inputs = tuple(x_shape), round_scale, 3
    ctx.x_is_block, ctx.x_is_block_t = x_is_block, x_is_block_t
    ctx.w_fp8_t = w_fp8_t if w_fp8_t.numel() else None
    ctx.weight_dtype = _DTYPES[weight_dtype]
    gx, gw, _ = K.FP8MatmulFunction.backward(ctx, grad_out)
    return gx, gw


@fp8_linear_bwd.register_fake
def _(grad_out, x_saved, x_scale, w_fp8, w_scale, w_fp8_t, x_shape, round_scale, x_is_block, x_is_block_t, weight_dtype):
    N, Kd = w_fp8.shape
    return (torch.empty(tuple(x_shape), dtype=torch.bfloat16, device=grad_out.device),
            torch.empty((N, Kd), dtype=torch.float32 if _DTYPES[weight_dtype] == torch.float32 else torch.bfloat16,
                        device=grad_out.device))


def _linear_setup(ctx, inputs, output):
    x, weight, round_scale, need_dgrad, need_wgrad = inputs
    _, _, _, want_wgrad, x_blk_t, _ = _linear_layout(x.shape, weight.shape, weight.stride(), weight.dtype, need_dgrad, need_wgrad)
    ctx.save_for_backward(*output[1:])
    ctx.x_shape, ctx.round_scale, ctx.weight_dtype = list(x.shape), round_scale, _tag(weight.dtype)
    ctx.x_is_block, ctx.x_is_block_t = want_wgrad, x_blk_t
    ctx.set_materialize_grads(False)


def _linear_backward(ctx, g_out, *ignored):
    x_saved, x_scale, w_fp8, w_scale, w_t = ctx.saved_tensors
    gx, gw = torch.ops.cinnamon_b200.fp8_linear_bwd(g_out, x_saved, x_scale, w_fp8, w_scale, w_t, ctx.x_shape, ctx.round_scale,
                                                    ctx.x_is_block, ctx.x_is_block_t, ctx.weight_dtype)
    return gx, gw, None, None, None


fp8_linear_fwd.register_autograd(_linear_backward, setup_context=_linear_setup)


def fp8_linear(x: Tensor, weight: Tensor, round_scale: bool) -> Tensor:
    """``FP8MatmulFunction.apply(x, weight, round_scale)`` as one opaque, differentiable graph node."""
    return torch.ops.cinnamon_b200.fp8_linear_fwd(x, weight, bool(round_scale), x.requires_grad, weight.requires_grad)[0]


# ---------------------------------------------------------------------------------------------------------------
# grouped GEMM
# ---------------------------------------------------------------------------------------------------------------
@torch.library.custom_op("cinnamon_b200::grouped_gemm_fwd", mutates_args=(), device_types="cuda")
def grouped_gemm_fwd(sorted_x: Tensor, weights: Tensor, expert_starts: Tensor, expert_ends: Tensor,
                     out_dtype: int) -> Tuple[Tensor, Tensor, Tensor]:
    ctx = _Ctx()
    out = K.MoEGroupedGemmFunction.forward(ctx, sorted_x, weights, expert_starts, expert_ends, _DTYPES[out_dtype])
    x_fp8, x_scale = ctx.saved_tensors[0], ctx.saved_tensors[1]
    return out, x_fp8, x_scale          # the e4m3 weights live in the library's cache: the backward asks for them again


@grouped_gemm_fwd.register_fake
def _(sorted_x, weights, expert_starts, expert_ends, out_dtype):
    T, d_in = sorted_x.shape
    E, d_out, _ = weights.shape
    e = lambda shape, dt: torch.empty(shape, dtype=dt, device=sorted_x.device)                  # noqa: E731
    return e((T, d_out), _DTYPES[out_dtype]), e((T, d_in), F8), e((T, _nb(d_in)), torch.float32)


@torch.library.custom_op("cinnamon_b200::grouped_gemm_bwd", mutates_args=(), device_types="cuda")
def grouped_gemm_bwd(grad_out: Tensor, x_fp8: Tensor, x_scale: Tensor, weights: Tensor, expert_starts: Tensor,
                     expert_ends: Tensor, x_dtype: int) -> Tuple[Tensor, Tensor]:
    ctx = _Ctx()
    w_fp8, w_scale = K.cached_expert_weights(weights)
    ctx.saved_tensors = (x_fp8, x_scale, w_fp8, w_scale, expert_starts, expert_ends)
    ctx.x_dtype, ctx.w_dtype = _DTYPES[x_dtype], weights.dtype
    gx, gw = K.MoEGroupedGemmFunction.backward(ctx, grad_out)[:2]
    return gx, gw


@grouped_gemm_bwd.register_fake
def _(grad_out, x_fp8, x_scale, weights, expert_starts, expert_ends, x_dtype):
    return (torch.empty(x_fp8.shape, dtype=_DTYPES[x_dtype], device=grad_out.device), torch.empty_like(weights))


def _grouped_setup(ctx, inputs, output):
    sorted_x, weights, starts, ends, _ = inputs
    ctx.save_for_backward(output[1], output[2], weights, starts, ends)
    ctx.x_dtype = _tag(sorted_x.dtype)
    ctx.set_materialize_grads(False)


def _grouped_backward(ctx, g_out, *ignored):
    x_fp8, x_scale, weights, starts, ends = ctx.saved_tensors
    gx, gw = torch.ops.cinnamon_b200.grouped_gemm_bwd(g_out, x_fp8, x_scale, weights, starts, ends, ctx.x_dtype)
    return gx, gw, None, None, None


grouped_gemm_fwd.register_autograd(_grouped_backward, setup_context=_grouped_setup)


def grouped_gemm(sorted_x: Tensor, weights: Tensor, expert_starts: Tensor, expert_ends: Tensor, dtype: torch.dtype) -> Tensor:
    return torch.ops.cinnamon_b200.grouped_gemm_fwd(sorted_x, weights, expert_starts, expert_ends, _tag(dtype))[0]


# ---------------------------------------------------------------------------------------------------------------
# sparse attention
# ---------------------------------------------------------------------------------------------------------------
@torch.library.custom_op("cinnamon_b200::sparse_attn_fwd", mutates_args=(), device_types="cuda")
def sparse_attn_fwd(q: Tensor, k: Tensor, v: Tensor, idx: Tensor, scale: float) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    ctx = _Ctx()
    out, attn = SA.SparseAttentionFunction.forward(ctx, q, k, v, idx, scale)
    _, _, _, _, out32, lse = ctx.saved_tensors
    return out, attn, out32 if out32.data_ptr() != out.data_ptr() else out32.clone(), lse


@sparse_attn_fwd.register_fake
def _(q, k, v, idx, scale):
    B, H, L, _ = q.shape
    e = lambda shape, dt: torch.empty(shape, dtype=dt, device=q.device)                        # noqa: E731
    return (e((B, H, L, v.shape[-1]), q.dtype), e((B, H, L, idx.shape[-1]), torch.float32),
            e((B, H, L, v.shape[-1]), torch.float32), e((B, H, L), torch.float32))


@torch.library.custom_op("cinnamon_b200::sparse_attn_bwd", mutates_args=(), device_types="cuda")
def sparse_attn_bwd(grad_out: Tensor, q: Tensor, k: Tensor, v: Tensor, idx: Tensor, out32: Tensor, lse: Tensor,
                    scale: float) -> Tuple[Tensor, Tensor, Tensor]:
    ctx = _Ctx()
    in_dtype = q.dtype
    work = in_dtype if in_dtype in SA._TAG else torch.float32
    ctx.saved_tensors = tuple(t.to(work).contiguous() for t in (q, k, v)) + (idx.to(torch.int64).contiguous(), out32, lse)
    ctx.scale, ctx.in_dtype = float(scale), in_dtype
    gq, gk, gv = SA.SparseAttentionFunction.backward(ctx, grad_out, None)[:3]
    return gq, gk, gv


@sparse_attn_bwd.register_fake
def _(grad_out, q, k, v, idx, out32, lse, scale):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _attn_setup(ctx, inputs, output):
    q, k, v, idx, scale = inputs
    ctx.save_for_backward(q, k, v, idx, output[2], output[3])
    ctx.scale = scale
    ctx.set_materialize_grads(False)


def _attn_backward(ctx, g_out, *ignored):
    q, k, v, idx, out32, lse = ctx.saved_tensors
    if g_out is None:
        return None, None, None, None, None
    gq, gk, gv = torch.ops.cinnamon_b200.sparse_attn_bwd(g_out, q, k, v, idx, out32, lse, ctx.scale)
    return gq, gk, gv, None, None


sparse_attn_fwd.register_autograd(_attn_backward, setup_context=_attn_setup)


def sparse_attention(q: Tensor, k: Tensor, v: Tensor, idx: Tensor, scale: float):
    out, attn, _, _ = torch.ops.cinnamon_b200.sparse_attn_fwd(q, k, v, idx, float(scale))
    return out, attn
