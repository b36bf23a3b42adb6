"""DSA sparse attention (reference src/kernels.py:913-1312) on the hand-written kernels.

``sparse_attention(q, k, v, idx, scale=None)`` and ``SparseAttentionFunction`` keep the reference's names,
argument order, return values and dtypes: ``(output [B, H, L, D_v] in the inputs' dtype, attn_weights
[B, H, L, K] fp32)``, gradients for q, k, v in the inputs' dtype.  One forward launch, one backward launch.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_L = _lib.lib
_TAG = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32, torch.float16: _lib.F16}


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


class SparseAttentionFunction(torch.autograd.Function):
    """Autograd function with the reference's signature (src/kernels.py:1189-1289)."""

    @staticmethod
    def forward(ctx, q, k, v, idx, scale):
        assert q.is_cuda and k.is_cuda and v.is_cuda and idx.is_cuda, "Inputs must be on CUDA"
        B, H, L, d_qk = q.shape
        d_v = v.shape[-1]
        K = idx.shape[-1]
        in_dtype = q.dtype
        work = in_dtype if in_dtype in _TAG else torch.float32
        q, k, v = (t.to(work).contiguous() for t in (q, k, v))          # :1220-1223
        idx = idx.to(torch.int64).contiguous()
        with torch.cuda.device(q.device):
            out = torch.empty((B, H, L, d_v), dtype=torch.float32, device=q.device)
            lse = torch.empty((B, H, L), dtype=torch.float32, device=q.device)
            attn = torch.empty((B, H, L, K), dtype=torch.float32, device=q.device)
            _lib.check(_L.cinn_sparse_attn_fwd(_ptr(q), _ptr(k), _ptr(v), _TAG[work], _ptr(idx), _ptr(out), _ptr(lse),
                                               _ptr(attn), B, H, L, K, d_qk, d_v, float(scale), _stream(q)),
                       "cinn_sparse_attn_fwd")
        ctx.save_for_backward(q, k, v, idx, out, lse)
        ctx.scale = float(scale)
        ctx.in_dtype = in_dtype
        ctx.mark_non_differentiable(attn)
        return out.to(in_dtype), attn

    @staticmethod
    def backward(ctx, grad_output, grad_attn_weights):
        q, k, v, idx, out, lse = ctx.saved_tensors
        B, H, L, d_qk = q.shape
        d_v = v.shape[-1]
        K = idx.shape[-1]
        g = grad_output.contiguous()
        if g.dtype != q.dtype and g.dtype != torch.float32:
            g = g.float()
        with torch.cuda.device(q.device):
            gq = torch.empty((B, H, L, d_qk), dtype=torch.float32, device=q.device)
            gk = torch.zeros((B, H, L, d_qk), dtype=torch.float32, device=q.device)     # accumulated into (:1257-1259)
            gv = torch.zeros((B, H, L, d_v), dtype=torch.float32, device=q.device)
            _lib.check(_L.cinn_sparse_attn_bwd(_ptr(g), _TAG[g.dtype], _ptr(out), _ptr(lse), _ptr(q), _ptr(k), _ptr(v),
                                               _TAG[q.dtype], _ptr(idx), _ptr(gq), _ptr(gk), _ptr(gv), B, H, L, K, d_qk, d_v,
                                               ctx.scale, _stream(q)), "cinn_sparse_attn_bwd")
        dt = ctx.in_dtype
        return gq.to(dt), gk.to(dt), gv.to(dt), None, None


def sparse_attention(q, k, v, idx, scale=None):
    """Attention over the K selected positions of every query (reference src/kernels.py:1292-1312).
    q, k: [B, H, L, D_qk]; v: [B, H, L, D_v]; idx: [B, L, K] int64.  Returns ``(output, attn_weights)``."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return SparseAttentionFunction.apply(q, k, v, idx, scale)
