"""Fused input prologue and output epilogue of the delta-rule attention layer.

The reference's layers (language_modeling/src/utils/cuda_fast_weight_layer.py:106-125, 152-163;
algorithmic/layers.py:110-137) turn the fused projection ``qkvb`` of shape (len, B, H, 3d+1) into the op's
arguments with a chain of split / sigmoid / permute / elu+1 / sum-normalise launches, and turn the op's
output back into (len, B, H*d) with a scale, a transpose and a reshape.  The two autograd Functions here do
each direction in one launch; ``delta_attention`` strings them around ``fast_weight_delta``:

    out = delta_attention(qkvb.view(len, B, H, 3*d + 1), W, scale)      # (len, B, H*d); W updated in place

fp32 only (the op's state and saved tensors are fp32 as well).
"""
import ctypes

import torch

from recurrent_fwp_b200 import _lib
from recurrent_fwp_b200.fast_weight import fast_weight_delta


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


class DeltaLayerPrologue(torch.autograd.Function):
    """qkvb (len, B, H, 3d+1) -> q, k (elu+1, sum-normalised), v, beta = sigmoid, each (B, H, len, .)."""

    @staticmethod
    def forward(ctx, qkvb):
        _lib.require_cuda(qkvb)
        if qkvb.dtype != torch.float32 or qkvb.dim() != 4 or (qkvb.shape[3] - 1) % 3:
            raise RuntimeError('qkvb must be float32 of shape (len, B, H, 3*d + 1)')
        x = qkvb.detach().contiguous()
        L, B, H, w = x.shape
        D = (w - 1) // 3
        q, k, v = (torch.empty((B, H, L, D), device=x.device, dtype=torch.float32) for _ in range(3))
        beta = torch.empty((B, H, L, 1), device=x.device, dtype=torch.float32)
        stream, dev = _lib.stream_and_device(x)
        _lib.check(_lib.lib.fwp_delta_layer_prologue_forward(L, B, H, D, _p(x), _p(q), _p(k), _p(v), _p(beta), stream, dev),
                   'delta_layer_prologue_forward')
        ctx.save_for_backward(x)
        return q, k, v, beta

    @staticmethod
    def backward(ctx, gq, gk, gv, gb):
        (x,) = ctx.saved_tensors
        L, B, H, w = x.shape
        D = (w - 1) // 3
        gq, gk, gv, gb = (g.contiguous() for g in (gq, gk, gv, gb))
        gx = torch.empty_like(x)
        stream, dev = _lib.stream_and_device(x)
        _lib.check(_lib.lib.fwp_delta_layer_prologue_backward(L, B, H, D, _p(x), _p(gq), _p(gk), _p(gv), _p(gb), _p(gx), stream, dev),
                   'delta_layer_prologue_backward')
        return gx


class DeltaLayerEpilogue(torch.autograd.Function):
    """out (B, H, len, d) -> scale * out as (len, B, H*d)."""

    @staticmethod
    def forward(ctx, out, scale):
        _lib.require_cuda(out)
        if out.dtype != torch.float32 or out.dim() != 4:
            raise RuntimeError('out must be float32 of shape (B, H, len, d)')
        src = out.detach().contiguous()
        B, H, L, D = src.shape
        dst = torch.empty((L, B, H * D), device=src.device, dtype=torch.float32)
        stream, dev = _lib.stream_and_device(src)
        _lib.check(_lib.lib.fwp_delta_layer_transpose(L, B, H, D, _p(src), _p(dst), float(scale), 1, stream, dev),
                   'delta_layer_transpose')
        ctx.scale = float(scale)
        ctx.dims = (L, B, H, D)
        return dst

    @staticmethod
    def backward(ctx, g):
        L, B, H, D = ctx.dims
        g = g.contiguous()
        dst = torch.empty((B, H, L, D), device=g.device, dtype=torch.float32)
        stream, dev = _lib.stream_and_device(g)
        _lib.check(_lib.lib.fwp_delta_layer_transpose(L, B, H, D, _p(g), _p(dst), ctx.scale, 0, stream, dev),
                   'delta_layer_transpose')
        return dst, None


delta_layer_prologue = DeltaLayerPrologue.apply
delta_layer_epilogue = DeltaLayerEpilogue.apply


def delta_attention(qkvb, W, scale):
    """Prologue, delta-rule fast weight memory, epilogue.  qkvb: (len, B, H, 3d+1); W: (B, H, d, d), updated in place."""
    q, k, v, beta = delta_layer_prologue(qkvb)
    return delta_layer_epilogue(fast_weight_delta(q, k, v, beta, W), scale)
