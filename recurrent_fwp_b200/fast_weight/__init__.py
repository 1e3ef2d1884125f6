"""Delta-rule fast weight memory: drop-in for the reference's ``fast_weight`` module.

Mirrors ``DeltaFastWeight`` / ``fast_weight_delta`` of
algorithmic/fast_weight/__init__.py:26-96 (also language_modeling/src/utils/fast_fast_weight
and reinforcement_learning/torchbeast/fast_weight): same positional arguments,
same saved tensors, same in-place state semantics --

  * ``W`` [N,H,E,M] enters as the start-of-segment state and is overwritten with
    the end-of-segment state;
  * ``backward`` rewinds that same tensor in place to the start-of-segment state
    (callers that carry the state clone it before backward, as the reference's
    layers do), and returns no gradient for it.

Differences a caller can observe: inputs may be float32 or bfloat16 (the state
and the tensors saved for backward stay float32); the work runs on the current
CUDA stream of the inputs' device instead of the legacy default stream.
"""
import torch

from recurrent_fwp_b200 import _lib


class DeltaFastWeight(torch.autograd.Function):
    """Fast weight using the delta update rule."""

    @staticmethod
    def forward(ctx, Q, K, V, beta, W):
        N, H, L, E = Q.shape
        M = V.shape[3]
        dt = _lib.io_dtype(Q)
        _lib.require_streams(Q, {'K': (K, (N, H, L, E)), 'V': (V, (N, H, L, M)), 'beta': (beta, (N, H, L, 1))})
        _lib.require_f32(Q, {'W': (W, (N, H, E, M))})
        _lib.require_cuda(Q, K, V, beta, W)
        Qc, Kc, Vc, bc = (_lib.unit_inner(t.detach()) for t in (Q, K, V, beta))
        Wd = W.detach()
        if Wd.stride(3) != 1:
            raise RuntimeError('W must have a unit innermost stride (it is updated in place)')
        out = torch.empty((N, H, L, M), device=Q.device, dtype=Q.dtype)
        V_old = torch.empty((N, H, L, M), device=Q.device, dtype=torch.float32)
        # The reference also stores u_t = beta_t (v_t - v_old_t) ("V_insert"); the backward here rebuilds it from
        # V, V_old and beta, so that tensor is neither allocated nor written (an empty placeholder keeps the
        # reference's saved-tensor order).
        V_insert = torch.empty(0, device=Q.device, dtype=torch.float32)
        stream, dev = _lib.stream_and_device(Q)
        _lib.check(_lib.lib.fwp_fast_weight_forward(
            N, H, L, E, M, _lib.desc(Qc), _lib.desc(Kc), _lib.desc(Vc), _lib.desc(bc),
            _lib.desc(V_old), _lib.desc(None), _lib.desc(Wd), _lib.desc(out),
            dt, stream, dev), 'fast_weight_forward')
        _lib.raise_on_device_fault('fast_weight_forward')
        ctx.save_for_backward(Qc, Kc, Vc, bc, V_old, V_insert, W)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V, beta, V_old, V_insert, W = ctx.saved_tensors
        N, H, L, E = Q.shape
        M = V.shape[3]
        grad_out = _lib.grad_like(grad_out, Q, (N, H, L, M))
        grad_Q = torch.empty_like(Q, memory_format=torch.contiguous_format)
        grad_K = torch.empty_like(K, memory_format=torch.contiguous_format)
        grad_V = torch.empty_like(V, memory_format=torch.contiguous_format)
        grad_beta = torch.empty_like(beta, memory_format=torch.contiguous_format)
        stream, dev = _lib.stream_and_device(Q)
        _lib.check(_lib.lib.fwp_fast_weight_backward(
            N, H, L, E, M, _lib.desc(Q), _lib.desc(K), _lib.desc(V), _lib.desc(beta),
            _lib.desc(V_old), _lib.desc(None), _lib.desc(grad_out), _lib.desc(W.detach()),
            _lib.desc(grad_Q), _lib.desc(grad_K), _lib.desc(grad_V), _lib.desc(grad_beta),
            _lib.io_dtype(Q), stream, dev), 'fast_weight_backward')
        _lib.raise_on_device_fault('fast_weight_backward')
        return grad_Q, grad_K, grad_V, grad_beta, None


# Alias the autograd function to the reference's snake-case name
fast_weight_delta = DeltaFastWeight.apply
