"""Sum-rule causal product with carried state: drop-in for the reference's
``fast_transformers`` module (``FastWeightSum`` / ``fast_weight_sum``,
algorithmic/fast_transformers/__init__.py:25-84).

``W`` [N,H,E,M] is updated in place to the end-of-segment state.  As in the
reference, the backward takes no state: its prefix sums restart from zero, so a
carried non-zero ``W`` contributes nothing to ``grad_Q`` and ``W`` is not rewound.
"""
import torch

from recurrent_fwp_b200 import _lib


class FastWeightSum(torch.autograd.Function):
    """Fast weight using the purely additive (sum) update rule."""

    @staticmethod
    def forward(ctx, Q, K, V, W):
        N, H, L, E = Q.shape
        M = V.shape[3]
        _lib.io_dtype(Q)
        _lib.require_streams(Q, {'K': (K, (N, H, L, E)), 'V': (V, (N, H, L, M))})
        _lib.require_f32(Q, {'W': (W, (N, H, E, M))})
        _lib.require_cuda(Q, K, V, W)
        Qc, Kc, Vc = (_lib.unit_inner(t.detach()) for t in (Q, K, V))
        out = torch.empty((N, H, L, M), device=Q.device, dtype=Q.dtype)
        stream, dev = _lib.stream_and_device(Q)
        _lib.check(_lib.lib.fwp_causal_dot_product(
            N, H, L, E, M, _lib.desc(Qc), _lib.desc(Kc), _lib.desc(Vc), _lib.desc(W.detach()),
            _lib.desc(out), _lib.io_dtype(Q), stream, dev), 'causal_dot_product')
        ctx.save_for_backward(Qc, Kc, Vc)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V = ctx.saved_tensors
        N, H, L, E = Q.shape
        M = V.shape[3]
        grad_out = _lib.grad_like(grad_out, Q, (N, H, L, M))
        grad_Q = torch.empty_like(Q, memory_format=torch.contiguous_format)
        grad_K = torch.empty_like(K, memory_format=torch.contiguous_format)
        grad_V = torch.empty_like(V, memory_format=torch.contiguous_format)
        stream, dev = _lib.stream_and_device(Q)
        _lib.check(_lib.lib.fwp_causal_dot_backward(
            N, H, L, E, M, _lib.desc(Q), _lib.desc(K), _lib.desc(V), _lib.desc(grad_out),
            _lib.desc(grad_Q), _lib.desc(grad_K), _lib.desc(grad_V),
            _lib.io_dtype(Q), stream, dev), 'causal_dot_backward')
        return grad_Q, grad_K, grad_V, None


fast_weight_sum = FastWeightSum.apply
