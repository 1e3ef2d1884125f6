"""Delta RNN v1: drop-in for the reference's ``fast_weight_rnn`` module.

Mirrors ``FastRNN`` / ``fast_rnn`` of language_modeling/src/utils/fast_weight_rnn/__init__.py:41-118
(argument order ``Z, K, V, W, beta, h0``): ``h_t = softmax(W_t h_{t-1} + z_t)`` with
``W_t`` written by the delta rule.  ``W`` and ``h0`` are updated in place; backward
rewinds ``W`` and returns no gradient for W and h0.
"""
import torch

from recurrent_fwp_b200 import _lib
from recurrent_fwp_b200.fast_weight_rnn_v2 import _check


class FastRNN(torch.autograd.Function):
    """Fast RNN with the FWM update rule (v1: softmax on the output)."""

    @staticmethod
    def forward(ctx, Z, K, V, W, beta, h0):
        N, H, L, M = _check(Z, K, V, W, beta, h0)
        Zc, Kc, Vc, bc = (_lib.unit_inner(t.detach()) for t in (Z, K, V, beta))
        kw = dict(device=Z.device, dtype=torch.float32)
        rnn_out = torch.empty((N, H, L, M), **kw)
        V_old = torch.empty((N, H, L, M), **kw)
        h_init = h0.detach().clone()
        stream, dev = _lib.stream_and_device(Z)
        D = _lib.desc
        _lib.check(_lib.lib.fwp_fast_rnn_forward(
            N, H, L, M, D(Zc), D(Kc), D(Vc), D(bc), D(V_old), D(h0.detach()), D(W.detach()),
            D(rnn_out), _lib.F32, stream, dev), 'fast_rnn_forward')
        ctx.save_for_backward(rnn_out, Kc, Vc, bc, V_old, W, h_init)
        return rnn_out

    @staticmethod
    def backward(ctx, grad_out):
        rnn_out, K, V, beta, V_old, W, h0 = ctx.saved_tensors
        N, H, L, M = K.shape
        grad_out = _lib.grad_like(grad_out, rnn_out, (N, H, L, M))
        rnn_out_delayed = _lib.delayed(rnn_out, h0)      # cat([h0, rnn_out[:, :, :-1]], dim=2) in one pass
        grad_Z = torch.empty_like(rnn_out)
        grad_K = torch.empty_like(rnn_out)
        grad_V = torch.empty_like(rnn_out)
        grad_beta = torch.empty((N, H, L, 1), device=K.device, dtype=torch.float32)
        stream, dev = _lib.stream_and_device(K)
        D = _lib.desc
        _lib.check(_lib.lib.fwp_fast_rnn_backward(
            N, H, L, M, D(K), D(V), D(beta), D(V_old), D(grad_out), D(rnn_out), D(rnn_out_delayed),
            D(W.detach()), D(grad_Z), D(grad_K), D(grad_V), D(grad_beta), _lib.F32, stream, dev),
            'fast_rnn_backward')
        return grad_Z, grad_K, grad_V, None, grad_beta, None


fast_rnn = FastRNN.apply
