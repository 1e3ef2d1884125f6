"""Delta RNN v2: drop-in for the reference's ``fast_weight_rnn_v2`` module.

Mirrors ``FastRNNv2`` / ``fast_rnn_v2`` of algorithmic/fast_weight_rnn_v2/__init__.py:29-121
(argument order ``Z, K, V, W, beta, h0`` -- W before beta).  Per step the fast
matrix is written by the delta rule from (k, v, beta) and read with the
softmax-normalised previous hidden state: ``h_t = W_t softmax_eps(h_{t-1}) + z_t``.
``W`` [N,H,d,d] and ``h0`` [N,H,1,d] are updated in place to the end-of-segment
state; backward rewinds ``W`` in place and returns no gradient for W and h0.
"""
import torch

from recurrent_fwp_b200 import _lib


def _check(Z, K, V, W, beta, h0):
    N, H, L, _ = Z.shape
    M = V.shape[3]
    assert K.shape == (N, H, L, M)
    assert V.shape == (N, H, L, M)
    assert h0.shape == (N, H, 1, M)
    assert W.shape == (N, H, M, M)
    if Z.dtype != torch.float32:
        raise TypeError('the recurrent fast-weight kernels take float32 tensors')
    _lib.require_streams(Z, {'Z': (Z, (N, H, L, M)), 'K': (K, (N, H, L, M)), 'V': (V, (N, H, L, M)),
                             'beta': (beta, (N, H, L, 1))})
    _lib.require_f32(Z, {'W': (W, (N, H, M, M)), 'h0': (h0, (N, H, 1, M))})
    _lib.require_cuda(Z, K, V, W, beta, h0)
    if W.stride(3) != 1 or h0.stride(3) != 1:
        raise RuntimeError('W and h0 must have a unit innermost stride (they are updated in place)')
    return N, H, L, M


class FastRNNv2(torch.autograd.Function):
    """Fast RNN with the FWM update rule (v2: softmax on the delayed state)."""

    @staticmethod
    def forward(ctx, Z, K, V, W, beta, h0):
        N, H, L, M = _check(Z, K, V, W, beta, h0)
        Zc, Kc, Vc, bc = (_lib.unit_inner(t.detach()) for t in (Z, K, V, beta))
        kw = dict(device=Z.device, dtype=torch.float32)
        rnn_out = torch.empty((N, H, L, M), **kw)
        rnn_out_nmz = torch.empty((N, H, L, M), **kw)
        V_old = torch.empty((N, H, L, M), **kw)
        stream, dev = _lib.stream_and_device(Z)
        D = _lib.desc
        _lib.check(_lib.lib.fwp_fast_rnn_v2_forward(
            N, H, L, M, D(Zc), D(Kc), D(Vc), D(bc), D(V_old), D(h0.detach()), D(W.detach()),
            D(rnn_out), D(rnn_out_nmz), _lib.F32, stream, dev), 'fast_rnn_v2_forward')
        ctx.save_for_backward(rnn_out, rnn_out_nmz, Kc, Vc, bc, V_old, W)
        return rnn_out

    @staticmethod
    def backward(ctx, grad_out):
        rnn_out, rnn_out_nmz, K, V, beta, V_old, W = ctx.saved_tensors
        N, H, L, M = K.shape
        grad_out = _lib.grad_like(grad_out, rnn_out, (N, H, L, M))
        grad_Z = torch.empty_like(rnn_out)
        grad_K = torch.empty_like(rnn_out)
        grad_V = torch.empty_like(rnn_out)
        grad_beta = torch.empty((N, H, L, 1), device=K.device, dtype=torch.float32)
        stream, dev = _lib.stream_and_device(K)
        D = _lib.desc
        _lib.check(_lib.lib.fwp_fast_rnn_v2_backward(
            N, H, L, M, D(K), D(V), D(beta), D(V_old), D(grad_out), D(rnn_out), D(rnn_out_nmz),
            D(W.detach()), D(grad_Z), D(grad_K), D(grad_V), D(grad_beta), _lib.F32, stream, dev),
            'fast_rnn_v2_backward')
        return grad_Z, grad_K, grad_V, None, grad_beta, None


fast_rnn_v2 = FastRNNv2.apply
