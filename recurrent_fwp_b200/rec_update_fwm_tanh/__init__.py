"""Recurrent delta net: drop-in for the reference's ``rec_update_fwm_tanh`` module.

Mirrors ``FastWeightRecUpdateTanh`` / ``rec_update_fwm_tanh`` of
algorithmic/rec_update_fwm_tanh/__init__.py:31-139 (same file in language_modeling/src/utils
and reinforcement_learning/torchbeast): ``forward(ctx, qx, kx, vx, bx, R_q, R_k, R_v, r_b, W, h0)``.
The inputs are *pre-activations*: softmax on query/key, sigmoid on beta and the
``R . tanh(y_{t-1})`` feedback are applied inside the kernel.  ``W`` [N,H,d,d] and
``h0`` [N,H,1,d] are updated in place; backward rewinds ``W`` and returns gradients
for the four streams and the four recurrent parameters, ``None`` for W and h0.
"""
import torch

from recurrent_fwp_b200 import _lib


class FastWeightRecUpdateTanh(torch.autograd.Function):
    """Delta-rule fast weight memory with tanh feedback from the previous output."""

    @staticmethod
    def forward(ctx, qx, kx, vx, bx, R_q, R_k, R_v, r_b, W, h0):
        N, H, L, E = qx.shape
        M = vx.shape[3]
        assert E == M, "Current kernel only support this case."
        assert R_q.shape == (1, H, M, M), "Reshape/unsqueeze if needed."
        assert R_k.shape == (1, H, M, M), "Reshape/unsqueeze if needed."
        assert R_v.shape == (1, H, M, M), "Reshape/unsqueeze if needed."
        assert r_b.shape == (1, H, 1, M), "Reshape/unsqueeze if needed."
        if qx.dtype != torch.float32:
            raise TypeError('the recurrent fast-weight kernels take float32 tensors')
        _lib.require_streams(qx, {'kx': (kx, (N, H, L, E)), 'vx': (vx, (N, H, L, M)), 'bx': (bx, (N, H, L, 1))})
        _lib.require_f32(qx, {'R_q': (R_q, (1, H, M, M)), 'R_k': (R_k, (1, H, M, M)), 'R_v': (R_v, (1, H, M, M)),
                              'r_b': (r_b, (1, H, 1, M)), 'W': (W, (N, H, E, M)), 'h0': (h0, (N, H, 1, M))})
        _lib.require_cuda(qx, kx, vx, bx, R_q, R_k, R_v, r_b, W, h0)
        if W.stride(3) != 1 or h0.stride(3) != 1:
            raise RuntimeError('W and h0 must have a unit innermost stride (they are updated in place)')
        qc, kc, vc, bc = (_lib.unit_inner(t.detach()) for t in (qx, kx, vx, bx))
        Rq, Rk, Rv = (t.detach().contiguous() for t in (R_q, R_k, R_v))
        rb = r_b.detach().contiguous()
        kw = dict(device=qx.device, dtype=torch.float32)
        out = torch.empty((N, H, L, M), **kw)
        v_old = torch.empty((N, H, L, M), **kw)
        q_out = torch.empty((N, H, L, E), **kw)
        k_out = torch.empty((N, H, L, E), **kw)
        v_out = torch.empty((N, H, L, M), **kw)
        beta_out = torch.empty((N, H, L, 1), **kw)
        h_init = h0.detach().clone()
        stream, dev = _lib.stream_and_device(qx)
        D = _lib.desc
        _lib.check(_lib.lib.fwp_rec_update_fwm_tanh_forward(
            N, H, L, M, D(qc), D(kc), D(vc), D(bc), D(Rq), D(Rk), D(Rv), D(rb),
            D(q_out), D(k_out), D(v_out), D(beta_out), D(v_old), D(h0.detach()), D(W.detach()), D(out),
            _lib.F32, stream, dev), 'rec_update_fwm_tanh_forward')
        ctx.save_for_backward(out, q_out, k_out, v_out, beta_out, v_old, Rq, Rk, Rv, rb, W, h_init)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (out, Q, K, V, beta, V_old, R_q, R_k, R_v, r_b, W, h0) = ctx.saved_tensors
        N, H, L, M = out.shape
        grad_out = _lib.grad_like(grad_out, out, (N, H, L, M))
        grad_Q = torch.empty_like(Q)
        grad_K = torch.empty_like(K)
        grad_V = torch.empty_like(V)
        grad_beta = torch.empty_like(beta)
        grad_R_q = torch.empty_like(R_q)
        grad_R_k = torch.empty_like(R_k)
        grad_R_v = torch.empty_like(R_v)
        grad_r_b = torch.empty_like(r_b)
        out_delayed = _lib.delayed(out, h0, op=1)       # tanh(cat([h0, out[:, :, :-1]], dim=2)) in one pass
        n_scratch = int(_lib.lib.fwp_rec_update_fwm_tanh_scratch_floats(N, H, M))
        scratch = torch.empty(n_scratch, device=out.device, dtype=torch.float32)
        stream, dev = _lib.stream_and_device(out)
        D = _lib.desc
        import ctypes
        _lib.check(_lib.lib.fwp_rec_update_fwm_tanh_backward(
            N, H, L, M, D(Q), D(K), D(V), D(beta), D(V_old), D(out_delayed), D(grad_out),
            D(R_q), D(R_k), D(R_v), D(r_b), D(W.detach()),
            D(grad_Q), D(grad_K), D(grad_V), D(grad_beta), D(grad_R_q), D(grad_R_k), D(grad_R_v), D(grad_r_b),
            ctypes.cast(scratch.data_ptr(), ctypes.POINTER(ctypes.c_float)), n_scratch,
            _lib.F32, stream, dev), 'rec_update_fwm_tanh_backward')
        return (grad_Q, grad_K, grad_V, grad_beta, grad_R_q, grad_R_k, grad_R_v, grad_r_b, None, None)


rec_update_fwm_tanh = FastWeightRecUpdateTanh.apply
