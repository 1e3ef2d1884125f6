"""Delta LSTM v1: drop-in for the reference's ``fast_lstm`` module.

Mirrors ``FastLSTM`` / ``fast_lstm`` of language_modeling/src/utils/fast_lstm/__init__.py:36-205:
``forward(ctx, Zi,Ki,Vi,bi,Wi, Zu,Ku,Vu,bu,Wu, Zo,Ko,Vo,bo,Wo, h0, c0) -> (rnn_out, cell_out)``.
The three fast matrices and ``h0``/``c0`` are updated in place to the end-of-segment
state; backward rewinds the matrices in place, ignores ``grad_cell`` (as the
reference does) and returns 12 gradients and 5 ``None``.

The sibling modules ``fast_lstm_v2`` / ``_v3`` / ``_v4`` are built from the same
factory below; they differ in where softmax / sigmoid / the skip term sit
(language_modeling/src/utils/fast_lstm_v{2,3,4}/__init__.py).
"""
import torch

from recurrent_fwp_b200 import _lib


def make_lstm_function(variant, name):
    def forward(ctx, Zi, Ki, Vi, bi, Wi, Zu, Ku, Vu, bu, Wu, Zo, Ko, Vo, bo, Wo, h0, c0):
        N, H, L, _ = Zi.shape
        M = Vi.shape[3]
        assert Ki.shape == (N, H, L, M)
        assert Vi.shape == (N, H, L, M)
        assert h0.shape == (N, H, 1, M)
        assert Wi.shape == (N, H, M, M)
        if Zi.dtype != torch.float32:
            raise TypeError('the recurrent fast-weight kernels take float32 tensors')
        for g, (z, k, v, b, w) in zip('iuo', ((Zi, Ki, Vi, bi, Wi), (Zu, Ku, Vu, bu, Wu), (Zo, Ko, Vo, bo, Wo))):
            _lib.require_streams(Zi, {'Z' + g: (z, (N, H, L, M)), 'K' + g: (k, (N, H, L, M)),
                                      'V' + g: (v, (N, H, L, M)), 'b' + g: (b, (N, H, L, 1))})
            _lib.require_f32(Zi, {'W' + g: (w, (N, H, M, M))})
            if w.stride(3) != 1:
                raise RuntimeError('the fast matrices must have a unit innermost stride (they are updated in place)')
        _lib.require_f32(Zi, {'h0': (h0, (N, H, 1, M)), 'c0': (c0, (N, H, 1, M))})
        _lib.require_cuda(Zi, Ki, Vi, bi, Wi, Zu, Ku, Vu, bu, Wu, Zo, Ko, Vo, bo, Wo, h0, c0)
        Z = [_lib.unit_inner(t.detach()) for t in (Zi, Zu, Zo)]
        K = [_lib.unit_inner(t.detach()) for t in (Ki, Ku, Ko)]
        V = [_lib.unit_inner(t.detach()) for t in (Vi, Vu, Vo)]
        B = [_lib.unit_inner(t.detach()) for t in (bi, bu, bo)]
        W = [Wi, Wu, Wo]
        kw = dict(device=Zi.device, dtype=torch.float32)
        new = lambda: torch.empty((N, H, L, M), **kw)
        rnn_out, cell_out = new(), new()
        gates = [new(), new(), new()]          # gate_i, update_u, gate_o
        v_old = [new(), new(), new()]
        out_del_nmz = new() if variant != 1 else None
        h_init = h0.detach().clone()
        c_init = c0.detach().clone()
        stream, dev = _lib.stream_and_device(Zi)
        D, D3 = _lib.desc, _lib.desc3
        _lib.check(_lib.lib.fwp_fast_lstm_forward(
            variant, N, H, L, M, D3(Z), D3(K), D3(V), D3(B), D(h0.detach()), D(c0.detach()),
            D3([w.detach() for w in W]), D(rnn_out), D(out_del_nmz), D(cell_out), D3(gates), D3(v_old),
            _lib.F32, stream, dev), name + '_forward')
        saved = [rnn_out, cell_out] + gates + K + V + B + W + v_old + [h_init, c_init]
        if variant != 1:
            saved.append(out_del_nmz)
        ctx.save_for_backward(*saved)
        return rnn_out, cell_out

    def backward(ctx, grad_out, grad_cell):
        t = ctx.saved_tensors
        rnn_out, cell_out = t[0], t[1]
        gates, K, V, B, W, v_old = list(t[2:5]), list(t[5:8]), list(t[8:11]), list(t[11:14]), list(t[14:17]), list(t[17:20])
        h0, c0 = t[20], t[21]
        N, H, L, M = rnn_out.shape
        grad_out = _lib.grad_like(grad_out, rnn_out, (N, H, L, M))
        # cat([h0, out[:, :, :-1]]) and update - cat([c0, cell[:, :, :-1]]), one pass each
        out_delayed = _lib.delayed(rnn_out, h0) if variant == 1 else t[22]
        u_minus_c = _lib.delayed(cell_out, c0, minuend=gates[1])
        gZ = [torch.empty_like(rnn_out) for _ in range(3)]
        gK = [torch.empty_like(rnn_out) for _ in range(3)]
        gV = [torch.empty_like(rnn_out) for _ in range(3)]
        gB = [torch.empty((N, H, L, 1), device=rnn_out.device, dtype=torch.float32) for _ in range(3)]
        stream, dev = _lib.stream_and_device(rnn_out)
        D, D3 = _lib.desc, _lib.desc3
        _lib.check(_lib.lib.fwp_fast_lstm_backward(
            variant, N, H, L, M, D(grad_out), D3(K), D3(V), D3(B), D3(v_old), D(rnn_out), D(out_delayed),
            D(cell_out), D(u_minus_c), D3(gates), D3([w.detach() for w in W]),
            D3(gZ), D3(gK), D3(gV), D3(gB), _lib.F32, stream, dev), name + '_backward')
        return (gZ[0], gK[0], gV[0], gB[0], None,
                gZ[1], gK[1], gV[1], gB[1], None,
                gZ[2], gK[2], gV[2], gB[2], None,
                None, None)

    cls = type(name, (torch.autograd.Function,), {
        '__doc__': 'Fast LSTM with the FWM update rule (variant %d).' % variant,
        'forward': staticmethod(forward), 'backward': staticmethod(backward)})
    return cls


FastLSTM = make_lstm_function(1, 'FastLSTM')
fast_lstm = FastLSTM.apply
