"""The autograd wrappers reject streams, states and parameters whose dtype, shape or device
differs from what the kernels will assume -- on the host, before any pointer reaches the C ABI
(which sees raw pointers plus one element type and cannot check).  CPU tensors are enough to
reach every rejection: the dtype and shape checks run before the CUDA-only check."""
import pytest
import torch

import recurrent_fwp_b200 as fwp

N, H, L, d = 2, 3, 5, 16


def streams(dtype=torch.float32):
    return [torch.rand(N, H, L, d, dtype=dtype) for _ in range(3)] + [torch.rand(N, H, L, 1, dtype=dtype)]


def test_delta_rule_rejects_a_mixed_dtype_stream():
    q, k, v, b = streams()
    W = torch.zeros(N, H, d, d)
    # the autocast case: fp32 q/k (a sum promoted them) beside a bf16 v
    with pytest.raises(TypeError, match='V is torch.bfloat16'):
        fwp.fast_weight_delta(q, k, v.bfloat16(), b, W)
    with pytest.raises(TypeError, match='beta'):
        fwp.fast_weight_delta(q, k, v, b.half(), W)
    with pytest.raises(TypeError, match='float32 or bfloat16'):
        fwp.fast_weight_delta(q.double(), k.double(), v.double(), b.double(), W)


def test_delta_rule_rejects_short_or_misshapen_streams():
    q, k, v, b = streams()
    W = torch.zeros(N, H, d, d)
    with pytest.raises(RuntimeError, match='K has shape'):
        fwp.fast_weight_delta(q, k[:, :, :-1], v, b, W)
    with pytest.raises(RuntimeError, match='beta has shape'):
        fwp.fast_weight_delta(q, k, v, b[..., 0], W)
    with pytest.raises(RuntimeError, match='W has shape'):
        fwp.fast_weight_delta(q, k, v, b, torch.zeros(N, H, d, d + 1))
    with pytest.raises(TypeError, match='W must be float32'):
        fwp.fast_weight_delta(q, k, v, b, W.bfloat16())
    # consistent arguments reach the CUDA-only check
    with pytest.raises(RuntimeError, match='no CPU path'):
        fwp.fast_weight_delta(q, k, v, b, W)


def test_sum_rule_rejections():
    q, k, v, _ = streams()
    W = torch.zeros(N, H, d, d)
    with pytest.raises(TypeError, match='V is'):
        fwp.fast_weight_sum(q, k, v.bfloat16(), W)
    with pytest.raises(RuntimeError, match='K has shape'):
        fwp.fast_weight_sum(q, k[:, :1], v, W)
    with pytest.raises(RuntimeError, match='no CPU path'):
        fwp.fast_weight_sum(q, k, v, W)


def test_recurrent_delta_net_rejections():
    q, k, v, b = streams()
    R = [torch.rand(1, H, d, d) for _ in range(3)]
    rb = torch.rand(1, H, 1, d)
    W, h0 = torch.zeros(N, H, d, d), torch.zeros(N, H, 1, d)
    with pytest.raises(TypeError, match='vx is'):
        fwp.rec_update_fwm_tanh(q, k, v.bfloat16(), b, *R, rb, W, h0)
    with pytest.raises(TypeError, match='R_k must be float32'):
        fwp.rec_update_fwm_tanh(q, k, v, b, R[0], R[1].double(), R[2], rb, W, h0)
    with pytest.raises(RuntimeError, match='bx has shape'):
        fwp.rec_update_fwm_tanh(q, k, v, b[:, :, :2], *R, rb, W, h0)
    with pytest.raises(RuntimeError, match='h0 has shape'):
        fwp.rec_update_fwm_tanh(q, k, v, b, *R, rb, W, torch.zeros(N, H, d))
    with pytest.raises(TypeError, match='W must be float32'):
        fwp.rec_update_fwm_tanh(q, k, v, b, *R, rb, W.double(), h0)
    with pytest.raises(RuntimeError, match='no CPU path'):
        fwp.rec_update_fwm_tanh(q, k, v, b, *R, rb, W, h0)


@pytest.mark.parametrize('op', ['fast_rnn_v2', 'fast_rnn'])
def test_delta_rnn_rejections(op):
    f = getattr(fwp, op)
    z, k, v, b = streams()
    W, h0 = torch.zeros(N, H, d, d), torch.zeros(N, H, 1, d)
    with pytest.raises(TypeError, match='K is'):
        f(z, k.bfloat16(), v, W, b, h0)
    with pytest.raises(RuntimeError, match='beta has shape'):
        f(z, k, v, W, b[:, :, :-1], h0)
    with pytest.raises(TypeError, match='h0 must be float32'):
        f(z, k, v, W, b, h0.half())
    with pytest.raises(RuntimeError, match='no CPU path'):
        f(z, k, v, W, b, h0)


@pytest.mark.parametrize('op', ['fast_lstm', 'fast_lstm_v2', 'fast_lstm_v3', 'fast_lstm_v4'])
def test_delta_lstm_rejections(op):
    f = getattr(fwp, op)

    def args():
        a = []
        for _ in range(3):
            a += streams() + [torch.zeros(N, H, d, d)]
        return a + [torch.zeros(N, H, 1, d), torch.zeros(N, H, 1, d)]
    a = args()
    a[7] = a[7].bfloat16()          # Vu
    with pytest.raises(TypeError, match='Vu is'):
        f(*a)
    a = args()
    a[13] = a[13][:, :, :-1]        # bo, one step short
    with pytest.raises(RuntimeError, match='bo has shape'):
        f(*a)
    a = args()
    a[9] = a[9].double()            # Wu
    with pytest.raises(TypeError, match='Wu must be float32'):
        f(*a)
    a = args()
    a[16] = torch.zeros(N, H, d)    # c0
    with pytest.raises(RuntimeError, match='c0 has shape'):
        f(*a)
    with pytest.raises(RuntimeError, match='no CPU path'):
        f(*args())


def test_incoming_gradient_is_checked():
    from recurrent_fwp_b200 import _lib
    ref = torch.zeros(N, H, L, d)
    with pytest.raises(RuntimeError, match='grad_out'):
        _lib.grad_like(torch.zeros(N, H, L - 1, d), ref, (N, H, L, d))
    g = _lib.grad_like(torch.zeros(N, H, L, d, dtype=torch.bfloat16).transpose(2, 3).transpose(2, 3), ref, (N, H, L, d))
    assert g.dtype == torch.float32 and g.stride(-1) == 1
