"""GPU parity of the delta-RNN kernels (v2 and v1) against the CPU oracle and the golden fixtures.
Tolerances: outputs max-abs <= 1e-4; gradients through ``util.check_grads`` (scaled-rel <= 1e-3 vs the fp64
oracle, strict element-wise measure above 4 x the fp32 CPU recurrence's own noise floor, all
figures recorded); the reference's own self-test threshold for these ops is 1e-3."""
import pytest
import torch

from oracle import kernels as K, loops
from tests import util

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def _ops(fwp):
    from recurrent_fwp_b200.fast_weight_rnn_v2 import fast_rnn_v2
    from recurrent_fwp_b200.fast_weight_rnn import fast_rnn
    return {2: fast_rnn_v2, 1: fast_rnn}


def oracle64(ver, z, k, v, b, W0, h0, gy, dtype=torch.float64):
    """Explicit oracle (the kernels' own formulas, epsilon included) in ``dtype``: fp64 is the ground truth,
    fp32 the reference's own arithmetic."""
    z, k, v, b, W0, h0, gy = (t.to(dtype) for t in (z, k, v, b, W0, h0, gy))
    N, H, L, d = z.shape
    W, st = W0.clone(), h0.clone()
    out, nmz, vold = (torch.zeros(N, H, L, d, dtype=dtype) for _ in range(3))
    if ver == 2:
        K.fast_rnn_v2_forward(z, k, v, b, vold, st, W, out, nmz)
        od = nmz
    else:
        K.fast_rnn_forward(z, k, v, b, vold, st, W, out)
        od = torch.cat([h0, out[:, :, :-1]], 2)
    W_end = W.clone()
    g = [torch.zeros_like(t) for t in (z, k, v, b)]
    (K.fast_rnn_v2_backward if ver == 2 else K.fast_rnn_backward)(k, v, b, vold, gy, out, od, W, *g)
    return out, g, W_end, st


@pytest.mark.parametrize('ver', [2, 1])
@pytest.mark.parametrize('B,H,L,d', [(2, 3, 37, 32), (2, 2, 19, 16), (1, 2, 11, 64), (2, 2, 1, 32), (1, 2, 9, 18)])
def test_parity_vs_oracle(fwp, ver, B, H, L, d):
    z, k, v, b, gy = util.rnn_inputs(3, B, H, L, d)
    W0 = torch.randn(B, H, d, d, generator=util.gen(4)) * 0.1
    h0 = torch.randn(B, H, 1, d, generator=util.gen(5))
    leaves = [t.clone().to(DEV).requires_grad_() for t in (z, k, v, b)]
    W, hs = W0.to(DEV), h0.to(DEV)
    y = _ops(fwp)[ver](leaves[0], leaves[1], leaves[2], W, leaves[3], hs)
    W_end = W.clone()
    y.backward(gy.to(DEV))
    out, g, S_end, st = oracle64(ver, z, k, v, b, W0, h0, gy)
    _, g32, _, _ = oracle64(ver, z, k, v, b, W0, h0, gy, torch.float32)
    assert util.max_abs(y, out) <= 1e-4
    assert util.max_abs(W_end, S_end) <= 1e-4 and util.max_abs(hs, st) <= 1e-4
    util.check_grads('rnn_v%d B%d H%d L%d d%d' % (ver, B, H, L, d), 'zkvb', [l.grad for l in leaves], g32, g)
    assert util.max_abs(W, W0) <= 1e-5


@pytest.mark.parametrize('name,ver', [('rnn_v2', 2), ('rnn_v1', 1)])
def test_golden_reference_selftest_case(fwp, name, ver):
    gd = util.golden(name)
    z, k, v, b = (gd['in_' + n] for n in ('z0', 'k0', 'v0', 'beta0'))
    N, H, L, d = z.shape
    leaves = [t.to(DEV).requires_grad_() for t in (z, k, v, b)]
    W, hs = torch.zeros(N, H, d, d, device=DEV), torch.zeros(N, H, 1, d, device=DEV)
    y = _ops(fwp)[ver](leaves[0], leaves[1], leaves[2], W, leaves[3], hs)
    if 'rand_targets' in gd:
        torch.nn.CrossEntropyLoss()(y.permute(2, 0, 1, 3).reshape(-1, d), gd['rand_targets'].to(DEV)).backward()
    else:
        y.sum().backward()
    assert util.max_rel(y, gd['out_LBHd'].permute(1, 2, 0, 3)) < 1e-3
    for leaf, n in zip(leaves, ('z2', 'k2', 'v2', 'beta2')):
        assert util.max_rel(leaf.grad, gd['grad_' + n]) < 1e-3


@pytest.mark.parametrize('ver', [2, 1])
def test_config4_shape_slice(fwp, ver):
    """The fast-weight RNN benchmark shape (B=128,H=4,L=512,d=32) on a batch slice the CPU oracle finishes
    quickly, for both versions."""
    B, H, L, d = 8, 4, 512, 32
    z, k, v, b, gy = util.rnn_inputs(13, B, H, L, d)
    leaves = [t.clone().to(DEV).requires_grad_() for t in (z, k, v, b)]
    W, hs = torch.zeros(B, H, d, d, device=DEV), torch.zeros(B, H, 1, d, device=DEV)
    y = _ops(fwp)[ver](leaves[0], leaves[1], leaves[2], W, leaves[3], hs)
    W_end = W.clone()
    y.backward(gy.to(DEV))
    zero = (torch.zeros(B, H, d, d), torch.zeros(B, H, 1, d))
    out, g, S_end, _ = oracle64(ver, z, k, v, b, *zero, gy)
    out32, g32, _, _ = oracle64(ver, z, k, v, b, *zero, gy, torch.float32)
    util.record('rnn_v%d benchmark shape slice' % ver, y_cuda=util.max_abs(y, out), y_cpu32=util.max_abs(out32, out),
                y_max=out.abs().max().item())
    assert util.max_abs(y, out) <= 1e-4 * max(1.0, out.abs().max().item())
    assert util.max_abs(W_end, S_end) <= 1e-4 * max(1.0, S_end.abs().max().item())
    util.check_grads('rnn_v%d benchmark shape slice' % ver, 'zkvb', [l.grad for l in leaves], g32, g)
    assert util.max_abs(W, zero[0]) <= 1e-5 * max(1.0, S_end.abs().max().item())
