"""CPU checks of the oracle: explicit kernels vs autograd loops (fp64), and both
against the golden fixtures captured from the reference's own self-test loops."""
import pytest
import torch

from oracle import kernels as K, loops
from tests import util

DT = torch.float64


def _z(*s, dtype=DT):
    return torch.zeros(*s, dtype=dtype)


def test_delta_explicit_matches_autograd_fp64():
    N, H, L, E, M = 2, 3, 9, 6, 4
    q, k, v, b, gy = util.delta_inputs(1, N, H, L, E, M, DT)
    W0 = torch.randn(N, H, E, M, dtype=DT, generator=util.gen(2)) * 0.1
    leaves = [t.clone().requires_grad_() for t in (q, k, v, b)]
    y, S = loops.delta_rule(*leaves, W0)
    (y * gy).sum().backward()
    W, out, vo, vi = W0.clone(), _z(N, H, L, M), _z(N, H, L, M), _z(N, H, L, M)
    K.fast_weight_forward(q, k, v, b, vo, vi, W, out)
    assert util.max_abs(out, y) < 1e-12 and util.max_abs(W, S) < 1e-12
    g = [_z(*t.shape) for t in (q, k, v, b)]
    K.fast_weight_backward(q, k, v, b, vo, vi, gy, W, *g)
    for got, leaf in zip(g, leaves):
        assert util.max_abs(got, leaf.grad) < 1e-12
    assert util.max_abs(W, W0) < 1e-12      # rewound to the start-of-segment state


def test_rec_delta_explicit_matches_autograd_fp64():
    N, H, L, d = 2, 3, 7, 5
    ins = [t.to(DT) for t in util.rec_inputs(3, N, H, L, d)]
    gy = ins[-1]
    W0 = torch.randn(N, H, d, d, dtype=DT, generator=util.gen(4)) * 0.1
    h0 = torch.randn(N, H, 1, d, dtype=DT, generator=util.gen(5))
    leaves = [t.clone().requires_grad_() for t in ins[:8]]
    y, S, hL = loops.rec_delta(*leaves, W0, h0)
    (y * gy).sum().backward()
    W, st = W0.clone(), h0.clone()
    qo, ko, vo_, out, vold = (_z(N, H, L, d) for _ in range(5))
    bo = _z(N, H, L, 1)
    K.rec_update_fwm_tanh_forward(*ins[:8], qo, ko, vo_, bo, vold, st, W, out)
    assert util.max_abs(out, y) < 1e-12 and util.max_abs(st, hL) < 1e-12
    od = torch.tanh(torch.cat([h0, out[:, :, :-1]], 2))
    g = [_z(*t.shape) for t in ins[:8]]
    K.rec_update_fwm_tanh_backward(qo, ko, vo_, bo, vold, od, gy, *ins[4:8], W, *g)
    for got, leaf in zip(g, leaves):
        assert util.max_abs(got, leaf.grad) < 1e-11
    assert util.max_abs(W, W0) < 1e-12


@pytest.mark.parametrize('ver', [1, 2])
def test_rnn_explicit_matches_autograd_fp64(ver, monkeypatch):
    monkeypatch.setattr(K, 'EPS_SOFTMAX', 0.0)   # the backward formulas ignore the epsilon
    N, H, L, d = 2, 3, 7, 5
    z, k, v, b, gy = [t.to(DT) for t in util.rnn_inputs(6, N, H, L, d)]
    W0 = torch.randn(N, H, d, d, dtype=DT, generator=util.gen(7)) * 0.1
    h0 = torch.randn(N, H, 1, d, dtype=DT, generator=util.gen(8))
    leaves = [t.clone().requires_grad_() for t in (z, k, v, b)]
    if ver == 2:
        y, S, hL = loops.delta_rnn_v2(leaves[0], leaves[1], leaves[2], W0, leaves[3], h0, eps_softmax=False)
    else:
        y, S, hL = loops.delta_rnn_v1(leaves[0], leaves[1], leaves[2], W0, leaves[3], h0)
    (y * gy).sum().backward()
    W, st = W0.clone(), h0.clone()
    out, nmz, vold = (_z(N, H, L, d) for _ in range(3))
    if ver == 2:
        K.fast_rnn_v2_forward(z, k, v, b, vold, st, W, out, nmz)
        od = nmz
    else:
        K.fast_rnn_forward(z, k, v, b, vold, st, W, out)
        od = torch.cat([h0, out[:, :, :-1]], 2)
    assert util.max_abs(out, y) < 1e-12 and util.max_abs(st, hL) < 1e-12
    g = [_z(*t.shape) for t in (z, k, v, b)]
    (K.fast_rnn_v2_backward if ver == 2 else K.fast_rnn_backward)(k, v, b, vold, gy, out, od, W, *g)
    for got, leaf in zip(g, leaves):
        assert util.max_abs(got, leaf.grad) < 1e-12
    assert util.max_abs(W, W0) < 1e-12


@pytest.mark.parametrize('variant', [1, 2, 3, 4])
def test_lstm_explicit_matches_autograd_fp64(variant, monkeypatch):
    monkeypatch.setattr(K, 'EPS_SOFTMAX', 0.0)
    N, H, L, d = 2, 2, 6, 5
    gates, gy = util.lstm_inputs(9, N, H, L, d)
    gates = [[t.to(DT) for t in g] for g in gates]
    gy = gy.to(DT)
    Ws = [torch.randn(N, H, d, d, dtype=DT, generator=util.gen(10 + i)) * 0.1 for i in range(3)]
    h0 = torch.randn(N, H, 1, d, dtype=DT, generator=util.gen(20))
    c0 = torch.randn(N, H, 1, d, dtype=DT, generator=util.gen(21))
    leaves = [[t.clone().requires_grad_() for t in g] for g in gates]
    args = []
    for g, W in zip(leaves, Ws):
        args += [g[0], g[1], g[2], g[3], W]
    hs, cs, Sf, hL, cL = loops.delta_lstm(variant, *args, h0, c0, eps_softmax=False)
    (hs * gy).sum().backward()
    W = [w.clone() for w in Ws]
    st, ce = h0.clone(), c0.clone()
    out, nmz, cell, gi, uu, go, voi, vou, voo = (_z(N, H, L, d) for _ in range(9))
    flat = [t for g in gates for t in g]   # Zi,Ki,Vi,bi, Zu,...
    K.fast_lstm_forward(variant, *flat, st, ce, *W, out, None if variant == 1 else nmz, cell, gi, uu, go,
                        voi, vou, voo)
    assert util.max_abs(out, hs) < 1e-12 and util.max_abs(cell, cs) < 1e-12
    assert util.max_abs(st, hL) < 1e-12 and util.max_abs(ce, cL) < 1e-12
    od = torch.cat([h0, out[:, :, :-1]], 2) if variant == 1 else nmz
    umc = uu - torch.cat([c0, cell[:, :, :-1]], 2)
    g = [[_z(*t.shape) for t in gt] for gt in gates]
    K.fast_lstm_backward(variant, gy,
                         gates[0][1], gates[0][2], gates[0][3], gates[1][1], gates[1][2], gates[1][3],
                         gates[2][1], gates[2][2], gates[2][3], voi, vou, voo, out, od, cell, umc, gi, uu, go,
                         *W, *[t for gt in g for t in gt])
    for gt, lt in zip(g, leaves):
        for got, leaf in zip(gt, lt):
            assert util.max_abs(got, leaf.grad) < 1e-12
    for a, b in zip(W, Ws):
        assert util.max_abs(a, b) < 1e-12


# ---- golden fixtures: inputs and results of the reference's own self-test loops ----

def test_golden_delta():
    gd = util.golden('delta')
    q, k, v, b = (gd['in_' + n] for n in ('q0', 'k0', 'v0', 'beta0'))
    N, H, L, E = q.shape
    M = v.shape[3]
    ref_out = gd['out_LBHd'].permute(1, 2, 0, 3)
    # autograd-loop layer
    leaves = [t.clone().requires_grad_() for t in (q, k, v, b)]
    y, _ = loops.delta_rule(*leaves, torch.zeros(N, H, E, M))
    y.sum().backward()
    assert util.max_rel(y, ref_out) < 1e-4
    for leaf, n in zip(leaves, ('q2', 'k2', 'v2', 'beta2')):
        assert util.max_rel(leaf.grad, gd['grad_' + n]) < 1e-3
    # explicit-kernel layer
    W, out, vo, vi = torch.zeros(N, H, E, M), torch.zeros(N, H, L, M), torch.zeros(N, H, L, M), torch.zeros(N, H, L, M)
    K.fast_weight_forward(q, k, v, b, vo, vi, W, out)
    assert util.max_rel(out, ref_out) < 1e-4
    g = [torch.zeros_like(t) for t in (q, k, v, b)]
    K.fast_weight_backward(q, k, v, b, vo, vi, torch.ones_like(out), W, *g)
    for got, n in zip(g, ('q2', 'k2', 'v2', 'beta2')):
        assert util.max_rel(got, gd['grad_' + n]) < 1e-3


def test_golden_rec_delta():
    gd = util.golden('rec_delta')
    ins = [gd['in_' + n] for n in ('q0', 'k0', 'v0', 'beta0', 'R_q0', 'R_k0', 'R_v0', 'r_b0')]
    N, H, L, d = ins[0].shape
    ref_out = gd['out_LBHd'].permute(1, 2, 0, 3)
    leaves = [t.clone().requires_grad_() for t in ins]
    y, _, _ = loops.rec_delta(*leaves, torch.zeros(N, H, d, d), torch.zeros(N, H, 1, d))
    y.sum().backward()
    assert util.max_rel(y, ref_out) < 1e-3
    for leaf, n in zip(leaves, ('q2', 'k2', 'v2', 'beta2', 'Rq2', 'Rk2', 'Rv2', 'rb2')):
        assert util.max_rel(leaf.grad, gd['grad_' + n]) < 1e-2   # the reference's own threshold for this op


@pytest.mark.parametrize('name', ['rnn_v1', 'rnn_v2'])
def test_golden_rnn(name):
    gd = util.golden(name)
    z, k, v, b = (gd['in_' + n] for n in ('z0', 'k0', 'v0', 'beta0'))
    N, H, L, d = z.shape
    ref_out = gd['out_LBHd'].permute(1, 2, 0, 3)
    leaves = [t.clone().requires_grad_() for t in (z, k, v, b)]
    W0, h0 = torch.zeros(N, H, d, d), torch.zeros(N, H, 1, d)
    if name == 'rnn_v2':
        y, _, _ = loops.delta_rnn_v2(leaves[0], leaves[1], leaves[2], W0, leaves[3], h0, eps_softmax=False)
    else:
        y, _, _ = loops.delta_rnn_v1(leaves[0], leaves[1], leaves[2], W0, leaves[3], h0)
    if 'rand_targets' in gd:   # v1's outputs are softmax rows: its self-test uses cross-entropy
        torch.nn.CrossEntropyLoss()(y.permute(2, 0, 1, 3).reshape(-1, d), gd['rand_targets']).backward()
    else:
        y.sum().backward()
    assert util.max_rel(y, ref_out) < 1e-3
    for leaf, n in zip(leaves, ('z2', 'k2', 'v2', 'beta2')):
        assert util.max_rel(leaf.grad, gd['grad_' + n]) < 1e-3


@pytest.mark.parametrize('variant', [1, 2, 3, 4])
def test_golden_lstm(variant):
    gd = util.golden('lstm_v%d' % variant)
    gates = [[gd['in_%s0%s' % (p, g)] for p in 'zkvb'] for g in 'iuo']
    N, H, L, d = gates[0][0].shape
    ref_out = gd['out_LBHd'].permute(1, 2, 0, 3)
    leaves = [[t.clone().requires_grad_() for t in g] for g in gates]
    args = []
    for g in leaves:
        args += [g[0], g[1], g[2], g[3], torch.zeros(N, H, d, d)]
    hs, _, _, _, _ = loops.delta_lstm(variant, *args, torch.zeros(N, H, 1, d), torch.zeros(N, H, 1, d),
                                      eps_softmax=False)
    if variant == 1:   # the reference's v1 self-test uses cross-entropy on stored random targets
        loss = torch.nn.CrossEntropyLoss()(hs.permute(2, 0, 1, 3).reshape(-1, d), gd['rand_targets'])
    else:
        loss = hs.sum()
    loss.backward()
    assert util.max_rel(hs, ref_out) < 1e-3
    thr = 1e-3 if variant == 1 else 1e-2
    for gname, lv in zip('iuo', leaves):
        for p, leaf in zip('zkvb', lv):
            assert util.max_rel(leaf.grad, gd['grad_%s2%s' % (p, gname)], eps=1e-6 if variant == 1 else 1e-8) < thr


def test_golden_sum():
    gd = util.golden('sum')
    q, k, v = gd['in_q0'], gd['in_k0'], gd['in_v0']
    N, H, L, E = q.shape
    M = v.shape[3]
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    y, _ = loops.sum_rule(*leaves, torch.zeros(N, H, E, M))
    y.sum().backward()
    ref = gd['out_LBHd']
    ref = ref.permute(1, 2, 0, 3) if ref.shape[0] == L and ref.shape != y.shape else ref
    assert util.max_rel(y, ref.reshape(y.shape) if ref.shape != y.shape else ref) < 1e-3
    for leaf, n in zip(leaves, ('q2', 'k2', 'v2')):
        assert util.max_rel(leaf.grad, gd['grad_' + n]) < 1e-3
