"""GPU parity of the delta-LSTM kernels (v1..v4) against the fp64 CPU oracle and the golden fixtures.
Tolerances: outputs max-abs <= 1e-4; gradients scaled-rel <= 1e-3 vs fp64; on the golden cases the
reference's own thresholds (1e-3 for v1, 1e-2 for v2-v4)."""
import importlib

import pytest
import torch

from oracle import kernels as K
from tests import util

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def op(variant):
    name = 'fast_lstm' if variant == 1 else 'fast_lstm_v%d' % variant
    return getattr(importlib.import_module('recurrent_fwp_b200.' + name), name)


def oracle64(variant, gates, Ws, h0, c0, gy):
    gates = [[t.double() for t in g] for g in gates]
    W = [w.double().clone() for w in Ws]
    st, ce, gy = h0.double().clone(), c0.double().clone(), gy.double()
    N, H, L, d = gates[0][0].shape
    z = lambda: torch.zeros(N, H, L, d, dtype=torch.float64)
    out, nmz, cell, gi, uu, go, voi, vou, voo = (z() for _ in range(9))
    flat = [t for g in gates for t in g]
    K.fast_lstm_forward(variant, *flat, st, ce, *W, out, None if variant == 1 else nmz, cell, gi, uu, go,
                        voi, vou, voo)
    W_end = [w.clone() for w in W]
    od = torch.cat([h0.double(), out[:, :, :-1]], 2) if variant == 1 else nmz
    umc = uu - torch.cat([c0.double(), cell[:, :, :-1]], 2)
    g = [[torch.zeros_like(t) for t in gt] for gt in gates]
    K.fast_lstm_backward(variant, gy,
                         gates[0][1], gates[0][2], gates[0][3], gates[1][1], gates[1][2], gates[1][3],
                         gates[2][1], gates[2][2], gates[2][3], voi, vou, voo, out, od, cell, umc, gi, uu, go,
                         *W, *[t for gt in g for t in gt])
    return out, cell, g, W_end, st, ce


@pytest.mark.parametrize('variant', [1, 2, 3, 4])
@pytest.mark.parametrize('B,H,L,d', [(2, 2, 21, 16), (2, 2, 13, 32), (1, 2, 7, 64), (2, 2, 9, 18), (1, 2, 1, 32)])
def test_parity_vs_oracle(fwp, variant, B, H, L, d):
    gates, gy = util.lstm_inputs(5, B, H, L, d)
    Ws = [torch.randn(B, H, d, d, generator=util.gen(30 + i)) * 0.1 for i in range(3)]
    h0 = torch.randn(B, H, 1, d, generator=util.gen(40))
    c0 = torch.randn(B, H, 1, d, generator=util.gen(41))
    leaves = [[t.clone().to(DEV).requires_grad_() for t in g] for g in gates]
    Wd = [w.to(DEV) for w in Ws]
    hd, cd = h0.to(DEV), c0.to(DEV)
    args = []
    for lv, w in zip(leaves, Wd):
        args += [lv[0], lv[1], lv[2], lv[3], w]
    y, cell = op(variant)(*args, hd, cd)
    W_end = [w.clone() for w in Wd]
    y.backward(gy.to(DEV))
    out, cell_ref, g, S_end, st, ce = oracle64(variant, gates, Ws, h0, c0, gy)
    assert util.max_abs(y, out) <= 1e-4 and util.max_abs(cell, cell_ref) <= 1e-4
    assert util.max_abs(hd, st) <= 1e-4 and util.max_abs(cd, ce) <= 1e-4
    for a, b in zip(W_end, S_end):
        assert util.max_abs(a, b) <= 1e-4
    for lv, gt in zip(leaves, g):
        for leaf, ref in zip(lv, gt):
            assert util.scaled_rel(leaf.grad, ref) <= 1e-3
    for a, b in zip(Wd, Ws):
        assert util.max_abs(a, b) <= 1e-5


@pytest.mark.parametrize('variant', [1, 2, 3, 4])
def test_golden_reference_selftest_case(fwp, variant):
    gd = util.golden('lstm_v%d' % variant)
    gates = [[gd['in_%s0%s' % (p, g)] for p in 'zkvb'] for g in 'iuo']
    N, H, L, d = gates[0][0].shape
    leaves = [[t.to(DEV).requires_grad_() for t in g] for g in gates]
    args = []
    for lv in leaves:
        args += [lv[0], lv[1], lv[2], lv[3], torch.zeros(N, H, d, d, device=DEV)]
    y, _ = op(variant)(*args, torch.zeros(N, H, 1, d, device=DEV), torch.zeros(N, H, 1, d, device=DEV))
    if variant == 1:
        torch.nn.CrossEntropyLoss()(y.permute(2, 0, 1, 3).reshape(-1, d), gd['rand_targets'].to(DEV)).backward()
    else:
        y.sum().backward()
    assert util.max_rel(y, gd['out_LBHd'].permute(1, 2, 0, 3)) < 1e-3
    thr, eps = (1e-3, 1e-6) if variant == 1 else (1e-2, 1e-8)
    for gname, lv in zip('iuo', leaves):
        for pname, leaf in zip('zkvb', lv):
            assert util.max_rel(leaf.grad, gd['grad_%s2%s' % (pname, gname)], eps=eps) < thr
