"""GPU parity of the delta-LSTM kernels (v1..v4) against the fp64 CPU oracle and the golden fixtures.
Tolerances: outputs max-abs <= 1e-4; gradients through ``util.check_grads`` (scaled-rel <= 1e-3 vs fp64,
strict element-wise measure above 4 x the fp32 CPU recurrence's own noise floor, all figures
recorded); on the golden cases the reference's own thresholds (1e-3 for v1, 1e-2 for v2-v4)."""
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


def oracle64(variant, gates, Ws, h0, c0, gy, dtype=torch.float64):
    """The explicit recurrences in ``dtype``: fp64 is the ground truth, fp32 the reference's own arithmetic."""
    gates = [[t.to(dtype) for t in g] for g in gates]
    W = [w.to(dtype).clone() for w in Ws]
    h0, c0 = h0.to(dtype), c0.to(dtype)
    st, ce, gy = h0.clone(), c0.clone(), gy.to(dtype)
    N, H, L, d = gates[0][0].shape
    z = lambda: torch.zeros(N, H, L, d, dtype=dtype)
    out, nmz, cell, gi, uu, go, voi, vou, voo = (z() for _ in range(9))
    flat = [t for g in gates for t in g]
    K.fast_lstm_forward(variant, *flat, st, ce, *W, out, None if variant == 1 else nmz, cell, gi, uu, go,
                        voi, vou, voo)
    W_end = [w.clone() for w in W]
    od = torch.cat([h0, out[:, :, :-1]], 2) if variant == 1 else nmz
    umc = uu - torch.cat([c0, cell[:, :, :-1]], 2)
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
    g32 = oracle64(variant, gates, Ws, h0, c0, gy, torch.float32)[2]
    for gname, lv, gt, gt32 in zip('iuo', leaves, g, g32):
        util.check_grads('lstm_v%d B%d H%d L%d d%d gate %s' % (variant, B, H, L, d, gname), 'zkvb',
                         [l.grad for l in lv], gt32, gt)
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


@pytest.mark.parametrize('variant', [1, 2, 3, 4])
def test_benchmark_shape_slice(fwp, variant):
    """The fast-LSTM benchmark shape (B=128,H=4,L=512,d=32) on a batch slice: 512 steps through the six-matrix
    backward, zero start states, all outputs, end states, gradients and the rewound matrices."""
    B, H, L, d = 4, 4, 512, 32
    gates, gy = util.lstm_inputs(9, B, H, L, d)
    Ws = [torch.zeros(B, H, d, d) for _ in range(3)]
    h0, c0 = torch.zeros(B, H, 1, d), torch.zeros(B, H, 1, d)
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
    out32, cell32, g32 = oracle64(variant, gates, Ws, h0, c0, gy, torch.float32)[:3]
    scale = max(1.0, out.abs().max().item(), cell_ref.abs().max().item())
    util.record('lstm_v%d benchmark shape slice' % variant, y_cuda=util.max_abs(y, out), y_cpu32=util.max_abs(out32, out),
                cell_cuda=util.max_abs(cell, cell_ref), cell_cpu32=util.max_abs(cell32, cell_ref), scale=scale)
    assert util.max_abs(y, out) <= 1e-4 * scale and util.max_abs(cell, cell_ref) <= 1e-4 * scale
    assert util.max_abs(hd, st) <= 1e-4 * scale and util.max_abs(cd, ce) <= 1e-4 * scale
    for a, b in zip(W_end, S_end):
        assert util.max_abs(a, b) <= 1e-4 * max(1.0, b.abs().max().item())
    for gname, lv, gt, gt32 in zip('iuo', leaves, g, g32):
        util.check_grads('lstm_v%d benchmark shape slice gate %s' % (variant, gname), 'zkvb',
                         [l.grad for l in lv], gt32, gt)
    for a, b in zip(Wd, S_end):
        assert util.max_abs(a, Ws[0]) <= 1e-5 * max(1.0, b.abs().max().item())
