"""The d = 32 execution plans of the recurrent families against the general kernels on the same inputs.

The short-chain / multi-warp kernels (``rec_fwd_warp32_kernel``, ``rec_bwd_roles32_kernel``, ``rnn_bwd_roles32_kernel``,
``lstm_fwd_gates32_kernel``, ``lstm_bwd_roles32_kernel``) are the default at a head dimension of exactly 32 with
16-byte aligned rows.  Each test runs the op twice, with the plan on and switched off through ``fwp_tune``, checks
which kernel ran (``fwp_last_kernel``) and that outputs, end states, rewound states and gradients agree to 2e-5 of
the tensor's scale (both paths are fp32 and differ in summation order and in the exp / tanh forms); sequence counts
that are not multiples of the sequences per CTA and lengths on both sides of the chunk boundaries are covered.
Rows that are not 16-byte aligned must take the general kernel and still give the same numbers.  Parity with the
fp64 oracle is in test_rnn_gpu.py, test_lstm_gpu.py and test_rec_delta_gpu.py (their d = 32 cases run these plans)."""
import importlib

import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'
SHAPES = [(1, 3, 15), (2, 2, 16), (1, 1, 17), (2, 4, 33), (1, 2, 1)]
D = 32
TOL = 2e-5


def close(a, b):
    scale = max(b.abs().max().item(), 1e-6)
    return (a - b).abs().max().item() <= TOL * scale


def note_backward_kernel(leaf, into):
    """fwp_last_kernel is per host thread and autograd runs backward on its own thread: ask from inside it."""
    from recurrent_fwp_b200 import _lib
    leaf.register_hook(lambda g: into.append(_lib.last_kernel()))


def misalign(t):
    """The same values behind rows that start 4 bytes off a 16-byte boundary (unit inner stride kept)."""
    wide = torch.zeros(*t.shape[:-1], t.shape[-1] + 4, device=t.device, dtype=t.dtype)
    view = wide[..., 1:t.shape[-1] + 1]
    view.copy_(t)
    return view


def run_rnn(ver, z, k, v, b, W0, h0, gy, mis=False):
    from recurrent_fwp_b200 import _lib
    from recurrent_fwp_b200.fast_weight_rnn_v2 import fast_rnn_v2
    from recurrent_fwp_b200.fast_weight_rnn import fast_rnn
    leaves = [(misalign(t.to(DEV)) if mis else t.clone().to(DEV)).requires_grad_() for t in (z, k, v, b)]
    W, hs = W0.clone().to(DEV), h0.clone().to(DEV)
    y = (fast_rnn_v2 if ver == 2 else fast_rnn)(leaves[0], leaves[1], leaves[2], W, leaves[3], hs)
    kf, kb = _lib.last_kernel(), []
    note_backward_kernel(leaves[0], kb)
    W_end = W.clone()
    y.backward(gy.to(DEV))
    return dict(y=y.detach(), W_end=W_end, W_back=W.clone(), h=hs, g=[l.grad for l in leaves], kf=kf, kb=kb[0])


@pytest.mark.parametrize('ver', [2, 1])
@pytest.mark.parametrize('B,H,L', SHAPES)
def test_rnn_backward_plans_agree(fwp, ver, B, H, L):
    from recurrent_fwp_b200 import _lib
    z, k, v, b, gy = util.rnn_inputs(11, B, H, L, D)
    W0 = torch.randn(B, H, D, D, generator=util.gen(12)) * 0.1
    h0 = torch.randn(B, H, 1, D, generator=util.gen(13))
    try:
        fast = run_rnn(ver, z, k, v, b, W0, h0, gy)
        _lib.tune('rnn_bwd.32.roles', 2)
        short = run_rnn(ver, z, k, v, b, W0, h0, gy)        # eight steps per chunk instead of sixteen
        _lib.tune('rnn_bwd.32.roles', 0)
        ref = run_rnn(ver, z, k, v, b, W0, h0, gy)
    finally:
        _lib.tune('rnn_bwd.32.roles', 1)
    off = run_rnn(ver, z, k, v, b, W0, h0, gy, mis=True)
    assert fast['kb'] == 'rnn_bwd_roles32_kernel' and short['kb'] == 'rnn_bwd_roles32_kernel'
    assert ref['kb'] == 'rnn_bwd_kernel' and off['kb'] == 'rnn_bwd_kernel'
    for got in (fast, short, off):
        assert close(got['y'], ref['y']) and close(got['W_end'], ref['W_end']) and close(got['h'], ref['h'])
        assert close(got['W_back'], ref['W_back'])
        for a, r in zip(got['g'], ref['g']):
            assert close(a, r)


def run_lstm(variant, gates, Ws, h0, c0, gy, mis=False):
    from recurrent_fwp_b200 import _lib
    name = 'fast_lstm' if variant == 1 else 'fast_lstm_v%d' % variant
    op = getattr(importlib.import_module('recurrent_fwp_b200.' + name), name)
    leaves = [[(misalign(t.to(DEV)) if mis else t.clone().to(DEV)).requires_grad_() for t in g] for g in gates]
    Wd = [w.clone().to(DEV) for w in Ws]
    hd, cd = h0.clone().to(DEV), c0.clone().to(DEV)
    args = []
    for lv, w in zip(leaves, Wd):
        args += [lv[0], lv[1], lv[2], lv[3], w]
    y, cell = op(*args, hd, cd)
    kf, kb = _lib.last_kernel(), []
    note_backward_kernel(leaves[0][0], kb)
    W_end = [w.clone() for w in Wd]
    y.backward(gy.to(DEV))
    return dict(y=y.detach(), cell=cell.detach(), W_end=W_end, W_back=[w.clone() for w in Wd], h=hd, c=cd,
                g=[l.grad for lv in leaves for l in lv], kf=kf, kb=kb[0])


@pytest.mark.parametrize('variant', [1, 2, 3, 4])
@pytest.mark.parametrize('B,H,L', SHAPES)
def test_lstm_plans_agree(fwp, variant, B, H, L):
    from recurrent_fwp_b200 import _lib
    gates, gy = util.lstm_inputs(21, B, H, L, D)
    Ws = [torch.randn(B, H, D, D, generator=util.gen(22 + i)) * 0.1 for i in range(3)]
    h0 = torch.randn(B, H, 1, D, generator=util.gen(25))
    c0 = torch.randn(B, H, 1, D, generator=util.gen(26))
    try:
        fast = run_lstm(variant, gates, Ws, h0, c0, gy)
        _lib.tune('lstm_fwd.32.gates', 0)
        _lib.tune('lstm_bwd.32.roles', 0)
        ref = run_lstm(variant, gates, Ws, h0, c0, gy)
    finally:
        _lib.tune('lstm_fwd.32.gates', 1)
        _lib.tune('lstm_bwd.32.roles', 1)
    off = run_lstm(variant, gates, Ws, h0, c0, gy, mis=True)
    assert fast['kf'] == 'lstm_fwd_gates32_kernel' and fast['kb'] == 'lstm_bwd_roles32_kernel'
    assert ref['kf'] == 'lstm_fwd_kernel' and ref['kb'] == 'lstm_bwd_kernel'
    assert off['kf'] == 'lstm_fwd_kernel' and off['kb'] == 'lstm_bwd_kernel'
    for got in (fast, off):
        assert close(got['y'], ref['y']) and close(got['cell'], ref['cell'])
        assert close(got['h'], ref['h']) and close(got['c'], ref['c'])
        for a, r in zip(got['W_end'] + got['W_back'] + got['g'], ref['W_end'] + ref['W_back'] + ref['g']):
            assert close(a, r)


@pytest.mark.parametrize('B,H,L', SHAPES)
def test_recurrent_delta_backward_plans_agree(fwp, B, H, L):
    """The chain-warp + trailing-warp backward against the two-warp split kernel on the same saved tensors:
    stream gradients, parameter gradients and the rewound state."""
    from recurrent_fwp_b200 import _lib
    from recurrent_fwp_b200.rec_update_fwm_tanh import rec_update_fwm_tanh
    *ins, gy = util.rec_inputs(41, B, H, L, D)
    W0 = torch.randn(B, H, D, D, generator=util.gen(42)) * 0.1
    h0 = torch.randn(B, H, 1, D, generator=util.gen(43))

    def run(mis=False):
        leaves = [(misalign(t.to(DEV)) if (mis and i < 3) else t.clone().to(DEV)).requires_grad_()
                  for i, t in enumerate(ins)]
        W, hs = W0.clone().to(DEV), h0.clone().to(DEV)
        y = rec_update_fwm_tanh(*leaves, W, hs)
        kb = []
        note_backward_kernel(leaves[0], kb)
        y.backward(gy.to(DEV))
        return dict(W_back=W.clone(), g=[l.grad for l in leaves], kb=kb[0])
    try:
        fast = run()
        _lib.tune('rec_bwd.32.roles', 0)
        ref = run()
    finally:
        _lib.tune('rec_bwd.32.roles', 1)
    assert fast['kb'] == 'rec_bwd_roles32_kernel' and ref['kb'] == 'rec_bwd_kernel'
    assert close(fast['W_back'], ref['W_back'])
    for a, r in zip(fast['g'], ref['g']):
        assert close(a, r)


@pytest.mark.parametrize('B,H,L', SHAPES)
def test_recurrent_delta_forward_plans_agree(fwp, B, H, L):
    from recurrent_fwp_b200 import _lib
    from recurrent_fwp_b200.rec_update_fwm_tanh import rec_update_fwm_tanh
    *ins, gy = util.rec_inputs(31, B, H, L, D)
    W0 = torch.randn(B, H, D, D, generator=util.gen(32)) * 0.1
    h0 = torch.randn(B, H, 1, D, generator=util.gen(33))

    def run():
        leaves = [t.clone().to(DEV).requires_grad_() for t in ins]
        W, hs = W0.clone().to(DEV), h0.clone().to(DEV)
        y = rec_update_fwm_tanh(*leaves, W, hs)
        kf = _lib.last_kernel()
        W_end = W.clone()
        y.backward(gy.to(DEV))
        return dict(y=y.detach(), W_end=W_end, h=hs, g=[l.grad for l in leaves], kf=kf)
    try:
        fast = run()
        _lib.tune('rec_fwd.32.warp', 0)
        ref = run()
    finally:
        _lib.tune('rec_fwd.32.warp', 1)
    assert fast['kf'] == 'rec_fwd_warp32_kernel' and ref['kf'] == 'rec_fwd_kernel'
    assert close(fast['y'], ref['y']) and close(fast['W_end'], ref['W_end']) and close(fast['h'], ref['h'])
    for a, r in zip(fast['g'], ref['g']):      # the backward is the same kernel: it sees the two forwards' saved tensors
        assert (a - r).abs().max().item() <= 1e-4 * max(r.abs().max().item(), 1e-6)
