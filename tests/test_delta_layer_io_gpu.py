"""The one-launch prologue / epilogue of the delta-rule layer against the chain of PyTorch ops the
reference's layers run (split, sigmoid, permute, elu+1, sum-normalise; scale, transpose, reshape), values
and gradients, and the language-model harness with them switched on against the reference fixture."""
import pytest
import torch
import torch.nn.functional as F

from tests import util
from tests.test_lm_harness_cpu import build

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def chain(qkvb, d):
    q, k, v, beta = torch.split(qkvb, (d, d, d, 1), dim=-1)
    q, k, v, beta = (t.permute(1, 2, 0, 3) for t in (q, k, v, torch.sigmoid(beta)))
    q = F.elu(q) + 1.0
    k = F.elu(k) + 1.0
    return q / q.sum(-1, keepdim=True), k / k.sum(-1, keepdim=True), v, beta


@pytest.mark.parametrize('L,B,H,d', [(37, 3, 2, 16), (5, 2, 8, 32), (11, 1, 3, 64), (3, 2, 2, 20), (2, 1, 1, 128), (1, 1, 1, 7)])
def test_prologue_matches_the_elementwise_chain(fwp, L, B, H, d):
    from recurrent_fwp_b200.delta_layer_io import delta_layer_prologue
    g = util.gen(5)
    x = (torch.randn(L, B, H, 3 * d + 1, generator=g) * 2).to(DEV)
    grads = [torch.randn(B, H, L, w, generator=g).to(DEV) for w in (d, d, d, 1)]
    res = {}
    for name, fn in (('fused', delta_layer_prologue), ('chain', lambda t: chain(t, d))):
        leaf = x.clone().requires_grad_()
        outs = fn(leaf)
        torch.autograd.backward(outs, grads)
        res[name] = ([o.detach() for o in outs], leaf.grad)
    for a, b in zip(res['fused'][0], res['chain'][0]):
        assert a.shape == b.shape and a.is_contiguous()
        assert util.max_abs(a, b) <= 2e-6
    assert util.scaled_rel(res['fused'][1], res['chain'][1]) <= 1e-5


@pytest.mark.parametrize('L,B,H,d', [(37, 3, 2, 16), (5, 2, 8, 32), (3, 2, 2, 21)])
def test_epilogue_matches_scale_transpose_reshape(fwp, L, B, H, d):
    from recurrent_fwp_b200.delta_layer_io import delta_layer_epilogue
    g = util.gen(6)
    x = torch.randn(B, H, L, d, generator=g).to(DEV)
    gy = torch.randn(L, B, H * d, generator=g).to(DEV)
    a = x.clone().requires_grad_()
    b = x.clone().requires_grad_()
    ya = delta_layer_epilogue(a, 0.25)
    yb = (0.25 * b).transpose(1, 2).reshape(B, L, H * d).transpose(0, 1)
    ya.backward(gy)
    yb.backward(gy)
    assert torch.equal(ya, yb) and torch.equal(a.grad, b.grad)


def test_language_model_with_fused_layer_io_matches_the_reference_fixture(fwp):
    gd = util.golden('lm_delta')
    from recurrent_fwp_b200.lm_harness import DeltaNetLM
    cfg = {k[4:]: int(v) for k, v in gd.items() if k.startswith('cfg_')}
    model = DeltaNetLM(fused_io=True, **cfg)
    model.load_state_dict({k[len('param/'):]: v for k, v in gd.items() if k.startswith('param/')})
    model = model.to(DEV).eval()
    tokens = gd['tokens'].to(DEV)
    L = gd['loss_plain'].shape[0]
    with torch.no_grad():
        loss, _ = model(tokens[:L], tokens[1:L + 1])
        assert util.max_abs(loss, gd['loss_plain']) <= 1e-4
        mems = None
        for seg in range(2):
            data, target = tokens[seg * L:(seg + 1) * L], tokens[seg * L + 1:(seg + 1) * L + 1]
            loss, mems = model(data, target, mems, carry_over_fast_weight=True)
            assert util.max_abs(loss, gd['loss_carry_%d' % seg]) <= 1e-4
    # and a training step: parameter gradients agree with the unfused path
    grads = {}
    for fused in (True, False):
        m = DeltaNetLM(fused_io=fused, **cfg)
        m.load_state_dict({k[len('param/'):]: v for k, v in gd.items() if k.startswith('param/')})
        m = m.to(DEV).train()
        loss, _ = m(tokens[:L], tokens[1:L + 1])
        loss.mean().backward()
        grads[fused] = {n: p.grad.detach() for n, p in m.named_parameters()}
    for n, gref in grads[False].items():
        assert util.scaled_rel(grads[True][n], gref) <= 1e-4, n


@pytest.mark.parametrize('shape', [(2, 3, 7, 32), (1, 2, 5, 20), (2, 2, 1, 16)])
def test_delayed_copies_match_the_torch_chain(fwp, shape):
    """fwp_delayed against cat / tanh / subtraction as the reference's wrappers write them; a strided source and a
    head dimension that is not a multiple of four take the element path."""
    from recurrent_fwp_b200 import _lib
    N, H, L, M = shape
    g = torch.Generator().manual_seed(3)
    src = torch.randn(N, H, L, M, generator=g).to('cuda:0')
    first = torch.randn(N, H, 1, M, generator=g).to('cuda:0')
    other = torch.randn(N, H, L, M, generator=g).to('cuda:0')
    cat = torch.cat([first, src[:, :, :-1]], dim=2)
    assert torch.equal(_lib.delayed(src, first), cat)
    assert (_lib.delayed(src, first, op=1) - torch.tanh(cat)).abs().max().item() <= 2e-7
    assert torch.equal(_lib.delayed(src, first, minuend=other), other - cat)
    wide = torch.randn(N, H, L, M + 3, generator=g).to('cuda:0')
    view = wide[..., 1:M + 1]                       # unit inner stride, rows not 16-byte aligned
    assert torch.equal(_lib.delayed(view, first), torch.cat([first, view[:, :, :-1]], dim=2))
