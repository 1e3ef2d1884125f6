"""End-to-end check of the boundary under its real caller: the delta-rule language model forward
(recurrent_fwp_b200/lm_harness.py) with the CUDA op, against the fixture produced by the reference's
MemTransformerLM, and a training step through the op's backward against the CPU checker."""
import pytest
import torch

from recurrent_fwp_b200.lm_harness import DeltaNetLM
from tests import util
from tests.test_lm_harness_cpu import CHECKER_OPS, RECURRENT, build, checker_delta, run_recurrent_fixture

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def test_forward_and_carried_segments_match_the_reference_fixture(fwp):
    gd = util.golden('lm_delta')
    model = build(gd, None, DEV)                    # default op: the CUDA library
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
            for i, (W, _) in enumerate(mems):
                assert util.max_abs(W, gd['mem_%d_layer_%d' % (seg, i)]) <= 1e-4


def test_training_step_gradients_match_the_checker(fwp):
    gd = util.golden('lm_delta')
    tokens = gd['tokens']
    L = gd['loss_plain'].shape[0]
    grads = {}
    for name, fn, dev in (('gpu', None, DEV), ('cpu', checker_delta, 'cpu')):
        model = build(gd, fn, dev).train()
        loss, _ = model(tokens[:L].to(dev), tokens[1:L + 1].to(dev))
        loss.mean().backward()
        grads[name] = {n: p.grad.detach().cpu() for n, p in model.named_parameters()}
    for n, g in grads['cpu'].items():
        assert util.scaled_rel(grads['gpu'][n], g) <= 1e-3, n


@pytest.mark.parametrize('name', sorted(RECURRENT))
def test_recurrent_layers_match_the_reference_fixture(fwp, name):
    """attn_type 134 / 254 / 934 with the CUDA ops (delta rule + delta RNN v2, delta rules + delta LSTM v4, recurrent
    delta net) under their layer classes: plain forward and two carried segments against the reference's fixture."""
    gd = util.golden(name)
    model = build(gd, None, DEV, attn_type=RECURRENT[name])     # default ops: the CUDA library
    run_recurrent_fixture(gd, model, gd['tokens'].to(DEV), 1e-4)


@pytest.mark.parametrize('name', sorted(RECURRENT))
def test_recurrent_layers_training_step_gradients_match_the_checker(fwp, name):
    gd = util.golden(name)
    tokens = gd['tokens']
    L = gd['loss_plain'].shape[0]
    grads = {}
    for arm, ops, dev in (('gpu', None, DEV), ('cpu', CHECKER_OPS, 'cpu')):
        model = build(gd, None, dev, attn_type=RECURRENT[name], ops=ops).train()
        loss, _ = model(tokens[:L].to(dev), tokens[1:L + 1].to(dev))
        loss.mean().backward()
        grads[arm] = {n: p.grad.detach().cpu() for n, p in model.named_parameters()}
    for n, g in grads['cpu'].items():
        assert util.scaled_rel(grads['gpu'][n], g) <= 1e-3, n


def test_configs4_language_model_shape_runs_at_reduced_depth(fwp):
    """d_model 256, 8 heads of 32, FF 1024, vocab 32768, L=512 (the end-to-end language-model shape of the scale-out benchmark) at
    2 layers and batch 2: finite losses near log(vocab) for random weights."""
    torch.manual_seed(3)
    model = DeltaNetLM(32768, 2, 8, 256, 32, 1024).to(DEV).eval()
    tokens = torch.randint(0, 32768, (513, 2), device=DEV)
    with torch.no_grad():
        loss, _ = model(tokens[:-1], tokens[1:])
    assert loss.shape == (512, 2) and torch.isfinite(loss).all()
    assert abs(loss.mean().item() - 10.4) < 0.5
