"""The language-model harness against the fixture made with the reference's own MemTransformerLM
(tests/golden/make_lm_golden.py): same parameters, same token ids, the CPU checker standing in for
the CUDA op.  Pins the harness (embedding scale, backwards-counted positions, pre-LayerNorm layers,
tied output layer, carried fast weights), not the kernels."""
import torch

from oracle import loops
from recurrent_fwp_b200.lm_harness import DeltaNetLM
from tests import util


def checker_delta(q, k, v, beta, W):
    """Same calling convention as fast_weight_delta: returns y and leaves the end state in W."""
    y, S = loops.delta_rule(q, k, v, beta, W.clone())
    W.copy_(S.detach())
    return y


def build(gd, delta_fn, device='cpu'):
    cfg = {k[4:]: int(v) for k, v in gd.items() if k.startswith('cfg_')}
    model = DeltaNetLM(delta_fn=delta_fn, **cfg)
    state = {k[len('param/'):]: v for k, v in gd.items() if k.startswith('param/')}
    missing, unexpected = model.load_state_dict(state, strict=True)
    assert not missing and not unexpected
    return model.to(device).eval()


def test_reference_state_dict_loads_and_plain_forward_matches():
    gd = util.golden('lm_delta')
    model = build(gd, checker_delta)
    tokens = gd['tokens']
    L = gd['loss_plain'].shape[0]
    with torch.no_grad():
        loss, mems = model(tokens[:L], tokens[1:L + 1])
    assert mems is None
    assert util.max_abs(loss, gd['loss_plain']) <= 2e-5


def test_carried_fast_weights_over_two_segments_match():
    gd = util.golden('lm_delta')
    model = build(gd, checker_delta)
    tokens = gd['tokens']
    L = gd['loss_plain'].shape[0]
    mems = None
    with torch.no_grad():
        for seg in range(2):
            data, target = tokens[seg * L:(seg + 1) * L], tokens[seg * L + 1:(seg + 1) * L + 1]
            loss, mems = model(data, target, mems, carry_over_fast_weight=True)
            assert util.max_abs(loss, gd['loss_carry_%d' % seg]) <= 2e-5
            for i, (W, _) in enumerate(mems):
                assert util.max_abs(W, gd['mem_%d_layer_%d' % (seg, i)]) <= 2e-5


def test_short_last_batch_uses_the_leading_rows_of_the_carried_state():
    gd = util.golden('lm_delta')
    model = build(gd, checker_delta)
    tokens = gd['tokens']
    L = gd['loss_plain'].shape[0]
    with torch.no_grad():
        _, mems = model(tokens[:L], tokens[1:L + 1], None, carry_over_fast_weight=True)
        full, _ = model(tokens[L:2 * L], tokens[L + 1:2 * L + 1], [(W.clone(), None) for W, _ in mems], carry_over_fast_weight=True)
        part, _ = model(tokens[L:2 * L, :2], tokens[L + 1:2 * L + 1, :2], mems, carry_over_fast_weight=True)
    assert util.max_abs(part, full[:, :2]) <= 1e-6
