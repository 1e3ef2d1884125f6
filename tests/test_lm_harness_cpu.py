"""The language-model harness against the fixture made with the reference's own MemTransformerLM
(tests/golden/make_lm_golden.py): same parameters, same token ids, the CPU checker standing in for
the CUDA op.  Pins the harness (embedding scale, backwards-counted positions, pre-LayerNorm layers,
tied output layer, carried fast weights), not the kernels.  One fixture per layer type: the delta
rule (attn_type 24), delta rule + delta RNN v2 (134), delta rules + delta LSTM v4 (254) and the
recurrent delta net (934)."""
import pytest
import torch

from oracle import loops
from recurrent_fwp_b200.lm_harness import DeltaNetLM
from tests import util


def checker_delta(q, k, v, beta, W):
    """Same calling convention as fast_weight_delta: returns y and leaves the end state in W."""
    y, S = loops.delta_rule(q, k, v, beta, W.clone())
    W.copy_(S.detach())
    return y


def checker_rnn_v2(Z, K, V, W, beta, h0):
    """fast_rnn_v2's convention: returns the outputs, leaves the end state in W."""
    y, S, _ = loops.delta_rnn_v2(Z, K, V, W.clone(), beta, h0)
    W.copy_(S.detach())
    return y


def checker_lstm_v4(Zi, Ki, Vi, bi, Wi, Zu, Ku, Vu, bu, Wu, Zo, Ko, Vo, bo, Wo, h0, c0):
    """fast_lstm_v4's convention: returns (outputs, cells), leaves the end states in Wi, Wu, Wo."""
    hs, cs, S, _, _ = loops.delta_lstm(4, Zi, Ki, Vi, bi, Wi.clone(), Zu, Ku, Vu, bu, Wu.clone(), Zo, Ko, Vo, bo,
                                       Wo.clone(), h0, c0)
    for W, Se in zip((Wi, Wu, Wo), S):
        W.copy_(Se.detach())
    return hs, cs


def checker_rec_delta(qx, kx, vx, bx, R_q, R_k, R_v, r_b, W, h0):
    y, S, _ = loops.rec_delta(qx, kx, vx, bx, R_q, R_k, R_v, r_b, W.clone(), h0)
    W.copy_(S.detach())
    return y


CHECKER_OPS = dict(delta=checker_delta, rnn_v2=checker_rnn_v2, lstm_v4=checker_lstm_v4, rec_delta=checker_rec_delta)
RECURRENT = {'lm_rnn_v2': 134, 'lm_lstm_v4': 254, 'lm_rec_delta': 934}


def build(gd, delta_fn, device='cpu', attn_type=24, ops=None):
    cfg = {k[4:]: int(v) for k, v in gd.items() if k.startswith('cfg_')}
    model = DeltaNetLM(delta_fn=delta_fn, attn_type=attn_type, ops=ops, **cfg)
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


def run_recurrent_fixture(gd, model, tokens, tol):
    """Plain forward, then two carried segments: losses and every carried tensor against the fixture."""
    L = gd['loss_plain'].shape[0]
    with torch.no_grad():
        loss, mems = model(tokens[:L], tokens[1:L + 1])
        assert mems is None
        assert util.max_abs(loss, gd['loss_plain']) <= tol
        for seg in range(2):
            data, target = tokens[seg * L:(seg + 1) * L], tokens[seg * L + 1:(seg + 1) * L + 1]
            loss, mems = model(data, target, mems, carry_over_fast_weight=True)
            assert util.max_abs(loss, gd['loss_carry_%d' % seg]) <= tol
            seen = 0
            for i, mem in enumerate(mems):
                for j, t in enumerate(mem):
                    key = 'mem_%d_layer_%d_%d' % (seg, i, j)
                    assert (t is None) == (key not in gd), key
                    if t is not None:
                        assert util.max_abs(t, gd[key]) <= tol, key
                        seen += 1
            assert seen == sum(k.startswith('mem_%d_' % seg) for k in gd)


@pytest.mark.parametrize('name', sorted(RECURRENT))
def test_recurrent_layers_match_the_reference_fixture(name):
    gd = util.golden(name)
    model = build(gd, None, attn_type=RECURRENT[name], ops=CHECKER_OPS)
    run_recurrent_fixture(gd, model, gd['tokens'], 3e-5)


@pytest.mark.parametrize('name', sorted(RECURRENT))
def test_recurrent_fixture_is_outside_the_linear_regime(name):
    """The fixture would pin little if the feedback paths saw near-zero inputs: the carried outputs must be of order
    0.1 or more, and the second segment must depend on the carried memory."""
    gd = util.golden(name)
    top = max(float(v.abs().max()) for k, v in gd.items() if k.startswith('mem_1_'))
    assert top > 0.1
    model = build(gd, None, attn_type=RECURRENT[name], ops=CHECKER_OPS)
    tokens = gd['tokens']
    L = gd['loss_plain'].shape[0]
    with torch.no_grad():
        fresh, _ = model(tokens[L:2 * L], tokens[L + 1:2 * L + 1])
    assert util.max_abs(fresh, gd['loss_carry_1']) > 1e-3
