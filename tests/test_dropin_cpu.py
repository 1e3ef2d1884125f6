"""The drop-in executed: the reference's own layer files, unchanged, import this package's ops.

Needs a recurrent-fwp checkout (FWP_REFERENCE_ROOT, or a sibling directory named ``reference``); skipped where
there is none.  Each case runs in a child interpreter, because the overlay registers modules named ``utils`` /
``torchbeast`` / ``fast_weight`` process-wide.  Importing the layer file is the whole test on CPU: the ops
themselves have no CPU path (their parity is the GPU tests' business)."""
import os
import subprocess
import sys
import textwrap

import pytest

from tests.conftest import ROOT

REF = os.environ.get('FWP_REFERENCE_ROOT', os.path.join(os.path.dirname(ROOT), 'reference'))
needs_reference = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, 'algorithmic')),
                                     reason='no recurrent-fwp checkout reachable')


def run_child(code):
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, '-c', textwrap.dedent(code)], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


@needs_reference
def test_algorithmic_layers_file_imports_these_ops():
    """algorithmic/layers.py:7-10 and the layer classes that call the ops (:133, :380-384, :461-463)."""
    out = run_child('''
        import recurrent_fwp_b200 as fwp
        from recurrent_fwp_b200 import dropin
        dropin.activate('algorithmic', %r)
        import layers
        assert layers.fast_weight_delta is fwp.fast_weight_delta
        assert layers.fast_weight_sum is fwp.fast_weight_sum
        assert layers.fast_rnn_v2 is fwp.fast_rnn_v2
        assert layers.rec_update_fwm_tanh is fwp.rec_update_fwm_tanh
        assert layers.__file__.startswith(%r)
        for cls in ('FastFFlayer', 'FastRNNlayer', 'RecUpdateTanhFastFFlayer'):
            assert hasattr(layers, cls)
        layer = layers.FastFFlayer(num_head=2, dim_head=16, in_dim=32, dropout=0.0)
        print('ok', type(layer).__name__)
    ''' % (REF, REF))
    assert 'ok FastFFlayer' in out


@needs_reference
def test_language_model_layer_file_imports_these_ops():
    """language_modeling/src/utils/cuda_fast_weight_layer.py:9-25: every kernel module it names resolves here, the
    rest of ``utils`` (performer_helper) still comes from the reference."""
    out = run_child('''
        import recurrent_fwp_b200 as fwp
        from recurrent_fwp_b200 import dropin
        dropin.activate('language_modeling', %r)
        import utils.cuda_fast_weight_layer as m
        assert m.fast_weight_delta is fwp.fast_weight_delta
        assert m.fast_weight_sum is fwp.fast_weight_sum
        assert m.fast_rnn is fwp.fast_rnn and m.fast_rnn_v2 is fwp.fast_rnn_v2
        assert m.fast_lstm is fwp.fast_lstm and m.fast_lstm_v2 is fwp.fast_lstm_v2
        assert m.fast_lstm_v3 is fwp.fast_lstm_v3 and m.fast_lstm_v4 is fwp.fast_lstm_v4
        assert m.rec_update_fwm_tanh is fwp.rec_update_fwm_tanh
        assert m.__file__.startswith(%r)
        import utils.performer_helper as ph
        assert ph.__file__.startswith(%r)
        print('ok')
    ''' % (REF, REF, REF))
    assert 'ok' in out


@needs_reference
def test_reinforcement_learning_layer_file_imports_these_ops():
    """reinforcement_learning/torchbeast/layer.py:7-10."""
    out = run_child('''
        import recurrent_fwp_b200 as fwp
        from recurrent_fwp_b200 import dropin
        dropin.activate('reinforcement_learning', %r)
        import torchbeast.layer as m
        assert m.fast_weight_delta is fwp.fast_weight_delta
        assert m.fast_weight_sum is fwp.fast_weight_sum
        assert m.fast_rnn_v2 is fwp.fast_rnn_v2
        assert m.rec_update_fwm_tanh is fwp.rec_update_fwm_tanh
        assert m.__file__.startswith(%r)
        print('ok')
    ''' % (REF, REF))
    assert 'ok' in out


def test_unknown_project_and_missing_checkout_are_errors():
    from recurrent_fwp_b200 import dropin
    with pytest.raises(ValueError):
        dropin.activate('vision', REF)
    with pytest.raises(FileNotFoundError):
        dropin.activate('algorithmic', os.path.join(ROOT, 'no_such_checkout'))
