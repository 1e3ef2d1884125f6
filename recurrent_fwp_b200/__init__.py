"""B200-native (sm_100a) fast-weight update kernels behind the reference's
``torch.autograd.Function`` entry points.

Sub-packages carry the reference's module names so that its layer code imports
them unchanged: ``fast_weight`` (delta rule), ``fast_transformers`` (sum rule),
``rec_update_fwm_tanh``, ``fast_weight_rnn_v2``, ``fast_weight_rnn``,
``fast_lstm``, ``fast_lstm_v2``, ``fast_lstm_v3``, ``fast_lstm_v4``.
Importing this package loads ``libfwp.so``; it raises if the library has not
been built (there is no CPU path).
"""
from . import _lib  # noqa: F401  (loads the shared library or raises)
from .fast_weight import DeltaFastWeight, fast_weight_delta  # noqa: F401
from .fast_transformers import FastWeightSum, fast_weight_sum  # noqa: F401
from .rec_update_fwm_tanh import FastWeightRecUpdateTanh, rec_update_fwm_tanh  # noqa: F401
from .fast_weight_rnn_v2 import FastRNNv2, fast_rnn_v2  # noqa: F401
from .fast_weight_rnn import FastRNN, fast_rnn  # noqa: F401
from .fast_lstm import FastLSTM, fast_lstm  # noqa: F401
from .fast_lstm_v2 import FastLSTMv2, fast_lstm_v2  # noqa: F401
from .fast_lstm_v3 import FastLSTMv3, fast_lstm_v3  # noqa: F401
from .fast_lstm_v4 import FastLSTMv4, fast_lstm_v4  # noqa: F401

__all__ = ['DeltaFastWeight', 'fast_weight_delta', 'FastWeightSum', 'fast_weight_sum',
           'FastWeightRecUpdateTanh', 'rec_update_fwm_tanh', 'FastRNNv2', 'fast_rnn_v2', 'FastRNN', 'fast_rnn',
           'FastLSTM', 'fast_lstm', 'FastLSTMv2', 'fast_lstm_v2', 'FastLSTMv3', 'fast_lstm_v3',
           'FastLSTMv4', 'fast_lstm_v4']
