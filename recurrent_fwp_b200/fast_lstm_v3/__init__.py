"""Delta LSTM v3: drop-in for the reference's ``fast_lstm_v3`` module
(language_modeling/src/utils/fast_lstm_v3/__init__.py, ``FastLSTMv3`` / ``fast_lstm_v3``).
Same signature and in-place state semantics as ``fast_lstm``; see that module."""
from recurrent_fwp_b200.fast_lstm import make_lstm_function

FastLSTMv3 = make_lstm_function(3, 'FastLSTMv3')
fast_lstm_v3 = FastLSTMv3.apply
