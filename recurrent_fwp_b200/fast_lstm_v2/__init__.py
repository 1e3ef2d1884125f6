"""Delta LSTM v2: drop-in for the reference's ``fast_lstm_v2`` module
(language_modeling/src/utils/fast_lstm_v2/__init__.py, ``FastLSTMv2`` / ``fast_lstm_v2``).
Same signature and in-place state semantics as ``fast_lstm``; see that module."""
from recurrent_fwp_b200.fast_lstm import make_lstm_function

FastLSTMv2 = make_lstm_function(2, 'FastLSTMv2')
fast_lstm_v2 = FastLSTMv2.apply
