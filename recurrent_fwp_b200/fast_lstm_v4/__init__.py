"""Delta LSTM v4: drop-in for the reference's ``fast_lstm_v4`` module
(language_modeling/src/utils/fast_lstm_v4/__init__.py, ``FastLSTMv4`` / ``fast_lstm_v4``).
Same signature and in-place state semantics as ``fast_lstm``; see that module."""
from recurrent_fwp_b200.fast_lstm import make_lstm_function

FastLSTMv4 = make_lstm_function(4, 'FastLSTMv4')
fast_lstm_v4 = FastLSTMv4.apply
