"""Golden fixture for the language-model harness, made with the reference's own model code.

Run where the reference checkout is present:

    python tests/golden/make_lm_golden.py /path/to/reference

It imports the reference's ``MemTransformerLM`` (language_modeling/src/model_main.py) on the CPU with
``torch.utils.cpp_extension.load`` replaced by a stub whose functions are ``oracle.kernels`` (the
CPU restatement stands where the JIT-compiled CUDA module stands; the wrapper's device-type
dispatch table gets a "cpu" entry pointing at the same functions), builds one small model per
fast-weight layer type -- attn_type 24 (delta rule), 134 (delta rule + delta RNN v2), 254 (delta rules +
delta LSTM v4), 934 (recurrent delta net) -- with seeded ``weights_init``-style parameters, and stores in
``tests/golden/lm_<name>.npz``: the parameters, seeded token ids, the per-token loss of a plain forward,
and the losses and carried memories (every tensor of every layer's tuple) of two consecutive segments
evaluated with ``carry_over_fast_weight=True``.
"""
import os
import sys
import types

import numpy as np
import torch
import torch.nn as nn
import torch.utils.cpp_extension as cpp_ext

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
from oracle import kernels as K  # noqa: E402

CFG = dict(n_token=211, n_layer=2, n_head=2, d_model=32, d_head=16, d_inner=64)
LEN, BSZ = 24, 3


MODELS = {24: 'lm_delta', 134: 'lm_rnn_v2', 254: 'lm_lstm_v4', 934: 'lm_rec_delta'}


class _Stub(types.ModuleType):
    def __getattr__(self, name):
        if name == 'fast_lstm_v4_forward':
            def fwd(Zi, Ki, Vi, bi, Zu, Ku, Vu, bu, Zo, Ko, Vo, bo, states, cells, kvi, kvu, kvo, out, nmz, cell, gi,
                    uu, go, voi, vou, voo):
                K.fast_lstm_forward(4, Zi, Ki, Vi, bi, Zu, Ku, Vu, bu, Zo, Ko, Vo, bo, states, cells, kvi, kvu, kvo,
                                    out, nmz, cell, gi, uu, go, voi, vou, voo)
            return fwd
        if name == 'fast_lstm_v4_backward':
            return lambda *a: K.fast_lstm_backward(4, *a)
        if hasattr(K, name):
            return getattr(K, name)

        def missing(*a, **k):
            raise RuntimeError('kernel %s is not part of this fixture' % name)
        return missing


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get('FWP_REFERENCE_ROOT')
    if not ref or not os.path.isdir(ref):
        raise SystemExit('usage: make_lm_golden.py /path/to/reference')
    sys.dont_write_bytecode = True
    cpp_ext.load = lambda name=None, **kw: _Stub(name or 'stub')
    sys.path.insert(0, os.path.join(ref, 'language_modeling', 'src'))
    import model_main
    from utils import fast_fast_weight, fast_weight_rnn_v2, fast_lstm_v4, rec_update_fwm_tanh
    # the wrappers dispatch on the device type and only list "cuda": let CPU tensors take the same entries
    for cls in (fast_fast_weight.DeltaFastWeight, fast_weight_rnn_v2.FastRNNv2, fast_lstm_v4.FastLSTMv4,
                rec_update_fwm_tanh.FastWeightRecUpdateTanh):
        for table in (cls.dot, cls.dot_backward):
            table['cpu'] = table['cuda']
    for attn_type, fname in MODELS.items():
        torch.manual_seed(20240 + attn_type - 24)
        model = model_main.MemTransformerLM(
            attn_type=attn_type, pre_lnorm=True, skip_attn_normalization=True, tgt_len=LEN, ext_len=0, mem_len=0,
            cutoffs=[], dropout=0.0, dropatt=0.0, device='cpu', **CFG)
        for m in model.modules():       # what weights_init does with --init normal --init_std 0.02
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, 0.0, 0.02)
                if getattr(m, 'bias', None) is not None:
                    nn.init.normal_(m.bias, 0.0, 0.02)      # non-zero so that the fixture also pins the bias paths
            elif isinstance(m, nn.LayerNorm):
                nn.init.normal_(m.weight, 1.0, 0.02)
                nn.init.normal_(m.bias, 0.0, 0.02)
        if attn_type != 24:
            # the recurrent layers see projections of near-zero size with std 0.02: scale the layer inputs' weights up
            # so that the feedback paths (softmax of the state, gates, tanh) leave their linear regime in the fixture
            for n, p_ in model.named_parameters():
                if n.endswith(('qkvb_net.weight', 'qkv_net.weight', 'slow_net.weight')):
                    p_.data.mul_(12.0)
        model.eval()
        g = torch.Generator().manual_seed(7)
        tokens = torch.randint(0, CFG['n_token'], (2 * LEN + 1, BSZ), generator=g)
        out = {'cfg_' + k: np.int64(v) for k, v in CFG.items()}
        out['tokens'] = tokens.numpy()
        with torch.no_grad():
            loss = model(tokens[:LEN], tokens[1:LEN + 1])[0]
            out['loss_plain'] = loss.numpy()
            mems = tuple()
            for seg in range(2):
                data, target = tokens[seg * LEN:(seg + 1) * LEN], tokens[seg * LEN + 1:(seg + 1) * LEN + 1]
                ret = model(data, target, *mems, carry_over_fast_weight=True)
                out['loss_carry_%d' % seg] = ret[0].numpy()
                mems = ret[1:]
                for i, mem in enumerate(mems):
                    for j, t in enumerate(mem):
                        if t is None:
                            continue
                        key = 'mem_%d_layer_%d' % (seg, i) if (attn_type == 24 and j == 0) else \
                              'mem_%d_layer_%d_%d' % (seg, i, j)
                        out[key] = t.clone().numpy()      # the next segment updates the matrices in place
        for name, p_ in model.state_dict().items():
            out['param/' + name] = p_.numpy()
        np.savez_compressed(os.path.join(HERE, fname + '.npz'), **out)
        print('wrote %s.npz:' % fname, {k: v.shape for k, v in out.items() if not k.startswith('param/')})


if __name__ == '__main__':
    main()
