"""Pin the CPU oracle against the reference itself and write the golden fixtures.

Runs only where the reference checkout is present (pass its root as argv[1] or
set FWP_REFERENCE_ROOT).  For every kernel family it executes the reference
wrapper file's own ``__main__`` self-test *on CPU*: the file's text is read,
the device strings are redirected to the CPU, ``torch.utils.cpp_extension.load``
is replaced by a stub whose functions are ``oracle.kernels`` (so the oracle
stands exactly where the JIT-compiled CUDA module stands), and the file is
executed as ``__main__``.  The reference's own per-timestep autograd loop and
its own assertions (relative error < 1e-3 / 1e-2) then decide whether the oracle stands.

After each run the seeded inputs and the *reference loop's* outputs and
gradients are taken from the executed module's globals and stored under
``tests/golden/<op>.npz``; the test-suite checks both oracle layers and the
CUDA path against these files without needing the reference checkout.

Usage:  python -m oracle.pin_against_reference /path/to/reference [--out DIR]
(``--out`` writes the fixtures to DIR instead of ``tests/golden``, e.g. to compare a fresh run with the
committed files.)
"""
import contextlib
import io
import os
import sys
import types

import numpy as np
import torch
import torch.utils.cpp_extension as cpp_ext

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
sys.path.insert(0, REPO)
from oracle import kernels as K  # noqa: E402

GOLDEN = os.path.join(REPO, 'tests', 'golden')


def _lstm_fwd(variant):
    def f(Zi, Ki, Vi, bi, Zu, Ku, Vu, bu, Zo, Ko, Vo, bo, states, cells, kvi, kvu, kvo, out, *rest):
        if variant == 1:
            cell, gi, uu, go, voi, vou, voo = rest
            nmz = None
        else:
            nmz, cell, gi, uu, go, voi, vou, voo = rest
        K.fast_lstm_forward(variant, Zi, Ki, Vi, bi, Zu, Ku, Vu, bu, Zo, Ko, Vo, bo, states, cells,
                            kvi, kvu, kvo, out, nmz, cell, gi, uu, go, voi, vou, voo)
    return f


def _lstm_bwd(variant):
    return lambda *a: K.fast_lstm_backward(variant, *a)


# reference wrapper file -> (names the file asks ``load`` for, python functions that stand in)
FAMILIES = {
    'delta': ('algorithmic/fast_weight/__init__.py', {
        'fast_weight_forward': K.fast_weight_forward,
        'fast_weight_backward': K.fast_weight_backward}),
    'sum': ('algorithmic/fast_transformers/__init__.py', {
        'causal_dot_product': K.causal_dot_product,
        'causal_dot_backward': K.causal_dot_backward}),
    'rec_delta': ('algorithmic/rec_update_fwm_tanh/__init__.py', {
        'rec_update_fwm_tanh_forward': K.rec_update_fwm_tanh_forward,
        'rec_update_fwm_tanh_backward': K.rec_update_fwm_tanh_backward}),
    'rnn_v2': ('algorithmic/fast_weight_rnn_v2/__init__.py', {
        'fast_rnn_v2_forward': K.fast_rnn_v2_forward,
        'fast_rnn_v2_backward': K.fast_rnn_v2_backward}),
    'rnn_v1': ('language_modeling/src/utils/fast_weight_rnn/__init__.py', {
        'fast_rnn_forward': K.fast_rnn_forward,
        'fast_rnn_backward': K.fast_rnn_backward}),
    'lstm_v1': ('language_modeling/src/utils/fast_lstm/__init__.py', {
        'fast_lstm_forward': _lstm_fwd(1), 'fast_lstm_backward': _lstm_bwd(1)}),
    'lstm_v2': ('language_modeling/src/utils/fast_lstm_v2/__init__.py', {
        'fast_lstm_v2_forward': _lstm_fwd(2), 'fast_lstm_v2_backward': _lstm_bwd(2)}),
    'lstm_v3': ('language_modeling/src/utils/fast_lstm_v3/__init__.py', {
        'fast_lstm_v3_forward': _lstm_fwd(3), 'fast_lstm_v3_backward': _lstm_bwd(3)}),
    'lstm_v4': ('language_modeling/src/utils/fast_lstm_v4/__init__.py', {
        'fast_lstm_v4_forward': _lstm_fwd(4), 'fast_lstm_v4_backward': _lstm_bwd(4)}),
}

# which globals of the executed self-test hold (inputs, reference-loop output, leaves with .grad)
CAPTURE = {
    'delta': dict(inputs=['q0', 'k0', 'v0', 'beta0'], out='out2', leaves=['q2', 'k2', 'v2', 'beta2']),
    'sum': dict(inputs=['q0', 'k0', 'v0'], out='out2', leaves=['q2', 'k2', 'v2']),
    'rec_delta': dict(inputs=['q0', 'k0', 'v0', 'beta0', 'R_q0', 'R_k0', 'R_v0', 'r_b0'], out='out2',
                      leaves=['q2', 'k2', 'v2', 'beta2', 'Rq2', 'Rk2', 'Rv2', 'rb2']),
    'rnn_v2': dict(inputs=['z0', 'k0', 'v0', 'beta0'], out='out2', leaves=['z2', 'k2', 'v2', 'beta2']),
    'rnn_v1': dict(inputs=['z0', 'k0', 'v0', 'beta0'], out='out2', leaves=['z2', 'k2', 'v2', 'beta2']),
}
for _v in (1, 2, 3, 4):
    CAPTURE['lstm_v%d' % _v] = dict(
        inputs=[p + '0' + g for g in 'iuo' for p in 'zkvb'], out='out2',
        leaves=[p + '2' + g for g in 'iuo' for p in 'zkvb'])


def run_selftest(ref_root, family):
    rel, fns = FAMILIES[family]
    path = os.path.join(ref_root, rel)
    with open(path) as fh:
        text = fh.read()
    # redirect the devices named in the file to the CPU; nothing else is touched
    text = (text.replace('"cuda":', '"cpu":')
                .replace("device='cuda'", "device='cpu'")
                .replace('torch.cuda.FloatTensor', 'torch.FloatTensor')
                .replace('.to(0)', ".to('cpu')"))
    stub = types.SimpleNamespace(**fns)
    saved = cpp_ext.load
    cpp_ext.load = lambda *a, **k: stub
    env = {'__name__': '__main__', '__file__': path}
    try:
        with contextlib.redirect_stdout(io.StringIO()):
            exec(compile(text, path, 'exec'), env)
    finally:
        cpp_ext.load = saved
    return env


def to_np(t):
    return t.detach().cpu().numpy()


def capture(family, env):
    spec = CAPTURE[family]
    rec = {}
    if spec['inputs'] is None:
        return None
    for name in spec['inputs']:
        rec['in_' + name] = to_np(env[name])
    # the self-tests permute their outputs to (L, B, H, d) before comparing
    rec['out_LBHd'] = to_np(env[spec['out']])
    for name in spec['leaves']:
        rec['grad_' + name] = to_np(env[name].grad)
    if 'rand_targets' in env:
        rec['rand_targets'] = to_np(env['rand_targets'])
    return rec


def main():
    argv = list(sys.argv[1:])
    out_dir = GOLDEN
    if '--out' in argv:
        i = argv.index('--out')
        out_dir = os.path.abspath(argv[i + 1])
        del argv[i:i + 2]
    ref_root = argv[0] if argv else os.environ.get('FWP_REFERENCE_ROOT', '')
    if not os.path.isdir(ref_root):
        raise SystemExit('reference checkout not found: pass its root as the first argument')
    os.makedirs(out_dir, exist_ok=True)
    for family in FAMILIES:
        try:
            env = run_selftest(ref_root, family)
        except AssertionError:
            print('%-10s reference self-test FAILED against the oracle' % family)
            raise
        rec = capture(family, env)
        note = ''
        if rec is not None:
            out = os.path.join(out_dir, family + '.npz')
            np.savez_compressed(out, **rec)
            note = ' -> %s (%d KB)' % (out, os.path.getsize(out) // 1024)
        print('%-10s reference self-test passed with the oracle as the kernel%s' % (family, note))


if __name__ == '__main__':
    main()
