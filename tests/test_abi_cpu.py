"""No-GPU checks of the C-ABI library: it loads, exports every symbol the header
declares, and rejects bad arguments on the host before touching CUDA."""
import ctypes
import os
import re

import pytest
import torch

from tests.conftest import ROOT


@pytest.fixture(scope='module')
def L():
    from recurrent_fwp_b200 import _lib
    return _lib


def test_every_declared_symbol_is_exported(L):
    header = open(os.path.join(ROOT, 'include', 'fwp.h')).read()
    declared = set(re.findall(r'\b(fwp_[a-z0-9_]+)\s*\(', header))
    assert len(declared) >= 19
    for name in sorted(declared):
        assert hasattr(L.lib, name), 'libfwp.so does not export %s' % name
    assert declared == set(L.SIGNATURES) | set(L.OTHER_SYMBOLS)


def test_status_strings(L):
    assert L.lib.fwp_status_string(0) == b'ok'
    for code in range(1, 11):
        assert L.lib.fwp_status_string(code) not in (b'ok', b'unknown status')
    assert L.lib.fwp_status_string(999) == b'unknown status'
    assert L.lib.fwp_version() >= 100
    assert L.lib.fwp_max_head_dim() == 64


def _fake(stride3=1, ptr=0x1000):
    t = L_mod.FwpTensor()
    t.data = ptr
    t.stride[0], t.stride[1], t.stride[2], t.stride[3] = 4096, 1024, 16, stride3
    return t


def test_host_validation_rejects_before_any_launch(L):
    global L_mod
    L_mod = L
    ok = _fake()
    null = L.FwpTensor()
    f = L.lib.fwp_fast_weight_forward
    args = lambda **kw: [kw.get(n, ok) for n in ('Q', 'K', 'V', 'beta', 'v_old', 'v_insert', 'kv', 'out')]
    before = L.launch_count()
    assert f(0, 8, 16, 16, 16, *args(), 0, None, -1) == 2          # shape
    assert f(2, 8, 16, 16, 16, *args(), 7, None, -1) == 5          # dtype
    assert f(2, 8, 16, 2048, 64, *args(), 0, None, -1) == 6        # beyond every kernel's head dimensions
    assert f(2, 8, 16, 16, 16, *args(Q=null), 0, None, -1) == 1    # NULL
    assert f(2, 8, 16, 16, 16, *args(K=_fake(stride3=2)), 0, None, -1) == 3   # stride
    assert f(2, 8, 16, 16, 16, *args(V=_fake(ptr=0x1002)), 0, None, -1) == 4  # alignment
    assert L.launch_count() == before


def test_ops_refuse_cpu_tensors(L):
    from recurrent_fwp_b200 import fast_weight_delta
    q = torch.rand(1, 1, 4, 16)
    with pytest.raises(RuntimeError, match='no CPU path'):
        fast_weight_delta(q, q, q, torch.rand(1, 1, 4, 1), torch.zeros(1, 1, 16, 16))


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, 'recurrent_fwp_b200')
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith(('.py', '.cu', '.cuh')):
                text = open(os.path.join(dirpath, fn)).read()
                assert 'oracle' not in text, '%s mentions the oracle' % fn


def test_plan_switches_are_a_closed_set(L):
    """fwp_tune accepts the library's own switches and refuses anything else (no table that grows)."""
    assert L.lib.fwp_tune(b'delta.blocked', -1) == 0
    assert L.lib.fwp_tune(b'delta_bwd.16.chunk', 32) == 0
    assert L.lib.fwp_tune(b'delta.tc64', -1) == 0
    for key in (b'sum_bwd.roles', b'launch.dependent', b'step.spread', b'rec_bwd.32.roles', b'rnn_bwd.32.roles',
                b'lstm_bwd.32.roles', b'lstm_fwd.32.gates', b'rec_fwd.32.warp', b'delta.pipe64'):
        assert L.lib.fwp_tune(key, 1) == 0      # 1 is every one of these switches' default
    assert L.lib.fwp_tune(b'no.such.switch', 1) == 6
    assert L.lib.fwp_tune(None, 1) == 1
    assert L.lib.fwp_last_kernel() == b''      # nothing launched on this thread
