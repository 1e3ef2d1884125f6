"""The no-allocation backward of the recurrent delta net (collected last on purpose).

`fwp_rec_update_fwm_tanh_backward_noalloc` is for hosts that cannot allocate device memory
at call time: it keeps its scratch in a fixed array inside the library.  The test drives
both backward entry points through the C ABI on the same saved tensors, twice in a row with
different inputs (the built-in array is shared between calls and keeps old contents), and
requires the same gradients from both (max-abs 1e-6; they run the same kernels) and checks those of the
no-allocation call against the fp64 oracle with the measure of the other parity tests.
It also checks that an oversized problem is refused with the dedicated status.
"""
import ctypes

import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def _forward(L_, ins, W, h):
    N, H, T, d = ins[0].shape
    kw = dict(device=DEV, dtype=torch.float32)
    out, q_out, k_out, v_out, v_old = (torch.empty(N, H, T, d, **kw) for _ in range(5))
    b_out = torch.empty(N, H, T, 1, **kw)
    D = L_.desc
    stream, dev = L_.stream_and_device(ins[0])
    L_.check(L_.lib.fwp_rec_update_fwm_tanh_forward(
        N, H, T, d, *[D(t) for t in ins], D(q_out), D(k_out), D(v_out), D(b_out), D(v_old), D(h), D(W), D(out),
        L_.F32, stream, dev), 'forward')
    return out, q_out, k_out, v_out, b_out, v_old


def _backward(L_, noalloc, saved, od, gy, params, W):
    out, q, k, v, b, v_old = saved
    N, H, T, d = q.shape
    grads = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(b)] + \
            [torch.empty_like(t) for t in params]
    D = L_.desc
    stream, dev = L_.stream_and_device(q)
    common = [N, H, T, d, D(q), D(k), D(v), D(b), D(v_old), D(od), D(gy)] + [D(t) for t in params] + [D(W)] + \
             [D(g) for g in grads]
    if noalloc:
        rc = L_.lib.fwp_rec_update_fwm_tanh_backward_noalloc(*common, L_.F32, stream, dev)
    else:
        n = int(L_.lib.fwp_rec_update_fwm_tanh_scratch_floats(N, H, d))
        scratch = torch.empty(n, device=DEV, dtype=torch.float32)
        rc = L_.lib.fwp_rec_update_fwm_tanh_backward(
            *common, ctypes.cast(scratch.data_ptr(), ctypes.POINTER(ctypes.c_float)), n, L_.F32, stream, dev)
    L_.check(rc, 'backward')
    torch.cuda.synchronize()
    return grads


def test_noalloc_backward_matches_regular_entry_point_twice(fwp):
    from recurrent_fwp_b200 import _lib as L_
    for call, (seed, shape) in enumerate([(5, (3, 4, 19, 32)), (6, (2, 3, 11, 16))]):
        N, H, T, d = shape
        *ins, gy = util.rec_inputs(seed, N, H, T, d)
        ins = [t.to(DEV) for t in ins]
        gy = gy.to(DEV)
        W0 = (torch.randn(N, H, d, d, generator=util.gen(seed + 10)) * 0.1).to(DEV)
        h0 = torch.randn(N, H, 1, d, generator=util.gen(seed + 20)).to(DEV)
        W, h = W0.clone(), h0.clone()
        saved = _forward(L_, ins, W, h)
        od = torch.tanh(torch.cat([h0, saved[0][:, :, :-1]], dim=2))
        W_end = W.clone()
        ref = _backward(L_, False, saved, od, gy, ins[4:8], W.clone())
        W_na = W_end.clone()
        got = _backward(L_, True, saved, od, gy, ins[4:8], W_na)
        for a, b in zip(got, ref):
            assert util.max_abs(a, b) <= 1e-6, 'call %d' % call
        assert util.max_abs(W_na, W0) <= 1e-5      # rewound like the regular entry point
        # and against the fp64 explicit recurrences themselves (fp32 recurrences as the noise floor)
        from tests.test_rec_delta_gpu import NAMES, oracle64
        cpu = [t.cpu() for t in ins]
        _, g64, _, _ = oracle64(cpu, W0.cpu(), h0.cpu(), gy.cpu())
        _, g32, _, _ = oracle64(cpu, W0.cpu(), h0.cpu(), gy.cpu(), torch.float32)
        util.check_grads('rec_delta no-alloc call %d' % call, NAMES, got, g32, g64)


def test_noalloc_refuses_oversized_problem(fwp):
    from recurrent_fwp_b200 import _lib as L_
    N, H, T, d = 4096, 16, 1, 64          # 4096*16*(3*64*64+64) floats >> the built-in array
    t = L_.FwpTensor()
    t.data = 0x1000
    t.stride[0], t.stride[1], t.stride[2], t.stride[3] = 1, 1, 1, 1
    before = L_.launch_count()
    rc = L_.lib.fwp_rec_update_fwm_tanh_backward_noalloc(N, H, T, d, *([t] * 20), L_.F32, None, 0)
    assert rc == 10 and b'built-in scratch' in L_.lib.fwp_status_string(rc)
    assert L_.launch_count() == before


def test_no_bounded_wait_ran_out_during_the_gpu_tests(fwp):
    """The delta-rule kernels bound every wait on their bulk copies; a wait that ran out would have raised this flag."""
    from recurrent_fwp_b200 import _lib as L_
    assert L_.device_fault() == 0
