"""The library under several host threads at once, as its callers use it.

``nn.DataParallel`` runs one worker thread per replica (language_modeling/src/train.py:525-533) and the RL learner
and inference threads call the same ops from different threads (RL/polybeast_learner.py:387-390,421).  Nothing in the
library is per-process state that a call mutates except the plan switches (atomic integers) and the name of the
last kernel (per thread), so calls from different threads on their own CUDA streams must give the bits they give
one after the other, whatever mix of families runs at the same time.  Autograd's own backward thread is part of the
picture: every worker's ``.backward()`` runs the backward kernels on it."""
import threading

import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'
ROUNDS = 6


def job_delta(fwp, seed, d):
    q, k, v, b, gy = (t.to(DEV) for t in util.delta_inputs(seed, 3, 4, 70, d))

    def run():
        leaves = [t.clone().requires_grad_() for t in (q, k, v, b)]
        W = torch.zeros(3, 4, d, d, device=DEV)
        y = fwp.fast_weight_delta(*leaves, W)
        W_end = W.clone()
        y.backward(gy)
        return [y.detach(), W_end, W.clone()] + [l.grad for l in leaves]
    return run


def job_delta_bf16(fwp, seed):
    """bf16 streams at d = 64 with fewer sequences than SMs: the tcgen05 forward (tensor maps encoded per call on the
    calling thread) and the warp-level chunkwise backward."""
    q, k, v, b, gy = (t.to(torch.bfloat16).to(DEV) for t in util.delta_inputs(seed, 2, 3, 200, 64))

    def run():
        leaves = [t.clone().requires_grad_() for t in (q, k, v, b)]
        W = torch.zeros(2, 3, 64, 64, device=DEV)
        y = fwp.fast_weight_delta(*leaves, W)
        W_end = W.clone()
        y.backward(gy)
        return [y.detach(), W_end, W.clone()] + [l.grad for l in leaves]
    return run


def job_sum(fwp, seed):
    q, k, v, _, gy = (t.to(DEV) for t in util.delta_inputs(seed, 2, 4, 50, 16))

    def run():
        leaves = [t.clone().requires_grad_() for t in (q, k, v)]
        W = torch.zeros(2, 4, 16, 16, device=DEV)
        y = fwp.fast_weight_sum(*leaves, W)
        y.backward(gy)
        return [y.detach(), W.clone()] + [l.grad for l in leaves]
    return run


def job_rnn(fwp, seed):
    from recurrent_fwp_b200.fast_weight_rnn_v2 import fast_rnn_v2
    z, k, v, b, gy = (t.to(DEV) for t in util.rnn_inputs(seed, 2, 3, 40, 32))

    def run():
        leaves = [t.clone().requires_grad_() for t in (z, k, v, b)]
        W = torch.zeros(2, 3, 32, 32, device=DEV)
        h0 = torch.zeros(2, 3, 1, 32, device=DEV)
        y = fast_rnn_v2(leaves[0], leaves[1], leaves[2], W, leaves[3], h0)
        y.backward(gy)
        return [y.detach(), W.clone(), h0.clone()] + [l.grad for l in leaves]
    return run


def job_lstm(fwp, seed):
    from recurrent_fwp_b200.fast_lstm import fast_lstm
    gates, gy = util.lstm_inputs(seed, 2, 2, 24, 32)
    gates = [[t.to(DEV) for t in g] for g in gates]
    gy = gy.to(DEV)

    def run():
        leaves = [[t.clone().requires_grad_() for t in g] for g in gates]
        Ws = [torch.zeros(2, 2, 32, 32, device=DEV) for _ in range(3)]
        h0, c0 = torch.zeros(2, 2, 1, 32, device=DEV), torch.zeros(2, 2, 1, 32, device=DEV)
        args = []
        for lv, w in zip(leaves, Ws):
            args += [lv[0], lv[1], lv[2], lv[3], w]
        y, cell = fast_lstm(*args, h0, c0)
        (y * gy).sum().backward()
        return [y.detach(), cell.detach(), h0.clone(), c0.clone()] + Ws + [l.grad for lv in leaves for l in lv]
    return run


def job_rec(fwp, seed):
    from recurrent_fwp_b200.rec_update_fwm_tanh import rec_update_fwm_tanh
    *ins, gy = util.rec_inputs(seed, 2, 2, 33, 32)
    ins = [t.to(DEV) for t in ins]
    gy = gy.to(DEV)

    def run():
        leaves = [t.clone().requires_grad_() for t in ins]
        W = torch.zeros(2, 2, 32, 32, device=DEV)
        h0 = torch.zeros(2, 2, 1, 32, device=DEV)
        y = rec_update_fwm_tanh(*leaves, W, h0)
        y.backward(gy)
        return [y.detach(), W.clone(), h0.clone()] + [l.grad for l in leaves]
    return run


def test_calls_from_concurrent_host_threads_give_the_serial_bits(fwp):
    jobs = [job_delta(fwp, 901, 16), job_delta(fwp, 902, 32), job_sum(fwp, 903), job_rnn(fwp, 904), job_lstm(fwp, 905),
            job_rec(fwp, 906), job_delta(fwp, 907, 16), job_rnn(fwp, 908), job_delta_bf16(fwp, 909),
            job_delta_bf16(fwp, 910)]
    serial = [job() for job in jobs]
    torch.cuda.synchronize()
    results = [[None] * ROUNDS for _ in jobs]
    errors = []
    start = threading.Barrier(len(jobs))

    def worker(i):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream(DEV)
            stream.wait_stream(torch.cuda.default_stream(DEV))
            start.wait(timeout=120)
            with torch.cuda.stream(stream):
                for r in range(ROUNDS):
                    results[i][r] = jobs[i]()
            stream.synchronize()
        except Exception as e:       # surfaced by the main thread
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,), daemon=True) for i in range(len(jobs))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not any(t.is_alive() for t in threads), 'a worker did not finish'
    assert not errors, errors
    torch.cuda.synchronize()
    for i, want in enumerate(serial):
        for r in range(ROUNDS):
            got = results[i][r]
            assert len(got) == len(want)
            for a, b in zip(got, want):
                assert torch.equal(a, b), 'job %d round %d differs from the serial run' % (i, r)
