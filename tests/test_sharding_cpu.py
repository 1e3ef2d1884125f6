"""World-size-2 gloo test of the multi-GPU partition: ranks own batch slices, run the recurrence
on their slice (here the CPU oracle stands in for the kernels), and the gathered result equals
the unsharded one; the only cross-rank sum is the recurrent delta net's parameter gradient."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import loops
from tests import util


def test_batch_slices_cover_and_balance():
    from recurrent_fwp_b200.sharding import batch_slice
    for n in (1, 7, 64, 257):
        for w in (1, 2, 3, 8):
            sl = [batch_slice(n, r, w) for r in range(w)]
            assert sl[0].start == 0 and sl[-1].stop == n
            assert all(a.stop == b.start for a, b in zip(sl, sl[1:]))
            sizes = [s.stop - s.start for s in sl]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from recurrent_fwp_b200 import sharding
        torch.set_num_threads(1)
        N, H, L, d = 5, 2, 9, 8          # odd batch: ranks get 3 and 2 rows
        *ins, gy = util.rec_inputs(3, N, H, L, d)
        W0 = torch.randn(N, H, d, d, generator=util.gen(4)) * 0.1
        h0 = torch.randn(N, H, 1, d, generator=util.gen(5))
        # full problem (every rank computes it for the comparison)
        full = [t.clone().requires_grad_() for t in ins]
        y_full, S_full, _ = loops.rec_delta(*full, W0, h0)
        (y_full * gy).sum().backward()
        # sharded problem: streams and states sliced along the batch, parameters replicated
        streams = sharding.shard(ins[:4] + [gy, W0, h0], rank, world)
        loc = [t.clone().requires_grad_() for t in streams[:4]] + [t.clone().requires_grad_() for t in ins[4:]]
        y_loc, S_loc, _ = loops.rec_delta(*loc, streams[5], streams[6])
        (y_loc * streams[4]).sum().backward()
        y_all = sharding.gather_outputs(y_loc.detach(), N)
        pgrads = sharding.reduce_parameter_grads([t.grad.clone() for t in loc[4:]])
        ok = util.max_abs(y_all, y_full) < 1e-6
        sl = sharding.batch_slice(N, rank, world)
        ok = ok and util.max_abs(S_loc, S_full[sl]) < 1e-6
        ok = ok and all(util.max_abs(a.grad, b.grad[sl]) < 1e-5 for a, b in zip(loc[:4], full[:4]))
        ok = ok and all(util.max_abs(a, b.grad) < 1e-4 for a, b in zip(pgrads, full[4:]))
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo_partition_matches_unsharded():
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=5) for _ in range(2))
    assert results == {0: True, 1: True}
