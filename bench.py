#!/usr/bin/env python
"""Benchmark of the fast-weight hot path: delta-rule forward+backward tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One *step* is one pass of the hot path over one batch: forward and backward of
four consecutive carried segments at the language-model shape (B=64, H=8, L=256,
d=16, fp32; the state is handed from segment i to i+1 as a clone, exactly as the
reference's layers do).  Tokens per step = 4*B*L per GPU.  With N > 1 every rank
runs the same per-GPU workload on its own (batch x head) shard -- there is no
collective on the data path -- so scaling is weak and `value` is the sum over
ranks divided by the slowest rank's device time.

The line printed by rank 0 carries, besides the contract keys:
  roofline      the dominant kernel (the fused backward) against the measured HBM peak
  roofline_fwd_bwd  forward+backward kernels together (the figure the 60% target is stated on)
  cpu_baseline  the reference's per-timestep PyTorch formulation timed on this host's cores
  e2e           the same metric through the public autograd API with pinned host buffers,
                host->device copies of the inputs and device->host copies of the results timed

  configs       (N = 1) every other benchmark shape timed in the same run: the small delta-rule case, the
                scale-out delta-rule shape, the recurrent delta net, the fast-weight RNN and LSTM, and the
                end-to-end language-model forward -- forward / backward ms, tokens/s, fraction of the HBM roofline
  long_strong   (every N) the scale-out delta-rule shape with its FIXED batch of 256 split over the ranks
                (256/N batch rows per rank, no collective): ms per fwd+bwd step (max over ranks) and tokens/s, so
                that value(N) / value(1) is the strong-scaling speed-up

`--impl reference` times the reference's CPU formulation (the oracle's per-timestep
loops, forward+backward through autograd) on all host threads, on the same step: four
carried segments of the language-model shape.
"""
import argparse
import collections
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, L, d, segments, dtype)
    'lm': (64, 8, 256, 16, 4, 'fp32'),            # language-model training shape, four carried segments
    'small': (2, 8, 256, 16, 1, 'fp32'),          # the reference's own CPU-runnable case
    'long': (256, 16, 4096, 64, 1, 'bf16'),       # scale-out shape, kernel part
    'long_slice': (32, 16, 4096, 64, 1, 'bf16'),  # an eighth of it (one GPU's shard at N=8)
    'long_few': (8, 16, 4096, 64, 1, 'bf16'),     # 128 sequences: fewer than SMs (small-batch use of the scale-out kernels)
    # the other execution plans of the delta and sum rules, for --kernels-only timing and the ncu captures
    'lm_d32': (64, 8, 256, 32, 1, 'fp32'),        # fp32 at d = 32: per-step forward, blocked backward
    'lm_d64': (64, 8, 256, 64, 1, 'fp32'),        # fp32 at d = 64
    'wide': (16, 8, 256, 128, 1, 'fp32'),         # E = M = 128: matrices in shared memory (the generic kernels)
    'sum_d16': (64, 8, 256, 16, 1, 'fp32'),       # sum rule (causal product and its backward), LM shape
    'sum_wide': (16, 8, 256, 128, 1, 'fp32'),     # sum rule, E = M = 128
}

# DRAM read+write bytes of one launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture), keyed by
# the kernel the dispatch picked (fwp_last_kernel) and the number of (batch, head) sequences and steps captured.
# Traffic of these kernels grows in proportion to sequences x steps, so a capture is scaled to the timed launch
# by that product; a kernel without a capture reports null.  Each entry names where its capture is summarised.
NCU_TRAFFIC = {
    'delta_bwd_kernel': dict(bytes=44221312, seqs=512, steps=256, d=16, dtype='fp32',
                             source='profiles/delta_fwd_bwd_lm_shape_ncu.md'),
    'delta_bwd_chunk_bf16_inv_kernel': dict(bytes=2430927000, seqs=512, steps=4096, d=64, dtype='bf16',
                                            source='profiles/delta_chunkwise_bf16_d64_ncu.md'),
    'delta_bwd_chunk_bf16_pipe_kernel': dict(bytes=2429864960, seqs=512, steps=4096, d=64, dtype='bf16',
                                             source='profiles/delta_chunkwise_bf16_d64_ncu.md'),
}


def ncu_traffic(kernel, seqs, steps, d, dts):
    """Per-launch DRAM traffic of `kernel` from its ncu capture, scaled by sequences x steps; None without one."""
    e = NCU_TRAFFIC.get(kernel)
    if not e or e['d'] != d or e['dtype'] != dts:
        return None, None
    return int(e['bytes'] * (seqs * steps) / (e['seqs'] * e['steps'])), e['source']


def peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        with open(p) as fh:
            return float(json.load(fh)['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
         'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
         'clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', '-i', str(index), '--query-gpu=' + self.Q, '--format=csv,noheader,nounits', '-lms', '100'],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(',')])

    def stop(self):
        if not self.proc:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for nme, val in zip(names, r[3:7]):
                if val.lower().startswith('active'):
                    reasons.add(nme)
        return {'sm_mhz': statistics.median(sm) if sm else None,
                'sm_max_mhz': max(mx) if mx else None, 'samples': len(sm), 'reasons': sorted(reasons)}


def make_inputs(seed, B, H, L, d, dtype, device=None, pin=False):
    """q,k ~ sum_norm(elu(N(0,1))+1), v ~ N(0,1), beta = sigmoid(N(0,1)), gy ~ N(0,1); seeded on the CPU generator."""
    import torch.nn.functional as F
    big = B * H * L * d > 2 ** 27 and device is not None and not pin
    gdev = device if big else 'cpu'     # very large shapes are drawn on the device to spare host RAM and time
    g = torch.Generator(device=gdev)
    g.manual_seed(seed)

    def phi(x):
        x = F.elu(x) + 1.
        return x / x.sum(-1, keepdim=True)
    q = phi(torch.randn(B, H, L, d, generator=g, device=gdev)).to(dtype)
    k = phi(torch.randn(B, H, L, d, generator=g, device=gdev)).to(dtype)
    v = torch.randn(B, H, L, d, generator=g, device=gdev).to(dtype)
    beta = torch.sigmoid(torch.randn(B, H, L, 1, generator=g, device=gdev)).to(dtype)
    gy = torch.randn(B, H, L, d, generator=g, device=gdev).to(dtype)
    out = [q, k, v, beta, gy]
    if pin:
        out = [t.pin_memory() for t in out]
    if device is not None:
        out = [t.to(device) for t in out]
    return out


def workload_config(name, B, H, L, d, segs, dts, **extra):
    """The `config` object of the JSON line; both arms print the same `workload` string for the same step."""
    cfg = {'workload': 'delta-rule fast weight memory fwd+bwd, B=%d,H=%d,L=%d,d_k=d_v=%d, %d carried segment(s) per '
                       'step, %s streams, fp32 state' % (B, H, L, d, segs, dts),
           'name': name, 'tokens_per_step_per_gpu': segs * B * L}
    cfg.update(extra)
    return cfg


def delta_bytes(B, H, L, d, esz):
    """Algorithmic bytes of one forward and one backward launch: the streams that cross the autograd boundary
    ((4d+1) and (7d+2) elements per (batch, head, step)) plus the fp32 state read and written once per launch."""
    units = B * H * L
    state = B * H * 2 * d * d * 4
    return units * (4 * d + 1) * esz + state, units * (7 * d + 2) * esz + state


# ----------------------------------------------------------------------- CPU arm
def cpu_loop_tokens_per_s(B, H, L, d, reps, warm=1, segs=1):
    """The reference's CPU path: per-timestep PyTorch loop, fp32, forward+backward by autograd, over `segs`
    carried segments per step (the end state of one segment is the detached start state of the next, as the
    reference's layers hand it on)."""
    from oracle import loops
    torch.set_num_threads(os.cpu_count() or 1)
    times = []
    for i in range(warm + reps):
        inputs = [make_inputs(1000 + 10 * i + s, B, H, L, d, torch.float32) for s in range(segs)]
        t0 = time.perf_counter()
        W = torch.zeros(B, H, d, d)
        for q, k, v, beta, gy in inputs:
            leaves = [t.requires_grad_() for t in (q, k, v, beta)]
            y, S = loops.delta_rule(*leaves, W)
            W = S.detach()
            (y * gy).sum().backward()
        dt = time.perf_counter() - t0
        if i >= warm:
            times.append(dt)
    return segs * B * L / statistics.mean(times), statistics.mean(times)


def run_reference_arm(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    B, H, L, d, segs, dts = WORKLOADS[args.workload]
    # the same step as the GPU arm (all carried segments); shapes too large for the host are capped and say so
    Bs = min(B, 64)
    Ls = min(L, 256)
    steps = max(1, min(args.steps, 8))          # about 3.5 s per step on 16 cores: keeps the run within minutes
    warm = max(1, min(args.warmup, 1))
    tps, sec = cpu_loop_tokens_per_s(Bs, H, Ls, d, reps=steps, warm=warm, segs=segs)
    sample = 'per-timestep PyTorch loop (oracle port of the reference formulation), fwd+bwd by autograd, fp32, ' \
             '%d carried segment(s) of B=%d,H=%d,L=%d,d=%d per step, %d timed steps' % (segs, Bs, H, Ls, d, steps)
    line = {
        'impl': 'reference', 'metric': 'fast-weight fwd+bwd tokens/s', 'value': tps, 'unit': 'tokens/s',
        'n_gpus': args.gpus, 'steps': steps, 'warmup': warm, 'ms_per_step': sec * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': dts, 'data': 'synthetic',
        'config': workload_config(args.workload, B, H, L, d, segs, dts, sample=sample),
        'cpu_baseline': {'value': tps, 'unit': 'tokens/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                         'sample': sample},
        'e2e': {'value': tps, 'unit': 'tokens/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------- GPU arm
class DeltaStep:
    """Device-resident fwd+bwd over `segs` carried segments through the C ABI, pre-allocated buffers."""

    def __init__(self, B, H, L, d, segs, dtype, device, seed, rule='delta'):
        from recurrent_fwp_b200 import _lib
        self.L_ = _lib
        self.rule = rule
        self.shape = (B, H, L, d)
        self.segs = segs
        self.dtype = dtype
        self.device = device
        self.inp = [make_inputs(seed + s, B, H, L, d, dtype, device) for s in range(segs)]
        f32 = dict(device=device, dtype=torch.float32)
        io = dict(device=device, dtype=dtype)
        # Ws[s] is the state segment s starts from; its forward leaves the end state there, a clone of it becomes
        # Ws[s+1] (the carried memory, as the reference's layers hand it on) and its backward rewinds Ws[s] in place.
        self.Ws = [torch.zeros(B, H, d, d, **f32) for _ in range(segs + 1)]
        self.W = self.Ws[0]
        self.y = [torch.empty(B, H, L, d, **io) for _ in range(segs)]
        self.vo = [torch.empty(B, H, L, d, **f32) for _ in range(segs)]
        self.g = [[torch.empty(B, H, L, d, **io) for _ in range(3)] + [torch.empty(B, H, L, 1, **io)]
                  for _ in range(segs)]
        self.code = _lib.io_dtype(self.inp[0][0])
        D = _lib.desc
        self.d_in = [[D(t) for t in seg] for seg in self.inp]
        self.d_Ws = [D(t) for t in self.Ws]
        self.d_y = [D(t) for t in self.y]
        self.d_vo = [D(t) for t in self.vo]
        self.d_none = D(None)     # u_t ("v_insert") is rebuilt by the backward: not stored
        self.d_g = [[D(t) for t in seg] for seg in self.g]
        self.dev_index = device.index
        self.kernels = {}

    def fwd(self, s, stream):
        B, H, L, d = self.shape
        q, k, v, b, _ = self.d_in[s]
        if self.rule == 'sum':
            self.L_.check(self.L_.lib.fwp_causal_dot_product(
                B, H, L, d, d, q, k, v, self.d_Ws[s], self.d_y[s], self.code, stream, self.dev_index), 'sum fwd')
            self.kernels['fwd'] = self.L_.last_kernel()
            return
        self.L_.check(self.L_.lib.fwp_fast_weight_forward(
            B, H, L, d, d, q, k, v, b, self.d_vo[s], self.d_none, self.d_Ws[s], self.d_y[s],
            self.code, stream, self.dev_index), 'fwd')
        self.kernels['fwd'] = self.L_.last_kernel()

    def bwd(self, s, stream):
        B, H, L, d = self.shape
        q, k, v, b, gy = self.d_in[s]
        gq, gk, gv, gb = self.d_g[s]
        if self.rule == 'sum':
            self.L_.check(self.L_.lib.fwp_causal_dot_backward(
                B, H, L, d, d, q, k, v, gy, gq, gk, gv, self.code, stream, self.dev_index), 'sum bwd')
            self.kernels['bwd'] = self.L_.last_kernel()
            return
        self.L_.check(self.L_.lib.fwp_fast_weight_backward(
            B, H, L, d, d, q, k, v, b, self.d_vo[s], self.d_none, gy, self.d_Ws[s], gq, gk, gv, gb,
            self.code, stream, self.dev_index), 'bwd')
        self.kernels['bwd'] = self.L_.last_kernel()

    def step(self):
        """Per segment: fwd, clone the end state as the next segment's start state (the carried memory; the reference's
        layers do the same clone because the backward rewinds the state in place), bwd."""
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        self.Ws[0].zero_()
        for s in range(self.segs):
            self.fwd(s, stream)
            self.Ws[s + 1].copy_(self.Ws[s])
            self.bwd(s, stream)


def time_kernels(ds, flush, reps):
    """Average device time of one forward and one backward launch: CUDA events on the launching stream around the
    launches of all segments back to back (their inputs are distinct tensors: 4 x 35 MB forward, 4 x 61 MB backward
    at the LM shape, more than the 126 MB L2), L2 flushed before each event pair.  Events are created before the
    flush so that the host is ahead of the device when the first launch is due."""
    stream_obj = torch.cuda.current_stream(ds.device)
    stream = ctypes.c_void_p(stream_obj.cuda_stream)
    tf, tb = [], []
    for i in range(reps + 2):     # the first two rounds are warm-up (clock ramp, cold instruction cache)
        e0, e1, e2, e3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
        for W in ds.Ws:
            W.zero_()
        flush()
        e0.record(stream_obj)
        for s in range(ds.segs):
            ds.fwd(s, stream)
        e1.record(stream_obj)
        flush()
        e2.record(stream_obj)
        for s in range(ds.segs):
            ds.bwd(s, stream)
        e3.record(stream_obj)
        torch.cuda.synchronize(ds.device)
        if i >= 2:
            tf.append(e0.elapsed_time(e1) / ds.segs)
            tb.append(e2.elapsed_time(e3) / ds.segs)
    return statistics.mean(tf) * 1e-3, statistics.mean(tb) * 1e-3, min(tf) * 1e-3, min(tb) * 1e-3


# ---- the recurrent families at their benchmark shapes; timed through their autograd Functions
FAMILY_SHAPES = {
    'rec_delta': (64, 8, 256, 32),     # recurrent delta net
    'rnn_v2': (128, 4, 512, 32),       # fast-weight RNN / LSTM shape
    'rnn_v1': (128, 4, 512, 32),
    'lstm_v1': (128, 4, 512, 32),
    'lstm_v2': (128, 4, 512, 32),
    'lstm_v3': (128, 4, 512, 32),
    'lstm_v4': (128, 4, 512, 32),
}


FAMILY_HEAD_START = 8      # 256 MB memsets queued before each timed call (about 0.6 ms of device work)


def time_family(name, steps, dev, flush_buf):
    """Forward and backward device time of one recurrent family at its benchmark shape (fp32, W0 = h0 = 0),
    CUDA events around the autograd Function's forward and around .backward(), L2 flushed before each."""
    import recurrent_fwp_b200 as fwp
    from recurrent_fwp_b200 import _lib
    B, H, L, d = FAMILY_SHAPES[name]
    g = torch.Generator(device='cpu')
    g.manual_seed(7)
    rn = lambda *s: torch.randn(*s, generator=g).to(dev)
    z = lambda *s: torch.zeros(*s, device=dev)

    def gate():
        return [rn(B, H, L, d), torch.softmax(rn(B, H, L, d), -1), rn(B, H, L, d), torch.sigmoid(rn(B, H, L, 1))]

    if name == 'rec_delta':
        ins = [rn(B, H, L, d), rn(B, H, L, d), rn(B, H, L, d), rn(B, H, L, 1)] + \
              [rn(1, H, d, d) / d ** 0.5 for _ in range(3)] + [rn(1, H, 1, d) / d ** 0.5]
        call = lambda x: fwp.rec_update_fwm_tanh(*x, z(B, H, d, d), z(B, H, 1, d))
        elems = 11 * d + 3
    elif name.startswith('rnn'):
        zz, k, v, b = gate()
        ins = [zz, k, v, b]
        op = fwp.fast_rnn_v2 if name == 'rnn_v2' else fwp.fast_rnn
        call = lambda x: op(x[0], x[1], x[2], z(B, H, d, d), x[3], z(B, H, 1, d))
        elems = 11 * d + 3
    else:
        ins = gate() + gate() + gate()
        op = getattr(fwp, 'fast_lstm' if name == 'lstm_v1' else 'fast_lstm_' + name[-2:])
        call = lambda x: op(x[0], x[1], x[2], x[3], z(B, H, d, d), x[4], x[5], x[6], x[7], z(B, H, d, d),
                            x[8], x[9], x[10], x[11], z(B, H, d, d), z(B, H, 1, d), z(B, H, 1, d))[0]
        elems = 29 * d + 9
    gy = rn(B, H, L, d)
    tf, tb, launches = [], [], 0
    for i in range(3 + max(steps, 5)):
        leaves = [t.detach().requires_grad_() for t in ins]
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        n0 = _lib.launch_count()
        for _ in range(FAMILY_HEAD_START):     # the host runs ahead of the device: the events see device time only
            flush_buf.zero_()
        e[0].record()
        y = call(leaves)
        e[1].record()
        for _ in range(FAMILY_HEAD_START):
            flush_buf.zero_()
        e[2].record()
        y.backward(gy)
        e[3].record()
        torch.cuda.synchronize(dev)
        launches = _lib.launch_count() - n0
        if i >= 3:
            tf.append(e[0].elapsed_time(e[1]) * 1e-3)
            tb.append(e[2].elapsed_time(e[3]) * 1e-3)
    peak, kind = peaks()
    f, b_ = statistics.mean(tf), statistics.mean(tb)
    nbytes = B * H * L * elems * 4
    return {'workload': name, 'shape': {'B': B, 'H': H, 'L': L, 'd': d}, 'dtype': 'fp32', 'fwd_ms': f * 1e3,
            'bwd_ms': b_ * 1e3, 'tokens_per_s': B * L / (f + b_), 'algorithmic_bytes_fwd_bwd': nbytes,
            'frac': nbytes / (f + b_) / 1e9 / peak, 'peak_kind': kind, 'launches_per_step': int(launches),
            'timing': 'CUDA events around the autograd forward / backward calls (the wrappers\' small torch ops '
                      'included); before each, the L2 flush is queued several times so that the host has issued the '
                      'call before the device reaches it'}


def run_family(args):
    dev = torch.device('cuda', int(os.environ.get('LOCAL_RANK', '0')))
    torch.cuda.set_device(dev)
    flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    print(json.dumps(time_family(args.workload, args.steps, dev, flush_buf)), flush=True)


def time_delta(name, device, flush, reps, B=None, seed=77):
    """Forward and backward kernel time of one delta-rule workload (all of its segments launched back to back),
    with the kernels the dispatch picked and the fraction of the HBM roofline of both launches together."""
    Bw, H, L, d, segs, dts = WORKLOADS[name]
    B = Bw if B is None else B
    dtype = torch.float32 if dts == 'fp32' else torch.bfloat16
    esz = 4 if dts == 'fp32' else 2
    ds = DeltaStep(B, H, L, d, segs, dtype, device, seed=seed)
    tf, tb, tf_min, tb_min = time_kernels(ds, flush, reps=reps)
    peak, kind = peaks()
    bf, bb = delta_bytes(B, H, L, d, esz)
    out = {'workload': name, 'shape': {'B': B, 'H': H, 'L': L, 'd': d}, 'dtype': dts, 'fwd_ms': tf * 1e3,
           'bwd_ms': tb * 1e3, 'tokens_per_s': B * L / (tf + tb), 'algorithmic_bytes_fwd_bwd': bf + bb,
           'frac': (bf + bb) / (tf + tb) / 1e9 / peak, 'frac_fwd': bf / tf / 1e9 / peak, 'frac_bwd': bb / tb / 1e9 / peak,
           'peak_kind': kind, 'kernels': dict(ds.kernels),
           'timing': 'CUDA events around the launches, L2 flushed before each direction'}
    del ds
    torch.cuda.empty_cache()
    return out


# ---- end-to-end forward of a 16-layer delta-rule language model (second part of the scale-out configuration)
LM_E2E = dict(n_token=32768, n_layer=16, n_head=8, d_model=256, d_head=32, d_inner=1024, batch=32, seq_len=512)


def time_lm_e2e(steps, warmup, dev, rank=0, world=1, fused_io=True, sample_clocks=False):
    """Forward of the delta-rule language model (recurrent_fwp_b200/lm_harness.py: the reference's
    MemTransformerLM with attn_type 24, random-init weights, uniform random token ids, fp32), B=32, L=512.
    Each step copies the step's token ids from pinned host memory, runs the forward under no_grad and reads the
    mean loss back.  With N > 1 ranks the batch rows are split over ranks and the per-token losses are
    all-gathered over NCCL (the only collective; it is outside the fast-weight op)."""
    import torch.distributed as dist
    from recurrent_fwp_b200 import _lib
    from recurrent_fwp_b200.lm_harness import DeltaNetLM
    from recurrent_fwp_b200 import sharding
    c = LM_E2E
    torch.manual_seed(11)
    model = DeltaNetLM(c['n_token'], c['n_layer'], c['n_head'], c['d_model'], c['d_head'], c['d_inner'],
                       fused_io=fused_io).to(dev).eval()
    B, L = c['batch'], c['seq_len']
    rows = sharding.batch_slice(B, rank, world)
    g = torch.Generator().manual_seed(5)
    host = [torch.randint(0, c['n_token'], (L + 1, B), generator=g)[:, rows].contiguous().pin_memory()
            for _ in range(4)]
    flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    times, launches, loss_mean = [], 0, None
    sampler = None
    for i in range(warmup + steps):
        if i == warmup:
            sampler = ClockSampler(dev.index) if sample_clocks else None
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)
        flush_buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = _lib.launch_count()
        e0.record()
        tok = host[i % len(host)].to(dev, non_blocking=True)
        with torch.no_grad():
            loss, _ = model(tok[:-1], tok[1:])
            if world > 1:
                loss = sharding.gather_outputs(loss.t().contiguous(), B).t()
            loss_mean = loss.mean().item()        # device -> host read of the step's result
        e1.record()
        torch.cuda.synchronize(dev)
        if i >= warmup:
            times.append(e0.elapsed_time(e1) * 1e-3)
            launches += _lib.launch_count() - n0
    clocks = sampler.stop() if sampler else None
    tsum = torch.tensor([sum(times)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tsum, op=dist.ReduceOp.MAX)
        dist.barrier()
    sec = tsum.item() / steps
    del model
    torch.cuda.empty_cache()
    return {'ms_per_step': sec * 1e3, 'tokens_per_s': B * L / sec, 'launches': int(launches), 'mean_loss': loss_mean,
            'h2d_bytes_per_step': int(host[0].numel() * 8), 'clocks': clocks}


LM_E2E_WORKLOAD = ('end-to-end forward, 16-layer delta-rule LM (attn_type 24), d_model 256, 8 heads of 32, FF 1024, '
                   'vocab 32768, B=32, L=512, random-init weights, uniform random token ids')


def run_lm_e2e(args):
    import torch.distributed as dist
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    dev = torch.device('cuda', int(os.environ.get('LOCAL_RANK', '0')))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    r = time_lm_e2e(args.steps, args.warmup, dev, rank, world, fused_io=not args.unfused_layer_io, sample_clocks=True)
    if rank == 0:
        print(json.dumps({
            'metric': 'delta-net language model forward tokens/s', 'value': r['tokens_per_s'], 'unit': 'tokens/s',
            'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': r['ms_per_step'],
            'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'fp32', 'data': 'synthetic',
            'config': {'workload': LM_E2E_WORKLOAD,
                       'layer_io': 'torch elementwise chain' if args.unfused_layer_io else 'one-launch prologue and epilogue',
                       'sharding': 'batch rows split over ranks; per-token losses all-gathered (NCCL) outside the op',
                       'l2': 'flushed between timed steps (256 MiB write)'},
            'e2e': {'value': r['tokens_per_s'], 'unit': 'tokens/s', 'h2d_bytes_per_step': r['h2d_bytes_per_step'],
                    'd2h_bytes_per_step': 4, 'api': 'recurrent_fwp_b200.lm_harness.DeltaNetLM.forward'},
            'gpu_launches': r['launches'], 'mean_loss': r['mean_loss'], 'clocks': r['clocks']}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_single_step(args):
    """`--workload rl_step`: the delta rule called one time step at a time (L = 1) at the RL callers' shape (32
    environments, 4 heads of 32; RL/model.py:436-448), the state carried in place.  Launch latency is the cost here, so
    two numbers per direction of use: a call through the C ABI from the host loop, and the same call replayed from
    a CUDA graph.  Device time by CUDA events around `reps` back-to-back steps, host time by the wall clock."""
    from recurrent_fwp_b200 import _lib
    dev = torch.device('cuda', int(os.environ.get('LOCAL_RANK', '0')))
    torch.cuda.set_device(dev)
    B, H, d, reps = 32, 4, 32, 400
    ds = DeltaStep(B, H, 1, d, 1, torch.float32, dev, seed=77)
    stream_obj = torch.cuda.Stream(dev)
    stream = ctypes.c_void_p(stream_obj.cuda_stream)

    def timed(fn):
        for _ in range(20):
            fn()
        stream_obj.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        a.record(stream_obj)
        for _ in range(reps):
            fn()
        b.record(stream_obj)
        host = (time.perf_counter() - t0) / reps
        stream_obj.synchronize()
        return a.elapsed_time(b) * 1e3 / reps, host * 1e6

    out = {}
    with torch.cuda.stream(stream_obj):
        out['abi_call'] = dict(zip(('device_us_per_step', 'host_us_per_step'), timed(lambda: ds.fwd(0, stream))))
        kernel = _lib.last_kernel()
        ds.fwd(0, stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream_obj):
            ds.fwd(0, stream)
        out['graph_replay'] = dict(zip(('device_us_per_step', 'host_us_per_step'), timed(graph.replay)))
        eight = torch.cuda.CUDAGraph()
        with torch.cuda.graph(eight, stream=stream_obj):
            for _ in range(8):
                ds.fwd(0, stream)
        dev_us, host_us = timed(eight.replay)
        out['graph_of_8_steps'] = {'device_us_per_step': dev_us / 8, 'host_us_per_step': host_us / 8}
    print(json.dumps({'workload': 'rl_step', 'shape': {'B': B, 'H': H, 'L': 1, 'd': d}, 'dtype': 'fp32', 'kernel': kernel,
                      'forward': out,
                      'timing': 'CUDA events on the launching stream around %d back-to-back steps; host time by the '
                                'wall clock around the same loop' % reps}), flush=True)


def long_strong(device, flush, rank, world, barrier, steps=5, warmup=3):
    """The scale-out delta-rule shape with its fixed batch of 256 split over the ranks (256 / N batch rows each,
    all 16 heads, no collective): fwd+bwd device time per step, max over ranks."""
    import torch.distributed as dist
    Bw, H, L, d, segs, dts = WORKLOADS['long']
    if Bw % world:
        return None
    B = Bw // world
    ds = DeltaStep(B, H, L, d, segs, torch.bfloat16, device, seed=900 + rank)
    tot = []
    for i in range(warmup + steps):
        if i == warmup:
            torch.cuda.synchronize(device)
            barrier()
        flush()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        ds.step()
        b_.record()
        torch.cuda.synchronize(device)
        if i >= warmup:
            tot.append(a.elapsed_time(b_) * 1e-3)
    t = torch.tensor([sum(tot)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec = float(t.item()) / steps
    kernels = dict(ds.kernels)
    del ds
    torch.cuda.empty_cache()
    peak, kind = peaks()
    bf, bb = delta_bytes(Bw, H, L, d, 2)
    return {'workload': 'delta-rule fwd+bwd, B=%d (fixed, %d per rank),H=%d,L=%d,d=%d, bf16 streams, fp32 state'
                        % (Bw, B, H, L, d),
            'scaling': 'strong', 'n_gpus': world, 'ms_per_step': sec * 1e3, 'tokens_per_s': Bw * L / sec,
            'frac_of_n_gpu_hbm': (bf + bb) / sec / 1e9 / (peak * world), 'peak_kind': kind, 'steps': steps,
            'kernels': kernels,
            'timing': 'CUDA events around forward, state copy and backward of each step, L2 flushed between steps, '
                      'summed, max over ranks'}


def run_gpu_arm(args):
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        raise SystemExit('bench.py: no CUDA device; the product has no CPU path (use --impl reference for the CPU arm)')
    device = torch.device('cuda', local)
    torch.cuda.set_device(device)
    import torch.distributed as dist
    if world > 1:
        # gloo for the host-side barriers, NCCL for device tensors.  No device_id, so the NCCL communicator comes up
        # with the first device collective, which is the max-over-ranks of the timed steps: measured here, a process
        # with a live NCCL communicator replays the graph-captured step 2.7 % slower (0.292 against 0.284 ms, one
        # rank), and the ranks of this benchmark exchange nothing on the data path.
        dist.init_process_group('cpu:gloo,cuda:nccl')
    import recurrent_fwp_b200 as fwp
    from recurrent_fwp_b200 import _lib

    B, H, L, d, segs, dts = WORKLOADS[args.workload]
    dtype = torch.float32 if dts == 'fp32' else torch.bfloat16
    esz = 4 if dts == 'fp32' else 2
    ds = DeltaStep(B, H, L, d, segs, dtype, device, seed=1234 + 100 * rank,
                   rule='sum' if args.workload.startswith('sum_') else 'delta')
    flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    def flush():
        flush_buf.zero_()

    if args.kernels_only:
        tf, tb, tf_min, tb_min = time_kernels(ds, flush, reps=max(3, args.steps))
        print(json.dumps({'workload': args.workload, 'fwd_us': tf * 1e6, 'bwd_us': tb * 1e6,
                          'fwd_min_us': tf_min * 1e6, 'bwd_min_us': tb_min * 1e6, 'kernels': dict(ds.kernels)}), flush=True)
        return

    # ---- the step, captured in a CUDA graph (launch gaps would otherwise dominate microsecond kernels)
    use_graph = not args.no_graph
    graph = None
    for _ in range(2):
        n0 = _lib.launch_count()
        ds.step()
        per_step_launches = _lib.launch_count() - n0
    torch.cuda.synchronize(device)
    if use_graph:
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                ds.step()
            torch.cuda.current_stream(device).wait_stream(side)
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                ds.step()
        except Exception as exc:  # report, and time eager launches instead
            sys.stderr.write('bench.py: CUDA graph capture failed (%r); timing eager launches\n' % (exc,))
            graph = None
            torch.cuda.synchronize(device)
    run_step = graph.replay if graph is not None else ds.step

    def barrier():
        if world > 1:
            dist.all_reduce(torch.zeros(1))     # a host-side barrier (gloo)

    for _ in range(max(args.warmup, 3)):
        flush()
        run_step()
    torch.cuda.synchronize(device)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = _lib.launch_count()
    evs = []
    t_wall0 = time.perf_counter()
    for _ in range(args.steps):
        flush()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run_step()
        b_.record()
        evs.append((a, b_))
    torch.cuda.synchronize(device)
    barrier()
    t_wall = time.perf_counter() - t_wall0
    launches = _lib.launch_count() - launches0
    if graph is not None:
        launches = per_step_launches * args.steps      # replays re-issue the launches counted in one eager step
    dev_s = sum(a.elapsed_time(b_) for a, b_ in evs) * 1e-3
    tmax = torch.tensor([dev_s], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dev_s = float(tmax.item())
    tokens_per_step = segs * B * L
    value = world * tokens_per_step * args.steps / dev_s

    # ---- e2e: public autograd API, pinned host buffers, copies inside the timed region
    Be = B if B * H * L * d <= 2 ** 27 else 8     # very large shapes: the end-to-end leg runs a batch slice
    host_in = [make_inputs(4321 + s + 100 * rank, Be, H, L, d, dtype, pin=True) for s in range(segs)]
    host_out = [[torch.empty(Be, H, L, d, dtype=dtype).pin_memory() for _ in range(4)] +
                [torch.empty(Be, H, L, 1, dtype=dtype).pin_memory()] for _ in range(segs)]
    h2d = sum(t.numel() * t.element_size() for seg in host_in for t in seg)
    d2h = sum(t.numel() * t.element_size() for seg in host_out for t in seg)

    # Three streams: segment s+1 is uploaded and segment s-1 downloaded while segment s computes (PCIe is full
    # duplex); every byte still crosses inside the timed region.  Device-side input buffers are double-buffered and
    # the steps are not separated by a device-wide synchronisation: the first upload of a step overlaps the last
    # download of the step before it, as a training loop that prefetches its next batch does.  An event per device
    # buffer (its last reader) keeps an upload from overwriting inputs that a backward still needs.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    dev_in = [[torch.empty(t.shape, dtype=t.dtype, device=device) for t in host_in[0]] for _ in range(2)]
    # One copy each way per segment: the five input tensors of a segment lie behind one another in one pinned
    # buffer (and in one device buffer), the five results are gathered into one device buffer before they leave.
    packed = not args.e2e_unpacked

    def carve(flat, like):
        """Views of `flat` with the shapes of `like`, each starting on a 256-byte boundary."""
        views, off = [], 0
        for t in like:
            views.append(flat[off:off + t.numel()].view(t.shape))
            off += (t.numel() + 127) // 128 * 128
        return views

    if packed:
        total_in = sum((t.numel() + 127) // 128 * 128 for t in host_in[0])
        total_out = sum((t.numel() + 127) // 128 * 128 for t in host_out[0])
        host_in_flat = [torch.empty(total_in, dtype=dtype).pin_memory() for _ in range(segs)]
        for flat, seg in zip(host_in_flat, host_in):
            for view, t in zip(carve(flat, seg), seg):
                view.copy_(t)
        host_in = [carve(flat, host_in[0]) for flat in host_in_flat]
        dev_in_flat = [torch.empty(total_in, dtype=dtype, device=device) for _ in range(2)]
        dev_in = [carve(flat, host_in[0]) for flat in dev_in_flat]
        host_out_flat = [torch.empty(total_out, dtype=dtype).pin_memory() for _ in range(segs)]
        like_out = host_out[0]
        host_out = [carve(flat, like_out) for flat in host_out_flat]
        dev_out_flat = [torch.empty(total_out, dtype=dtype, device=device) for _ in range(2)]
        dev_out = [carve(flat, like_out) for flat in dev_out_flat]
        out_free = [None, None]         # per staging buffer: its last download
    last_reader = [None, None]
    counter = [0]
    in_flight = collections.deque()     # download-complete events of the segments the host has queued

    def e2e_step():
        cur = torch.cuda.current_stream(device)
        W = torch.zeros(Be, H, d, d, device=device)

        def upload(seg, buf):
            with torch.cuda.stream(s_in):
                if last_reader[buf] is not None:
                    s_in.wait_event(last_reader[buf])   # the buffer's previous reader (saved tensors of that segment)
                if packed:
                    dev_in_flat[buf].copy_(host_in_flat[seg], non_blocking=True)
                else:
                    for dst, src in zip(dev_in[buf], host_in[seg]):
                        dst.copy_(src, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
            return ev

        ready = upload(0, counter[0] % 2)
        for seg in range(segs):
            # The host stays at most three segments ahead of the downloads (a bounded prefetch, as a trainer's
            # loader has): the caching allocator then reuses the same blocks every segment instead of growing
            # its pool inside the timed region.  Three queued segments are about 3 ms of device work.
            while len(in_flight) >= 3:
                in_flight.popleft().synchronize()
            buf = counter[0] % 2
            counter[0] += 1
            nxt = upload(seg + 1, counter[0] % 2) if seg + 1 < segs else None
            cur.wait_event(ready)
            q, k, v, b = (t.detach().requires_grad_() for t in dev_in[buf][:4])
            gy = dev_in[buf][4]
            y = fwp.fast_weight_delta(q, k, v, b, W)
            W_next = W.clone()
            y.backward(gy)
            results = (y.detach(), q.grad, k.grad, v.grad, b.grad)
            if packed:
                if out_free[buf] is not None:
                    cur.wait_event(out_free[buf])       # the staging buffer's previous download
                for dst, src in zip(dev_out[buf], results):
                    dst.copy_(src)
            done = torch.cuda.Event()
            done.record(cur)
            last_reader[buf] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                if packed:
                    host_out_flat[seg].copy_(dev_out_flat[buf], non_blocking=True)
                else:
                    for dst, src in zip(host_out[seg], results):
                        dst.copy_(src, non_blocking=True)
                        src.record_stream(s_out)
                landed = torch.cuda.Event()
                landed.record(s_out)
            if packed:
                out_free[buf] = landed
            in_flight.append(landed)
            W = W_next
            ready = nxt

    def e2e_drain():
        cur = torch.cuda.current_stream(device)
        cur.wait_stream(s_out)
        cur.wait_stream(s_in)

    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(2):
        e2e_step()
    e2e_drain()
    torch.cuda.synchronize(device)
    barrier()
    t0 = time.perf_counter()
    ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ea.record()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_drain()                     # the last downloads are inside the timed region
    eb.record()
    torch.cuda.synchronize(device)
    e2e_s = max(ea.elapsed_time(eb) * 1e-3, 1e-9)
    # what arrived on the host is what the op computes: segment 0 again, straight on the device (outside the timing)
    chk = [t.to(device).requires_grad_() for t in host_in[0][:4]]
    y_chk = fwp.fast_weight_delta(*chk, torch.zeros(Be, H, d, d, device=device))
    y_chk.backward(host_in[0][4].to(device))
    torch.cuda.synchronize(device)
    for got, want in zip(host_out[0], [y_chk.detach()] + [t.grad for t in chk]):
        if not torch.equal(got, want.cpu()):
            raise SystemExit('bench.py: the end-to-end leg returned other numbers than the op computes')
    barrier()
    te = torch.tensor([e2e_s], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = world * segs * Be * L * e2e_steps / float(te.item())
    clocks = sampler.stop() if sampler else None

    # ---- the scale-out shape with its fixed batch split over the ranks (every N)
    strong = None
    if args.workload == 'lm' and not args.skip_configs:
        strong = long_strong(device, flush, rank, world, barrier)

    # ---- per-kernel timing for the roofline (rank 0 only; separate from the step timing)
    if rank == 0:
        tf, tb, tf_min, tb_min = time_kernels(ds, flush, reps=max(10, min(4 * args.steps, 40)))
        peak, peak_kind = peaks()
        bytes_fwd, bytes_bwd = delta_bytes(B, H, L, d, esz)
        ach_b = bytes_bwd / tb / 1e9
        ach_fb = (bytes_fwd + bytes_bwd) / (tf + tb) / 1e9
        bwd_kernel = ds.kernels.get('bwd')
        traffic, traffic_src = ncu_traffic(bwd_kernel, B * H, L, d, dts)
        configs = None
        if world == 1 and args.workload == 'lm' and not args.skip_configs:
            configs = {'small': time_delta('small', device, flush, reps=10),
                       'long': time_delta('long', device, flush, reps=3)}
            for fam in ('rec_delta', 'rnn_v2', 'lstm_v1'):
                configs[fam] = time_family(fam, 5, device, flush_buf)
            r = time_lm_e2e(5, 3, device)
            configs['lm_e2e'] = {'workload': LM_E2E_WORKLOAD, 'fwd_ms': r['ms_per_step'], 'bwd_ms': None,
                                 'tokens_per_s': r['tokens_per_s'], 'frac': None, 'launches_per_step': r['launches'] // 5,
                                 'h2d_bytes_per_step': r['h2d_bytes_per_step'], 'd2h_bytes_per_step': 4,
                                 'timing': 'CUDA events around token upload, forward under no_grad and the read of '
                                           'the mean loss; L2 flushed between steps'}
        cpu = None
        if world == 1 and not args.skip_cpu:
            Bs, Ls = min(B, 64), min(L, 256)
            tps, sec = cpu_loop_tokens_per_s(Bs, H, Ls, d, reps=6, warm=1, segs=segs)
            cpu = {'value': tps, 'unit': 'tokens/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                   'sample': 'per-timestep PyTorch loop (oracle port of the reference formulation), fwd+bwd by '
                             'autograd, fp32, 6 repetitions of the step (%d carried segment(s) of B=%d,H=%d,L=%d,d=%d; '
                             '%.2f s each)' % (segs, Bs, H, Ls, d, sec)}
        line = {
            'metric': 'fast-weight fwd+bwd tokens/s', 'value': value, 'unit': 'tokens/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': dev_s / args.steps * 1e3,
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': dts, 'data': 'synthetic',
            'config': workload_config(
                args.workload, B, H, L, d, segs, dts,
                sharding='batch x head units split over ranks, no collective on the data path',
                l2='flushed between timed steps (256 MiB write)', cuda_graph=graph is not None,
                timing='CUDA events per step, summed; max over ranks'),
            'roofline': {'bound': 'hbm', 'kernel': bwd_kernel, 'achieved': ach_b, 'peak': peak, 'unit': 'GB/s',
                         'frac': ach_b / peak, 'peak_kind': peak_kind, 'traffic': traffic, 'traffic_source': traffic_src,
                         'algorithmic_bytes_per_launch': bytes_bwd, 'launch_s': tb, 'launch_s_min': tb_min,
                         'timing': 'CUDA events around the %d segments launched back to back (distinct inputs, '
                                   'L2 flushed before the first), divided by %d' % (segs, segs)},
            'roofline_fwd_bwd': {'achieved': ach_fb, 'peak': peak, 'unit': 'GB/s', 'frac': ach_fb / peak,
                                 'algorithmic_bytes': bytes_fwd + bytes_bwd, 'fwd_s': tf, 'bwd_s': tb,
                                 'fwd_s_min': tf_min, 'bwd_s_min': tb_min, 'kernels': dict(ds.kernels)},
            'cpu_baseline': cpu,
            'e2e': {'value': e2e_value, 'unit': 'tokens/s', 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h,
                    'steps': e2e_steps, 'batch': Be, 'api': 'recurrent_fwp_b200.fast_weight_delta (autograd) + .backward()',
                    'pipeline': 'uploads, compute and downloads on three streams, consecutive steps overlap (no device-wide synchronisation between them), the host at most three segments ahead of the downloads; pinned host buffers, ' + ('one copy per segment and direction (inputs packed in one buffer, results gathered on the device)' if packed else 'one copy per tensor')},
            'gpu_launches': int(launches), 'clocks': clocks, 'wall_s_timed_region': t_wall,
            'long_strong': strong, 'configs': configs,
        }
        if _lib.device_fault() != 0:
            raise SystemExit('bench.py: a bounded wait inside a kernel ran out; the numbers above are invalid')
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.all_reduce(torch.zeros(1))
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='fwp', choices=['fwp', 'reference'])
    ap.add_argument('--workload', default='lm', choices=sorted(WORKLOADS) + sorted(FAMILY_SHAPES) + ['lm_e2e', 'rl_step'])
    ap.add_argument('--no-graph', action='store_true')
    ap.add_argument('--tune', action='append', default=[], metavar='KEY=INT',
                    help='set an execution-plan switch of the library before the run (repeatable), e.g. delta.chunk=1')
    ap.add_argument('--skip-cpu', action='store_true')
    ap.add_argument('--e2e-unpacked', action='store_true',
                    help='end-to-end leg: one host-device copy per tensor instead of one per segment and direction')
    ap.add_argument('--skip-configs', action='store_true',
                    help='leave out the `configs` and `long_strong` objects (the other benchmark shapes)')
    ap.add_argument('--unfused-layer-io', action='store_true',
                    help='lm_e2e: run the chain of torch ops around the op instead of the fused prologue / epilogue')
    ap.add_argument('--kernels-only', action='store_true',
                    help='run the forward and backward kernels a few times and print their device times '
                         '(the command the ncu captures under profiles/ use)')
    args = ap.parse_args()
    if args.tune and args.impl != 'reference':      # execution-plan switches of the library, e.g. delta.chunk=1
        from recurrent_fwp_b200 import _lib
        for kv in args.tune:
            key, _, val = kv.partition('=')
            _lib.tune(key, int(val))
    if args.workload == 'lm_e2e':
        run_lm_e2e(args)
    elif args.workload == 'rl_step':
        run_single_step(args)
    elif args.workload in FAMILY_SHAPES:
        run_family(args)
    elif args.impl == 'reference':
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == '__main__':
    main()
