"""GPU parity of the delta-rule (and sum-rule) kernels, through the C ABI, against
the CPU oracle on identical seeded inputs and against the golden fixtures.

Tolerances (fp32): max |dy| <= 1e-4; gradients: the reference self-test's measure
max |d| / (|ref| + 1e-6) <= 1e-3 on the reference-shaped golden case; on the N(0,1)-driven
configurations ``util.check_grads`` gates max |d| / (|ref| + mean|ref|) <= 1e-3 and the strict
measure for every entry above 4 x the noise floor of the fp32 CPU loop (its largest absolute error against
fp64 on the same inputs), recording all figures.

bf16 streams (fp32 state): the oracle is the fp64 recurrence on the bf16-rounded inputs.  Outputs are
themselves rounded to bf16 (half an ulp is 2^-9 = 2e-3 of the value) on top of products taken with bf16
operands, so the bounds are |dy| <= 8e-3 max|y| and gradients 2e-2 (scaled); the error of the fp32 CPU
recurrence with its outputs rounded to bf16 is recorded beside every figure as the anchor.
"""
import pytest
import torch

from oracle import kernels as K, loops
from tests import util

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def run_cuda(fwp, q, k, v, b, W, gy):
    leaves = [t.detach().to(DEV).requires_grad_() for t in (q, k, v, b)]
    y = fwp.fast_weight_delta(*leaves, W)
    W_end = W.clone()
    y.backward(gy.to(DEV))
    return y.detach(), [l.grad for l in leaves], W_end


def run_loop(q, k, v, b, W0, gy, dtype):
    leaves = [t.detach().to(dtype).clone().requires_grad_() for t in (q, k, v, b)]
    y, S = loops.delta_rule(*leaves, W0.to(dtype))
    (y * gy.to(dtype)).sum().backward()
    return y.detach(), [l.grad for l in leaves], S.detach()


def test_golden_reference_selftest_case(fwp):
    gd = util.golden('delta')
    q, k, v, b = (gd['in_' + n] for n in ('q0', 'k0', 'v0', 'beta0'))
    N, H, L, E = q.shape
    W = torch.zeros(N, H, E, v.shape[3], device=DEV)
    y, grads, _ = run_cuda(fwp, q, k, v, b, W, torch.ones(N, H, L, v.shape[3]))
    assert util.max_rel(y, gd['out_LBHd'].permute(1, 2, 0, 3)) < 1e-3
    for g, n in zip(grads, ('q2', 'k2', 'v2', 'beta2')):
        assert util.max_rel(g, gd['grad_' + n]) < 1e-3
    assert W.abs().max().item() < 1e-4     # rewound to the zero start state


@pytest.mark.parametrize('B,H,L,E,M', [
    (2, 8, 256, 16, 16),     # configs[0]
    (3, 2, 37, 32, 32),
    (2, 2, 41, 64, 64),
    (2, 3, 1, 16, 16),       # single step (the RL callers)
    (2, 2, 19, 18, 18),      # not a power of two
    (2, 2, 23, 20, 5),       # E != M
    (1, 2, 17, 16, 49),      # M = 3d+1
    (1, 1, 9, 64, 3),
])
def test_parity_vs_oracle(fwp, B, H, L, E, M):
    q, k, v, b, gy = util.delta_inputs(11, B, H, L, E, M)
    W0 = torch.randn(B, H, E, M, generator=util.gen(12)) * 0.1
    W = W0.to(DEV)
    y, grads, W_end = run_cuda(fwp, q, k, v, b, W, gy)
    y32, g32, S32 = run_loop(q, k, v, b, W0, gy, torch.float32)
    y64, g64, S64 = run_loop(q, k, v, b, W0, gy, torch.float64)
    assert util.max_abs(y, y32) <= 1e-4 and util.max_abs(y, y64) <= 1e-4
    assert util.max_abs(W_end, S64) <= 1e-4
    util.check_grads('delta B%d H%d L%d E%d M%d' % (B, H, L, E, M), 'qkvb', grads, g32, g64)
    for g, r32 in zip(grads, g32):
        assert util.scaled_rel(g, r32) <= 1e-3
    assert util.max_abs(W, W0) <= 1e-5     # backward rewound the state in place


def test_four_carried_segments_lm_shape(fwp):
    """configs[1]: B=64,H=8,L=256,d=16, state handed over 4 segments, fwd+bwd per segment."""
    B, H, L, d = 64, 8, 256, 16
    W = torch.zeros(B, H, d, d, device=DEV)
    S = torch.zeros(B, H, d, d, dtype=torch.float64)
    for seg in range(4):
        q, k, v, b, gy = util.delta_inputs(100 + seg, B, H, L, d)
        W_in = W.clone()
        y, grads, W_end = run_cuda(fwp, q, k, v, b, W, gy)
        assert util.max_abs(W, W_in) <= 1e-5
        y64, g64, S_next = run_loop(q, k, v, b, S, gy, torch.float64)
        y32, g32, _ = run_loop(q, k, v, b, S, gy, torch.float32)
        assert util.max_abs(y, y64) <= 1e-4
        util.record('delta lm shape segment %d' % seg, y_cuda=util.max_abs(y, y64), y_cpu32=util.max_abs(y32, y64))
        util.check_grads('delta lm shape segment %d' % seg, 'qkvb', grads, g32, g64)
        W = W_end            # the caller's clone of the end state, as the reference layers do
        S = S_next
        assert util.max_abs(W, S) <= 1e-4


def test_strided_views_of_a_fused_projection(fwp):
    """Callers pass permuted views of one (L, B, H, 3d+1) projection; no copy is required."""
    L, B, H, d = 33, 2, 4, 16
    g = util.gen(5)
    fused = torch.randn(L, B, H, 3 * d + 1, generator=g)
    hq, hk, hv, hb = torch.split(fused, (d, d, d, 1), -1)
    q = loops.sum_norm(loops.elu_p1(hq)).permute(1, 2, 0, 3)
    k = loops.sum_norm(loops.elu_p1(hk)).permute(1, 2, 0, 3)
    v = hv.permute(1, 2, 0, 3)
    b = torch.sigmoid(hb).permute(1, 2, 0, 3)
    gy = torch.randn(L, B, H, d, generator=g).permute(1, 2, 0, 3)
    assert not v.is_contiguous()
    fused_dev = fused.to(DEV)
    vq = fused_dev[..., 2 * d:3 * d].permute(1, 2, 0, 3).requires_grad_()   # a true strided view on the device
    qd, kd, bd = (t.to(DEV).requires_grad_() for t in (q, k, b))
    W = torch.zeros(B, H, d, d, device=DEV)
    y = fwp.fast_weight_delta(qd, kd, vq, bd, W)
    y.backward(gy.to(DEV))
    y64, g64, _ = run_loop(q, k, v, b, torch.zeros(B, H, d, d), gy, torch.float64)
    assert util.max_abs(y, y64) <= 1e-4
    for got, ref in zip((qd.grad, kd.grad, vq.grad, bd.grad), g64):
        assert util.scaled_rel(got, ref) <= 1e-3


def test_batch_prefix_slice_of_a_larger_state(fwp):
    """`mems[:bsz]`: the state may be a prefix slice of a bigger buffer; only that slice is touched."""
    B, H, L, d = 2, 3, 12, 16
    big = torch.full((4, H, d, d), 7.0, device=DEV)
    big[:B] = 0
    q, k, v, b, gy = util.delta_inputs(21, B, H, L, d)
    y = fwp.fast_weight_delta(q.to(DEV), k.to(DEV), v.to(DEV), b.to(DEV), big[:B])
    y64, _, S64 = run_loop(q, k, v, b, torch.zeros(B, H, d, d), gy, torch.float64)
    assert util.max_abs(y, y64) <= 1e-4 and util.max_abs(big[:B], S64) <= 1e-4
    assert (big[B:] == 7.0).all()


def test_bitwise_reproducible(fwp):
    q, k, v, b, gy = util.delta_inputs(31, 4, 4, 64, 32)
    outs = []
    for _ in range(2):
        W = torch.zeros(4, 4, 32, 32, device=DEV)
        y, grads, _ = run_cuda(fwp, q, k, v, b, W, gy)
        outs.append([y] + grads)
    for a, c in zip(*outs):
        assert torch.equal(a, c)


BF16_Y, BF16_G = 8e-3, 2e-2     # |dy| / max|y| and scaled-rel gradient bounds for bf16 streams


def bf16_anchor(case, y, grads, y64, g64, y32, g32):
    """Record the CUDA path's error against fp64 beside the error of the fp32 CPU recurrence whose outputs are
    rounded to bf16 (what a perfect kernel with bf16 outputs could do), and gate the CUDA path."""
    ym = y64.abs().max().item()
    e_cuda = util.max_abs(y.float(), y64) / ym
    e_cpu = util.max_abs(y32.to(torch.bfloat16).float(), y64) / ym
    util.record(case, tensor='y', rel_to_max_cuda=e_cuda, rel_to_max_cpu32_rounded=e_cpu)
    assert e_cuda <= BF16_Y, (case, e_cuda, e_cpu)
    for n, g, r32, r64 in zip('qkvb', grads, g32, g64):
        s_cuda = util.scaled_rel(g.float(), r64)
        s_cpu = util.scaled_rel(r32.to(torch.bfloat16).float(), r64)
        util.record(case, tensor='d' + n, scaled_cuda=s_cuda, scaled_cpu32_rounded=s_cpu)
        assert s_cuda <= BF16_G, (case, n, s_cuda, s_cpu)


def test_bf16_streams_fp32_state(fwp):
    """bf16 q/k/v/beta/gy with an fp32 state: oracle = fp64 loop on the bf16-rounded inputs."""
    B, H, L, d = 2, 4, 128, 64
    q, k, v, b, gy = [t.to(torch.bfloat16) for t in util.delta_inputs(41, B, H, L, d)]
    W = torch.zeros(B, H, d, d, device=DEV)
    y, grads, W_end = run_cuda(fwp, q, k, v, b, W, gy)
    assert y.dtype == torch.bfloat16
    f = [t.float() for t in (q, k, v, b)]
    y64, g64, S64 = run_loop(*f, torch.zeros(B, H, d, d), gy.float(), torch.float64)
    y32, g32, _ = run_loop(*f, torch.zeros(B, H, d, d), gy.float(), torch.float32)
    bf16_anchor('delta bf16 d64 L128', y, grads, y64, g64, y32, g32)
    assert util.max_abs(W_end, S64) <= 1e-4


def test_sum_rule_golden_and_oracle(fwp):
    gd = util.golden('sum')
    q, k, v = gd['in_q0'], gd['in_k0'], gd['in_v0']
    N, H, L, E = q.shape
    M = v.shape[3]
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
    W = torch.zeros(N, H, E, M, device=DEV)
    y = fwp.fast_weight_sum(*leaves, W)
    y.sum().backward()
    ref = [t.clone().requires_grad_() for t in (q, k, v)]
    y2, S2 = loops.sum_rule(*ref, torch.zeros(N, H, E, M))
    y2.sum().backward()
    assert util.max_rel(y, y2) < 1e-3 and util.max_abs(W, S2) < 1e-4
    for leaf, n in zip(leaves, ('q2', 'k2', 'v2')):
        assert util.max_rel(leaf.grad, gd['grad_' + n]) < 1e-3


def test_unsupported_head_dim_is_an_error_not_a_fallback(fwp):
    q = torch.rand(1, 1, 4, 512, device=DEV)
    with pytest.raises(RuntimeError, match='head dimension'):
        fwp.fast_weight_delta(q, q, q, torch.rand(1, 1, 4, 1, device=DEV), torch.zeros(1, 1, 512, 512, device=DEV))


@pytest.mark.parametrize('B,H,L,E,M', [
    (2, 2, 13, 128, 16),     # Performer / DPFP feature maps: wide keys, narrow values
    (1, 2, 9, 96, 32),       # E = 2 * n_roll * d
    (1, 2, 11, 16, 97),      # M = 3d+1 above the register-resident limit
    (1, 1, 7, 200, 10),
    (1, 2, 5, 128, 128),
])
def test_shapes_above_64_use_the_shared_memory_kernels(fwp, B, H, L, E, M):
    q, k, v, b, gy = util.delta_inputs(61, B, H, L, E, M)
    W0 = torch.randn(B, H, E, M, generator=util.gen(62)) * 0.1
    W = W0.to(DEV)
    y, grads, W_end = run_cuda(fwp, q, k, v, b, W, gy)
    y64, g64, S64 = run_loop(q, k, v, b, W0, gy, torch.float64)
    assert util.max_abs(y, y64) <= 1e-4 and util.max_abs(W_end, S64) <= 1e-4
    for g, r in zip(grads, g64):
        assert util.scaled_rel(g, r) <= 1e-3
    assert util.max_abs(W, W0) <= 1e-5


@pytest.mark.parametrize('B,H,L,E,M', [(2, 2, 13, 128, 16), (1, 2, 9, 96, 32), (1, 2, 11, 16, 97), (1, 1, 7, 300, 10)])
def test_sum_rule_above_64_both_directions(fwp, B, H, L, E, M):
    """The sum rule takes any E, M in the reference (causal_product_cuda.cu:369-445); above 64 both directions run
    on the shared-memory kernels.  A carried non-zero state enters the forward only, as in the reference."""
    q, k, v, _, gy = util.delta_inputs(63, B, H, L, E, M)
    W0 = torch.randn(B, H, E, M, generator=util.gen(64)) * 0.1
    leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
    W = W0.to(DEV)
    y = fwp.fast_weight_sum(*leaves, W)
    y.backward(gy.to(DEV))
    ref = [t.double().requires_grad_() for t in (q, k, v)]
    y64, S64 = loops.sum_rule(*ref, W0.double())
    y0, _ = loops.sum_rule(*ref, torch.zeros(B, H, E, M, dtype=torch.float64))   # the backward restarts from zero
    (y0 * gy.double()).sum().backward()
    assert util.max_abs(y, y64) <= 1e-4 and util.max_abs(W, S64) <= 1e-4
    for leaf, r in zip(leaves, ref):
        assert util.scaled_rel(leaf.grad, r.grad) <= 1e-3


@pytest.mark.parametrize('B,H,L,E,M', [(2, 2, 37, 16, 16), (1, 3, 16, 12, 16), (3, 1, 17, 32, 20), (1, 2, 9, 24, 32),
                                       (1, 1, 13, 64, 64), (1, 2, 1, 16, 16), (1, 1, 5, 40, 64)])
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_sum_rule_backward_side_by_side_equals_one_after_the_other(fwp, B, H, L, E, M, dtype):
    """The sum rule's dq, dk, dv are independent prefix sums (causal_product_cuda.cu:369-445).  The default kernel
    gives each of them warps of its own; with ``sum_bwd.roles`` = 0 the same warps compute them one after the other.
    Both do the same additions in the same order, so the gradients are equal bit for bit; and they meet the oracle."""
    from recurrent_fwp_b200 import _lib
    q, k, v, _, gy = util.delta_inputs(71, B, H, L, E, M)
    q, k, v, gy = (t.to(dtype) for t in (q, k, v, gy))
    res, names = {}, {}
    try:
        for roles in (1, 0):
            _lib.tune('sum_bwd.roles', roles)
            leaves = [t.to(DEV).requires_grad_() for t in (q, k, v)]
            y = fwp.fast_weight_sum(*leaves, torch.zeros(B, H, E, M, device=DEV))
            seen = []
            leaves[0].register_hook(lambda g: seen.append(_lib.last_kernel()))
            y.backward(gy.to(DEV))
            res[roles], names[roles] = [l.grad for l in leaves], seen[0]
    finally:
        _lib.tune('sum_bwd.roles', 1)
    assert names[1] == 'sum_bwd_roles_kernel' and names[0] == 'sum_bwd_kernel'
    for a, b in zip(res[1], res[0]):
        assert torch.equal(a, b)
    ref = [t.double().requires_grad_() for t in (q, k, v)]
    y0, _ = loops.sum_rule(*ref, torch.zeros(B, H, E, M, dtype=torch.float64))
    (y0 * gy.double()).sum().backward()
    for a, r in zip(res[1], ref):
        assert util.scaled_rel(a.double(), r.grad) <= (1e-3 if dtype == torch.float32 else 2e-2)


def test_single_step_calls_replayed_from_a_cuda_graph(fwp):
    """The RL callers advance one environment step per call (L = 1, RL/model.py:436-448: 4 heads of 32, the state
    carried in place).  One such call captured in a CUDA graph and replayed over static input buffers -- the way
    an inference loop avoids the launch path -- gives the bits of eager stepping and meets the fp64 loop over the
    whole sequence."""
    B, H, T, d = 32, 4, 12, 32
    q, k, v, b, _ = util.delta_inputs(91, B, H, T, d)
    qd, kd, vd, bd = (t.to(DEV) for t in (q, k, v, b))
    # eager: one call per step on a state carried in place
    W_eager = torch.zeros(B, H, d, d, device=DEV)
    ys_eager = [fwp.fast_weight_delta(qd[:, :, t:t + 1], kd[:, :, t:t + 1], vd[:, :, t:t + 1], bd[:, :, t:t + 1], W_eager)
                for t in range(T)]
    # graph: static one-step buffers, the state updated in place by every replay
    sq, sk, sv = (torch.zeros(B, H, 1, d, device=DEV) for _ in range(3))
    sb = torch.zeros(B, H, 1, 1, device=DEV)
    W = torch.zeros(B, H, d, d, device=DEV)
    side = torch.cuda.Stream(DEV)
    side.wait_stream(torch.cuda.current_stream(DEV))
    with torch.cuda.stream(side), torch.no_grad():
        fwp.fast_weight_delta(sq, sk, sv, sb, W)           # warm-up outside the capture
        W.zero_()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=side):
            sy = fwp.fast_weight_delta(sq, sk, sv, sb, W)
        W.zero_()
        ys_graph = []
        for t in range(T):
            sq.copy_(qd[:, :, t:t + 1]); sk.copy_(kd[:, :, t:t + 1]); sv.copy_(vd[:, :, t:t + 1]); sb.copy_(bd[:, :, t:t + 1])
            gr.replay()
            ys_graph.append(sy.clone())
    side.synchronize()
    torch.cuda.synchronize()
    for a, e in zip(ys_graph, ys_eager):
        assert torch.equal(a, e)
    assert torch.equal(W, W_eager)
    y64, S64 = loops.delta_rule(q.double(), k.double(), v.double(), b.double(), torch.zeros(B, H, d, d, dtype=torch.float64))
    assert util.max_abs(torch.cat(ys_graph, dim=2), y64) <= 1e-4 and util.max_abs(W, S64) <= 1e-4


@pytest.mark.parametrize('graph', [False, True])
@pytest.mark.parametrize('B,H,L', [(8, 8, 96), (64, 32, 48)])      # one wave of CTAs; several waves (512 CTAs)
def test_dependent_launches_hand_results_on_like_plain_ones(fwp, graph, B, H, L):
    """The blocked kernels are launched so that their prologue may overlap the kernel before them in the stream
    (programmatic stream serialisation; they wait before touching global memory and let their own dependents in
    early).  A chain in which every launch consumes what the one before it wrote -- four forwards that carry the
    state in place, then the four backwards that rewind it, back to back with no other kernel between them --
    must give the same bits as with plain launches (``launch.dependent`` = 0), eagerly and replayed from a CUDA
    graph."""
    from recurrent_fwp_b200 import _lib
    d, segs = 16, 4
    ins = [[t.to(DEV) for t in util.delta_inputs(81 + s, B, H, L, d)] for s in range(segs)]
    D = _lib.desc

    def chain(out):
        stream, dev = _lib.stream_and_device(ins[0][0])
        W = out['W']
        for s in range(segs):
            q, k, v, b, _ = ins[s]
            _lib.check(_lib.lib.fwp_fast_weight_forward(B, H, L, d, d, D(q), D(k), D(v), D(b), D(out['vo'][s]), D(None),
                                                        D(W), D(out['y'][s]), _lib.F32, stream, dev), 'fwd')
        for s in reversed(range(segs)):
            q, k, v, b, gy = ins[s]
            _lib.check(_lib.lib.fwp_fast_weight_backward(B, H, L, d, d, D(q), D(k), D(v), D(b), D(out['vo'][s]), D(None),
                                                         D(gy), D(W), *(D(g) for g in out['g'][s]), _lib.F32, stream, dev),
                       'bwd')

    def buffers():
        new = lambda w=d: torch.zeros(B, H, L, w, device=DEV)
        return dict(W=torch.zeros(B, H, d, d, device=DEV), vo=[new() for _ in range(segs)], y=[new() for _ in range(segs)],
                    g=[[new(), new(), new(), new(1)] for _ in range(segs)])

    res = {}
    try:
        for dep in (1, 0):
            _lib.tune('launch.dependent', dep)
            out = buffers()
            if graph:
                side = torch.cuda.Stream(DEV)
                with torch.cuda.stream(side):
                    chain(out)                      # warm-up outside the capture
                    out['W'].zero_()
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr, stream=side):
                        chain(out)
                    out['W'].fill_(7.0)             # the replay must start from the state it finds
                    out['W'].zero_()
                    gr.replay()
                side.synchronize()
            else:
                chain(out)
            torch.cuda.synchronize()
            assert _lib.last_kernel() == 'delta_bwd_kernel'
            res[dep] = out
    finally:
        _lib.tune('launch.dependent', 1)
    assert util.max_abs(res[1]['W'], torch.zeros_like(res[1]['W'])) <= 1e-4      # rewound to the initial state
    for s in range(segs):
        assert torch.equal(res[1]['y'][s], res[0]['y'][s]) and torch.equal(res[1]['vo'][s], res[0]['vo'][s])
        for a, b in zip(res[1]['g'][s], res[0]['g'][s]):
            assert torch.equal(a, b)
    assert torch.equal(res[1]['W'], res[0]['W'])


@pytest.mark.parametrize('B,H,L,d', [(2, 2, 37, 16), (1, 2, 21, 32), (1, 1, 13, 64)])
def test_per_step_kernels_agree_with_blocked_form(fwp, B, H, L, d):
    """The four-step blocked kernels and the per-step kernels are two execution plans
    of the same recurrence; both must meet the oracle tolerance and agree with each other."""
    from recurrent_fwp_b200 import _lib
    q, k, v, b, gy = util.delta_inputs(51, B, H, L, d)
    W0 = torch.randn(B, H, d, d, generator=util.gen(52)) * 0.1
    res = {}
    try:
        for blocked in (1, 0):
            _lib.tune('delta.blocked', blocked)
            W = W0.to(DEV)
            res[blocked] = run_cuda(fwp, q, k, v, b, W, gy)
    finally:
        _lib.tune('delta.blocked', -1)
    y64, g64, _ = run_loop(q, k, v, b, W0, gy, torch.float64)
    for blocked in (1, 0):
        y, grads, _ = res[blocked]
        assert util.max_abs(y, y64) <= 1e-4
        for g, r in zip(grads, g64):
            assert util.scaled_rel(g, r) <= 1e-3
    assert util.max_abs(res[1][0], res[0][0]) <= 1e-5






@pytest.mark.parametrize('key,value', [('delta_bwd.bulk', 0), ('delta_bwd.16.chunk', 16)])
@pytest.mark.parametrize('B,H,L', [(2, 3, 100), (1, 2, 257)])
def test_alternative_backward_staging_plans_give_the_same_bits(fwp, key, value, B, H, L):
    """d = 16 backward: cp.async instead of bulk-copy staging, and 16-step chunks staged two ahead instead of
    32-step chunks staged one ahead.  Staging does not touch the arithmetic: results are bit-identical."""
    from recurrent_fwp_b200 import _lib
    d = 16
    q, k, v, b, gy = util.delta_inputs(97, B, H, L, d)
    W0 = torch.randn(B, H, d, d, generator=util.gen(98)) * 0.1
    res = []
    try:
        for setting in (None, value):
            if setting is not None:
                _lib.tune(key, setting)
            W = W0.to(DEV)
            y, grads, W_end = run_cuda(fwp, q, k, v, b, W, gy)
            res.append([y, W_end, W] + grads)
    finally:
        _lib.tune(key, 1 if key.endswith('bulk') else 32)
    for a, c in zip(*res):
        assert torch.equal(a, c)
    assert _lib.device_fault() == 0


@pytest.mark.parametrize('B,H,L', [(2, 3, 100), (1, 2, 17), (1, 2, 300), (3, 1, 64)])
def test_chunkwise_bf16_plan_at_d64_meets_the_oracle(fwp, B, H, L):
    """Default plan for bf16 streams at E = M = 64 beyond 16 steps: 16-step chunks, bf16 tensor-core products,
    fp32 state, one launch per direction.  Checked against the fp64 loop on the bf16-rounded inputs and
    against the per-step plan ('delta.chunk64' = 0).  Bounds: the bf16-stream bounds stated at the top of this
    file, end state 2e-4, rewound start state 1e-5."""
    from recurrent_fwp_b200 import _lib
    d = 64
    q, k, v, b, gy = [t.to(torch.bfloat16) for t in util.delta_inputs(301, B, H, L, d)]
    W0 = torch.randn(B, H, d, d, generator=util.gen(302)) * 0.1
    res = {}
    try:
        # 1: chunkwise plan (the default); 0: per-step plan
        for chunk in (1, 0):
            _lib.tune('delta.chunk64', chunk)
            before = _lib.lib.fwp_launch_count()
            W = W0.to(DEV)
            res[chunk] = run_cuda(fwp, q, k, v, b, W, gy) + (W, _lib.lib.fwp_launch_count() - before)
    finally:
        _lib.tune('delta.chunk64', 1)
    y64, g64, S64 = run_loop(q.float(), k.float(), v.float(), b.float(), W0, gy.float(), torch.float64)
    y32, g32, _ = run_loop(q.float(), k.float(), v.float(), b.float(), W0, gy.float(), torch.float32)
    for chunk in (1, 0):
        y, grads, W_end, W_back, launches = res[chunk]
        assert launches == 2
        bf16_anchor('delta bf16 d64 B%d H%d L%d plan %d' % (B, H, L, chunk), y, grads, y64, g64, y32, g32)
        assert util.max_abs(W_end, S64) <= 2e-4
        assert util.max_abs(W_back, W0) <= 1e-5
    # the two plans agree far inside the bf16 output rounding
    assert util.max_abs(res[1][0].float(), res[0][0].float()) <= 1e-2 * y64.abs().max().item()


def test_chunkwise_bf16_plan_leaves_unaligned_rows_to_the_per_step_plan(fwp):
    """Views of a fused (L,B,H,3d+1) projection have rows that are not 16-byte aligned: the chunkwise bf16 plan
    does not apply and the call takes the per-step kernels; same numbers as on contiguous copies within the
    bf16 bounds."""
    L, B, H, d = 40, 2, 2, 64
    g = util.gen(303)
    qkvb = torch.randn(L, B, H, 3 * d + 1, generator=g).to(DEV)
    q, k, v, beta = torch.split(qkvb, (d, d, d, 1), dim=-1)
    q, k, v, beta = (t.permute(1, 2, 0, 3) for t in (q, k, v, torch.sigmoid(beta)))
    fused = torch.cat([torch.softmax(q, -1), torch.softmax(k, -1), v, beta], -1).to(torch.bfloat16)
    q, k, v, beta = torch.split(fused, (d, d, d, 1), dim=-1)
    gy = torch.randn(B, H, L, d, generator=g).to(DEV).to(torch.bfloat16)
    res = []
    for contiguous in (False, True):
        leaves = [(t.contiguous() if contiguous else t).detach().requires_grad_() for t in (q, k, v, beta)]
        W = torch.zeros(B, H, d, d, device=DEV)
        y = fwp.fast_weight_delta(*leaves, W)
        W_end = W.clone()
        y.backward(gy)
        res.append([y.detach(), W_end] + [t.grad for t in leaves])
    ym = res[1][0].float().abs().max().item()
    assert util.max_abs(res[0][0].float(), res[1][0].float()) <= 2 * BF16_Y * ym
    assert util.max_abs(res[0][1], res[1][1]) <= 2e-4
    for a, c in zip(res[0][2:], res[1][2:]):
        assert util.scaled_rel(a.float(), c.float()) <= 2 * BF16_G


def explicit_oracle(q, k, v, b, W0, gy, dtype):
    """Forward and backward by the explicit recurrences (O(L) memory, no autograd graph), for long sequences."""
    q, k, v, b, gy = (t.to(dtype) for t in (q, k, v, b, gy))
    N, H, L, E = q.shape
    M = v.shape[3]
    z = lambda *s: torch.zeros(*s, dtype=dtype)
    y, vo, vi = z(N, H, L, M), z(N, H, L, M), z(N, H, L, M)
    S = W0.to(dtype).clone()
    K.fast_weight_forward(q, k, v, b, vo, vi, S, y)
    S_end = S.clone()
    g = [z(N, H, L, E), z(N, H, L, E), z(N, H, L, M), z(N, H, L, 1)]
    K.fast_weight_backward(q, k, v, b, vo, vi, gy, S, *g)
    return y, g, S_end, S


@pytest.mark.parametrize('tc64,forward', [(-1, 'delta_fwd_tc_kernel'), (0, 'delta_fwd_chunk_bf16_pipe_kernel')])
def test_chunkwise_bf16_plan_at_the_scale_out_length(fwp, tc64, forward):
    """The scale-out configuration's own sequence length (L = 4096, E = M = 64, bf16 streams) on a 1 x 2 slice:
    256 chunks of in-place rewinding.  Outputs, all four gradients, the end state and the *rewound* start state
    against the fp64 explicit recurrence on the bf16-rounded inputs, with the fp32 recurrence beside it.  Two
    sequences are fewer than the SMs, so the default forward here is the tcgen05 kernel; the warp-level forward
    (what a full shard of the configuration runs) is checked with the switch at 0."""
    from recurrent_fwp_b200 import _lib
    B, H, L, d = 1, 2, 4096, 64
    q, k, v, b, gy = [t.to(torch.bfloat16) for t in util.delta_inputs(401, B, H, L, d)]
    W0 = torch.randn(B, H, d, d, generator=util.gen(402)) * 0.1
    W = W0.to(DEV)
    try:
        _lib.tune('delta.tc64', tc64)
        leaves = [t.detach().to(DEV).requires_grad_() for t in (q, k, v, b)]
        y = fwp.fast_weight_delta(*leaves, W)
        assert _lib.last_kernel() == forward
        W_end = W.clone()
        y.backward(gy.to(DEV))
        y, grads = y.detach(), [l.grad for l in leaves]
    finally:
        _lib.tune('delta.tc64', -1)
    assert _lib.device_fault() == 0
    f = [t.float() for t in (q, k, v, b)]
    y64, g64, S64, S64_back = explicit_oracle(*f, W0, gy.float(), torch.float64)
    y32, g32, S32, S32_back = explicit_oracle(*f, W0, gy.float(), torch.float32)
    assert util.max_abs(S64_back, W0) <= 1e-12
    bf16_anchor('delta bf16 d64 L4096 tc64=%d' % tc64, y, grads, y64, g64, y32, g32)
    util.record('delta bf16 d64 L4096 tc64=%d' % tc64, tensor='state', end_cuda=util.max_abs(W_end, S64),
                end_cpu32=util.max_abs(S32, S64), rewound_cuda=util.max_abs(W, W0),
                rewound_cpu32=util.max_abs(S32_back, W0))
    assert util.max_abs(W_end, S64) <= 2e-4
    assert util.max_abs(W, W0) <= 5e-5      # 4096 reversed rank-1 updates in fp32


@pytest.mark.parametrize('d', [16, 32])
def test_fp32_plans_at_4096_steps(fwp, d):
    """fp32 streams at L = 4096 (d = 16: four-step blocked plan, d = 32: blocked backward): the rewind over the
    whole length stays inside the fp32 bounds."""
    B, H, L = 1, 2, 4096
    q, k, v, b, gy = util.delta_inputs(411, B, H, L, d)
    W0 = torch.randn(B, H, d, d, generator=util.gen(412)) * 0.1
    W = W0.to(DEV)
    y, grads, W_end = run_cuda(fwp, q, k, v, b, W, gy)
    y64, g64, S64, _ = explicit_oracle(q, k, v, b, W0, gy, torch.float64)
    y32, g32, S32, S32_back = explicit_oracle(q, k, v, b, W0, gy, torch.float32)
    assert util.max_abs(y, y64) <= 1e-4 and util.max_abs(W_end, S64) <= 1e-4
    util.check_grads('delta fp32 d%d L4096' % d, 'qkvb', grads, g32, g64)
    util.record('delta fp32 d%d L4096' % d, tensor='state', rewound_cuda=util.max_abs(W, W0),
                rewound_cpu32=util.max_abs(S32_back, W0))
    assert util.max_abs(W, W0) <= 5e-5


@pytest.mark.parametrize('B,H,L', [(1, 1, 64), (2, 3, 100), (1, 2, 17), (1, 2, 300), (3, 1, 128), (4, 16, 1024)])
def test_tcgen05_forward_plan_meets_the_oracle(fwp, B, H, L):
    """Opt-in forward for bf16 streams at E = M = 64 ('delta.tc64' = 1): 64-step chunks, every 64-wide product a
    tcgen05.mma with accumulators in tensor memory, K / Q / V tiles by TMA, five warp roles meeting at mbarriers.
    Same bounds as the warp-level chunkwise plan; the backward (warp-level) consumes its v_old, so the gradients
    check that tensor too.  No bounded wait may run out."""
    from recurrent_fwp_b200 import _lib
    d = 64
    q, k, v, b, gy = [t.to(torch.bfloat16) for t in util.delta_inputs(501, B, H, L, d)]
    W0 = torch.randn(B, H, d, d, generator=util.gen(502)) * 0.1
    res = {}
    try:
        for tc in (1, 0):
            _lib.tune('delta.tc64', tc)
            W = W0.to(DEV)
            leaves = [t.detach().to(DEV).requires_grad_() for t in (q, k, v, b)]
            y = fwp.fast_weight_delta(*leaves, W)
            kernel = _lib.last_kernel()
            W_end = W.clone()
            y.backward(gy.to(DEV))
            res[tc] = (y.detach(), [l.grad for l in leaves], W_end, W, kernel)
    finally:
        _lib.tune('delta.tc64', -1)
    assert _lib.device_fault() == 0
    assert res[1][4] == 'delta_fwd_tc_kernel' and res[0][4] == 'delta_fwd_chunk_bf16_pipe_kernel'
    f = [t.float() for t in (q, k, v, b)]
    y64, g64, S64 = run_loop(*f, W0, gy.float(), torch.float64)
    y32, g32, _ = run_loop(*f, W0, gy.float(), torch.float32)
    for tc in (1, 0):
        y, grads, W_end, W_back, _ = res[tc]
        bf16_anchor('delta bf16 d64 B%d H%d L%d tcgen05=%d' % (B, H, L, tc), y, grads, y64, g64, y32, g32)
        assert util.max_abs(W_end, S64) <= 2e-4
        assert util.max_abs(W_back, W0) <= 1e-5
    assert util.max_abs(res[1][0].float(), res[0][0].float()) <= 1e-2 * y64.abs().max().item()


@pytest.mark.parametrize('B,H,L', [(1, 1, 17), (2, 3, 33), (1, 2, 48), (3, 2, 300), (2, 16, 1024)])
def test_preparing_warp_kernels_equal_the_self_preparing_ones_bit_for_bit(fwp, B, H, L):
    """The chunkwise bf16 kernels with a preparing warp ('delta.pipe64' = 1, the default) do the same arithmetic as the
    kernels in which every warp prepares for itself ('delta.pipe64' = 0), only in another warp and one chunk earlier:
    outputs, v_old, end state, rewound state and all four gradients must be identical bit for bit, for two-chunk
    sequences, ragged last chunks and many chunks alike."""
    from recurrent_fwp_b200 import _lib
    d = 64
    q, k, v, b, gy = [t.to(torch.bfloat16) for t in util.delta_inputs(601, B, H, L, d)]
    W0 = torch.randn(B, H, d, d, generator=util.gen(602)) * 0.1
    res = {}
    names = {}
    try:
        _lib.tune('delta.tc64', 0)          # the warp-level forward whatever the sequence count
        for pipe in (1, 0):
            _lib.tune('delta.pipe64', pipe)
            W = W0.to(DEV)
            leaves = [t.detach().to(DEV).requires_grad_() for t in (q, k, v, b)]
            y = fwp.fast_weight_delta(*leaves, W)
            kf, kb = _lib.last_kernel(), []
            leaves[0].register_hook(lambda g, kb=kb: kb.append(_lib.last_kernel()))
            W_end = W.clone()
            y.backward(gy.to(DEV))
            res[pipe] = [y.detach(), W_end, W.clone()] + [l.grad for l in leaves]
            names[pipe] = (kf, kb[0])
    finally:
        _lib.tune('delta.pipe64', 1)
        _lib.tune('delta.tc64', -1)
    assert names[1] == ('delta_fwd_chunk_bf16_pipe_kernel', 'delta_bwd_chunk_bf16_pipe_kernel')
    assert names[0] == ('delta_fwd_chunk_bf16_inv_kernel', 'delta_bwd_chunk_bf16_inv_kernel')
    for a, r in zip(res[1], res[0]):
        assert torch.equal(a, r)


def test_tcgen05_forward_is_the_kernel_that_ran(fwp):
    """With the switch on, an eligible call runs delta_fwd_tc_kernel; a caller that asks for v_insert, or whose
    state is not 8-byte aligned, gets the warp-level kernel (the tcgen05 plan does not apply), never an error."""
    from recurrent_fwp_b200 import _lib
    B, H, L, d = 1, 2, 64, 64
    q, k, v, b, _ = [t.to(torch.bfloat16).to(DEV) for t in util.delta_inputs(503, B, H, L, d)]
    D = _lib.desc
    y = torch.empty(B, H, L, d, device=DEV, dtype=torch.bfloat16)
    vo = torch.empty(B, H, L, d, device=DEV)
    vi = torch.empty(B, H, L, d, device=DEV)
    stream, dev = _lib.stream_and_device(q)
    try:
        _lib.tune('delta.tc64', 1)
        for v_ins, want in ((None, 'delta_fwd_tc_kernel'), (vi, 'delta_fwd_chunk_bf16_pipe_kernel')):
            W = torch.zeros(B, H, d, d, device=DEV)
            _lib.check(_lib.lib.fwp_fast_weight_forward(B, H, L, d, d, D(q), D(k), D(v), D(b), D(vo), D(v_ins), D(W), D(y),
                                                        _lib.BF16, stream, dev), 'forward')
            assert _lib.last_kernel() == want
    finally:
        _lib.tune('delta.tc64', -1)
    torch.cuda.synchronize()
    assert _lib.device_fault() == 0


def test_a_wait_that_runs_out_is_reported_not_hung(fwp):
    """Failure detection without a fault: a probe kernel waits (64 polls) on a barrier nothing completes; it returns,
    the device flag reads 1 once, and the context keeps working."""
    from recurrent_fwp_b200 import _lib
    assert _lib.device_fault() == 0
    stream, dev = _lib.stream_and_device(torch.zeros(1, device=DEV))
    _lib.check(_lib.lib.fwp_debug_bounded_wait_probe(64, stream, dev), 'probe')
    torch.cuda.synchronize()
    assert _lib.device_fault() == 1
    assert _lib.device_fault() == 0
    assert _lib.lib.fwp_debug_bounded_wait_probe(0, stream, dev) == 2      # poll limit out of range: refused
    q, k, v, b, gy = util.delta_inputs(504, 1, 2, 33, 16)
    y, _, _ = run_cuda(fwp, q, k, v, b, torch.zeros(1, 2, 16, 16, device=DEV), gy)
    y64, _, _ = run_loop(q, k, v, b, torch.zeros(1, 2, 16, 16), gy, torch.float64)
    assert util.max_abs(y, y64) <= 1e-4
