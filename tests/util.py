"""Seeded input generators (the BASELINE configurations) and error measures."""
import os

import numpy as np
import torch

from oracle import loops

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')


def golden(name):
    z = np.load(os.path.join(GOLDEN, name + '.npz'))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def gen(seed):
    g = torch.Generator(device='cpu')
    g.manual_seed(seed)
    return g


def delta_inputs(seed, B, H, L, E, M=None, dtype=torch.float32):
    """q,k,v ~ N(0,1); q,k <- sum_norm(elu+1); beta = sigmoid(N(0,1)); gy ~ N(0,1)."""
    M = E if M is None else M
    g = gen(seed)
    q = loops.sum_norm(loops.elu_p1(torch.randn(B, H, L, E, generator=g)))
    k = loops.sum_norm(loops.elu_p1(torch.randn(B, H, L, E, generator=g)))
    v = torch.randn(B, H, L, M, generator=g)
    beta = torch.sigmoid(torch.randn(B, H, L, 1, generator=g))
    gy = torch.randn(B, H, L, M, generator=g)
    return [t.to(dtype) for t in (q, k, v, beta, gy)]


def rec_inputs(seed, B, H, L, d):
    g = gen(seed)
    qx, kx, vx = (torch.randn(B, H, L, d, generator=g) for _ in range(3))
    bx = torch.randn(B, H, L, 1, generator=g)
    Rq, Rk, Rv = (torch.randn(1, H, d, d, generator=g) / d ** 0.5 for _ in range(3))
    rb = torch.randn(1, H, 1, d, generator=g) / d ** 0.5
    gy = torch.randn(B, H, L, d, generator=g)
    return qx, kx, vx, bx, Rq, Rk, Rv, rb, gy


def rnn_inputs(seed, B, H, L, d):
    g = gen(seed)
    z = torch.randn(B, H, L, d, generator=g)
    k = torch.softmax(torch.randn(B, H, L, d, generator=g), dim=-1)
    v = torch.randn(B, H, L, d, generator=g)
    beta = torch.sigmoid(torch.randn(B, H, L, 1, generator=g))
    gy = torch.randn(B, H, L, d, generator=g)
    return z, k, v, beta, gy


def lstm_inputs(seed, B, H, L, d):
    gates = [rnn_inputs(seed * 7 + i, B, H, L, d)[:4] for i in range(3)]
    gy = torch.randn(B, H, L, d, generator=gen(seed + 1000))
    return gates, gy


def max_abs(a, b):
    return (a.double().cpu() - b.double().cpu()).abs().max().item()


def max_rel(a, b, eps=1e-6):
    """The reference self-tests' measure: max |b - a| / (|b| + eps), b the trusted value."""
    a, b = a.double().cpu(), b.double().cpu()
    return ((b - a).abs() / (b.abs() + eps)).max().item()


def scaled_rel(a, b):
    """max |b - a| / (|b| + mean|b|): element-wise relative error with the tensor's own
    scale as the floor, for N(0,1)-driven gradients whose smallest entries are pure
    cancellation noise in any fp32 implementation."""
    a, b = a.double().cpu(), b.double().cpu()
    return ((b - a).abs() / (b.abs() + b.abs().mean())).max().item()
