"""Per-timestep PyTorch formulation of every fast-weight op (TEST INFRASTRUCTURE ONLY).

This is the reference's CPU path: the loops its wrapper files use to check
their CUDA kernels (one autograd-tracked step per token, gradients by
``backward()``).  Only the test-suite, the smoke check and the benchmark's
CPU-baseline / ``--impl reference`` legs may import this file; the shipped ops
never do.

Each function takes tensors laid out as the ops take them, ``(N, H, L, d)``,
and returns the outputs plus the end-of-segment states.  Gradients come from
autograd, so these loops are an independent check on the explicit backward
formulas in ``oracle/kernels.py``.

Restated from (paths inside the reference project):
  delta rule      algorithmic/fast_weight/__init__.py:178-190
  recurrent delta algorithmic/rec_update_fwm_tanh/__init__.py:263-302
  delta RNN v2    algorithmic/fast_weight_rnn_v2/__init__.py:205-217
  delta RNN v1    language_modeling/src/utils/fast_weight_rnn/__init__.py:205-215
  delta LSTM v1   language_modeling/src/utils/fast_lstm/__init__.py:394-429
  delta LSTM v2-4 language_modeling/src/utils/fast_lstm_v{2,3,4}/__init__.py:404-435
  sum rule        algorithmic/fast_transformers/__init__.py (self-test loop)
  input maps      algorithmic/layers.py:13-20 (elu_p1, sum_norm)
The reference loops hold the transposed matrix ``W[b, m, e]``; here the matrix
is ``S[n, h, e, m]`` as the ops store it.  The reference's RNN-v2 / LSTM-v2-4
loops use a plain softmax where its kernels add 1e-6 to the denominator;
``eps_softmax=True`` selects the kernel's form.
"""
import torch
import torch.nn.functional as F

from .kernels import EPS_SOFTMAX


def elu_p1(x):
    return F.elu(x, 1., False) + 1.


def sum_norm(x):
    return x / x.sum(-1, keepdim=True)


def _sm(x, eps_softmax):
    if not eps_softmax:
        return F.softmax(x, dim=-1)
    e = torch.exp(x - x.max(dim=-1, keepdim=True).values.detach())
    return e / (e.sum(-1, keepdim=True) + EPS_SOFTMAX)


def _delta_step(S, k, v, b):
    v_old = torch.einsum('nhem,nhe->nhm', S, k)
    return S + k.unsqueeze(-1) * (b * (v - v_old)).unsqueeze(-2)


def _read(S, x):
    return torch.einsum('nhem,nhe->nhm', S, x)


def delta_rule(Q, K, V, beta, W0):
    S = W0
    ys = []
    for t in range(Q.shape[2]):
        S = _delta_step(S, K[:, :, t], V[:, :, t], beta[:, :, t])
        ys.append(_read(S, Q[:, :, t]))
    return torch.stack(ys, dim=2), S


def sum_rule(Q, K, V, W0):
    S = W0
    ys = []
    for t in range(Q.shape[2]):
        S = S + K[:, :, t].unsqueeze(-1) * V[:, :, t].unsqueeze(-2)
        ys.append(_read(S, Q[:, :, t]))
    return torch.stack(ys, dim=2), S


def rec_delta(qx, kx, vx, bx, R_q, R_k, R_v, r_b, W0, h0):
    S, h = W0, h0[:, :, 0]
    ys = []
    for t in range(qx.shape[2]):
        ht = torch.tanh(h)
        q = F.softmax(qx[:, :, t] + torch.einsum('nhe,hem->nhm', ht, R_q[0]), dim=-1)
        k = F.softmax(kx[:, :, t] + torch.einsum('nhe,hem->nhm', ht, R_k[0]), dim=-1)
        v = vx[:, :, t] + torch.einsum('nhe,hem->nhm', ht, R_v[0])
        b = torch.sigmoid(bx[:, :, t] + (ht * r_b[0, :, 0]).sum(-1, keepdim=True))
        S = _delta_step(S, k, v, b)
        h = _read(S, q)
        ys.append(h)
    return torch.stack(ys, dim=2), S, h.unsqueeze(2)


def delta_rnn_v2(Z, K, V, W0, beta, h0, eps_softmax=True):
    S, h = W0, h0[:, :, 0]
    ys = []
    for t in range(Z.shape[2]):
        S = _delta_step(S, K[:, :, t], V[:, :, t], beta[:, :, t])
        h = _read(S, _sm(h, eps_softmax)) + Z[:, :, t]
        ys.append(h)
    return torch.stack(ys, dim=2), S, h.unsqueeze(2)


def delta_rnn_v1(Z, K, V, W0, beta, h0):
    S, h = W0, h0[:, :, 0]
    ys = []
    for t in range(Z.shape[2]):
        S = _delta_step(S, K[:, :, t], V[:, :, t], beta[:, :, t])
        h = F.softmax(_read(S, h) + Z[:, :, t], dim=-1)
        ys.append(h)
    return torch.stack(ys, dim=2), S, h.unsqueeze(2)


def delta_lstm(variant, Zi, Ki, Vi, bi, Wi, Zu, Ku, Vu, bu, Wu, Zo, Ko, Vo, bo, Wo, h0, c0,
               eps_softmax=True):
    Si, Su, So = Wi, Wu, Wo
    h, c = h0[:, :, 0], c0[:, :, 0]
    hs, cs = [], []
    for t in range(Zi.shape[2]):
        Si = _delta_step(Si, Ki[:, :, t], Vi[:, :, t], bi[:, :, t])
        Su = _delta_step(Su, Ku[:, :, t], Vu[:, :, t], bu[:, :, t])
        So = _delta_step(So, Ko[:, :, t], Vo[:, :, t], bo[:, :, t])
        x = h if variant == 1 else _sm(h, eps_softmax)
        gi = torch.sigmoid(_read(Si, x) + Zi[:, :, t])
        uu = _read(Su, x) + Zu[:, :, t]
        if variant != 4:
            uu = torch.sigmoid(uu)
        go = torch.sigmoid(_read(So, x) + Zo[:, :, t])
        c = gi * uu + (1. - gi) * c
        if variant == 1:
            h = F.softmax(c * go, dim=-1)
        elif variant == 3:
            h = c * go + Zu[:, :, t]
        else:
            h = c * go
        hs.append(h)
        cs.append(c)
    return torch.stack(hs, dim=2), torch.stack(cs, dim=2), (Si, Su, So), h.unsqueeze(2), c.unsqueeze(2)
