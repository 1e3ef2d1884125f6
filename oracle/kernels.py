"""CPU restatement of the reference's fast-weight CUDA kernels (TEST INFRASTRUCTURE ONLY).

This file is the checker, never the product: only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it.  The shipped ops call
the CUDA library and fail loudly when it is missing.

Every function below has the argument list of the native (pybind) function of
the reference that it restates, works on CPU tensors of any floating dtype
(fp32 to mimic the reference, fp64 as ground truth), mutates the state tensors
in place exactly as the CUDA kernels do, and *overwrites* its output buffers
(the reference accumulates into pre-zeroed buffers, which is the same thing for
the zero-initialised buffers its wrappers pass).

Notation: ``S[n,h,e,m]`` is the fast-weight matrix (``e`` = key/query index,
``m`` = value index).  ``colvec(S, x)[m] = sum_e S[e,m] x[e]`` and
``rowvec(S, y)[e] = sum_m S[e,m] y[m]``.

Parity pin: ``oracle/pin_against_reference.py`` runs the reference's own
``__main__`` self-tests on CPU with these functions standing in for the
JIT-compiled CUDA module, so each function is checked by the reference's own
per-timestep autograd loop under the reference's own thresholds.
"""
import torch

EPS_SOFTMAX = 1e-6  # fast_rnn_cuda.cu:71, fast_lstm_v2_cuda.cu (``esp``)


def colvec(S, x):
    """sum over the key index: [N,H,E,M] x [N,H,E] -> [N,H,M]."""
    return torch.einsum('nhem,nhe->nhm', S, x)


def rowvec(S, y):
    """sum over the value index: [N,H,E,M] x [N,H,M] -> [N,H,E]."""
    return torch.einsum('nhem,nhm->nhe', S, y)


def outer(x, y):
    return x.unsqueeze(-1) * y.unsqueeze(-2)


def softmax_max(x):
    """exp(x-max)/sum, the form of rec_update_fwm_tanh.cu:201-233 and fast_lstm_cuda.cu:299-338."""
    e = torch.exp(x - x.max(dim=-1, keepdim=True).values)
    return e / e.sum(dim=-1, keepdim=True)


def softmax_eps(x):
    """exp(x-max)/(sum+1e-6), the form of fast_rnn_cuda.cu:143-178 (v2) and fast_lstm_v2_cuda.cu:188-254."""
    e = torch.exp(x - x.max(dim=-1, keepdim=True).values)
    return e / (e.sum(dim=-1, keepdim=True) + EPS_SOFTMAX)


def softmax_bwd(p, g):
    """p * (g - <p,g>); every reference backward ignores the epsilon of softmax_eps."""
    return p * (g - (p * g).sum(dim=-1, keepdim=True))


def delta_bwd_block(S, G, k, v, beta, v_old):
    """One reversed delta-rule step, shared by every kernel family.

    ``S`` is the post-update state of the step and ``G = dL/dS`` with the
    step's upstream contribution already added.  Returns the pre-update state,
    the gradient w.r.t. it, and dk, dv, dbeta.  Follows
    fast_weight_cuda.cu:489-552 (value/beta pass) and :336-389 (query/key pass,
    including the in-place rewind of the state).
    """
    w = v - v_old
    u = beta * w
    r = colvec(G, k)
    br = beta * r
    dv = br
    dbeta = (r * w).sum(dim=-1, keepdim=True)
    dk = rowvec(G, u)
    S = S - outer(k, u)
    dk = dk - rowvec(S, br)
    G = G - outer(k, br)
    return S, G, dk, dv, dbeta


# --------------------------------------------------------------------------
# Delta rule: algorithmic/fast_weight/fast_weight_cuda.cu
# --------------------------------------------------------------------------

def fast_weight_forward(Q, K, V, beta, v_old, v_insert, kv, out):
    """fast_weight_forward, fast_weight_cuda.cu:182-240 (kernel :17-178)."""
    L = Q.shape[2]
    S = kv.clone()
    for t in range(L):
        k, q, v, b = K[:, :, t], Q[:, :, t], V[:, :, t], beta[:, :, t]
        vo = colvec(S, k)
        u = b * (v - vo)
        S = S + outer(k, u)
        out[:, :, t] = colvec(S, q)
        v_old[:, :, t] = vo
        v_insert[:, :, t] = u
    kv.copy_(S)


def fast_weight_backward(Q, K, V, beta, v_old, v_insert, grad_out, fw_mem,
                         grad_Q, grad_K, grad_V, grad_beta):
    """fast_weight_backward, fast_weight_cuda.cu:564-664.  ``fw_mem`` enters as
    the end-of-segment state and leaves rewound to the start-of-segment state."""
    L = Q.shape[2]
    S = fw_mem.clone()
    G = torch.zeros_like(S)
    for t in range(L - 1, -1, -1):
        k, q, v, b = K[:, :, t], Q[:, :, t], V[:, :, t], beta[:, :, t]
        gy = grad_out[:, :, t]
        G = G + outer(q, gy)
        grad_Q[:, :, t] = rowvec(S, gy)
        S, G, dk, dv, db = delta_bwd_block(S, G, k, v, b, v_old[:, :, t])
        grad_K[:, :, t] = dk
        grad_V[:, :, t] = dv
        grad_beta[:, :, t] = db
    fw_mem.copy_(S)


# --------------------------------------------------------------------------
# Sum rule: algorithmic/fast_transformers/causal_product_cuda.cu
# --------------------------------------------------------------------------

def causal_dot_product(Q, K, V, kv, out):
    """causal_dot_product with carried state, causal_product_cuda.cu:98-140."""
    L = Q.shape[2]
    S = kv.clone()
    for t in range(L):
        S = S + outer(K[:, :, t], V[:, :, t])
        out[:, :, t] = colvec(S, Q[:, :, t])
    kv.copy_(S)


def causal_dot_backward(Q, K, V, grad_out, grad_Q, grad_K, grad_V):
    """causal_dot_backward, causal_product_cuda.cu:369-445.  The reference takes
    no state argument here: the key/value prefix sums restart from zero, so a
    carried non-zero state contributes nothing to grad_Q."""
    N, H, L, E = Q.shape
    M = V.shape[3]
    S = torch.zeros(N, H, E, M, dtype=Q.dtype)
    for t in range(L):
        S = S + outer(K[:, :, t], V[:, :, t])
        grad_Q[:, :, t] = rowvec(S, grad_out[:, :, t])
    G = torch.zeros_like(S)
    for t in range(L - 1, -1, -1):
        G = G + outer(Q[:, :, t], grad_out[:, :, t])
        grad_K[:, :, t] = rowvec(G, V[:, :, t])
        grad_V[:, :, t] = colvec(G, K[:, :, t])


# --------------------------------------------------------------------------
# Recurrent delta net: algorithmic/rec_update_fwm_tanh/rec_update_fwm_tanh.cu
# --------------------------------------------------------------------------

def rec_update_fwm_tanh_forward(qx, kx, vx, bx, Rq, Rk, Rv, rb,
                                q_out, k_out, v_out, beta_out, v_old,
                                states, kv, out):
    """rec_update_fwm_tanh_forward, rec_update_fwm_tanh.cu:349-444 (kernel :25-345).
    R_* are [1,H,d,d] with the first index contracting with the fed-back
    vector; rb is [1,H,1,d]; ``states`` [N,H,1,d] and ``kv`` are in/out."""
    L = qx.shape[2]
    S = kv.clone()
    h = states[:, :, 0].clone()
    rq, rk, rv, rbv = Rq[0], Rk[0], Rv[0], rb[0, :, 0]
    for t in range(L):
        ht = torch.tanh(h)
        q = softmax_max(qx[:, :, t] + torch.einsum('nhe,hem->nhm', ht, rq))
        k = softmax_max(kx[:, :, t] + torch.einsum('nhe,hem->nhm', ht, rk))
        v = vx[:, :, t] + torch.einsum('nhe,hem->nhm', ht, rv)
        b = torch.sigmoid(bx[:, :, t] + (ht * rbv).sum(-1, keepdim=True))
        vo = colvec(S, k)
        S = S + outer(k, b * (v - vo))
        h = colvec(S, q)
        out[:, :, t] = h
        q_out[:, :, t], k_out[:, :, t], v_out[:, :, t] = q, k, v
        beta_out[:, :, t] = b
        v_old[:, :, t] = vo
    kv.copy_(S)
    states[:, :, 0] = h


def rec_update_fwm_tanh_backward(q, k, v, beta, v_old, o_delayed, grad_out,
                                 Rq, Rk, Rv, rb, fw_mem,
                                 grad_q, grad_k, grad_v, grad_beta,
                                 grad_Rq, grad_Rk, grad_Rv, grad_rb):
    """rec_update_fwm_tanh_backward, rec_update_fwm_tanh.cu:880-986 (kernel :448-876).
    q,k,v,beta are the post-activation tensors saved by the forward;
    ``o_delayed[t] = tanh(y_{t-1})`` (tanh(h0) at t=0)."""
    L = q.shape[2]
    S = fw_mem.clone()
    G = torch.zeros_like(S)
    g_h = torch.zeros_like(q[:, :, 0])
    rq, rk, rv, rbv = Rq[0], Rk[0], Rv[0], rb[0, :, 0]
    aq, ak, av = (torch.zeros_like(rq) for _ in range(3))
    ab = torch.zeros_like(rbv)
    for t in range(L - 1, -1, -1):
        qt, kt, vt, bt = q[:, :, t], k[:, :, t], v[:, :, t], beta[:, :, t]
        ht = o_delayed[:, :, t]
        g = grad_out[:, :, t] + g_h
        dq = softmax_bwd(qt, rowvec(S, g))
        G = G + outer(qt, g)
        S, G, dk, dv, db = delta_bwd_block(S, G, kt, vt, bt, v_old[:, :, t])
        db = db * bt * (1 - bt)
        dk = softmax_bwd(kt, dk)
        back = (torch.einsum('hem,nhm->nhe', rq, dq) + torch.einsum('hem,nhm->nhe', rk, dk)
                + torch.einsum('hem,nhm->nhe', rv, dv) + rbv * db)
        g_h = (1 - ht * ht) * back
        aq = aq + torch.einsum('nhe,nhm->hem', ht, dq)
        ak = ak + torch.einsum('nhe,nhm->hem', ht, dk)
        av = av + torch.einsum('nhe,nhm->hem', ht, dv)
        ab = ab + (ht * db).sum(0)
        grad_q[:, :, t], grad_k[:, :, t], grad_v[:, :, t] = dq, dk, dv
        grad_beta[:, :, t] = db
    fw_mem.copy_(S)
    grad_Rq[0], grad_Rk[0], grad_Rv[0] = aq, ak, av
    grad_rb[0, :, 0] = ab


# --------------------------------------------------------------------------
# Delta RNN v2: algorithmic/fast_weight_rnn_v2/fast_rnn_cuda.cu
# Delta RNN v1: language_modeling/src/utils/fast_weight_rnn/fast_rnn_cuda.cu
# --------------------------------------------------------------------------

def fast_rnn_v2_forward(Z, K, V, beta, v_old, states, kv, out, out_nmz):
    """fast_rnn_v2_forward, fast_weight_rnn_v2/fast_rnn_cuda.cu:233-293 (kernel :25-229)."""
    L = Z.shape[2]
    S = kv.clone()
    h = states[:, :, 0].clone()
    for t in range(L):
        k, v, b = K[:, :, t], V[:, :, t], beta[:, :, t]
        vo = colvec(S, k)
        S = S + outer(k, b * (v - vo))
        s = softmax_eps(h)
        h = colvec(S, s) + Z[:, :, t]
        out[:, :, t], out_nmz[:, :, t], v_old[:, :, t] = h, s, vo
    kv.copy_(S)
    states[:, :, 0] = h


def fast_rnn_v2_backward(K, V, beta, v_old, grad_out, out, out_delayed, fw_mem,
                         grad_Z, grad_K, grad_V, grad_beta):
    """fast_rnn_v2_backward, fast_weight_rnn_v2/fast_rnn_cuda.cu:592-659 (kernel :297-588).
    ``out_delayed`` is the normalised delayed state saved by the forward
    (softmax_eps(h_{t-1})); ``out`` is accepted for signature parity only."""
    L = K.shape[2]
    S = fw_mem.clone()
    G = torch.zeros_like(S)
    g_h = torch.zeros_like(K[:, :, 0])
    for t in range(L - 1, -1, -1):
        s = out_delayed[:, :, t]
        g = grad_out[:, :, t] + g_h
        grad_Z[:, :, t] = g
        G = G + outer(s, g)
        gs = rowvec(S, g)
        S, G, dk, dv, db = delta_bwd_block(S, G, K[:, :, t], V[:, :, t], beta[:, :, t], v_old[:, :, t])
        g_h = softmax_bwd(s, gs)
        grad_K[:, :, t], grad_V[:, :, t], grad_beta[:, :, t] = dk, dv, db
    fw_mem.copy_(S)


def fast_rnn_forward(Z, K, V, beta, v_old, states, kv, out):
    """fast_rnn_forward (v1), fast_weight_rnn/fast_rnn_cuda.cu: h_t = softmax(S_t^T h_{t-1} + z_t)."""
    L = Z.shape[2]
    S = kv.clone()
    h = states[:, :, 0].clone()
    for t in range(L):
        k, v, b = K[:, :, t], V[:, :, t], beta[:, :, t]
        vo = colvec(S, k)
        S = S + outer(k, b * (v - vo))
        h = softmax_max(colvec(S, h) + Z[:, :, t])
        out[:, :, t], v_old[:, :, t] = h, vo
    kv.copy_(S)
    states[:, :, 0] = h


def fast_rnn_backward(K, V, beta, v_old, grad_out, out, out_delayed, fw_mem,
                      grad_Z, grad_K, grad_V, grad_beta):
    """fast_rnn_backward (v1).  ``out_delayed = cat[h0, out[:-1]]`` is built by the wrapper."""
    L = K.shape[2]
    S = fw_mem.clone()
    G = torch.zeros_like(S)
    g_h = torch.zeros_like(K[:, :, 0])
    for t in range(L - 1, -1, -1):
        g = grad_out[:, :, t] + g_h
        dz = softmax_bwd(out[:, :, t], g)
        grad_Z[:, :, t] = dz
        G = G + outer(out_delayed[:, :, t], dz)
        g_h = rowvec(S, dz)
        S, G, dk, dv, db = delta_bwd_block(S, G, K[:, :, t], V[:, :, t], beta[:, :, t], v_old[:, :, t])
        grad_K[:, :, t], grad_V[:, :, t], grad_beta[:, :, t] = dk, dv, db
    fw_mem.copy_(S)


# --------------------------------------------------------------------------
# Delta LSTM v1..v4: language_modeling/src/utils/fast_lstm*/fast_lstm*_cuda.cu
# --------------------------------------------------------------------------

def fast_lstm_forward(variant,
                      Zi, Ki, Vi, bi, Zu, Ku, Vu, bu, Zo, Ko, Vo, bo,
                      states, cells, kv_i, kv_u, kv_o,
                      out, out_del_nmz, cell_out, gate_i, update_u, gate_o,
                      v_old_i, v_old_u, v_old_o):
    """fast_lstm*_forward.  variant 1: fast_lstm_cuda.cu:364-480 (kernel :28-360);
    variants 2-4 feed softmax_eps(h_{t-1}) to the fast matrices
    (fast_lstm_v2_cuda.cu:188-254) and differ in the output line
    (fast_lstm_v3_cuda.cu:293-295, fast_lstm_v4_cuda.cu:287-288).
    ``out_del_nmz`` is None for variant 1 (that native function has no such argument)."""
    L = Zi.shape[2]
    Si, Su, So = kv_i.clone(), kv_u.clone(), kv_o.clone()
    h = states[:, :, 0].clone()
    c = cells[:, :, 0].clone()
    for t in range(L):
        voi, vou, voo = colvec(Si, Ki[:, :, t]), colvec(Su, Ku[:, :, t]), colvec(So, Ko[:, :, t])
        Si = Si + outer(Ki[:, :, t], bi[:, :, t] * (Vi[:, :, t] - voi))
        Su = Su + outer(Ku[:, :, t], bu[:, :, t] * (Vu[:, :, t] - vou))
        So = So + outer(Ko[:, :, t], bo[:, :, t] * (Vo[:, :, t] - voo))
        x = h if variant == 1 else softmax_eps(h)
        gi = torch.sigmoid(colvec(Si, x) + Zi[:, :, t])
        uu = colvec(Su, x) + Zu[:, :, t]
        if variant != 4:
            uu = torch.sigmoid(uu)
        go = torch.sigmoid(colvec(So, x) + Zo[:, :, t])
        c = gi * uu + (1 - gi) * c
        if variant == 1:
            h = softmax_max(go * c)
        elif variant == 3:
            h = go * c + Zu[:, :, t]
        else:
            h = go * c
        out[:, :, t], cell_out[:, :, t] = h, c
        gate_i[:, :, t], update_u[:, :, t], gate_o[:, :, t] = gi, uu, go
        v_old_i[:, :, t], v_old_u[:, :, t], v_old_o[:, :, t] = voi, vou, voo
        if variant != 1:
            out_del_nmz[:, :, t] = x
    kv_i.copy_(Si)
    kv_u.copy_(Su)
    kv_o.copy_(So)
    states[:, :, 0] = h
    cells[:, :, 0] = c


def fast_lstm_backward(variant, grad_out,
                       Ki, Vi, bi, Ku, Vu, bu, Ko, Vo, bo,
                       v_old_i, v_old_u, v_old_o,
                       out, out_delayed, cell_out, u_minus_c,
                       gate_i, update_u, gate_o,
                       kv_i, kv_u, kv_o,
                       gZi, gKi, gVi, gbi, gZu, gKu, gVu, gbu, gZo, gKo, gVo, gbo):
    """fast_lstm*_backward.  variant 1: fast_lstm_cuda.cu:1061-1205 (kernel :484-1056);
    variants 2-4: fast_lstm_v2_cuda.cu:734-759,898-913 and the v3/v4 deltas.
    ``out_delayed`` is cat[h0, out[:-1]] for variant 1 and the saved
    softmax_eps(h_{t-1}) for variants 2-4; ``u_minus_c = update_u - c_{t-1}``."""
    L = Ki.shape[2]
    Si, Su, So = kv_i.clone(), kv_u.clone(), kv_o.clone()
    Gi, Gu, Go = torch.zeros_like(Si), torch.zeros_like(Su), torch.zeros_like(So)
    g_h = torch.zeros_like(Ki[:, :, 0])
    g_c = torch.zeros_like(g_h)
    for t in range(L - 1, -1, -1):
        x = out_delayed[:, :, t]
        gi, uu, go, c = gate_i[:, :, t], update_u[:, :, t], gate_o[:, :, t], cell_out[:, :, t]
        g = grad_out[:, :, t] + g_h
        a = softmax_bwd(out[:, :, t], g) if variant == 1 else g
        dzo = (c * a) * (1 - go) * go
        g_c = g_c + go * a
        Go = Go + outer(x, dzo)
        g_h = rowvec(So, dzo)
        dzi = (g_c * u_minus_c[:, :, t]) * (1 - gi) * gi
        dzu = g_c * gi
        if variant != 4:
            dzu = dzu * (1 - uu) * uu
        g_c = g_c * (1 - gi)
        Gi = Gi + outer(x, dzi)
        Gu = Gu + outer(x, dzu)
        g_h = g_h + rowvec(Si, dzi) + rowvec(Su, dzu)
        So, Go, dko, dvo, dbo = delta_bwd_block(So, Go, Ko[:, :, t], Vo[:, :, t], bo[:, :, t], v_old_o[:, :, t])
        Si, Gi, dki, dvi, dbi = delta_bwd_block(Si, Gi, Ki[:, :, t], Vi[:, :, t], bi[:, :, t], v_old_i[:, :, t])
        Su, Gu, dku, dvu, dbu = delta_bwd_block(Su, Gu, Ku[:, :, t], Vu[:, :, t], bu[:, :, t], v_old_u[:, :, t])
        if variant != 1:
            g_h = softmax_bwd(x, g_h)
        gZi[:, :, t], gZo[:, :, t] = dzi, dzo
        gZu[:, :, t] = dzu + g if variant == 3 else dzu
        gKi[:, :, t], gVi[:, :, t], gbi[:, :, t] = dki, dvi, dbi
        gKu[:, :, t], gVu[:, :, t], gbu[:, :, t] = dku, dvu, dbu
        gKo[:, :, t], gVo[:, :, t], gbo[:, :, t] = dko, dvo, dbo
    kv_i.copy_(Si)
    kv_u.copy_(Su)
    kv_o.copy_(So)
