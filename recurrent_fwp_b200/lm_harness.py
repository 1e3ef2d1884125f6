"""A delta-rule language model forward built on the public op: the caller-side harness for end-to-end checks.

This is the forward pass of the reference's ``MemTransformerLM`` for the configuration its
delta-rule language models use (language_modeling/src/model_main.py:898-1361 with
``attn_type=24, pre_lnorm=True, skip_attn_normalization=True, mem_len=0, cutoffs=[], div_val=1``):

* token embedding scaled by sqrt(d_model), tied with the output layer
  (model_main.py:833-896, utils/proj_adaptive_softmax.py:63-87 with no clusters);
* sinusoidal absolute positions counted backwards from the end of the segment
  (model_main.py:1271-1282, utils/model_utils.py:15-31);
* per layer: LayerNorm -> fused q/k/v/beta projection -> sigmoid(beta), elu+1 and sum
  normalisation of q and k -> ``fast_weight_delta`` -> scale by 1/sqrt(d_head) -> output
  projection -> residual onto the normalised input (utils/cuda_fast_weight_layer.py:57-189), then the position-wise
  feed-forward block with its own pre-LayerNorm and residual (utils/model_utils.py:34-67);
* per-token negative log-likelihood of shape (len, batch).

With ``carry_over_fast_weight=True`` every layer receives its fast weight matrix from the previous
segment and hands back a detached clone of the updated one, exactly like the reference's evaluation
loop (language_modeling/src/eval.py:97-118), including the ``[:bsz]`` slice for a short last batch.

``attn_type`` selects the fast-weight layer between the embedding and feed-forward blocks, numbered as in the
reference (model_main.py:744-758):
  24   delta rule                      (``CudaFastWeightLinearTransformerLayer``, cuda_fast_weight_layer.py:57-189)
  134  delta rule feeding a delta RNN  (``CudaFastRNNv2Layer``, :1830-1987)
  254  three delta rules feeding a delta LSTM, v4 (``CudaFastLSTMv4Layer``, :2763-3012)
  934  recurrent delta net             (``CudaFastWeightRecUpdateTanhLayer``, :3154-3290)
Each carries the reference's tuple of memories per layer (fast matrices, recurrent fast matrices, last hidden /
cell state) when ``carry_over_fast_weight=True``.

Parameter names equal the reference's ``state_dict`` keys, so weights exported from the reference
load with ``load_state_dict``.  The op is injectable (``delta_fn``) so that tests can run the same
module on the CPU with a checker in place of the CUDA op; the default is the CUDA op.  ``fused_io=True``
replaces the elementwise chain around the op by the one-launch prologue and epilogue of
``recurrent_fwp_b200/delta_layer_io.py``.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class _Named(nn.Module):
    """An empty container: only there to reproduce the reference's parameter paths."""


class _DeltaAttention(nn.Module):
    def __init__(self, n_head, d_model, d_head, delta_fn, fused_io):
        super().__init__()
        self.n_head, self.d_head = n_head, d_head
        self.fused_io = fused_io
        self.qkvb_net = nn.Linear(d_model, n_head * (3 * d_head + 1), bias=False)
        self.o_net = nn.Linear(n_head * d_head, d_model, bias=False)
        self.layer_norm = nn.LayerNorm(d_model)
        self.scale = 1.0 / math.sqrt(d_head)
        self.delta_fn = delta_fn

    def forward(self, h, mem, carry):
        slen, bsz, _ = h.shape
        x = self.layer_norm(h)
        qkvb = self.qkvb_net(x).view(slen, bsz, self.n_head, 3 * self.d_head + 1)
        if mem is None:
            W = torch.zeros(bsz, self.n_head, self.d_head, self.d_head, device=h.device, dtype=torch.float32)
        else:
            W = mem[0][:bsz]
        if self.fused_io:       # one launch before and one after the op instead of the chain below
            from recurrent_fwp_b200.delta_layer_io import delta_attention
            y = x + self.o_net(delta_attention(qkvb, W, self.scale))
            return y, ((W.clone().detach(), None) if carry else None)
        q, k, v, beta = torch.split(qkvb, (self.d_head, self.d_head, self.d_head, 1), dim=-1)
        # (len, B, H, d) -> (B, H, len, d); the op takes these strided views as they are
        q, k, v, beta = (t.permute(1, 2, 0, 3) for t in (q, k, v, torch.sigmoid(beta)))
        q = F.elu(q) + 1.0
        k = F.elu(k) + 1.0
        q = q / q.sum(-1, keepdim=True)
        k = k / k.sum(-1, keepdim=True)
        out = self.delta_fn(q, k, v, beta, W)                       # W now holds the end-of-segment state
        out = (self.scale * out).transpose(1, 2).reshape(bsz, slen, self.n_head * self.d_head).transpose(0, 1)
        y = x + self.o_net(out)     # the reference adds the *normalised* input back (cuda_fast_weight_layer.py:100-102,171-173)
        if carry:
            return y, (W.clone().detach(), None)
        return y, None


def _default_ops():
    from recurrent_fwp_b200.fast_weight import fast_weight_delta
    from recurrent_fwp_b200.fast_weight_rnn_v2 import fast_rnn_v2
    from recurrent_fwp_b200.fast_lstm_v4 import fast_lstm_v4
    from recurrent_fwp_b200.rec_update_fwm_tanh import rec_update_fwm_tanh
    return dict(delta=fast_weight_delta, rnn_v2=fast_rnn_v2, lstm_v4=fast_lstm_v4, rec_delta=rec_update_fwm_tanh)


def _bhld(t):
    """(len, B, H, d) -> (B, H, len, d); the ops take these strided views as they are."""
    return t.permute(1, 2, 0, 3)


def _phi(x):
    x = F.elu(x, 1., False) + 1.
    return x / x.sum(-1, keepdim=True)


class _RecurrentAttention(nn.Module):
    """What the three recurrent layer classes share: pre-LayerNorm, output projection, residual onto the
    normalised input, and the scale / transpose of the op's output."""

    def __init__(self, n_head, d_model, d_head, ops):
        super().__init__()
        self.n_head, self.d_head = n_head, d_head
        self.o_net = nn.Linear(n_head * d_head, d_model, bias=False)
        self.layer_norm = nn.LayerNorm(d_model)
        self.scale = 1.0 / math.sqrt(d_head)
        self.ops = ops

    def zeros(self, bsz, rows, like):
        return torch.zeros(bsz, self.n_head, rows, self.d_head, device=like.device, dtype=torch.float32)

    def finish(self, x, out):
        bsz, _, slen, _ = out.shape
        out = (self.scale * out).transpose(1, 2).reshape(bsz, slen, self.n_head * self.d_head).transpose(0, 1)
        return x + self.o_net(out)

    @staticmethod
    def last(out):
        return out[:, :, -1, :].clone().detach().unsqueeze(2)


class _DeltaRNNv2Attention(_RecurrentAttention):
    """attn_type 134: y = fast_rnn_v2(fast_weight_delta(q, k, v, beta), rec_k, rec_v, rec_beta)."""

    def __init__(self, n_head, d_model, d_head, ops):
        super().__init__(n_head, d_model, d_head, ops)
        self.qkvb_net = nn.Linear(d_model, n_head * (5 * d_head + 2), bias=False)

    def forward(self, h, mem, carry):
        slen, bsz, _ = h.shape
        d = self.d_head
        x = self.layer_norm(h)
        qkv = self.qkvb_net(x).view(slen, bsz, self.n_head, 5 * d + 2)
        q, k, v, rk, rv, b, rb = torch.split(qkv, (d,) * 5 + (1,) * 2, -1)
        q, k, v, rk, rv, b, rb = (_bhld(t) for t in (q, k, v, rk, rv, torch.sigmoid(b), torch.sigmoid(rb)))
        q, k, rk = _phi(q), _phi(k), F.softmax(rk, dim=-1)
        if mem is None:
            W, Wr, h0 = self.zeros(bsz, d, x), self.zeros(bsz, d, x), self.zeros(bsz, 1, x)
        else:
            W, Wr, h0 = (m[:bsz] for m in mem)
        z = self.ops['delta'](q, k, v, b, W)
        out = self.ops['rnn_v2'](z, rk, rv, Wr, rb, h0)
        y = self.finish(x, out)
        return y, ((W.clone().detach(), Wr.clone().detach(), self.last(out)) if carry else None)


class _DeltaLSTMv4Attention(_RecurrentAttention):
    """attn_type 254: three delta rules produce the gate inputs of a delta LSTM (v4: no sigmoid on the update)."""

    def __init__(self, n_head, d_model, d_head, ops):
        super().__init__(n_head, d_model, d_head, ops)
        self.qkv_net = nn.Linear(d_model, n_head * (15 * d_head + 6), bias=False)

    def forward(self, h, mem, carry):
        slen, bsz, _ = h.shape
        d = self.d_head
        x = self.layer_norm(h)
        parts = torch.split(self.qkv_net(x).view(slen, bsz, self.n_head, 15 * d + 6), (d,) * 15 + (1,) * 6, -1)
        gates = []
        for gi in range(3):          # input, update, output
            q, k, v, rk, rv = (_bhld(t) for t in parts[5 * gi:5 * gi + 5])
            b, rb = (_bhld(torch.sigmoid(t)) for t in parts[15 + 2 * gi:17 + 2 * gi])
            gates.append((_phi(q), _phi(k), v, b, F.softmax(rk, dim=-1), rv, rb))
        if mem is None:
            Wf = [self.zeros(bsz, d, x) for _ in range(3)]
            Wr = [self.zeros(bsz, d, x) for _ in range(3)]
            h0, c0 = self.zeros(bsz, 1, x), self.zeros(bsz, 1, x)
        else:
            Wf = [m[:bsz] for m in mem[0:3]]
            Wr = [m[:bsz] for m in mem[3:6]]
            h0, c0 = mem[6][:bsz], mem[7][:bsz]
        args = []
        for (q, k, v, b, rk, rv, rb), wf, wr in zip(gates, Wf, Wr):
            z = self.ops['delta'](q, k, v, b, wf)
            args += [z, rk, rv, rb, wr]
        out, cell = self.ops['lstm_v4'](*args, h0, c0)
        y = self.finish(x, out)
        if not carry:
            return y, None
        return y, tuple(w.clone().detach() for w in Wf + Wr) + (self.last(out), self.last(cell))


class _RecDeltaAttention(_RecurrentAttention):
    """attn_type 934: the recurrent delta net (softmax, sigmoid and the tanh feedback sit inside the op)."""

    def __init__(self, n_head, d_model, d_head, ops):
        super().__init__(n_head, d_model, d_head, ops)
        self.slow_net = nn.Linear(d_model, n_head * (3 * d_head + 1), bias=False)
        self.R_q = nn.Parameter(torch.empty(1, n_head, d_head, d_head))
        self.R_k = nn.Parameter(torch.empty(1, n_head, d_head, d_head))
        self.R_v = nn.Parameter(torch.empty(1, n_head, d_head, d_head))
        self.r_b = nn.Parameter(torch.empty(1, n_head, 1, d_head))
        for w in (self.R_q, self.R_k, self.R_v, self.r_b):       # reset_rec_parameters, :3203-3208
            nn.init.normal_(w, mean=0., std=1.0 / math.sqrt(d_head))

    def forward(self, h, mem, carry):
        slen, bsz, _ = h.shape
        d = self.d_head
        x = self.layer_norm(h)
        qkvb = self.slow_net(x).view(slen, bsz, self.n_head, 3 * d + 1)
        q, k, v, b = (_bhld(t) for t in torch.split(qkvb, (d,) * 3 + (1,), -1))
        if mem is None:
            W, h0 = self.zeros(bsz, d, x), self.zeros(bsz, 1, x)
        else:
            W, h0 = mem[0][:bsz], mem[2][:bsz]
        out = self.ops['rec_delta'](q, k, v, b, self.R_q, self.R_k, self.R_v, self.r_b, W, h0)
        y = self.finish(x, out)
        return y, ((W.clone().detach(), None, self.last(out)) if carry else None)


_RECURRENT = {134: _DeltaRNNv2Attention, 254: _DeltaLSTMv4Attention, 934: _RecDeltaAttention}


class _FeedForward(nn.Module):
    def __init__(self, d_model, d_inner):
        super().__init__()
        self.CoreNet = nn.Sequential(nn.Linear(d_model, d_inner), nn.ReLU(), nn.Dropout(0.0),
                                     nn.Linear(d_inner, d_model), nn.Dropout(0.0))
        self.layer_norm = nn.LayerNorm(d_model)

    def forward(self, x):
        return x + self.CoreNet(self.layer_norm(x))


class _Layer(nn.Module):
    def __init__(self, n_head, d_model, d_head, d_inner, delta_fn, fused_io, attn_type=24, ops=None):
        super().__init__()
        if attn_type == 24:
            self.dec_attn = _DeltaAttention(n_head, d_model, d_head, delta_fn, fused_io)
        else:
            self.dec_attn = _RECURRENT[attn_type](n_head, d_model, d_head, ops)
        self.pos_ff = _FeedForward(d_model, d_inner)


class DeltaNetLM(nn.Module):
    def __init__(self, n_token, n_layer, n_head, d_model, d_head, d_inner, delta_fn=None, init_std=0.02, fused_io=False,
                 attn_type=24, ops=None):
        """``ops`` (attn_type 134 / 254 / 934): dict with the callables 'delta', 'rnn_v2', 'lstm_v4', 'rec_delta'
        to run instead of the CUDA ops (tests pass CPU checkers); ``delta_fn`` plays that part for attn_type 24."""
        super().__init__()
        if attn_type not in (24,) + tuple(_RECURRENT):
            raise ValueError('attn_type %r is not covered (24, 134, 254, 934)' % (attn_type,))
        if fused_io and (delta_fn is not None or attn_type != 24):
            raise ValueError('the fused prologue / epilogue belongs to the CUDA op of the delta-rule layer')
        if attn_type != 24 and ops is None:
            ops = _default_ops()
        if delta_fn is None and attn_type == 24:
            from recurrent_fwp_b200.fast_weight import fast_weight_delta as delta_fn
        self.d_model = d_model
        self.word_emb = _Named()
        self.word_emb.emb_layers = nn.ModuleList([nn.Embedding(n_token, d_model)])
        self.layers = nn.ModuleList([_Layer(n_head, d_model, d_head, d_inner, delta_fn, fused_io, attn_type, ops)
                                     for _ in range(n_layer)])
        self.crit = _Named()
        self.crit.out_layers = nn.ModuleList([nn.Linear(d_model, n_token)])
        self.crit.out_layers[0].weight = self.word_emb.emb_layers[0].weight         # tied
        self.pos_emb = _Named()
        self.pos_emb.register_buffer('inv_freq', 1.0 / (10000 ** (torch.arange(0.0, d_model, 2.0) / d_model)))
        self.reset_parameters(init_std)

    def reset_parameters(self, std):
        """The reference's ``weights_init`` (language_modeling/src/train.py:378-432) with ``--init normal``."""
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, 0.0, std)
                if getattr(m, 'bias', None) is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.LayerNorm):
                nn.init.normal_(m.weight, 1.0, std)
                nn.init.zeros_(m.bias)

    def hidden(self, data, mems=None, carry_over_fast_weight=False):
        qlen = data.shape[0]
        emb = self.word_emb.emb_layers[0](data) * math.sqrt(self.d_model)
        pos = torch.arange(qlen - 1, -1, -1.0, device=emb.device, dtype=emb.dtype)
        ang = torch.outer(pos, self.pos_emb.inv_freq)
        h = emb + torch.cat([ang.sin(), ang.cos()], dim=-1)[:, None, :]
        new_mems = []
        for i, layer in enumerate(self.layers):
            h, mem = layer.dec_attn(h, None if mems is None else mems[i], carry_over_fast_weight)
            h = layer.pos_ff(h)
            new_mems.append(mem)
        return h, (new_mems if carry_over_fast_weight else None)

    def forward(self, data, target, mems=None, carry_over_fast_weight=False):
        """data, target: (len, batch) token ids.  Returns (loss of shape (len, batch), new_mems or None)."""
        h, new_mems = self.hidden(data, mems, carry_over_fast_weight)
        tgt_len = target.shape[0]
        out = self.crit.out_layers[0]
        logit = F.linear(h[-tgt_len:].reshape(-1, h.shape[-1]), out.weight, out.bias)
        nll = -F.log_softmax(logit, dim=-1).gather(1, target.reshape(-1, 1)).squeeze(1)
        return nll.view(tgt_len, -1), new_mems
