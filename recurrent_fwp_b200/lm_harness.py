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


class _FeedForward(nn.Module):
    def __init__(self, d_model, d_inner):
        super().__init__()
        self.CoreNet = nn.Sequential(nn.Linear(d_model, d_inner), nn.ReLU(), nn.Dropout(0.0),
                                     nn.Linear(d_inner, d_model), nn.Dropout(0.0))
        self.layer_norm = nn.LayerNorm(d_model)

    def forward(self, x):
        return x + self.CoreNet(self.layer_norm(x))


class _Layer(nn.Module):
    def __init__(self, n_head, d_model, d_head, d_inner, delta_fn, fused_io):
        super().__init__()
        self.dec_attn = _DeltaAttention(n_head, d_model, d_head, delta_fn, fused_io)
        self.pos_ff = _FeedForward(d_model, d_inner)


class DeltaNetLM(nn.Module):
    def __init__(self, n_token, n_layer, n_head, d_model, d_head, d_inner, delta_fn=None, init_std=0.02, fused_io=False):
        super().__init__()
        if fused_io and delta_fn is not None:
            raise ValueError('the fused prologue / epilogue belongs to the CUDA op')
        if delta_fn is None:
            from recurrent_fwp_b200.fast_weight import fast_weight_delta as delta_fn
        self.d_model = d_model
        self.word_emb = _Named()
        self.word_emb.emb_layers = nn.ModuleList([nn.Embedding(n_token, d_model)])
        self.layers = nn.ModuleList([_Layer(n_head, d_model, d_head, d_inner, delta_fn, fused_io) for _ in range(n_layer)])
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
