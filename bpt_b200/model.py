"""The callers of the attention path, re-hosted on plain tensors (no graph library).

`BPTBlock` keeps the parameters of the reference's block (modules/attention.py:22-52: proj_q/k/v/o
without bias, embed_ak of MAX_ETYPE rows, post-LN, FFN) under the same names, and the models keep
the reference's `embed.lut` / `generator.proj` / `norm` names, so a reference state dict of the
relative-position configurations with dim_embed == dim_model loads with strict=True; its forward (attention.py:54-81) takes the node features and an
`AttentionPlan` instead of a DGL graph + CSR tuple and replaces the four-operator chain by
the fused call.  `BPTMemBlock` (attention.py:84-172) adds attention to an encoder memory over the
sentence-aligned cross graph; the fused call takes distinct destination and source node sets, so
the reference's zero padding of the smaller side (attention.py:148-149, model.py:90-93) is not
needed.  `BPTEncoderDecoder` is the forward of BinaryPartitionEncoderDecoder
(modules/model.py:22-106) with relative positions.  `BPTLanguageModel` is the decoder-only use of
BinaryPartitionTransformer.forward (modules/model.py:240-280): token embedding on the leaves,
zeros on span nodes, `n_layers` blocks over all nodes, log-softmax generator on the leaves.
Projections, LayerNorm and the FFN are torch operators, as in the reference.
"""
import math

import torch
import torch.nn as nn

from . import _lib
from .attention import bpt_attention


class _AddLayerNorm(torch.autograd.Function):
    """y = LayerNorm(x + r) through bpt_add_layer_norm (one pass over memory).  The backward
    recomputes the sum and goes through torch's layer-norm derivative."""

    @staticmethod
    def forward(ctx, x, r, weight, bias, eps):
        y = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().bpt_add_layer_norm(x.data_ptr(), r.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                                     float(eps), y.data_ptr(), x.numel() // x.size(-1), x.size(-1),
                                                     _lib.dtype_code(x.dtype), _lib.stream()))
        ctx.save_for_backward(x, r, weight, bias)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, gy):
        x, r, weight, bias = ctx.saved_tensors
        with torch.enable_grad():
            s = (x + r).detach().requires_grad_(True)
            w, b = weight.detach().requires_grad_(True), bias.detach().requires_grad_(True)
            out = nn.functional.layer_norm(s, (s.size(-1),), w, b, ctx.eps)
            gs, gw, gb = torch.autograd.grad(out, (s, w, b), gy)
        return gs, gs, gw, gb, None


def add_layer_norm(x, r, norm):
    """norm(x + r) for an nn.LayerNorm over the last dimension; fused on CUDA when the kernel's
    shape rules hold (same dtype everywhere, last dimension a multiple of 8 up to 4096)."""
    dim = x.size(-1)
    if (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16, torch.float16) and dim % 8 == 0 and dim <= 4096
            and norm.weight is not None and norm.bias is not None and norm.weight.dtype == x.dtype
            and r.dtype == x.dtype and r.shape == x.shape and tuple(norm.normalized_shape) == (dim,)):
        return _AddLayerNorm.apply(x.contiguous(), r.contiguous(), norm.weight, norm.bias, norm.eps)
    return norm(x + r)


class PositionwiseFeedForward(nn.Module):  # modules/attention.py:8-19
    def __init__(self, dim_model, dim_ff, dropout=0.1, activation="relu"):
        super().__init__()
        self.w_1 = nn.Linear(dim_model, dim_ff)
        self.w_2 = nn.Linear(dim_ff, dim_model)
        self.dropout = nn.Dropout(dropout)
        if activation not in ("relu", "gelu", "gelu_tanh"):
            raise ValueError("activation must be relu, gelu or gelu_tanh")
        self.activation = activation
        self.act = {"relu": torch.relu, "gelu": nn.functional.gelu,
                    "gelu_tanh": lambda t: nn.functional.gelu(t, approximate="tanh")}[activation]

    def forward(self, x):
        if (x.is_cuda and x.dim() == 2 and self.activation != "gelu" and not torch.is_grad_enabled()
                and not (self.training and self.dropout.p > 0) and x.dtype == self.w_1.weight.dtype):
            # inference: bias and activation ride in the GEMM's epilogue (relu, or gelu in its tanh form)
            hidden = torch._addmm_activation(self.w_1.bias, x, self.w_1.weight.t(),
                                             use_gelu=self.activation == "gelu_tanh")
            return self.w_2(hidden)
        return self.w_2(self.dropout(self.act(self.w_1(x))))


class BPTBlock(nn.Module):
    MAX_ETYPE = 1000  # modules/attention.py:23

    def __init__(self, dim_model, h, dim_ff, rel_pos=False, drop_h=0.1, drop_a=0.0, activation="relu"):
        super().__init__()
        self.drop_a = float(drop_a)  # dropout on the attention weights, inside the fused call (attention.py:73)
        self.dim_model, self.h, self.dim_ff = dim_model, h, dim_ff
        self.d_k = dim_model // h
        self.rel_pos = rel_pos
        self.drop_h = nn.Dropout(drop_h)
        self.norm_in = nn.LayerNorm(dim_model)
        self.norm_inter = nn.LayerNorm(dim_model)
        self.proj_q = nn.Linear(dim_model, self.d_k * h, bias=False)
        self.proj_k = nn.Linear(dim_model, self.d_k * h, bias=False)
        self.proj_v = nn.Linear(dim_model, self.d_k * h, bias=False)
        self.proj_o = nn.Linear(self.d_k * h, dim_model, bias=False)
        if rel_pos:
            self.embed_ak = nn.Embedding(self.MAX_ETYPE, self.d_k)
        self.ffn = nn.Sequential(PositionwiseFeedForward(dim_model, dim_ff, dropout=drop_h, activation=activation),
                                 nn.Dropout(drop_h))

    def reset_parameters(self):  # modules/attention.py:49-52
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.xavier_uniform_(p)

    def forward(self, h, plan):
        """h: (N, dim_model) features of all nodes; returns the block's output (N, dim_model)."""
        q = self.proj_q(h).view(-1, self.h, self.d_k)
        k = self.proj_k(h).view(-1, self.h, self.d_k)
        v = self.proj_v(h).view(-1, self.h, self.d_k)
        ak = self.embed_ak.weight if self.rel_pos else None
        drop_a = self.drop_a if self.training else 0.0
        a = bpt_attention(plan, q, k, v, ak, 1.0 / math.sqrt(self.d_k), dropout_p=drop_a).view(-1, self.d_k * self.h)
        h = add_layer_norm(h, self.drop_h(self.proj_o(a)), self.norm_in)
        return add_layer_norm(h, self.ffn(h), self.norm_inter)


class BPTMemBlock(nn.Module):
    """modules/attention.py:84-172: self-attention over the node's own graph, then attention from
    every node to the memory nodes its cross graph names (no relative-position term there), then
    the FFN.  Parameter names and shapes follow the reference (lists of two for the two
    attentions), so a reference state dict loads."""
    MAX_ETYPE = 1000

    def __init__(self, dim_model, h, dim_ff, rel_pos=False, drop_h=0.1, drop_a=0.0, activation="relu"):
        super().__init__()
        self.drop_a = float(drop_a)  # dropout on the attention weights, inside the fused call (attention.py:73)
        self.dim_model, self.h, self.dim_ff = dim_model, h, dim_ff
        self.d_k = dim_model // h
        self.rel_pos = rel_pos
        self.drop_h = nn.ModuleList([nn.Dropout(drop_h) for _ in range(2)])
        self.norm_in = nn.ModuleList([nn.LayerNorm(dim_model) for _ in range(2)])
        self.norm_inter = nn.LayerNorm(dim_model)
        self.proj_q = nn.ModuleList([nn.Linear(dim_model, self.d_k * h, bias=False) for _ in range(2)])
        self.proj_k = nn.ModuleList([nn.Linear(dim_model, self.d_k * h, bias=False) for _ in range(2)])
        self.proj_v = nn.ModuleList([nn.Linear(dim_model, self.d_k * h, bias=False) for _ in range(2)])
        self.proj_o = nn.ModuleList([nn.Linear(self.d_k * h, dim_model, bias=False) for _ in range(2)])
        if rel_pos:
            self.embed_ak = nn.Embedding(self.MAX_ETYPE, self.d_k)
        self.ffn = nn.Sequential(PositionwiseFeedForward(dim_model, dim_ff, dropout=drop_h, activation=activation),
                                 nn.Dropout(drop_h))

    def reset_parameters(self):  # modules/attention.py:111-114
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.xavier_uniform_(p)

    def forward(self, h, plan, mem, plan_inter):
        """h: (N, dim_model) node features; plan: AttentionPlan of the nodes' own graph; mem:
        (M, dim_model) memory node features; plan_inter: AttentionPlan(src in [0, M), dst in [0, N),
        None, N, n_src=M) of the cross graph.  Nodes without a cross edge get a zero attention
        result, as in the reference."""
        shape = (-1, self.h, self.d_k)
        scale = 1.0 / math.sqrt(self.d_k)
        ak = self.embed_ak.weight if self.rel_pos else None
        drop_a = self.drop_a if self.training else 0.0
        a = bpt_attention(plan, self.proj_q[0](h).view(shape), self.proj_k[0](h).view(shape),
                          self.proj_v[0](h).view(shape), ak, scale, dropout_p=drop_a).view(-1, self.d_k * self.h)
        h = add_layer_norm(h, self.drop_h[0](self.proj_o[0](a)), self.norm_in[0])  # attention.py:131-141
        a = bpt_attention(plan_inter, self.proj_q[1](h).view(shape), self.proj_k[1](mem).view(shape),
                          self.proj_v[1](mem).view(shape), None, scale, dropout_p=drop_a).view(-1, self.d_k * self.h)
        h = add_layer_norm(h, self.drop_h[1](self.proj_o[1](a)), self.norm_in[1])  # attention.py:151-168
        return add_layer_norm(h, self.ffn(h), self.norm_inter)                     # attention.py:170-171


class Generator(nn.Module):  # modules/model.py:8-17
    def __init__(self, dim_model, n_classes):
        super().__init__()
        self.proj = nn.Linear(dim_model, n_classes)

    def forward(self, x):
        return torch.log_softmax(self.proj(x), dim=-1)


class Embedding(nn.Module):
    """modules/embedding.py:13-21: the token table sits in `.lut`, so its state-dict key is `<name>.lut.weight`
    as in the reference's checkpoints."""

    def __init__(self, vocab_size, dim_model):
        super().__init__()
        self.lut = nn.Embedding(vocab_size, dim_model)
        self.dim_model = dim_model

    def forward(self, x):
        return self.lut(x)


class BPTLanguageModel(nn.Module):
    """modules/model.py:197-280 with rel_pos=True and dim_embed == dim_model (the character-LM
    configuration): a state dict of that reference model loads as it is."""

    def __init__(self, vocab_size, dim_model, dim_ff, h, n_layers, dropout=0.0, activation="relu", dropout_a=0.0):
        super().__init__()
        self.embed = Embedding(vocab_size, dim_model)
        self.layers = nn.ModuleList([BPTBlock(dim_model, h, dim_ff, rel_pos=True, drop_h=dropout, drop_a=dropout_a,
                                              activation=activation) for _ in range(n_layers)])
        self.generator = Generator(dim_model, vocab_size)
        self.norm = nn.LayerNorm(dim_model)
        self.emb_dropout = nn.Dropout(dropout)

    def forward(self, tokens, leaf_ids, plan):
        """tokens: (n_leaves,) int64 in leaf order; leaf_ids: their node ids; plan.n_nodes nodes.
        Returns log-probabilities (n_leaves, vocab)."""
        x = self.norm(self.emb_dropout(self.embed(tokens)))                     # model.py:249-262
        h = x.new_zeros((plan.n_nodes, x.size(-1)))                             # span nodes start at zero
        h[leaf_ids] = x
        for layer in self.layers:                                              # model.py:268-269
            h = layer(h, plan)
        return self.generator(h[leaf_ids])                                      # model.py:275


class BPTClassifier(nn.Module):
    """The sequence classifier use of BinaryPartitionTransformer (modules/model.py:197-280 as
    driven by graph/text_classification.py): blocks over all nodes, then one vector per sequence
    into a linear head.  readout="root" reads each sequence's root node as the reference does
    (text_classification.py:48,77); readout="mean" averages the sequence's leaves."""

    def __init__(self, vocab_size, dim_model, dim_ff, h, n_layers, n_classes, dropout=0.0, activation="relu",
                 readout="root", dropout_a=0.0):
        super().__init__()
        if readout not in ("root", "mean"):
            raise ValueError("readout must be root or mean")
        self.readout = readout
        self.embed = Embedding(vocab_size, dim_model)
        self.layers = nn.ModuleList([BPTBlock(dim_model, h, dim_ff, rel_pos=True, drop_h=dropout, drop_a=dropout_a,
                                              activation=activation) for _ in range(n_layers)])
        self.generator = Generator(dim_model, n_classes)
        self.norm = nn.LayerNorm(dim_model)
        self.emb_dropout = nn.Dropout(dropout)

    def forward(self, tokens, leaf_ids, plan, root_ids, lengths=None):
        """tokens: (n_leaves,) in leaf order; root_ids: (B,) node id of every sequence's root;
        lengths: (B,) leaves per sequence (needed for readout="mean"; leaves of a sequence are
        contiguous in `tokens`).  Returns log-probabilities (B, n_classes)."""
        x = self.norm(self.emb_dropout(self.embed(tokens)))
        h = x.new_zeros((plan.n_nodes, x.size(-1)))
        h[leaf_ids] = x
        for layer in self.layers:
            h = layer(h, plan)
        if self.readout == "root":
            pooled = h[root_ids]
        else:
            seq = torch.repeat_interleave(torch.arange(lengths.numel(), device=h.device), lengths)
            pooled = torch.zeros((lengths.numel(), h.size(-1)), dtype=h.dtype, device=h.device)
            pooled.index_add_(0, seq, h[leaf_ids])
            pooled = pooled / lengths.to(h.dtype).unsqueeze(1)
        return self.generator(pooled)


class BPTEncoderDecoder(nn.Module):
    """Forward of BinaryPartitionEncoderDecoder (modules/model.py:22-106) with rel_pos=True:
    `n_layers` blocks over the encoder graph, `m_layers` memory blocks over the decoder graph
    reading the encoder's node features, generator on the read-out nodes."""

    def __init__(self, vocab_sizes, dim_model, dim_ff, h, n_layers, m_layers, dropout=0.0, activation="relu",
                 dropout_a=0.0):
        super().__init__()
        self.embed = nn.ModuleList([Embedding(v, dim_model) for v in vocab_sizes])
        self.enc_layers = nn.ModuleList([BPTBlock(dim_model, h, dim_ff, rel_pos=True, drop_h=dropout, drop_a=dropout_a,
                                                  activation=activation) for _ in range(n_layers)])
        self.dec_layers = nn.ModuleList([BPTMemBlock(dim_model, h, dim_ff, rel_pos=True, drop_h=dropout,
                                                     drop_a=dropout_a, activation=activation) for _ in range(m_layers)])
        self.generator = Generator(dim_model, vocab_sizes[-1])
        self.norm = nn.LayerNorm(dim_model)
        self.emb_dropout = nn.Dropout(dropout)

    def _embed(self, table, tokens, leaf_ids, n_nodes):
        x = self.norm(self.emb_dropout(table(tokens)))                              # model.py:80-83, 96-99
        h = x.new_zeros((n_nodes, x.size(-1)))
        h[leaf_ids] = x
        return h

    def forward(self, enc_tokens, enc_leaf_ids, enc_plan, dec_tokens, dec_leaf_ids, dec_plan, inter_plan,
                readout_ids):
        """Tokens in leaf order, their node ids, the three plans (inter_plan: sources = encoder
        nodes, destinations = decoder nodes) and the decoder nodes to read out.  Returns
        log-probabilities (len(readout_ids), vocab)."""
        h_enc = self._embed(self.embed[0], enc_tokens, enc_leaf_ids, enc_plan.n_nodes)
        for layer in self.enc_layers:                                              # model.py:85-86
            h_enc = layer(h_enc, enc_plan)
        h_dec = self._embed(self.embed[-1], dec_tokens, dec_leaf_ids, dec_plan.n_nodes)
        for layer in self.dec_layers:                                              # model.py:101-102
            h_dec = layer(h_dec, dec_plan, h_enc, inter_plan)
        return self.generator(h_dec[readout_ids])                                  # model.py:104
