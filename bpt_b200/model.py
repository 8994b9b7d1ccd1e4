"""The callers of the attention path, re-hosted on plain tensors (no graph library).

`BPTBlock` keeps the parameters of the reference's block (modules/attention.py:22-52: proj_q/k/v/o
without bias, embed_ak of MAX_ETYPE rows, post-LN, FFN) under the same names, so a reference
state dict loads; its forward (attention.py:54-81) takes the node features and an
`AttentionPlan` instead of a DGL graph + CSR tuple and replaces the four-operator chain by
the fused call.  `BPTLanguageModel` is the decoder-only use of
BinaryPartitionTransformer.forward (modules/model.py:240-280): token embedding on the leaves,
zeros on span nodes, `n_layers` blocks over all nodes, log-softmax generator on the leaves.
Projections, LayerNorm and the FFN are torch operators, as in the reference.
"""
import math

import torch
import torch.nn as nn

from .attention import bpt_attention


class PositionwiseFeedForward(nn.Module):  # modules/attention.py:8-19
    def __init__(self, dim_model, dim_ff, dropout=0.1, activation="relu"):
        super().__init__()
        self.w_1 = nn.Linear(dim_model, dim_ff)
        self.w_2 = nn.Linear(dim_ff, dim_model)
        self.dropout = nn.Dropout(dropout)
        self.act = torch.relu if activation == "relu" else nn.functional.gelu

    def forward(self, x):
        return self.w_2(self.dropout(self.act(self.w_1(x))))


class BPTBlock(nn.Module):
    MAX_ETYPE = 1000  # modules/attention.py:23

    def __init__(self, dim_model, h, dim_ff, rel_pos=False, drop_h=0.1, drop_a=0.0, activation="relu"):
        super().__init__()
        if drop_a != 0.0:
            raise ValueError("dropout on attention weights is not available in the fused call; "
                             "use bpt_b200.op (the operator chain) for drop_a > 0")
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
        a = bpt_attention(plan, q, k, v, ak, 1.0 / math.sqrt(self.d_k)).view(-1, self.d_k * self.h)
        h = self.norm_in(h + self.drop_h(self.proj_o(a)))
        return self.norm_inter(h + self.ffn(h))


class Generator(nn.Module):  # modules/model.py:8-17
    def __init__(self, dim_model, n_classes):
        super().__init__()
        self.proj = nn.Linear(dim_model, n_classes)

    def forward(self, x):
        return torch.log_softmax(self.proj(x), dim=-1)


class BPTLanguageModel(nn.Module):
    """modules/model.py:197-280 with rel_pos=True (the character-LM configuration)."""

    def __init__(self, vocab_size, dim_model, dim_ff, h, n_layers, dropout=0.0, activation="relu"):
        super().__init__()
        self.embed = nn.Embedding(vocab_size, dim_model)
        self.layers = nn.ModuleList([BPTBlock(dim_model, h, dim_ff, rel_pos=True, drop_h=dropout,
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
