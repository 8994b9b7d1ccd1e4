"""Incremental decoding for the encoder-decoder model (no graph library).

The reference decodes by running its message-passing `infer` path on the nodes whose position
equals the current step (modules/attention.py:174-231 driven by modules/beam.py:64-173): in a
causal binary-partition graph every edge goes from a node to a node of equal or later position
(`pos` of graph_builder/builder.pyx:57-62), so the nodes of position t -- leaf t and the span
nodes that end at t -- depend only on nodes of positions <= t.  Here the same schedule runs on
the fused attention call: per step and layer the new nodes' keys and values are written into
per-layer caches over all decoder nodes, and a small attention plan (destinations = the step's
nodes, sources = all decoder nodes, or all encoder nodes for the cross-attention) reads them.
Plans are built once per batch shape (`DecodeSchedule`) and reused by every decode call.

`teacher_forced` feeds given target tokens and must reproduce the full forward of
`BPTEncoderDecoder`; `greedy` feeds back the arg-max token; `beam_search` keeps `beam_size`
hypotheses per sequence as the reference's BinaryPartitionBeamSearch does (beam.py:64-173: scores
are sums of log-probabilities, the top `beam_size` of beam x vocabulary continuations survive a
step, only the first beam is alive at step 0, a surviving hypothesis inherits the K/V rows of the
hypothesis it extends).  Target lengths are given by the decoder graphs; the reference's
end-of-sentence bookkeeping, which moves the cross-attention to the next source sentence, is not
re-hosted: the cross graph is fixed by the schedule.
"""
import math

import torch

from .attention import AttentionPlan, bpt_attention
from .model import add_layer_norm


class DecodeSchedule:
    """Which decoder nodes are computed at which step, and the plans of their attentions.

    dec: csr.BatchedGraph of causal (triu=True) decoder graphs; inter_src / inter_dst: the cross
    graph's edges (encoder node -> decoder node, csr.inter_graph); n_enc: encoder node count."""

    def __init__(self, dec, inter_src, inter_dst, n_enc, n_etypes=1000):
        dev = dec.src.device
        self.n_dec, self.n_enc = dec.n_nodes, n_enc
        # step of every decoder node: its position inside its own sequence
        step_of = dec.pos.long()
        seq_of = torch.zeros(dec.n_nodes, dtype=torch.long, device=dev)
        for b, (n0, n1) in enumerate(zip(dec.node_offsets[:-1], dec.node_offsets[1:])):
            seq_of[n0:n1] = b
        lengths = torch.tensor(dec.lengths, device=dev)
        self.lengths = list(dec.lengths)
        self.n_steps = max(self.lengths) if self.lengths else 0
        leaf_of = torch.full((dec.n_nodes,), -1, dtype=torch.long, device=dev)  # leaf index inside the sequence
        for n0, n in zip(dec.node_offsets[:-1], dec.lengths):
            leaf_of[n0:n0 + n] = torch.arange(n, device=dev)
        if bool((step_of[dec.src.long()] > step_of[dec.dst.long()]).any()):
            raise ValueError("DecodeSchedule needs causal graphs (an edge runs to an earlier position)")
        order = torch.argsort(step_of, stable=True)
        counts = torch.bincount(step_of, minlength=self.n_steps).tolist()
        e_step = step_of[dec.dst.long()]
        e_order = torch.argsort(e_step, stable=True)
        e_counts = torch.bincount(e_step, minlength=self.n_steps).tolist()
        x_step = step_of[inter_dst.long()]
        x_order = torch.argsort(x_step, stable=True)
        x_counts = torch.bincount(x_step, minlength=self.n_steps).tolist()
        local = torch.empty(dec.n_nodes, dtype=torch.long, device=dev)           # index of a node inside its step
        self.rows, self.leaf_rows, self.leaf_seq, self.self_plans, self.cross_plans = [], [], [], [], []
        n0 = e0 = x0 = 0
        for t in range(self.n_steps):
            rows = order[n0:n0 + counts[t]]
            n0 += counts[t]
            local[rows] = torch.arange(rows.numel(), device=dev)
            self.rows.append(rows)
            is_leaf = leaf_of[rows] >= 0
            self.leaf_rows.append(torch.nonzero(is_leaf).squeeze(1))             # which of the step's rows are leaves
            self.leaf_seq.append(seq_of[rows][is_leaf])                          # and whose sequence they belong to
            e = e_order[e0:e0 + e_counts[t]]
            e0 += e_counts[t]
            self.self_plans.append(AttentionPlan(dec.src[e].contiguous(), local[dec.dst[e].long()].to(torch.int32),
                                                 dec.etype[e].contiguous(), int(rows.numel()), n_etypes=n_etypes,
                                                 n_src=dec.n_nodes))
            x = x_order[x0:x0 + x_counts[t]]
            x0 += x_counts[t]
            self.cross_plans.append(AttentionPlan(inter_src[x].contiguous(), local[inter_dst[x].long()].to(torch.int32),
                                                  None, int(rows.numel()), n_src=n_enc))
        self.n_seq = len(self.lengths)
        self.lengths_t = lengths
        self.seq_of = seq_of                                                     # sequence of every decoder node
        self.node_offsets = torch.tensor(list(dec.node_offsets), dtype=torch.long, device=dev)


def _encode(model, enc_tokens, enc_leaf_ids, enc_plan):
    h = model._embed(model.embed[0], enc_tokens, enc_leaf_ids, enc_plan.n_nodes)
    for layer in model.enc_layers:
        h = layer(h, enc_plan)
    return h


def _decoder_step(model, schedule, t, feed, k_cache, v_cache, k_mem, v_mem):
    """Computes the decoder nodes of step t for the fed tokens (one per sequence of the schedule), writes
    their K/V rows into the caches and returns (sequence ids of the step's leaves, their log-probabilities)."""
    layers = model.dec_layers
    h_, d_k = layers[0].h, layers[0].d_k
    shape = (-1, h_, d_k)
    scale = 1.0 / math.sqrt(d_k)
    rows, leaf_rows, leaf_seq = schedule.rows[t], schedule.leaf_rows[t], schedule.leaf_seq[t]
    x = model.norm(model.emb_dropout(model.embed[-1](feed[leaf_seq])))           # modules/model.py:96-99
    h = x.new_zeros((rows.numel(), x.size(-1)))
    h[leaf_rows] = x
    for li, layer in enumerate(layers):                                         # modules/attention.py:116-172
        q = layer.proj_q[0](h).view(shape)
        k_cache[li][rows] = layer.proj_k[0](h).view(shape)
        v_cache[li][rows] = layer.proj_v[0](h).view(shape)
        ak = layer.embed_ak.weight if layer.rel_pos else None
        a = bpt_attention(schedule.self_plans[t], q, k_cache[li], v_cache[li], ak, scale)
        h = add_layer_norm(h, layer.proj_o[0](a.reshape(-1, h_ * d_k)), layer.norm_in[0])
        a = bpt_attention(schedule.cross_plans[t], layer.proj_q[1](h).view(shape), k_mem[li], v_mem[li], None, scale)
        h = add_layer_norm(h, layer.proj_o[1](a.reshape(-1, h_ * d_k)), layer.norm_in[1])
        h = add_layer_norm(h, layer.ffn(h), layer.norm_inter)
    return leaf_seq, model.generator(h[leaf_rows])


@torch.no_grad()
def decode(model, schedule, enc_tokens, enc_leaf_ids, enc_plan, first_tokens, forced=None):
    """Runs the decoder step by step.  first_tokens: (n_seq,) the token fed at step 0 of every
    sequence.  forced: None for greedy decoding (the arg-max token of step t is fed at step t+1),
    or a list over steps of (n_seq,) tensors with the token to feed at that step (entry 0 is
    ignored in favour of first_tokens; entries of finished sequences are ignored).
    Returns (tokens, logp): per step the arg-max token of every sequence (-1 once a sequence is
    past its length) as (n_steps, n_seq), and the log-probabilities of the step's leaves as a list
    of (n_active, vocab) tensors with their sequence ids."""
    dev = enc_tokens.device
    mem = _encode(model, enc_tokens, enc_leaf_ids, enc_plan)
    layers = model.dec_layers
    h_, d_k = layers[0].h, layers[0].d_k
    shape = (-1, h_, d_k)
    dtype = mem.dtype
    k_cache = [torch.zeros((schedule.n_dec, h_, d_k), dtype=dtype, device=dev) for _ in layers]
    v_cache = [torch.zeros((schedule.n_dec, h_, d_k), dtype=dtype, device=dev) for _ in layers]
    k_mem = [layer.proj_k[1](mem).view(shape).contiguous() for layer in layers]
    v_mem = [layer.proj_v[1](mem).view(shape).contiguous() for layer in layers]
    out_tokens = torch.full((schedule.n_steps, schedule.n_seq), -1, dtype=torch.long, device=dev)
    out_logp = []
    feed = first_tokens.clone()
    for t in range(schedule.n_steps):
        if forced is not None and t > 0:
            feed = forced[t]
        leaf_seq, logp = _decoder_step(model, schedule, t, feed, k_cache, v_cache, k_mem, v_mem)
        best = logp.argmax(-1)
        out_tokens[t, leaf_seq] = best
        out_logp.append((leaf_seq, logp))
        if forced is None:
            feed = feed.clone()
            feed[leaf_seq] = best
    return out_tokens, out_logp


@torch.no_grad()
def beam_search(model, schedule, beam_size, enc_tokens, enc_leaf_ids, enc_plan, first_tokens):
    """Beam search over the fused attention with K/V caches (modules/beam.py:64-173).

    schedule: a DecodeSchedule whose decoder batch holds every target sequence `beam_size` times in a row
    (hypothesis j of sequence b is sequence b * beam_size + j of the batch; the cross graph is replicated the
    same way), so that each hypothesis has its own cache rows.  first_tokens: (n_sequences,) fed at step 0.
    Returns (tokens, scores): tokens (n_steps, n_sequences, beam_size) with -1 past a sequence's length,
    hypotheses ordered best first; scores (n_sequences, beam_size) their summed log-probabilities."""
    dev = enc_tokens.device
    beam = int(beam_size)
    if schedule.n_seq % beam:
        raise ValueError("beam_search: the schedule's batch must hold every sequence beam_size times")
    n_orig = schedule.n_seq // beam
    lengths = schedule.lengths_t.view(n_orig, beam)
    if not bool((lengths == lengths[:, :1]).all()):
        raise ValueError("beam_search: the copies of a sequence must have one length")
    mem = _encode(model, enc_tokens, enc_leaf_ids, enc_plan)
    layers = model.dec_layers
    h_, d_k = layers[0].h, layers[0].d_k
    shape = (-1, h_, d_k)
    k_cache = [torch.zeros((schedule.n_dec, h_, d_k), dtype=mem.dtype, device=dev) for _ in layers]
    v_cache = [torch.zeros((schedule.n_dec, h_, d_k), dtype=mem.dtype, device=dev) for _ in layers]
    k_mem = [layer.proj_k[1](mem).view(shape).contiguous() for layer in layers]
    v_mem = [layer.proj_v[1](mem).view(shape).contiguous() for layer in layers]
    scores = torch.zeros((n_orig, beam), dtype=torch.float32, device=dev)
    scores[:, 1:] = -float("inf")                                  # only the first beam is alive at step 0 (beam.py:133-134)
    hist = torch.full((schedule.n_steps, n_orig, beam), -1, dtype=torch.long, device=dev)
    feed = first_tokens.repeat_interleave(beam).clone()
    off, node_hyp = schedule.node_offsets, schedule.seq_of
    all_nodes = torch.arange(schedule.n_dec, device=dev)
    own = torch.arange(beam, device=dev).unsqueeze(0)
    for t in range(schedule.n_steps):
        leaf_seq, logp = _decoder_step(model, schedule, t, feed, k_cache, v_cache, k_mem, v_mem)
        vocab = logp.size(-1)
        full = torch.full((schedule.n_seq, vocab), -float("inf"), dtype=torch.float32, device=dev)
        full[leaf_seq] = logp.float()
        active = torch.zeros(schedule.n_seq, dtype=torch.bool, device=dev)
        active[leaf_seq] = True
        act = active.view(n_orig, beam)[:, 0]                      # a sequence's copies are active together
        cand = (scores.unsqueeze(-1) + full.view(n_orig, beam, vocab)).view(n_orig, beam * vocab)
        top, idx = cand.topk(beam, -1)                             # beam.py:136-137
        bp, tok = idx // vocab, idx % vocab                        # which hypothesis is extended, with which token
        bp = torch.where(act.unsqueeze(1), bp, own.expand(n_orig, beam))
        scores = torch.where(act.unsqueeze(1), top, scores)
        # hypothesis (b, j) continues hypothesis (b, bp[b, j]): it inherits that one's history and cache rows
        hist[:t] = hist[:t].gather(2, bp.unsqueeze(0).expand(t, n_orig, beam))
        hist[t] = torch.where(act.unsqueeze(1), tok, torch.full_like(tok, -1))
        src_hyp = (torch.arange(n_orig, device=dev).unsqueeze(1) * beam + bp).view(-1)
        shift = off[src_hyp] - off[:-1]
        gather = all_nodes + shift[node_hyp]
        for li in range(len(layers)):
            k_cache[li] = k_cache[li].index_select(0, gather)
            v_cache[li] = v_cache[li].index_select(0, gather)
        feed = torch.where(act.unsqueeze(1), tok, feed.view(n_orig, beam)).view(-1)
    return hist, scores


def greedy(model, schedule, enc_tokens, enc_leaf_ids, enc_plan, first_tokens):
    """Greedy decoding: tokens (n_steps, n_seq), -1 past a sequence's length."""
    return decode(model, schedule, enc_tokens, enc_leaf_ids, enc_plan, first_tokens)[0]


def teacher_forced(model, schedule, enc_tokens, enc_leaf_ids, enc_plan, dec_tokens_per_seq):
    """Feeds the given target tokens (list of (length_b,) tensors, one per sequence) and returns the
    log-probabilities of every target position in leaf order of the batch -- what the full forward
    of BPTEncoderDecoder computes for the same tokens."""
    dev = enc_tokens.device
    n_seq = schedule.n_seq
    forced = []
    for t in range(schedule.n_steps):
        col = torch.zeros(n_seq, dtype=torch.long, device=dev)
        for b, toks in enumerate(dec_tokens_per_seq):
            if t < toks.numel():
                col[b] = toks[t]
        forced.append(col)
    _, out = decode(model, schedule, enc_tokens, enc_leaf_ids, enc_plan, forced[0], forced=forced)
    offsets = [0]
    for n in schedule.lengths:
        offsets.append(offsets[-1] + n)
    vocab = out[0][1].size(-1)
    logp = torch.empty((offsets[-1], vocab), dtype=out[0][1].dtype, device=dev)
    off_t = torch.tensor(offsets[:-1], device=dev)
    for t, (leaf_seq, lp) in enumerate(out):
        logp[off_t[leaf_seq] + t] = lp
    return logp
