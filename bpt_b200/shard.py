"""Sharding of the attention path over GPUs (one process per GPU, torch.distributed).

Two cases, as the graph decides:
* Batches of independent graphs shard by graph: every rank builds and processes its own
  block-diagonal batch; nothing is exchanged on the data path (the reference's data
  parallelism, lm.py:39, shards its dataset the same way).
* One long sequence shards by destination node: every rank owns an equal slice of every
  level of the binary-partition tree, computes Q/K/V for the nodes it owns, and attends from
  its destinations to sources on any rank.  K and V are exchanged once per layer with an
  all-gather into local HBM (NCCL over NVLink); the backward returns the gradients of the
  gathered K/V to their owners with a reduce-scatter.  The reference has no counterpart: it
  keeps a sequence on one GPU.

Two exchanges are provided.  `sharded_attention` gathers every rank's K/V rows (simple, but a
shard reads only a few hundred remote rows: per level the k neighbours beyond each end of its
range).  `halo_attention` sends exactly those rows: each rank keeps [its own rows | the remote
rows its edges name] and one variable-size all-to-all per tensor replaces the all-gather;
gradients of the remote rows travel back the same way and are added to their owners' rows in
rank order.

Index spaces: "global" ids are the builder's node ids; rank r's "local" ids are positions in
its sorted list of owned nodes; the "gathered" space is what all_gather_into_tensor yields:
rank-major, every rank padded to the largest owner count, so that gathered id =
owner * max_owned + local id and the reduce-scatter of a gathered-space tensor hands every
rank exactly its own rows.
"""
import torch


def owned_nodes(n_nodes_arr, shift, rank, world):
    """Global ids owned by `rank`: at each level of n_j nodes the index range
    [floor(rank * n_j / world), floor((rank + 1) * n_j / world)).  Every node has one owner;
    levels with fewer nodes than ranks leave some ranks without a node of that level."""
    parts = []
    for n_j, s_j in zip(n_nodes_arr, shift):
        lo, hi = (rank * int(n_j)) // world, ((rank + 1) * int(n_j)) // world
        if hi > lo:
            parts.append(torch.arange(int(s_j) + lo, int(s_j) + hi, dtype=torch.int64))
    return torch.cat(parts) if parts else torch.zeros(0, dtype=torch.int64)


class SequenceShard:
    """One rank's share of a single sequence's graph.

    src, dst, etype: the whole graph's COO (any integer dtype, any device); n_nodes_arr,
    shift: its level table (graphbuilder.levels).  Attributes:
      owned          global ids owned by this rank (sorted)
      max_owned      rows every rank contributes to the gathered K/V
      n_gathered     world * max_owned
      src_g, dst_l   this rank's edges: source in gathered space, destination in local ids
      etype_l, eid   their types and their global edge ids (ascending)
    """

    def __init__(self, src, dst, etype, n_nodes_arr, shift, rank, world):
        dev = src.device
        self.rank, self.world = rank, world
        n_nodes = int(shift[-1]) + int(n_nodes_arr[-1])
        owners = [owned_nodes(n_nodes_arr, shift, r, world) for r in range(world)]
        self.owned = owners[rank].to(dev)
        self.max_owned = max(int(o.numel()) for o in owners)
        self.n_gathered = world * self.max_owned
        to_gathered = torch.empty(n_nodes, dtype=torch.int64)
        to_local = torch.full((n_nodes,), -1, dtype=torch.int64)
        for r, o in enumerate(owners):
            to_gathered[o] = r * self.max_owned + torch.arange(o.numel())
        to_local[owners[rank]] = torch.arange(owners[rank].numel())
        self.to_gathered = to_gathered.to(dev)
        local_dst = to_local.to(dev)[dst.long()]
        keep = local_dst >= 0
        self.eid = torch.nonzero(keep).squeeze(1)
        self.dst_l = local_dst[keep].to(torch.int32)
        self.src_g = self.to_gathered[src.long()[keep]].to(torch.int32)
        self.etype_l = None if etype is None else etype[keep].to(torch.int32)
        self.n_owned = int(self.owned.numel())
        self._etype = etype
        self._n_leaves = int(n_nodes_arr[0])

    # ---- halo exchange: only the remote rows this rank's edges name ----
    def build_halo(self, src, dst, split_straddlers=False):
        """Send/receive lists of the halo exchange, computed locally by every rank from the whole
        edge list (no communication).  With split_straddlers, span nodes whose source leaves lie
        on several ranks (the top log2(world) levels of the tree) are not computed by their owner
        alone: every rank attends from them to its own sources only and the partial results are
        merged (halo_attention does that); their rows are appended after this rank's other
        destinations.  Sets
          n_halo       remote rows this rank receives
          src_h        this rank's edges' sources in the local extended space [own | halo]
          recv_counts  rows received from each rank, in rank order (the halo rows' order)
          send_idx     per peer, the local indices of the own rows it needs (ascending global id)"""
        dev = src.device
        world, rank = self.world, self.rank
        n_nodes = self.to_gathered.numel()
        owner = (self.to_gathered // self.max_owned)                     # owner rank of every node
        local = (self.to_gathered % self.max_owned)                      # its index in the owner's list
        src64, dst64 = src.long(), dst.long()
        dst_owner = owner[dst64]
        needs = []                                                       # needs[r]: global ids r reads but does not own
        for r in range(world):
            s_r = torch.unique(src64[dst_owner == r])
            needs.append(s_r[owner[s_r] != r])
        self.split = bool(split_straddlers)
        if self.split:
            n_leaves = int(self._n_leaves)
            span = dst64 >= n_leaves
            lo = torch.full((n_nodes,), world, dtype=torch.int64, device=dev).scatter_reduce(
                0, dst64[span], owner[src64[span]], "amin")
            hi = torch.full((n_nodes,), -1, dtype=torch.int64, device=dev).scatter_reduce(
                0, dst64[span], owner[src64[span]], "amax")
            is_strad = hi > lo                                           # sources on more than one rank
            strad = torch.nonzero(is_strad).squeeze(1)                   # ascending global ids
            self.strad_ids = strad
            self.n_strad = int(strad.numel())
            # edges this rank computes: into its own non-straddling rows, and from its own sources
            # into any straddler
            edge_strad = is_strad[dst64]
            keep = (~edge_strad & (dst_owner == rank)) | (edge_strad & (owner[src64] == rank))
            self.eid = torch.nonzero(keep).squeeze(1)
            own_ns = ~is_strad[self.owned]
            self.ns_idx = torch.nonzero(own_ns).squeeze(1)               # positions of non-straddlers in `owned`
            self.s_own_idx = torch.nonzero(~own_ns).squeeze(1)           # positions of my straddlers in `owned`
            self.s_own_pos = torch.searchsorted(strad, self.owned[self.s_own_idx])
            self.n_ns = int(self.ns_idx.numel())
            # straddlers are top-level nodes: in the sorted `owned` list they normally come last
            self.ns_prefix = bool(self.n_ns == 0 or int(self.ns_idx[-1]) == self.n_ns - 1)
            loc = torch.full((n_nodes,), -1, dtype=torch.int64, device=dev)
            loc[self.owned[self.ns_idx]] = torch.arange(self.n_ns, device=dev)
            loc[strad] = self.n_ns + torch.arange(self.n_strad, device=dev)
            self.dst_l = loc[dst64[self.eid]].to(torch.int32)
            self.n_dst_local = self.n_ns + self.n_strad
            self.etype_l = None if self._etype is None else self._etype[self.eid].to(torch.int32)
            # remote rows are needed only by edges into non-straddling rows
            needs = []
            for r in range(world):
                s_r = torch.unique(src64[~edge_strad & (dst_owner == r)])
                needs.append(s_r[owner[s_r] != r])
        mine = needs[rank]
        order = torch.argsort(owner[mine] * n_nodes + mine)              # by owner rank, then id
        mine = mine[order]
        self.recv_counts = [int((owner[mine] == r).sum()) for r in range(world)]
        self.n_halo = int(mine.numel())
        ext = torch.full((n_nodes,), -1, dtype=torch.int64, device=dev)
        ext[self.owned] = torch.arange(self.n_owned, device=dev)
        ext[mine] = self.n_owned + torch.arange(self.n_halo, device=dev)
        self.src_h = ext[src64[self.eid]].to(torch.int32)
        self.send_idx = []
        for r in range(world):
            want = needs[r][owner[needs[r]] == rank]                     # ascending ids (torch.unique sorts)
            self.send_idx.append(local[want])
        self.send_counts = [int(t.numel()) for t in self.send_idx]
        self.send_all = torch.cat(self.send_idx) if self.send_idx else torch.zeros(0, dtype=torch.int64, device=dev)
        self.n_ext = self.n_owned + self.n_halo
        # Table for the way back (halo_return): row i of ret_mat lists the positions in send_all that
        # name own row ret_rows[i], in peer order, padded with n_send (an all-zero row appended to what
        # was received).  The returned gradients are then summed with a handful of launches instead of
        # three per peer, still in a fixed order.
        n_send = int(self.send_all.numel())
        order = torch.argsort(self.send_all, stable=True)
        self.ret_rows, counts = torch.unique_consecutive(self.send_all[order], return_counts=True)
        n_t = int(self.ret_rows.numel())
        width = int(counts.max()) if n_t else 0
        self.ret_mat = torch.full((n_t, width), n_send, dtype=torch.int64, device=dev)
        if n_t:
            starts = torch.cumsum(counts, 0) - counts
            group = torch.repeat_interleave(torch.arange(n_t, device=dev), counts)
            self.ret_mat[group, torch.arange(n_send, device=dev) - starts[group]] = order
        return self

    def pad_rows(self, x):
        """(n_owned, ...) -> (max_owned, ...) zero-padded: this rank's all-gather contribution."""
        if x.size(0) == self.max_owned:
            return x.contiguous()
        out = x.new_zeros((self.max_owned,) + tuple(x.shape[1:]))
        out[: x.size(0)] = x
        return out


def all_gather_rows(shard, x, group=None):
    """all_gather_into_tensor of every rank's padded rows: (n_gathered, ...)."""
    import torch.distributed as dist
    mine = shard.pad_rows(x)
    out = mine.new_empty((shard.n_gathered,) + tuple(mine.shape[1:]))
    dist.all_gather_into_tensor(out, mine, group=group)
    return out


def reduce_scatter_rows(shard, x_g, group=None):
    """Sums a gathered-space tensor over ranks and returns this rank's (n_owned, ...) rows."""
    import torch.distributed as dist
    out = x_g.new_empty((shard.max_owned,) + tuple(x_g.shape[1:]))
    dist.reduce_scatter_tensor(out, x_g.contiguous(), op=dist.ReduceOp.SUM, group=group)
    return out[: shard.n_owned]


class _GatherKV(torch.autograd.Function):
    """K or V rows of all ranks, differentiable: gradient = reduce-scatter to the owners."""

    @staticmethod
    def forward(ctx, shard, x):
        ctx.shard = shard
        return all_gather_rows(shard, x)

    @staticmethod
    def backward(ctx, g):
        return None, reduce_scatter_rows(ctx.shard, g)


def sharded_attention(shard, plan, q, k, v, embed_ak=None, scale=None):
    """Attention for this rank's destinations.  q, k, v: (n_owned, h, d) of the nodes this
    rank owns; plan: AttentionPlan(shard.src_g, shard.dst_l, shard.etype_l, shard.n_owned,
    n_src=shard.n_gathered).  Differentiable; returns (n_owned, h, d)."""
    from .attention import bpt_attention
    k_g = _GatherKV.apply(shard, k)
    v_g = _GatherKV.apply(shard, v)
    return bpt_attention(plan, q, k_g, v_g, embed_ak, scale)


def halo_exchange(shard, x, group=None):
    """(n_owned, ...) -> (n_owned + n_halo, ...): this rank's rows followed by the remote rows its
    edges name, fetched with one variable-size all-to-all."""
    import torch.distributed as dist
    if shard.world == 1:
        return x
    send = x.index_select(0, shard.send_all)
    recv = x.new_empty((shard.n_halo,) + tuple(x.shape[1:]))
    dist.all_to_all_single(recv, send, output_split_sizes=shard.recv_counts, input_split_sizes=shard.send_counts,
                           group=group)
    return torch.cat([x, recv], 0)


def _wide(x):
    """16-bit floats are summed in fp32."""
    return x.float() if x.dtype in (torch.bfloat16, torch.float16) else x


def halo_return(shard, g_ext, group=None):
    """Gradient of halo_exchange: sends the halo rows' gradients back to their owners and adds
    them to the owners' rows; a row named by several peers gets their contributions summed in
    fp32 in peer order (shard.ret_mat), so every sum has a fixed order."""
    import torch.distributed as dist
    if shard.world == 1:
        return g_ext
    g_own = g_ext[: shard.n_owned].clone()
    send = g_ext[shard.n_owned:].contiguous()
    n_send = int(shard.send_all.numel())
    recv = g_ext.new_zeros((n_send + 1,) + tuple(g_ext.shape[1:]))     # last row stays zero: the table's padding
    dist.all_to_all_single(recv[:n_send], send, output_split_sizes=shard.send_counts,
                           input_split_sizes=shard.recv_counts, group=group)
    if shard.ret_rows.numel():
        g_own[shard.ret_rows] += _wide(recv[shard.ret_mat]).sum(1).to(g_own.dtype)
    return g_own


def halo_exchange_pair(shard, a, b, group=None):
    """halo_exchange of two tensors of one shape with ONE all-to-all (K and V travel together)."""
    import torch.distributed as dist
    if shard.world == 1:
        return a, b
    send = torch.stack([a.index_select(0, shard.send_all), b.index_select(0, shard.send_all)], 1)
    recv = a.new_empty((shard.n_halo, 2) + tuple(a.shape[1:]))
    dist.all_to_all_single(recv, send, output_split_sizes=shard.recv_counts, input_split_sizes=shard.send_counts,
                           group=group)
    return torch.cat([a, recv[:, 0]], 0), torch.cat([b, recv[:, 1]], 0)


def halo_return_pair(shard, ga_ext, gb_ext, group=None):
    """halo_return of two gradients with ONE all-to-all; same fixed summation order."""
    import torch.distributed as dist
    if shard.world == 1:
        return ga_ext, gb_ext
    ga_own, gb_own = ga_ext[: shard.n_owned].clone(), gb_ext[: shard.n_owned].clone()
    send = torch.stack([ga_ext[shard.n_owned:], gb_ext[shard.n_owned:]], 1)
    n_send = int(shard.send_all.numel())
    recv = ga_ext.new_zeros((n_send + 1, 2) + tuple(ga_ext.shape[1:]))  # last row stays zero: the table's padding
    dist.all_to_all_single(recv[:n_send], send, output_split_sizes=shard.send_counts,
                           input_split_sizes=shard.recv_counts, group=group)
    if shard.ret_rows.numel():
        total = _wide(recv[shard.ret_mat]).sum(1).to(ga_own.dtype)      # (targets, 2, ...)
        ga_own[shard.ret_rows] += total[:, 0]
        gb_own[shard.ret_rows] += total[:, 1]
    return ga_own, gb_own


class _HaloKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, shard, x):
        ctx.shard = shard
        return halo_exchange(shard, x)

    @staticmethod
    def backward(ctx, g):
        return None, halo_return(ctx.shard, g)


# (forward, backward) callables used by _StraddleAttention instead of the GPU kernels; tests on
# CPU ranks install stand-ins with the signatures of attention_forward / attention_backward.
_KERNELS = None


def _all_ranks_rows(shard, x_own, group=None):
    """Rows of the straddling nodes, (n_strad, ...), on every rank: each owner fills its rows of
    a zero buffer and the buffers are summed (a sum with zeros is exact)."""
    import torch.distributed as dist
    buf = x_own.new_zeros((shard.n_strad,) + tuple(x_own.shape[1:]))
    buf[shard.s_own_pos] = x_own[shard.s_own_idx]
    if shard.world > 1 and shard.n_strad:
        dist.all_reduce(buf, group=group)
    return buf


def _local_rows(shard, x_own):
    """(n_owned, ...) -> this rank's destination rows [own non-straddlers | all straddlers]."""
    if shard.n_strad == 0:
        return x_own
    head = x_own[: shard.n_ns] if shard.ns_prefix else x_own[shard.ns_idx]
    return torch.cat([head, _all_ranks_rows(shard, x_own)], 0)


def _own_rows(shard, x_loc, x_strad):
    """Inverse of _local_rows for results: own non-straddlers from x_loc, own straddlers from x_strad."""
    if shard.n_strad == 0:
        return x_loc
    out = x_loc.new_empty((shard.n_owned,) + tuple(x_loc.shape[1:]))
    if shard.ns_prefix:
        out[: shard.n_ns] = x_loc[: shard.n_ns]
    else:
        out[shard.ns_idx] = x_loc[: shard.n_ns]
    out[shard.s_own_idx] = x_strad[shard.s_own_pos].to(out.dtype)
    return out


class _StraddleAttention(torch.autograd.Function):
    """Attention with the halo exchange and split straddlers, forward and backward spelled out
    because partial rows are merged between the kernels.  bf16 / head dim 64 only: the
    tensor-core backward takes the row term delta from the merged O, which a rank that sees only
    part of a row's edges cannot recompute."""

    @staticmethod
    def forward(ctx, shard, plan, q, k, v, embed_ak, scale):
        import torch.distributed as dist
        if _KERNELS is not None:
            attention_forward = _KERNELS[0]
        else:
            from .attention import attention_forward, tensor_core_eligible
            if not tensor_core_eligible(q, embed_ak, plan):
                raise RuntimeError("halo_attention with split straddlers needs bf16 tensors with head dim 64 "
                                   "and a tile plan that fits in shared memory")
        k_e, v_e = halo_exchange_pair(shard, k.contiguous(), v.contiguous())
        q_loc = _local_rows(shard, q)
        o_loc, lse_loc = attention_forward(plan, q_loc, k_e, v_e, embed_ak, scale)
        if shard.n_strad:
            # merge every rank's partial rows: lse = logsumexp_r lse_r, o = sum_r exp(lse_r - lse) o_r
            n, w = shard.n_strad, shard.world
            part = torch.cat([o_loc[-n:].float().flatten(1), lse_loc[-n:]], 1).contiguous()
            allp = part.new_empty((w * n, part.shape[1]))
            dist.all_gather_into_tensor(allp, part)
            allp = allp.view(w, n, part.shape[1])
            h, d = q.shape[1], q.shape[2]
            o_r, lse_r = allp[:, :, : h * d].view(w, n, h, d), allp[:, :, h * d:]
            lse = torch.logsumexp(lse_r, 0)
            wgt = torch.exp(lse_r - lse.unsqueeze(0)).nan_to_num(0.0)
            o_s = (wgt.unsqueeze(-1) * o_r).sum(0)
            o_loc = torch.cat([o_loc[:-n], o_s.to(o_loc.dtype)], 0)
            lse_loc = torch.cat([lse_loc[:-n], lse], 0)
        o = _own_rows(shard, o_loc, o_loc[shard.n_ns:])
        ctx.shard, ctx.plan, ctx.scale, ctx.has_ak = shard, plan, scale, embed_ak is not None
        ctx.save_for_backward(q_loc, k_e, v_e, embed_ak if ctx.has_ak else q.new_empty(0), o_loc, lse_loc)
        return o

    @staticmethod
    def backward(ctx, d_o):
        import torch.distributed as dist
        if _KERNELS is not None:
            attention_backward = _KERNELS[1]
        else:
            from .attention import attention_backward
        shard = ctx.shard
        q_loc, k_e, v_e, ak, o_loc, lse_loc = ctx.saved_tensors
        ak = ak if ctx.has_ak else None
        d_o = d_o.contiguous()
        do_loc = _local_rows(shard, d_o)
        dq_loc, dk_e, dv_e, dak = attention_backward(ctx.plan, q_loc, k_e, v_e, ak, ctx.scale, lse_loc, do_loc,
                                                     o=o_loc)
        dq_s = dq_loc[shard.n_ns:].float()
        if shard.n_strad and shard.world > 1:
            dist.all_reduce(dq_s)                       # every rank's share of the straddlers' dQ
        dq = _own_rows(shard, dq_loc, dq_s)
        dk, dv = halo_return_pair(shard, dk_e, dv_e)
        return None, None, dq, dk, dv, (dak.to(ak.dtype) if dak is not None else None), None


def halo_attention(shard, plan, q, k, v, embed_ak=None, scale=None):
    """Attention for this rank's destinations with the halo exchange.  After
    shard.build_halo(src, dst[, split_straddlers=True]) the plan is
    AttentionPlan(shard.src_h, shard.dst_l, shard.etype_l, n_dst, n_src=shard.n_ext) with n_dst =
    shard.n_dst_local when straddlers are split, else shard.n_owned.  q, k, v: (n_owned, h, d) of
    the nodes this rank owns.  Differentiable; returns (n_owned, h, d).  The gradient of embed_ak
    is this rank's share (sum it over ranks like any data-parallel parameter gradient)."""
    import math
    from .attention import bpt_attention
    if scale is None:
        scale = 1.0 / math.sqrt(q.size(-1))
    if getattr(shard, "split", False):
        return _StraddleAttention.apply(shard, plan, q, k, v, embed_ak, scale)
    return bpt_attention(plan, q, _HaloKV.apply(shard, k), _HaloKV.apply(shard, v), embed_ak, scale)


class HaloRunner:
    """One attention layer, forward and backward, of a destination-sharded sequence as a fixed schedule with
    four collectives per step instead of six and everything between them on static buffers:

      forward   pack  -> all-to-all (halo K and V rows + the straddlers' Q rows, owner to everyone)
                      -> unpack, fused forward, partial (o, lse) of the straddlers
                      -> all-gather of the partials -> merge
      backward  all-gather of the straddlers' dO rows (each owner contributes its rows, padded to the largest
                         share; an all-reduce of a zero-filled buffer took twice as long on eight ranks)
                      -> fused backward, pack -> all-to-all back (dK, dV of the halo rows + every rank's
                         share of the straddlers' dQ, to the owner) -> fixed-order sums

    The pieces between collectives are plain tensor programs over precomputed index lists, so on a GPU each
    of them can be captured once in a CUDA graph (graphs=True) and replayed with one launch; the collectives
    themselves are issued eagerly between the replays.  shard: a SequenceShard after
    build_halo(split_straddlers=True); plan: its AttentionPlan.  bf16 / head dim 64 on the GPU (the
    tensor-core kernels' row term <dO, O> is what lets a rank compute its share of a straddling row).
    """

    def __init__(self, shard, plan, h, d, dtype, device, scale, ak_rows, graphs=False, group=None):
        if not getattr(shard, "split", False):
            raise ValueError("HaloRunner needs shard.build_halo(..., split_straddlers=True)")
        s = self.shard = shard
        self.plan, self.h, self.d, self.dtype, self.dev, self.scale, self.group = plan, h, d, dtype, device, scale, group
        w, rank = s.world, s.rank
        dev = device
        i64 = dict(dtype=torch.int64, device=dev)
        # straddlers: global list (ascending ids), their owners, and which are mine
        self.n_strad, self.n_ns, self.n_my = s.n_strad, s.n_ns, int(s.s_own_idx.numel())
        owner_of = (s.to_gathered // s.max_owned)[s.strad_ids].to(dev)       # owner rank of every straddler
        n_str_of = [int((owner_of == r).sum()) for r in range(w)]
        pos_of = [torch.nonzero(owner_of == r).squeeze(1) for r in range(w)]   # positions in the straddler list
        # ---- forward all-to-all: to peer p [halo rows p needs | my straddlers' Q rows]
        self.f_send_counts = [s.send_counts[p] + self.n_my for p in range(w)]
        self.f_recv_counts = [s.recv_counts[p] + n_str_of[p] for p in range(w)]
        sb = [0]
        for c in self.f_send_counts:
            sb.append(sb[-1] + c)
        rb = [0]
        for c in self.f_recv_counts:
            rb.append(rb[-1] + c)
        self.n_fsend, self.n_frecv = sb[-1], rb[-1]
        self.send_pos_kv = torch.cat([torch.arange(sb[p], sb[p] + s.send_counts[p], **i64) for p in range(w)])
        self.send_pos_q = torch.cat([torch.arange(sb[p] + s.send_counts[p], sb[p + 1], **i64) for p in range(w)])
        self.send_src_q = s.s_own_idx.to(dev).repeat(w)
        self.recv_pos_kv = torch.cat([torch.arange(rb[p], rb[p] + s.recv_counts[p], **i64) for p in range(w)])
        self.recv_pos_q = torch.cat([torch.arange(rb[p] + s.recv_counts[p], rb[p + 1], **i64) for p in range(w)])
        self.recv_dst_q = s.n_ns + torch.cat(pos_of) if self.n_strad else torch.zeros(0, **i64)
        # ---- return all-to-all: to peer p [gradients of the halo rows p sent | my share of dQ of p's straddlers]
        self.r_send_counts, self.r_recv_counts = self.f_recv_counts, self.f_send_counts
        self.ret_src_q = self.recv_dst_q                        # rows of dq_loc, in the order of recv_pos_q
        # received: from peer p [gradients for my rows send_idx[p] | p's share of dQ of my straddlers]
        self.my_q_parts = self.send_pos_q.view(w, self.n_my) if self.n_my else torch.zeros((w, 0), **i64)
        self.send_all = s.send_all.to(dev)
        self.ret_rows, self.ret_mat = s.ret_rows.to(dev), s.ret_mat.to(dev)
        self.s_own_idx, self.s_own_pos = s.s_own_idx.to(dev), s.s_own_pos.to(dev)
        self.ns_idx = s.ns_idx.to(dev)
        # ---- static buffers.  The inputs live inside the buffers the kernels read: k_in / v_in are the head of
        # the extended K / V, q_in / do_in the head of the destination-row buffers (own non-straddlers first,
        # which is how the owned list is ordered for binary-partition trees), so nothing is copied around the
        # exchange; a caller can also write its projections straight into them and call forward() / backward()
        # without arguments.  The straddler rows of q_in / do_in are consumed by the pack step and then reused.
        if not s.ns_prefix:
            raise ValueError("HaloRunner expects the straddling nodes last in a rank's owned list")
        row = (h, d)
        mk = lambda n, dt=dtype: torch.zeros((n,) + row, dtype=dt, device=dev)
        n_rows = max(s.n_dst_local, s.n_owned)
        # K, V and Q rows live in one tensor [K (n_ext) | V (n_ext) | Q (n_rows) | zero row | dump row], so that the
        # pack step is one gather of rows into the send buffer and the unpack step one scatter of the received rows
        self._big = mk(2 * s.n_ext + n_rows + 2)
        self.k_e, self.v_e = self._big[: s.n_ext], self._big[s.n_ext: 2 * s.n_ext]
        self._q_buf, self._do_buf = self._big[2 * s.n_ext: 2 * s.n_ext + n_rows], mk(n_rows)
        q0, zero_row, dump_row = 2 * s.n_ext, 2 * s.n_ext + n_rows, 2 * s.n_ext + n_rows + 1
        # the gradients likewise: [dQ (n_dst_local) | dK (n_ext) | dV (n_ext) | zero row]
        self._gbig = mk(s.n_dst_local + 2 * s.n_ext + 1)
        self._dq_out = self._gbig[: s.n_dst_local]
        self._dk_out = self._gbig[s.n_dst_local: s.n_dst_local + s.n_ext]
        self._dv_out = self._gbig[s.n_dst_local + s.n_ext: s.n_dst_local + 2 * s.n_ext]
        g_dk0, g_dv0, g_zero = s.n_dst_local, s.n_dst_local + s.n_ext, s.n_dst_local + 2 * s.n_ext
        self.q_loc, self.do_loc = self._q_buf[: s.n_dst_local], self._do_buf[: s.n_dst_local]
        self.k_in, self.v_in = self.k_e[: s.n_owned], self.v_e[: s.n_owned]
        self.q_in, self.do_in = self._q_buf[: s.n_owned], self._do_buf[: s.n_owned]
        self.ak_in = None if ak_rows is None else torch.zeros((ak_rows, d), dtype=dtype, device=dev)
        self.o_loc = self.lse_loc = None                          # the forward kernel's outputs, kept for the backward
        self.f_send = torch.zeros((self.n_fsend, 2) + row, dtype=dtype, device=dev)
        self.f_recv = torch.zeros((self.n_frecv, 2) + row, dtype=dtype, device=dev)
        self.r_send = torch.zeros((self.n_frecv, 2) + row, dtype=dtype, device=dev)
        self.r_recv = torch.zeros((self.n_fsend + 1, 2) + row, dtype=dtype, device=dev)   # last row stays zero
        self.part = torch.zeros((self.n_strad, h * d + h), dtype=torch.float32, device=dev)
        self.allp = torch.zeros((w * self.n_strad, h * d + h), dtype=torch.float32, device=dev)
        self.do_strad = mk(self.n_strad)
        # dO rows of the straddlers travel by all-gather: every rank sends max_my rows (its own straddlers first),
        # straddler j is row do_pick[j] of the gathered buffer
        self.max_my = max(n_str_of) if n_str_of else 0
        self.do_mine = mk(self.max_my)
        self.do_all = mk(w * self.max_my)
        pick = torch.zeros(self.n_strad, **i64)
        for r in range(w):
            pick[pos_of[r]] = r * self.max_my + torch.arange(n_str_of[r], **i64)
        self.do_pick = pick
        self.dq_strad = mk(self.n_my)                             # summed dQ of my straddlers
        # row lists of the exchanges over those tensors; a send or receive buffer is (rows, 2, h, d), its flat row
        # 2 p + c is slot c of position p
        send_all = s.send_all.to(dev).to(torch.int64)
        pack = torch.full((2 * self.n_fsend,), zero_row, **i64)
        pack[2 * self.send_pos_kv] = send_all
        pack[2 * self.send_pos_kv + 1] = s.n_ext + send_all
        if self.n_my:
            pack[2 * self.send_pos_q] = q0 + self.send_src_q.to(torch.int64)
        self.pack_rows = pack
        unpack = torch.full((2 * self.n_frecv,), dump_row, **i64)
        n_kv_recv = int(self.recv_pos_kv.numel())
        unpack[2 * self.recv_pos_kv] = s.n_owned + torch.arange(n_kv_recv, **i64)
        unpack[2 * self.recv_pos_kv + 1] = s.n_ext + s.n_owned + torch.arange(n_kv_recv, **i64)
        if self.n_strad:
            unpack[2 * self.recv_pos_q] = q0 + self.recv_dst_q.to(torch.int64)
        self.unpack_rows = unpack
        ret = torch.full((2 * self.n_frecv,), g_zero, **i64)
        ret[2 * self.recv_pos_kv] = g_dk0 + s.n_owned + torch.arange(n_kv_recv, **i64)
        ret[2 * self.recv_pos_kv + 1] = g_dv0 + s.n_owned + torch.arange(n_kv_recv, **i64)
        if self.n_strad:
            ret[2 * self.recv_pos_q] = self.ret_src_q.to(torch.int64)
        self.ret_pack_rows = ret
        # returned halo gradients: ret_mat lists, per own row, positions among [kv part of the received buffer |
        # the all-zero last row]; as positions of the received buffer itself
        halo_pos = torch.cat([self.send_pos_kv, torch.tensor([self.n_fsend], **i64)])
        self.ret_mat_recv = halo_pos[self.ret_mat] if self.ret_rows.numel() else self.ret_mat
        self.ret_rows_kv = torch.stack([g_dk0 + self.ret_rows.to(torch.int64), g_dv0 + self.ret_rows.to(torch.int64)], 1)
        self.graphs = bool(graphs) and device.type == "cuda"
        self._g = {}

    def own_rows(self, x_loc, x_strad_own=None):
        """(n_owned, ...) rows of this rank from a destination-row tensor [own non-straddlers | all straddlers]:
        the straddlers this rank owns are taken from x_strad_own (n_my rows) when given, else from x_loc."""
        tail = x_strad_own if x_strad_own is not None else x_loc[self.n_ns + self.s_own_pos]
        return torch.cat([x_loc[: self.n_ns], tail.to(x_loc.dtype)], 0)

    # ---- the pieces between collectives (no communication inside)
    def _kernels(self):
        if _KERNELS is not None:
            return _KERNELS
        from .attention import attention_backward, attention_forward
        return attention_forward, attention_backward

    def _seg_pack(self):
        if self.n_fsend:
            torch.index_select(self._big, 0, self.pack_rows, out=self.f_send.view((-1,) + self._big.shape[1:]))

    def _seg_forward(self):
        s = self.shard
        if self.n_frecv:
            # halo K and V rows behind the own ones, the straddlers' Q rows over q_in's straddler rows
            self._big.index_copy_(0, self.unpack_rows, self.f_recv.view((-1,) + self._big.shape[1:]))
        self.o_loc, self.lse_loc = self._kernels()[0](self.plan, self.q_loc, self.k_e, self.v_e, self.ak_in, self.scale)
        if self.n_strad:
            n = self.n_strad
            self.part[:, : self.h * self.d].copy_(self.o_loc[-n:].flatten(1))   # widened by the copy
            self.part[:, self.h * self.d:] = self.lse_loc[-n:]

    def _seg_merge(self):
        if self.n_strad:
            # lse = logsumexp_r lse_r, o = sum_r exp(lse_r - lse) o_r over the ranks' partial rows
            n, w, hd = self.n_strad, self.shard.world, self.h * self.d
            allp = self.allp.view(w, n, hd + self.h)
            o_r, lse_r = allp[:, :, :hd].view(w, n, self.h, self.d), allp[:, :, hd:]
            # weights exp(lse_r - lse) are the softmax of the ranks' lse (rows no rank has an edge for: all -inf)
            wgt = torch.softmax(lse_r, 0).nan_to_num_(0.0)
            self.o_loc[-n:] = (wgt.unsqueeze(-1) * o_r).sum(0).to(self.o_loc.dtype)
            torch.logsumexp(lse_r, 0, out=self.lse_loc[-n:])

    def _seg_dout(self):
        if self.n_my:
            self.do_mine[: self.n_my] = self.do_in[self.s_own_idx]

    def _seg_dout_pick(self):
        self.do_strad.copy_(self.do_all[self.do_pick])

    def _seg_backward(self):
        s = self.shard
        if self.n_strad:
            self.do_loc[self.n_ns:] = self.do_strad                        # overwrites do_in's straddler rows
        if _KERNELS is None:
            # the library's kernels write straight into the gradient tensor the return step gathers from
            _, _, _, dak = self._kernels()[1](self.plan, self.q_loc, self.k_e, self.v_e, self.ak_in, self.scale,
                                              self.lse_loc, self.do_loc, o=self.o_loc,
                                              out=(self._dq_out, self._dk_out, self._dv_out))
        else:
            dq_loc, dk_e, dv_e, dak = self._kernels()[1](self.plan, self.q_loc, self.k_e, self.v_e, self.ak_in,
                                                         self.scale, self.lse_loc, self.do_loc, o=self.o_loc)
            self._dq_out.copy_(dq_loc)
            self._dk_out.copy_(dk_e)
            self._dv_out.copy_(dv_e)
        self.dq_loc, self.dk_e, self.dv_e, self.dak = self._dq_out, self._dk_out, self._dv_out, dak
        if self.n_frecv:
            torch.index_select(self._gbig, 0, self.ret_pack_rows, out=self.r_send.view((-1,) + self._gbig.shape[1:]))

    def _seg_return(self):
        n_send = self.n_fsend
        if self.ret_rows.numel():
            # row i of ret_mat_recv lists the positions of the received buffer that name own row ret_rows[i]
            # (padded with the all-zero last row); dK and dV rows are updated together
            total = self.r_recv[self.ret_mat_recv].sum(1, dtype=torch.float32)   # (targets, 2, h, d) in fp32
            self._gbig[self.ret_rows_kv] = (total + self._gbig[self.ret_rows_kv]).to(self._gbig.dtype)
        if self.n_my:
            parts = self.r_recv[self.my_q_parts, 0]                              # (world, n_my, h, d), rank order
            self.dq_strad.copy_(parts.sum(0, dtype=torch.float32))

    def _run(self, name, fn):
        """Runs a piece eagerly, or captures it in a CUDA graph on first use and replays it afterwards."""
        if not self.graphs:
            return fn()
        g = self._g.get(name)
        if g is None:
            side = torch.cuda.Stream(device=self.dev)
            side.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    fn()                                          # warm-up outside the capture (workspaces, handles)
            torch.cuda.current_stream(self.dev).wait_stream(side)
            torch.cuda.synchronize(self.dev)
            g = torch.cuda.CUDAGraph()
            # thread_local: other threads of the process (the collective library's watchdog queries events
            # while ranks wait for each other) may keep calling the CUDA runtime during the capture
            import warnings
            with warnings.catch_warnings():
                # a piece that has nothing to do on this rank (no straddlers, no peers) captures an empty graph
                warnings.filterwarnings("ignore", message="The CUDA Graph is empty")
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    fn()
            self._g[name] = g
        g.replay()

    # ---- the step
    def forward(self, q=None, k=None, v=None, embed_ak=None):
        """q, k, v: (n_owned, h, d) of the nodes this rank owns, embed_ak (rows, d); an argument left out means
        the caller has already written it into q_in / k_in / v_in / ak_in.  Returns o over this rank's
        destination rows [own non-straddlers | all straddlers]: own_rows(o) gives the (n_owned, h, d) result.
        The tensor is reused by the next forward."""
        import torch.distributed as dist
        s = self.shard
        for buf, x in ((self.q_in, q), (self.k_in, k), (self.v_in, v), (self.ak_in, embed_ak)):
            if x is not None and buf is not None:
                buf.copy_(x)
        self._run("pack", self._seg_pack)
        if s.world > 1:
            dist.all_to_all_single(self.f_recv, self.f_send, output_split_sizes=self.f_recv_counts,
                                   input_split_sizes=self.f_send_counts, group=self.group)
        else:
            self.f_recv.copy_(self.f_send)
        self._run("forward", self._seg_forward)
        if self.n_strad:
            if s.world > 1:
                dist.all_gather_into_tensor(self.allp, self.part, group=self.group)
            else:
                self.allp.copy_(self.part)
            self._run("merge", self._seg_merge)
        return self.o_loc

    def backward(self, d_o=None):
        """d_o: (n_owned, h, d) gradient of own_rows(forward()), or None when already written into do_in.
        Returns (dq_loc, dq_strad_own, dk, dv, d_embed_ak): dq over the destination rows with the summed dQ
        of this rank's straddlers apart -- own_rows(dq_loc, dq_strad_own) is the (n_owned, h, d) gradient --,
        dk and dv (n_owned, h, d), d_embed_ak this rank's share in fp32 or None.  Reused by the next backward."""
        import torch.distributed as dist
        s = self.shard
        if d_o is not None:
            self.do_in.copy_(d_o)
        if self.n_strad:
            self._run("dout", self._seg_dout)
            if s.world > 1:
                dist.all_gather_into_tensor(self.do_all, self.do_mine, group=self.group)
            else:
                self.do_all.copy_(self.do_mine)
            self._run("dout_pick", self._seg_dout_pick)
        self._run("backward", self._seg_backward)
        if s.world > 1:
            dist.all_to_all_single(self.r_recv[: self.n_fsend], self.r_send, output_split_sizes=self.r_recv_counts,
                                   input_split_sizes=self.r_send_counts, group=self.group)
        else:
            self.r_recv[: self.n_fsend].copy_(self.r_send)
        self._run("return", self._seg_return)
        return self.dq_loc, self.dq_strad, self.dk_e[: s.n_owned], self.dv_e[: s.n_owned], self.dak
