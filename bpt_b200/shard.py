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

    # ---- halo exchange: only the remote rows this rank's edges name ----
    def build_halo(self, src, dst):
        """Send/receive lists of the halo exchange, computed locally by every rank from the whole
        edge list (no communication).  Sets
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
    send = x.index_select(0, shard.send_all)
    recv = x.new_empty((shard.n_halo,) + tuple(x.shape[1:]))
    dist.all_to_all_single(recv, send, output_split_sizes=shard.recv_counts, input_split_sizes=shard.send_counts,
                           group=group)
    return torch.cat([x, recv], 0)


def halo_return(shard, g_ext, group=None):
    """Gradient of halo_exchange: sends the halo rows' gradients back to their owners and adds
    them to the owners' rows, peer by peer in rank order (rows of one peer are distinct, so
    every sum has a fixed order)."""
    import torch.distributed as dist
    g_own = g_ext[: shard.n_owned].clone()
    send = g_ext[shard.n_owned:].contiguous()
    recv = g_ext.new_empty((int(shard.send_all.numel()),) + tuple(g_ext.shape[1:]))
    dist.all_to_all_single(recv, send, output_split_sizes=shard.send_counts, input_split_sizes=shard.recv_counts,
                           group=group)
    off = 0
    for idx in shard.send_idx:
        n = int(idx.numel())
        if n:
            g_own[idx] += recv[off:off + n]
        off += n
    return g_own


class _HaloKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, shard, x):
        ctx.shard = shard
        return halo_exchange(shard, x)

    @staticmethod
    def backward(ctx, g):
        return None, halo_return(ctx.shard, g)


def halo_attention(shard, plan, q, k, v, embed_ak=None, scale=None):
    """Attention for this rank's destinations with the halo exchange.  plan:
    AttentionPlan(shard.src_h, shard.dst_l, shard.etype_l, shard.n_owned, n_src=shard.n_ext) after
    shard.build_halo(src, dst).  Differentiable; returns (n_owned, h, d)."""
    from .attention import bpt_attention
    return bpt_attention(plan, q, _HaloKV.apply(shard, k), _HaloKV.apply(shard, v), embed_ak, scale)
