"""CSR extraction and block-diagonal batching on the device.

`get_csrs` replaces get_csrs(g) of the reference's graph/base.py:71-86: from a COO edge
list (edge id = position) it returns the same 6-tuple
`(out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C)` of int64 tensors, each csr being
`(indptr, indices, eid)`; rows of out_csr are sources, rows of in_csr destinations, and
the chunk arrays come from partition_csr with the default chunk of 32 edges.  Inside a row
entries are in ascending edge-id order (the reference leaves that order to its graph
library).  Everything stays on the GPU: the reference builds these on the host and copies
them over every step (modules/model.py:244).

`batch_graphs` is the batching rule of graph/lm.py:59-98.
"""
import torch

from . import _lib
from .graphbuilder import BinaryPartition, partition_csr


def coo_to_csr(key, other, n_rows):
    """Stable bucket of edge ids by `key`: returns (indptr, indices=other[eid], eid)."""
    _lib.require_cuda(key, other)
    if key.dtype != other.dtype or key.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("coo_to_csr: key/other must both be int32 or both int64")
    e = key.numel()
    dev = key.device
    L = _lib.lib()
    with torch.cuda.device(dev):
        indptr = torch.empty(n_rows + 1, dtype=key.dtype, device=dev)
        indices = torch.empty(e, dtype=key.dtype, device=dev)
        eid = torch.empty(e, dtype=key.dtype, device=dev)
        ws = _lib.workspace(L.bpt_coo_to_csr_workspace_bytes(e, n_rows), dev)
        _lib.check(L.bpt_coo_to_csr(_lib.ptr(key), _lib.ptr(other), e, n_rows, key.element_size(),
                                    indptr.data_ptr(), _lib.ptr(indices), _lib.ptr(eid),
                                    ws.data_ptr(), ws.numel(), _lib.stream()))
    return indptr, indices, eid


def get_csrs(src, dst, n_nodes):
    """graph/base.py:71-86 on device tensors `src`, `dst` (int64, edge id = position)."""
    src = src.to(torch.int64).contiguous()
    dst = dst.to(torch.int64).contiguous()
    out_csr = coo_to_csr(src, dst, n_nodes)
    in_csr = coo_to_csr(dst, src, n_nodes)
    ROW, INDPTR_R = partition_csr(out_csr[0])
    COL, INDPTR_C = partition_csr(in_csr[0])
    return out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C


class GraphCache:
    """Per-length cache of built graphs, as GraphBatcher._get_graph keeps (graph/base.py:12-26)."""

    def __init__(self, triu=False, step=1, clip_dist=10, device=None):
        self.triu, self.step, self.clip_dist, self.device = triu, step, clip_dist, device
        self._cache = {}

    def get(self, length):
        g = self._cache.get(length)
        if g is None:
            g = BinaryPartition(length, self.triu, self.step, self.clip_dist, device=self.device)
            self._cache[length] = g
        return g


class BatchedGraph:
    """A block-diagonal batch: COO arrays on the device plus per-sequence offsets."""

    def __init__(self, src, dst, etype, pos, node_offsets, edge_offsets, lengths):
        self.src, self.dst, self.etype, self.pos = src, dst, etype, pos
        self.node_offsets, self.edge_offsets, self.lengths = node_offsets, edge_offsets, lengths
        self.n_nodes, self.n_edges = node_offsets[-1], edge_offsets[-1]

    def leaf_ids(self):
        """Concatenation of every sequence's leaf_ids(v_shift) (graph/lm.py:79-80)."""
        parts = [torch.arange(o, o + n, device=self.src.device)
                 for o, n in zip(self.node_offsets[:-1], self.lengths)]
        return torch.cat(parts)

    def root_ids(self):
        return torch.tensor([o - 1 for o in self.node_offsets[1:]], device=self.src.device)


def batch_graphs(graphs, dtype=torch.int32):
    """graph/lm.py:59-98: sequence b's nodes are shifted by the node count of sequences
    before it; its edges follow theirs, so edge id = position in the concatenation.
    `graphs` is a list of BinaryPartition (the same object may repeat)."""
    dev = graphs[0].device
    node_offsets, edge_offsets = [0], [0]
    for g in graphs:
        node_offsets.append(node_offsets[-1] + g.n_nodes)
        edge_offsets.append(edge_offsets[-1] + g.n_edges)
    N, E = node_offsets[-1], edge_offsets[-1]
    if dtype == torch.int32 and N >= 2 ** 31:
        raise RuntimeError("batch_graphs: node ids exceed int32")
    src = torch.empty(E, dtype=dtype, device=dev)
    dst = torch.empty(E, dtype=dtype, device=dev)
    etype = torch.empty(E, dtype=dtype, device=dev)
    pos = torch.empty(N, dtype=dtype, device=dev)
    for b, g in enumerate(graphs):
        e0, e1 = edge_offsets[b], edge_offsets[b + 1]
        n0, n1 = node_offsets[b], node_offsets[b + 1]
        g.fill_into(n0, src[e0:e1], dst[e0:e1], etype[e0:e1], pos[n0:n1])
    return BatchedGraph(src, dst, etype, pos, node_offsets, edge_offsets, [g.length for g in graphs])


def inter_graph(src_ranges, dst_ranges, device=None, dtype=torch.int32):
    """Sentence-aligned cross graph (graph/mt.py:318-321, graph/nli.py:84-87): every node of the
    i-th source range sends an edge to every node of the i-th destination range.  Ranges are
    (first id, count) pairs; returns (src, dst) device tensors with the reference's edge order
    (source slow, destination fast inside a block)."""
    if len(src_ranges) != len(dst_ranges):
        raise ValueError("inter_graph: as many source ranges as destination ranges")
    if not torch.cuda.is_available():
        raise RuntimeError("bpt_b200.csr.inter_graph needs a CUDA device (there is no CPU path)")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    blocks, offsets = [], [0]
    for (s0, ns), (d0, nd) in zip(src_ranges, dst_ranges):
        if ns < 0 or nd < 0:
            raise ValueError("inter_graph: negative range length")
        blocks.append((int(s0), int(ns), int(d0), int(nd)))
        offsets.append(offsets[-1] + int(ns) * int(nd))
    n_edges = offsets[-1]
    src = torch.empty(n_edges, dtype=dtype, device=dev)
    dst = torch.empty(n_edges, dtype=dtype, device=dev)
    if n_edges:
        with torch.cuda.device(dev):
            b = torch.tensor(blocks, dtype=torch.int64).to(dev)
            o = torch.tensor(offsets, dtype=torch.int64).to(dev)
            _lib.check(_lib.lib().bpt_dense_blocks_fill(b.data_ptr(), o.data_ptr(), len(blocks), n_edges,
                                                        src.element_size(), src.data_ptr(), dst.data_ptr(),
                                                        _lib.stream()))
    return src, dst
