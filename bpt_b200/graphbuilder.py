"""GPU counterpart of the reference's `graphbuilder` module (graph_builder/builder.pyx).

Same names, arguments and return types as the reference: `BinaryPartition(length,
triu=False, step=1, clip_dist=10)` with its properties and accessors (builder.pyx:29-152),
the baseline graphs `FullyConnected` (:228-303) and `OpenAISparse` (:154-225), and
`partition_csr(indptr, chunk_size=32)` (:305-321).
The graph is built on the current CUDA device by the kernels behind bpt_bp_count /
bpt_bp_fill and is bit-identical to the reference's.  The numpy-returning accessors copy to
the host as the reference's callers expect; the `*_device` accessors hand out the device
arrays for the fused path without a round trip.
"""
import ctypes

import numpy as np
import torch

from . import _lib


def _device(device=None):
    if not torch.cuda.is_available():
        raise RuntimeError("bpt_b200.graphbuilder needs a CUDA device (there is no CPU path)")
    return torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)


def levels(length):
    """Level sizes, first node id per level, node count (builder.pyx:41-56). Host only."""
    nn = (ctypes.c_uint32 * 64)()
    sh = (ctypes.c_uint32 * 64)()
    n_nodes = ctypes.c_int64(0)
    n_lvl = ctypes.c_int(0)
    _lib.check(_lib.lib().bpt_bp_levels(int(length), ctypes.addressof(nn), ctypes.addressof(sh),
                                        ctypes.addressof(n_nodes), ctypes.addressof(n_lvl)))
    k = n_lvl.value
    return list(nn[:k]), list(sh[:k]), int(n_nodes.value)


def count_edges(length, triu, step, clip_dist, device=None):
    """Runs the count pass; returns (leaf_offsets device int64[length+1], n_edges)."""
    dev = _device(device)
    L = _lib.lib()
    with torch.cuda.device(dev):
        offsets = torch.empty(length + 1, dtype=torch.int64, device=dev)
        ws = _lib.workspace(L.bpt_bp_count_workspace_bytes(int(length)), dev)
        n_edges = ctypes.c_int64(0)
        _lib.check(L.bpt_bp_count(int(length), int(bool(triu)), int(step), int(clip_dist),
                                  offsets.data_ptr(), ws.data_ptr(), ws.numel(),
                                  ctypes.addressof(n_edges), _lib.stream()))
    return offsets, int(n_edges.value)


def fill_edges(length, triu, step, clip_dist, offsets, v_shift, src, dst, etype, pos):
    """Runs the fill pass into (views of) preallocated device arrays, all int32 or all int64."""
    some = next(t for t in (src, dst, etype, pos) if t is not None)
    index_bytes = some.element_size()
    with torch.cuda.device(some.device):
        _lib.check(_lib.lib().bpt_bp_fill(int(length), int(bool(triu)), int(step), int(clip_dist),
                                          offsets.data_ptr(), int(v_shift), index_bytes,
                                          _lib.ptr(src), _lib.ptr(dst), _lib.ptr(etype), _lib.ptr(pos),
                                          _lib.stream()))


class BinaryPartition:
    """builder.pyx:23-152.  Built once on the GPU; int32 device arrays are kept."""

    def __init__(self, length, triu=False, step=1, clip_dist=10, device=None):
        length, step, clip_dist = int(length), int(step), int(clip_dist)
        if length < 1:
            raise ValueError("BinaryPartition: length must be >= 1")
        self.length, self.triu, self.step, self.clip_dist = length, bool(triu), step, clip_dist
        self.n_nodes_arr, self.shift, self.n_nodes = levels(length)
        self.n_lvl = len(self.n_nodes_arr)
        self.device = _device(device)
        self._offsets, self.n_edges = count_edges(length, triu, step, clip_dist, self.device)
        e = self.n_edges
        self._src = torch.empty(e, dtype=torch.int32, device=self.device)
        self._dst = torch.empty(e, dtype=torch.int32, device=self.device)
        self._etype = torch.empty(e, dtype=torch.int32, device=self.device)
        self._pos = torch.empty(self.n_nodes, dtype=torch.int32, device=self.device)
        fill_edges(length, triu, step, clip_dist, self._offsets, 0, self._src, self._dst, self._etype,
                   self._pos)

    def __reduce__(self):  # builder.pyx:38-39
        return BinaryPartition, (self.length, self.triu, self.step, self.clip_dist)

    @property
    def number_of_nodes(self):
        return self.n_nodes

    @property
    def number_of_edges(self):
        return self.n_edges

    @property
    def number_of_levels(self):
        return self.n_lvl

    @property
    def is_triu(self):
        return self.triu

    def get_pos(self):
        """builder.pyx:134-135 (int64 numpy array)."""
        return self._pos.cpu().numpy().astype(np.int64)

    def get_edges(self, v_shift=0):
        """builder.pyx:137-140: (src + v_shift, dst + v_shift, etype) as int64 numpy arrays."""
        return (self._src.cpu().numpy().astype(np.int64) + v_shift,
                self._dst.cpu().numpy().astype(np.int64) + v_shift,
                self._etype.cpu().numpy().astype(np.int64))

    def leaf_ids(self, v_shift=0, start=0):
        return np.arange(v_shift + start, v_shift + self.n_nodes_arr[0])

    def internal_ids(self, v_shift=0):
        return np.arange(v_shift + self.n_nodes_arr[0], v_shift + self.n_nodes)

    def root_id(self, v_shift=0):
        return v_shift + self.n_nodes - 1

    def number_of_nodes_at_lvl(self, i):
        return self.n_nodes_arr[i]

    # ---- device-side accessors (no counterpart in the reference) ----
    def edges_device(self):
        """(src, dst, etype) int32 device tensors in edge-id order."""
        return self._src, self._dst, self._etype

    def pos_device(self):
        return self._pos

    def fill_into(self, v_shift, src, dst, etype, pos):
        """Writes this graph, node ids shifted by v_shift, into slices of a batch's arrays:
        the block-diagonal placement of graph/lm.py:76-91."""
        fill_edges(self.length, self.triu, self.step, self.clip_dist, self._offsets, v_shift,
                   src, dst, etype, pos)


class _BaselineGraph:
    """Shared part of the two baseline graphs: `length` tokens plus one root node."""

    def _build(self, count, fill):
        L = _lib.lib()
        with torch.cuda.device(self.device):
            self._offsets = torch.empty(self.length + 1, dtype=torch.int64, device=self.device)
            ws = _lib.workspace(L.bpt_bp_count_workspace_bytes(self.length), self.device)
            n_edges = ctypes.c_int64(0)
            _lib.check(count(self._offsets.data_ptr(), ws.data_ptr(), ws.numel(), ctypes.addressof(n_edges),
                             _lib.stream()))
            self.n_edges = int(n_edges.value)
            self._src, self._dst, self._etype = [torch.empty(self.n_edges, dtype=torch.int32, device=self.device)
                                                 for _ in range(3)]
            self._pos = torch.empty(self.n_nodes, dtype=torch.int32, device=self.device)
            self._fill = fill
            self.fill_into(0, self._src, self._dst, self._etype, self._pos)

    def fill_into(self, v_shift, src, dst, etype, pos):
        some = next(t for t in (src, dst, etype, pos) if t is not None)
        with torch.cuda.device(some.device):
            _lib.check(self._fill(self._offsets.data_ptr(), int(v_shift), some.element_size(), _lib.ptr(src),
                                  _lib.ptr(dst), _lib.ptr(etype), _lib.ptr(pos), _lib.stream()))

    @property
    def number_of_nodes(self):
        return self.n_nodes

    @property
    def number_of_edges(self):
        return self.n_edges

    @property
    def is_triu(self):
        return self.triu

    def get_pos(self):
        return self._pos.cpu().numpy().astype(np.int64)

    def get_edges(self, v_shift=0):
        return (self._src.cpu().numpy().astype(np.int64) + v_shift,
                self._dst.cpu().numpy().astype(np.int64) + v_shift,
                self._etype.cpu().numpy().astype(np.int64))

    def root_id(self, v_shift=0):
        return v_shift + self.n_nodes - 1

    def leaf_ids(self, v_shift=0, start=0):
        return np.arange(v_shift + start, v_shift + self.length)

    def internal_ids(self, v_shift=0):
        return np.arange(v_shift + self.length, v_shift + self.n_nodes)

    def edges_device(self):
        return self._src, self._dst, self._etype

    def pos_device(self):
        return self._pos


class FullyConnected(_BaselineGraph):
    """builder.pyx:228-303: dense (or windowed) attention graph with a root node."""

    def __init__(self, length, triu=False, window=8192, device=None):
        self.length, self.triu, self.window = int(length), bool(triu), int(window)
        if self.length < 1:
            raise ValueError("FullyConnected: length must be >= 1")
        self.n_nodes = self.length + 1
        self.device = _device(device)
        L = _lib.lib()
        self._build(lambda *a: L.bpt_fc_count(self.length, int(self.triu), self.window, *a),
                    lambda *a: L.bpt_fc_fill(self.length, int(self.triu), self.window, *a))

    def __reduce__(self):
        return FullyConnected, (self.length, self.triu, self.window)


class OpenAISparse(_BaselineGraph):
    """builder.pyx:154-225: strided causal graph of the Sparse Transformer baseline."""

    def __init__(self, length, stride, c, triu=True, device=None):
        assert triu, "bidirectional model is not supported"  # builder.pyx:165
        self.length, self.stride, self.c, self.triu = int(length), int(stride), int(c), True
        if self.length < 1 or self.stride < 1:
            raise ValueError("OpenAISparse: length and stride must be >= 1")
        self.n_nodes = self.length + 1
        self.device = _device(device)
        L = _lib.lib()
        self._build(lambda *a: L.bpt_oas_count(self.length, self.stride, self.c, *a),
                    lambda *a: L.bpt_oas_fill(self.length, self.stride, self.c, *a))

    def __reduce__(self):
        return OpenAISparse, (self.length, self.stride, self.c, self.triu)


def partition_csr(indptr, chunk_size=32):
    """builder.pyx:305-321.  Takes a numpy int64 array and returns numpy arrays like the
    reference; given a CUDA int64 tensor it returns CUDA tensors and stays on the device."""
    as_numpy = isinstance(indptr, np.ndarray)
    if as_numpy:
        dev = _device()
        t = torch.from_numpy(np.ascontiguousarray(indptr, dtype=np.int64)).to(dev)
    else:
        t = indptr.contiguous()
        _lib.require_cuda(t)
        if t.dtype != torch.int64:
            raise RuntimeError("partition_csr: indptr must be int64")
        dev = t.device
    n_rows = t.numel() - 1
    L = _lib.lib()
    with torch.cuda.device(dev):
        offs = torch.empty(n_rows + 1, dtype=torch.int64, device=dev)
        ws = _lib.workspace(L.bpt_partition_csr_workspace_bytes(n_rows), dev)
        n_chunks = ctypes.c_int64(0)
        _lib.check(L.bpt_partition_csr_count(t.data_ptr(), n_rows, int(chunk_size), offs.data_ptr(),
                                             ws.data_ptr(), ws.numel(), ctypes.addressof(n_chunks),
                                             _lib.stream()))
        c = int(n_chunks.value)
        row = torch.empty(c, dtype=torch.int64, device=dev)
        ip = torch.empty(c + 1, dtype=torch.int64, device=dev)
        _lib.check(L.bpt_partition_csr_fill(t.data_ptr(), n_rows, int(chunk_size), offs.data_ptr(), c,
                                            _lib.ptr(row) if c else None, ip.data_ptr(), _lib.stream()))
    if as_numpy:
        return row.cpu().numpy(), ip.cpu().numpy()
    return row, ip
