"""Fused binary-partition graph attention: host side of bpt_attn_forward / bpt_attn_backward.

`AttentionPlan` is built once per graph (per batch layout) from the COO edge list and holds
the device blob the kernels walk.  `bpt_attention(plan, q, k, v, embed_ak, scale)` is one
autograd function that stands for the chain of four operators in the reference's
BPTBlock.forward (modules/attention.py:66-77, dropout off):

    e     = masked_mm(..., k, q)
    e_rel = node_mul_edge(..., q, embed_ak(etype))
    p     = sparse_softmax(..., (e_rel + e) / sqrt(d_k))
    a     = vec_spmm(..., p, v)

Unlike the chain it never materialises the (E, d) gather of embed_ak nor any (E, h) tensor
in the forward, and its results do not vary from run to run.
"""
import ctypes
import math
import os

import numpy as np
import torch

from . import _lib


class AttentionPlan:
    """Device-resident plan of one graph for the fused kernels.

    src, dst, etype: int32 CUDA tensors in edge-id order (etype may be None);
    n_etypes: rows of the relative-position table the graph may index (every etype must be
    smaller); defaults to max(etype) + 1.  n_src: number of source rows (k, v) when sources
    and destinations are different node sets (cross-attention, a shard attending to gathered
    K/V); defaults to n_nodes.
    """

    def __init__(self, src, dst, etype, n_nodes, n_etypes=None, n_src=None):
        src = src.to(torch.int32).contiguous()
        dst = dst.to(torch.int32).contiguous()
        _lib.require_cuda(src, dst)
        if etype is not None:
            etype = etype.to(torch.int32).contiguous()
            _lib.require_cuda(etype)
            if n_etypes is None:
                n_etypes = int(etype.max().item()) + 1 if etype.numel() else 1
        elif n_etypes is None:
            n_etypes = 1
        self.device = src.device
        self.n_nodes, self.n_edges, self.n_etypes = int(n_nodes), int(src.numel()), int(n_etypes)
        self.n_src = self.n_nodes if n_src is None else int(n_src)
        L = _lib.lib()
        with torch.cuda.device(self.device):
            self.blob = _lib.workspace(L.bpt_attn_plan_bytes(self.n_nodes, self.n_src, self.n_edges, self.n_etypes),
                                       self.device)
            ws = _lib.workspace(L.bpt_attn_plan_workspace_bytes(self.n_nodes, self.n_src, self.n_edges, self.n_etypes),
                                self.device)
            self._counts = (ctypes.c_int32 * 12)()
            _lib.check(L.bpt_attn_plan_build(_lib.ptr(src), _lib.ptr(dst), _lib.ptr(etype), self.n_edges,
                                             self.n_nodes, self.n_src, self.n_etypes, self.blob.data_ptr(),
                                             self.blob.numel(), ws.data_ptr(), ws.numel(),
                                             ctypes.addressof(self._counts), _lib.stream()))
        self.counts = list(self._counts)
        self._ws = {}
        self.tiles = None    # TilePlan of the tensor-core forward, built on first use
        self.tiles_t = None  # transposed TilePlan of the tensor-core dK/dV kernel
        self.tiles5 = None   # 128-row TilePlan of the tcgen05 forward
        self.segments = None  # node offsets of the graphs of a block-diagonal batch (from_batch), for the tile plans

    @classmethod
    def from_batch(cls, batch, n_etypes=None):
        """From a csr.BatchedGraph.  The tile plans count their blocks of source columns from each graph's first
        node, so a graph is cut into tiles where it is cut when it is planned alone."""
        plan = cls(batch.src, batch.dst, batch.etype, batch.n_nodes, n_etypes)
        offsets = [int(x) for x in batch.node_offsets]
        if TILE_ALIGN_GRAPHS and len(offsets) > 2:
            plan.segments = offsets
        return plan

    def workspace(self, h, d, backward):
        """Scratch for one call; cached per (h, d, direction) and reused by later calls on
        the same stream (calls on different streams must not share a plan's scratch)."""
        key = (h, d, bool(backward))
        ws = self._ws.get(key)
        if ws is None:
            n = _lib.lib().bpt_attn_workspace_bytes(self.n_nodes, self.n_edges, ctypes.addressof(self._counts), h, d,
                                                    int(bool(backward)))
            ws = _lib.workspace(n, self.device)
            self._ws[key] = ws
        return ws

    def tile_plan(self):
        """The tile plan of the tensor-core forward and of the destination side of the backward (built once
        per graph)."""
        if self.tiles is None:
            self.tiles = TilePlan(self, max_cols=TILE_MAX_COLS, col_segments=self.segments)
        return self.tiles

    def tile_plan5(self):
        """The tile plan of the tcgen05 forward: groups of 128 destination rows (one per thread and
        tensor-memory lane) over up to 512 source columns; rows outside dense groups bucketed by
        block of 128 consecutive sources."""
        if self.tiles5 is None:
            self.tiles5 = TilePlan(self, min_density=0.05, max_cols=512, group_rows=128, col_block=128,
                                   max_mblocks=8, col_segments=self.segments)
        return self.tiles5

    def tile_plan_t(self):
        """The transposed tile plan (rows = sources) of the tensor-core dK/dV kernel."""
        if self.tiles_t is None:
            self.tiles_t = TilePlan(self, transposed=True, min_density=0.15, simt_max_degree=0,
                                    max_cols=TILE_T_MAX_COLS, col_block=TILE_T_COL_BLOCK, col_segments=self.segments)
        return self.tiles_t

    def _args(self):
        return (self.blob.data_ptr(), ctypes.addressof(self._counts), self.n_nodes, self.n_edges, self.n_etypes)


class TilePlan:
    """Groups of columns shared by m-blocks of <= 16 rows, for the tensor-core kernels.
    Planned once per graph from a CSR of the plan (integer work; on the device by default), kept on the
    device.  transposed=False: rows are destinations, columns sources, cells carry edge types
    (bpt_attn_forward_tc).  transposed=True: rows are sources, columns destinations, cells
    carry the edge's position in the in-CSR (source side of bpt_attn_backward_tc)."""

    def __init__(self, plan, transposed=False, min_density=0.25, max_cols=384, group_rows=16, col_block=128,
                 simt_max_degree=0, max_mblocks=1, join_dense=False, planner=None, col_segments=None):
        """planner: "device" (the default; BPT_TILE_PLANNER overrides it) plans with CUDA kernels from the CSR
        arrays where the plan keeps them; "host" exports the CSR, plans in C++ on the host and uploads.  Both
        give the same arrays; simt_max_degree and join_dense exist on the host planner only.
        col_segments: ascending offsets [0, ..., number of columns] of the graphs of a block-diagonal batch;
        blocks of col_block columns are then counted from each graph's first column."""
        if col_segments is not None:
            col_segments = [int(x) for x in col_segments]
            n_col_space = plan.n_nodes if transposed else plan.n_src
            if len(col_segments) < 2 or col_segments[0] != 0 or col_segments[-1] != n_col_space or \
                    any(b < a for a, b in zip(col_segments, col_segments[1:])):
                raise ValueError("TilePlan: col_segments must ascend from 0 to the number of columns")
        self.col_segments = col_segments
        planner = planner or TILE_PLANNER
        if planner not in ("device", "host"):
            raise ValueError("TilePlan: planner must be 'device' or 'host'")
        if simt_max_degree or join_dense:
            planner = "host"
        self.planner = planner
        self.n_etypes = plan.n_etypes
        self.transposed = transposed
        self._ws = {}
        if planner == "device":
            self._plan_on_device(plan, transposed, min_density, max_cols, group_rows, col_block, max_mblocks,
                                 col_segments)
        else:
            self._plan_on_host(plan, transposed, min_density, max_cols, group_rows, col_block, simt_max_degree,
                               max_mblocks, join_dense, col_segments)

    def _plan_on_device(self, plan, transposed, min_density, max_cols, group_rows, col_block, max_mblocks,
                        col_segments=None):
        L = _lib.lib()
        dev = plan.device
        n_segs = 0 if col_segments is None else len(col_segments) - 1
        segs = (ctypes.c_int64 * (n_segs + 1))(*col_segments) if n_segs else None
        with torch.cuda.device(dev):
            handle = L.bpt_tile_plan_create_device_aligned(
                plan.blob.data_ptr(), ctypes.addressof(plan._counts), plan.n_nodes, plan.n_edges, plan.n_etypes,
                int(bool(transposed)), None if segs is None else ctypes.addressof(segs), n_segs, float(min_density),
                int(max_cols), int(group_rows), int(col_block), int(max_mblocks), _lib.stream())
            if not handle:
                _lib.check(1)
            try:
                sizes = (ctypes.c_int64 * 13)()
                _lib.check(L.bpt_tile_plan_device_sizes(handle, ctypes.addressof(sizes)))
                (self.n_groups, self.n_mblocks, n_cols, self.n_cells, self.n_split, self.n_slots, self.t_max,
                 self.max_cols_pad, self.max_mblocks, self.max_qr_slots, self.n_row_items,
                 self.n_dense_groups, max_et) = [int(x) for x in sizes]
                self.n_cols = n_cols
                self.et_bytes = 1 if transposed or max_et < 248 else 2
                i32 = dict(dtype=torch.int32, device=dev)
                self.groups = torch.empty(max(self.n_groups * 8, 1), **i32)
                self.mblocks = torch.empty(max(self.n_mblocks * 56, 1), **i32)
                self.cols = torch.empty(max(n_cols, 1), **i32)
                self.et = None if transposed else torch.empty(max(self.n_cells, 1) * self.et_bytes, dtype=torch.uint8,
                                                              device=dev)
                self.cellpos = torch.empty(max(self.n_cells, 1), **i32)
                self.split = torch.empty(max(self.n_split * 4, 1), **i32)
                self.items = torch.empty(1, **i32)
                _lib.check(L.bpt_tile_plan_device_export(
                    handle, self.groups.data_ptr(), self.mblocks.data_ptr(), self.cols.data_ptr(),
                    None if self.et is None else self.et.data_ptr(), self.et_bytes, self.cellpos.data_ptr(),
                    self.split.data_ptr(), _lib.stream()))
            finally:
                L.bpt_tile_plan_device_destroy(handle)

    def _plan_on_host(self, plan, transposed, min_density, max_cols, group_rows, col_block, simt_max_degree,
                      max_mblocks, join_dense, col_segments=None):
        L = _lib.lib()
        E, T = plan.n_edges, plan.n_etypes
        n_rows = plan.n_src if transposed else plan.n_nodes
        indptr = np.empty(n_rows + 1, np.int32)
        other = np.empty(max(E, 1), np.int32)
        extra = np.empty(max(E, 1), np.int32)
        export = L.bpt_export_out_csr if transposed else L.bpt_export_in_csr
        with torch.cuda.device(plan.device):
            _lib.check(export(plan.blob.data_ptr(), ctypes.addressof(plan._counts), plan.n_nodes, E, T,
                              indptr.ctypes.data, other.ctypes.data, extra.ctypes.data, _lib.stream()))
        seg_start = seg_shift = None
        if col_segments is not None and len(col_segments) > 1:
            # every graph's columns start at a multiple of col_block for the planner; shifted back below
            seg_start = np.asarray(col_segments[:-1], np.int64)
            sizes_seg = np.diff(np.asarray(col_segments, np.int64))
            padded = (sizes_seg + col_block - 1) // col_block * col_block
            vstart = np.concatenate([[0], np.cumsum(padded)[:-1]])
            seg_shift = vstart - seg_start
            seg = np.searchsorted(seg_start, other[:E], side="right") - 1
            other[:E] = (other[:E] + seg_shift[seg]).astype(np.int32)
        etype_ptr, payload_ptr = (None, extra.ctypes.data) if transposed else (extra.ctypes.data, None)
        handle = L.bpt_tile_plan_create(indptr.ctypes.data, other.ctypes.data, etype_ptr, payload_ptr, n_rows, E,
                                        float(min_density), int(max_cols), int(group_rows), int(col_block),
                                        int(simt_max_degree), int(max_mblocks), int(bool(join_dense)))
        if not handle:
            _lib.check(1)
        try:
            sizes = (ctypes.c_int64 * 12)()
            _lib.check(L.bpt_tile_plan_sizes(handle, ctypes.addressof(sizes)))
            (self.n_groups, self.n_mblocks, n_cols, self.n_cells, self.n_split, self.n_slots, self.t_max,
             self.max_cols_pad, self.max_mblocks, self.max_qr_slots, self.n_row_items,
             self.n_dense_groups) = [int(x) for x in sizes]
            self.n_cols = n_cols
            max_et = 0 if transposed or not E else int(extra[:E].max())
            self.et_bytes = 1 if max_et < 248 else 2  # 8-bit cells: types and the "no edge" table index fit a byte
            groups = np.empty(max(self.n_groups * 8, 1), np.int32)
            mblocks = np.empty(max(self.n_mblocks * 56, 1), np.int32)
            cols = np.empty(max(n_cols, 1), np.int32)
            et = np.empty(max(self.n_cells, 1), np.uint8 if self.et_bytes == 1 else np.uint16)
            cellpos = np.empty(max(self.n_cells, 1), np.int32)
            split = np.empty(max(self.n_split * 4, 1), np.int32)
            items = np.empty(max(self.n_row_items * 4, 1), np.int32)
            _lib.check(L.bpt_tile_plan_export(handle, groups.ctypes.data, mblocks.ctypes.data, cols.ctypes.data,
                                              et.ctypes.data, self.et_bytes,
                                              cellpos.ctypes.data, split.ctypes.data,
                                              items.ctypes.data))
        finally:
            L.bpt_tile_plan_destroy(handle)
        if seg_start is not None and n_cols > 0:
            seg = np.searchsorted(seg_start + seg_shift, cols[:n_cols], side="right") - 1
            cols[:n_cols] = (cols[:n_cols] - seg_shift[seg]).astype(np.int32)
        dev = plan.device
        self.groups = torch.from_numpy(groups).to(dev)
        self.mblocks = torch.from_numpy(mblocks).to(dev)
        self.cols = torch.from_numpy(cols).to(dev)
        self.et = None if transposed else torch.from_numpy(et.view(np.uint8)).to(dev)
        self.cellpos = torch.from_numpy(cellpos).to(dev)
        self.split = torch.from_numpy(split).to(dev)
        self.items = torch.from_numpy(items).to(dev)

    def struct(self):
        """The bpt_tile_plan_t view of the device arrays."""
        s = _lib.TilePlanStruct()
        s.groups, s.mblocks, s.cols = self.groups.data_ptr(), self.mblocks.data_ptr(), self.cols.data_ptr()
        s.et = None if self.et is None else self.et.data_ptr()
        s.cell_pos = self.cellpos.data_ptr()
        s.split_rows, s.row_items = self.split.data_ptr(), self.items.data_ptr()
        s.n_groups, s.n_split, s.n_slots, s.n_row_items = self.n_groups, self.n_split, self.n_slots, self.n_row_items
        s.et_bytes, s.max_cols_pad, s.t_max = self.et_bytes, self.max_cols_pad, self.t_max
        return s

    def workspace(self, h, device):
        ws = self._ws.get(h)
        if ws is None:
            L = _lib.lib()
            n = L.bpt_attn_forward_tc_workspace_bytes(self.n_slots, h)
            ws = _lib.workspace(n, device)
            self._ws[h] = ws
        return ws


# fp32 with head dim 64: "tc32" = forward on the tile plan with 3xTF32 products, "simt" = CUDA-core kernel
FP32_FORWARD = os.environ.get("BPT_FP32_FORWARD", "tc32")
# fp32 backward: "tc32" = destination side (p, dp, K part of dQ) on the tile plan with 3xTF32 products, the
# source-side and embed_ak passes on the CUDA-core kernels; "simt" = all CUDA-core
FP32_BACKWARD = os.environ.get("BPT_FP32_BACKWARD", "tc32")
FP32_BACKWARD_SOURCE_SIDE = os.environ.get("BPT_FP32_BACKWARD_SOURCE_SIDE", "tc32")  # with FP32_BACKWARD = "tc32"
TILE_PLANNER = os.environ.get("BPT_TILE_PLANNER", "device")
# Tile plans of a batch count their column blocks from each graph's first node (AttentionPlan.from_batch)
TILE_ALIGN_GRAPHS = os.environ.get("BPT_TILE_ALIGN_GRAPHS", "1") != "0"
# Widest column list of a 16-row tile; rows that would need more are cut by blocks of 128 source columns.
TILE_MAX_COLS = int(os.environ.get("BPT_TILE_MAX_COLS", "384"))
# The transposed plan (rows = sources): widest destination list of a tile, and the block of destinations by which
# sources with longer lists are cut (each block a source falls into is one partial dK/dV row to merge)
TILE_T_MAX_COLS = int(os.environ.get("BPT_TILE_T_MAX_COLS", "384"))
TILE_T_COL_BLOCK = int(os.environ.get("BPT_TILE_T_COL_BLOCK", "128"))
MAX_BLOCK_SMEM = 227 * 1024  # shared memory one thread block can have on this GPU


def _check_inputs(plan, q, k, v, embed_ak):
    """Shape, dtype and device rules shared by every entry of the fused call, checked before any path
    is chosen: q (n_nodes, h, d); k, v (n_src, h, d) of q's dtype; embed_ak (>= n_etypes, d) of q's dtype
    (the kernels read it as q's element type and index it with every edge type of the plan)."""
    _lib.require_cuda(q, k, v)
    if q.dim() != 3:
        raise RuntimeError("bpt_attention: q must be (n_nodes, h, d)")
    N, h, d = q.shape
    if N != plan.n_nodes or k.shape != (plan.n_src, h, d) or v.shape != k.shape:
        raise RuntimeError("bpt_attention: q must be (n_nodes, h, d) and k, v (n_src, h, d)")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise RuntimeError("bpt_attention: q, k and v must have one dtype")
    if embed_ak is not None:
        _lib.require_cuda(embed_ak)
        if (embed_ak.dim() != 2 or embed_ak.dtype != q.dtype or embed_ak.size(0) < plan.n_etypes
                or embed_ak.size(1) != d):
            raise RuntimeError("bpt_attention: embed_ak must be (>= n_etypes = %d, d = %d) of the dtype of q (%s); "
                               "got %s of %s" % (plan.n_etypes, d, q.dtype, tuple(embed_ak.shape), embed_ak.dtype))
    return N, h, d


def tensor_core_eligible(q, embed_ak, plan=None):
    """bf16 with head dim 64; and, when the plan is given, a tile plan whose per-head tables fit
    in shared memory (graphs with many hundreds of edge types stay on the CUDA-core kernels)."""
    if not (q.dtype == torch.bfloat16 and q.size(-1) == 64):
        return False
    if plan is None:
        return True
    tp = plan.tile_plan()
    need = _lib.lib().bpt_attn_tc_smem_bytes(tp.max_cols_pad, tp.t_max if embed_ak is not None else 0, tp.et_bytes)
    return 0 < need <= MAX_BLOCK_SMEM


def attention_forward_tc(plan, q, k, v, embed_ak, scale, dropout=None):
    """Forward through bpt_attn_forward_tc (bf16, head dim 64). Returns (o, lse)."""
    N, h, d = _check_inputs(plan, q, k, v, embed_ak)
    drop_keep, drop_ptr = _lib.dropout_arg(dropout)
    tp = plan.tile_plan()
    o = torch.empty_like(q)
    lse = torch.empty((N, h), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        ws = tp.workspace(h, q.device)
        _lib.check(_lib.lib().bpt_attn_forward_tc(
            tp.groups.data_ptr(), tp.n_groups, tp.mblocks.data_ptr(), tp.cols.data_ptr(), tp.et.data_ptr(),
            tp.et_bytes, tp.split.data_ptr(), tp.n_split, tp.n_slots, tp.items.data_ptr(), tp.n_row_items,
            plan.blob.data_ptr(), ctypes.addressof(plan._counts), plan.n_nodes, plan.n_edges, tp.max_cols_pad,
            tp.t_max, tp.max_mblocks, tp.max_qr_slots, tp.n_etypes, q.data_ptr(), k.data_ptr(), v.data_ptr(),
            _lib.ptr(embed_ak), float(scale), o.data_ptr(), lse.data_ptr(), h, d, _lib.dtype_code(q.dtype),
            ws.data_ptr(), ws.numel(), drop_ptr, _lib.stream()))
    return o, lse


def tc32_eligible(q, embed_ak, plan):
    """fp32 with head dim 64 and a tile plan that the 3xTF32 tile kernel takes: no CUDA-core row items and
    tables that fit in shared memory."""
    if not (q.dtype == torch.float32 and q.size(-1) == 64):
        return False
    tp = plan.tile_plan()
    if tp.n_row_items:
        return False
    need = _lib.lib().bpt_attn_forward_tc32_smem_bytes(tp.max_cols_pad, tp.t_max if embed_ak is not None else 0,
                                                       tp.et_bytes)
    return 0 < need <= MAX_BLOCK_SMEM


def attention_forward_tc32(plan, q, k, v, embed_ak, scale, dropout=None):
    """fp32 forward through bpt_attn_forward_tc32 (tile plan, every product as three TF32 products; within
    the fp32 tolerance of the CUDA-core kernel).  Returns (o, lse)."""
    N, h, d = _check_inputs(plan, q, k, v, embed_ak)
    drop_keep, drop_ptr = _lib.dropout_arg(dropout)
    tp = plan.tile_plan()
    o = torch.empty_like(q)
    lse = torch.empty((N, h), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        ws = tp.workspace(h, q.device)
        s = tp.struct()
        _lib.check(_lib.lib().bpt_attn_forward_tc32(
            ctypes.addressof(s), N, tp.n_etypes, q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr(embed_ak),
            float(scale), o.data_ptr(), lse.data_ptr(), h, d, ws.data_ptr(), ws.numel(), drop_ptr, _lib.stream()))
    return o, lse


def tc5_eligible(q, embed_ak, plan):
    """bf16, head dim 64, 8-bit cells (at most 248 edge types) and a 128-row tile plan that fits in
    shared memory: the tcgen05 forward applies."""
    if not (q.dtype == torch.bfloat16 and q.size(-1) == 64):
        return False
    tp = plan.tile_plan5()
    if tp.et_bytes != 1 or (embed_ak is not None and tp.t_max > 248):
        return False
    need = _lib.lib().bpt_attn_forward_tc5_smem_bytes(tp.max_cols_pad, tp.t_max if embed_ak is not None else 0)
    return 0 < need <= MAX_BLOCK_SMEM


def attention_forward_tc5(plan, q, k, v, embed_ak, scale):
    """Forward through bpt_attn_forward_tc5 (tcgen05.mma, accumulators in tensor memory). Returns (o, lse)."""
    N, h, d = _check_inputs(plan, q, k, v, embed_ak)
    tp = plan.tile_plan5()
    o = torch.empty_like(q)
    lse = torch.empty((N, h), dtype=torch.float32, device=q.device)
    L = _lib.lib()
    with torch.cuda.device(q.device):
        ws = tp._ws.get(("tc5", h))
        if ws is None:
            ws = _lib.workspace(L.bpt_attn_forward_tc5_workspace_bytes(tp.n_slots, h), q.device)
            ws[:16].zero_()  # the status word
            tp._ws[("tc5", h)] = ws
        tiles = tp.struct()
        _lib.check(L.bpt_attn_forward_tc5(ctypes.addressof(tiles), plan.n_nodes, plan.n_etypes, q.data_ptr(),
                                          k.data_ptr(), v.data_ptr(), _lib.ptr(embed_ak), float(scale), o.data_ptr(),
                                          lse.data_ptr(), h, d, _lib.dtype_code(q.dtype), ws.data_ptr(), ws.numel(),
                                          _lib.stream()))
    return o, lse


def tc5_status(plan, h):
    """0 when every bounded wait of the tcgen05 forward calls on this plan completed (waits for the stream)."""
    tp = plan.tiles5
    ws = None if tp is None else tp._ws.get(("tc5", h))
    if ws is None:
        return 0
    out = ctypes.c_int32(0)
    with torch.cuda.device(ws.device):
        _lib.check(_lib.lib().bpt_attn_forward_tc5_status(ws.data_ptr(), ctypes.addressof(out), _lib.stream()))
    return int(out.value)


# Which tensor-core forward bf16 / head-dim-64 calls take: "tc5" (tcgen05, 128-row tiles) where it
# applies, else "tile" (mma.sync, 16-row tiles).
FORWARD_IMPL = os.environ.get("BPT_FORWARD_IMPL", "tile")


def attention_forward(plan, q, k, v, embed_ak, scale, tensor_cores=None, dropout=None):
    """Returns (o, lse). q, k, v: (N, h, d) contiguous CUDA tensors of one dtype.
    bf16 with head dim 64 runs on the tensor-core kernel unless tensor_cores=False.
    dropout: None or (rate, seed) -- dropout on the attention weights (modules/attention.py:73); the same
    pair must be given to attention_backward."""
    N, h, d = _check_inputs(plan, q, k, v, embed_ak)
    if tensor_cores is None:
        tensor_cores = tensor_core_eligible(q, embed_ak, plan) or (FP32_FORWARD == "tc32" and
                                                                   tc32_eligible(q, embed_ak, plan))
    drop_keep, drop_ptr = _lib.dropout_arg(dropout)
    if tensor_cores:
        if q.dtype == torch.float32:
            return attention_forward_tc32(plan, q, k, v, embed_ak, scale, dropout)
        if FORWARD_IMPL == "tc5" and drop_ptr is None and tc5_eligible(q, embed_ak, plan):
            return attention_forward_tc5(plan, q, k, v, embed_ak, scale)
        return attention_forward_tc(plan, q, k, v, embed_ak, scale, dropout)
    o = torch.empty_like(q)
    lse = torch.empty((N, h), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        ws = plan.workspace(h, d, False)
        _lib.check(_lib.lib().bpt_attn_forward(*plan._args(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                               _lib.ptr(embed_ak), float(scale), o.data_ptr(), lse.data_ptr(),
                                               h, d, _lib.dtype_code(q.dtype), ws.data_ptr(), ws.numel(),
                                               drop_ptr, _lib.stream()))
    return o, lse


def attention_forward_static(plan, q, k, v, embed_ak, scale, out=None, lse_out=None):
    """attention_forward through bpt_attn_forward_static: the library call itself allocates no
    device memory (its scratch is an 8 MiB array built into the library).  For callers that
    pre-allocate everything, pass `out` (like q) and `lse_out` (fp32 (N, h)) so that this
    wrapper allocates nothing either.  Graphs whose split rows need more scratch than the
    built-in array raise; use attention_forward for those.  Calls on one GPU share that array
    and must not overlap in time."""
    N, h, d = _check_inputs(plan, q, k, v, embed_ak)
    o = torch.empty_like(q) if out is None else out
    lse = torch.empty((N, h), dtype=torch.float32, device=q.device) if lse_out is None else lse_out
    _lib.require_cuda(o, lse)
    # caller-supplied outputs go to the library as raw pointers: a wrong shape or dtype would be an
    # out-of-bounds device write
    if o.shape != q.shape or o.dtype != q.dtype or o.device != q.device:
        raise RuntimeError("bpt_attention: out must have the shape, dtype and device of q")
    if lse.shape != (N, h) or lse.dtype != torch.float32 or lse.device != q.device:
        raise RuntimeError("bpt_attention: lse_out must be float32 (n_nodes, h) on the device of q")
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().bpt_attn_forward_static(*plan._args(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                      _lib.ptr(embed_ak), float(scale), o.data_ptr(),
                                                      lse.data_ptr(), h, d, _lib.dtype_code(q.dtype),
                                                      _lib.stream()))
    return o, lse


def attention_backward(plan, q, k, v, embed_ak, scale, lse, d_o, o=None, tensor_cores=None, dropout=None, out=None):
    """Returns (dq, dk, dv, d_embed_ak or None); d_embed_ak is fp32 (rows of embed_ak, d).
    bf16 with head dim 64 runs on the tensor-core kernels when the forward's output `o` is given
    (they take delta = <dO, O> from it) unless tensor_cores=False.  out: optional (dq, dk, dv) tensors of the
    shapes and dtype of q, k, v (contiguous, on their device) that receive the gradients instead of new ones."""
    d_o = d_o.contiguous()
    N, h, d = _check_inputs(plan, q, k, v, embed_ak)
    _lib.require_cuda(lse, d_o)
    if d_o.shape != q.shape or d_o.dtype != q.dtype:
        raise RuntimeError("bpt_attention: d_o must have the shape and dtype of q")
    if lse.shape != (N, h) or lse.dtype != torch.float32:
        raise RuntimeError("bpt_attention: lse must be float32 (n_nodes, h)")
    tile32 = tensor_cores is not False and o is not None and FP32_BACKWARD == "tc32" and \
        tc32_eligible(q, embed_ak, plan) and plan.tile_plan().cellpos is not None
    if tensor_cores is None:
        tensor_cores = o is not None and tensor_core_eligible(q, embed_ak, plan)
    if out is None:
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    else:
        dq, dk, dv = out
        for name, t, like in (("dq", dq, q), ("dk", dk, k), ("dv", dv, v)):
            if t.shape != like.shape or t.dtype != like.dtype or t.device != like.device or not t.is_contiguous():
                raise RuntimeError("bpt_attention: out[%s] must be a contiguous tensor of the shape, dtype and device "
                                   "of its input" % name)
    drop_keep, drop_ptr = _lib.dropout_arg(dropout)
    dak = None
    if embed_ak is not None:
        dak = torch.zeros((embed_ak.size(0), d), dtype=torch.float32, device=q.device)
    L = _lib.lib()
    if tile32:
        _lib.require_cuda(o)
        tiles = plan.tile_plan().struct()
        src_tiles = plan.tile_plan_t().struct() if FP32_BACKWARD_SOURCE_SIDE == "tc32" else None
        src_ptr = None if src_tiles is None else ctypes.addressof(src_tiles)
        with torch.cuda.device(q.device):
            ws = plan._ws.get(("tc32_bwd", h))
            if ws is None:
                ws = _lib.workspace(L.bpt_attn_backward_tc32_workspace_bytes(
                    ctypes.addressof(tiles), src_ptr, ctypes.addressof(plan._counts), plan.n_nodes, plan.n_edges, h),
                    q.device)
                plan._ws[("tc32_bwd", h)] = ws
            _lib.check(L.bpt_attn_backward_tc32(
                ctypes.addressof(tiles), src_ptr, *plan._args(), q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr(embed_ak),
                float(scale), o.data_ptr(), lse.data_ptr(), d_o.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                dv.data_ptr(), _lib.ptr(dak), h, d, ws.data_ptr(), ws.numel(), drop_ptr, _lib.stream()))
        return dq, dk, dv, dak
    with torch.cuda.device(q.device):
        if tensor_cores:
            if o is None:
                raise RuntimeError("bpt_attention: the tensor-core backward needs the forward's output o")
            _lib.require_cuda(o)
            dst_tiles, src_tiles = plan.tile_plan().struct(), plan.tile_plan_t().struct()
            ws = plan._ws.get(("tc_bwd", h))
            if ws is None:
                ws = _lib.workspace(L.bpt_attn_backward_tc_workspace_bytes(
                    ctypes.addressof(dst_tiles), ctypes.addressof(src_tiles), ctypes.addressof(plan._counts),
                    plan.n_nodes, plan.n_edges, h), q.device)
                plan._ws[("tc_bwd", h)] = ws
            _lib.check(L.bpt_attn_backward_tc(
                ctypes.addressof(dst_tiles), ctypes.addressof(src_tiles), *plan._args(), q.data_ptr(), k.data_ptr(),
                v.data_ptr(), _lib.ptr(embed_ak), float(scale), o.data_ptr(), lse.data_ptr(), d_o.data_ptr(),
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _lib.ptr(dak), h, d, _lib.dtype_code(q.dtype),
                ws.data_ptr(), ws.numel(), drop_ptr, _lib.stream()))
        else:
            ws = plan.workspace(h, d, True)
            _lib.check(L.bpt_attn_backward(*plan._args(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                           _lib.ptr(embed_ak), float(scale), lse.data_ptr(), d_o.data_ptr(),
                                           dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), _lib.ptr(dak), h, d,
                                           _lib.dtype_code(q.dtype), ws.data_ptr(), ws.numel(), drop_ptr,
                                           _lib.stream()))
    return dq, dk, dv, dak


class _BPTAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, plan, q, k, v, embed_ak, scale, dropout):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        if embed_ak is not None:
            embed_ak = embed_ak.contiguous()
        o, lse = attention_forward(plan, q, k, v, embed_ak, scale, dropout=dropout)
        ctx.plan, ctx.scale, ctx.dropout = plan, scale, dropout
        ctx.has_ak = embed_ak is not None
        ctx.save_for_backward(q, k, v, embed_ak if ctx.has_ak else q.new_empty(0), lse, o)
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, ak, lse, o = ctx.saved_tensors
        ak = ak if ctx.has_ak else None
        dq, dk, dv, dak = attention_backward(ctx.plan, q, k, v, ak, ctx.scale, lse, d_o, o=o, dropout=ctx.dropout)
        return None, dq, dk, dv, (dak.to(ak.dtype) if dak is not None else None), None, None


def bpt_attention(plan, q, k, v, embed_ak=None, scale=None, dropout_p=0.0, seed=None):
    """o[i,h] = sum over i's incoming edges e of drop(softmax_e(scale * <q[i,h], k[src_e,h] +
    embed_ak[etype_e]>)) * v[src_e,h].  scale defaults to 1/sqrt(d) (modules/attention.py:73).
    dropout_p > 0 zeroes each attention weight with that probability and scales the rest by
    1 / (1 - dropout_p), as the reference's drop_att does between sparse_softmax and vec_spmm; the mask
    is regenerated in the backward from `seed` (drawn from torch's generator when not given)."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.size(-1))
    dropout = None
    if dropout_p:
        if seed is None:
            seed = int(torch.randint(0, 2 ** 62, (1,)).item())
        dropout = (float(dropout_p), int(seed))
    return _BPTAttention.apply(plan, q, k, v, embed_ak, scale, dropout)


def dropout_mask(plan_src, plan_dst, h, dropout_p, seed):
    """The (E, h) bool mask (True = kept) that bpt_attention(..., dropout_p, seed) applies, for edges given by
    their int32 source and destination ids in edge-id order."""
    src, dst = plan_src.to(torch.int32).contiguous(), plan_dst.to(torch.int32).contiguous()
    _lib.require_cuda(src, dst)
    out = torch.empty((src.numel(), h), dtype=torch.uint8, device=src.device)
    keep, ptr_ = _lib.dropout_arg((dropout_p, seed))
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().bpt_attn_dropout_mask(src.data_ptr(), dst.data_ptr(), src.numel(), h, ptr_,
                                                    out.data_ptr(), _lib.stream()))
    return out.bool()
