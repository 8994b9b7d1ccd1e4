"""The device tile planner (bpt_tile_plan_create_device) against the host planner (bpt_tile_plan_create,
pure integer host code): every exported array and every size must be identical, for the forward and the
transposed plans, on binary-partition batches (incl. duplicate edges and a 3000-edge root row), dense
cross-attention blocks with empty rows, the parameter sets the kernels use (16-row groups; 128-row groups
with eight m-blocks), parameters that force rows into column buckets with several group copies, and a graph
with more than 255 edge types (16-bit cells)."""
import numpy as np
import pytest
import torch

from helpers import fully_connected_blocks
from test_fused_gpu import GRAPHS

pytestmark = pytest.mark.gpu

PARAMS = {
    "forward16": dict(min_density=0.25, max_cols=384, group_rows=16, col_block=128, max_mblocks=1),
    "source16": dict(min_density=0.15, max_cols=384, group_rows=16, col_block=128, max_mblocks=1),
    "rows128": dict(min_density=0.05, max_cols=512, group_rows=128, col_block=128, max_mblocks=8),
    "buckets": dict(min_density=0.6, max_cols=64, group_rows=32, col_block=48, max_mblocks=2),
}
FIELDS = ("n_groups", "n_mblocks", "n_cells", "n_split", "n_slots", "t_max", "max_cols_pad", "max_mblocks",
          "max_qr_slots", "n_dense_groups", "et_bytes", "n_cols")


def _plan(src, dst, etype, N, T, n_src=None):
    from bpt_b200.attention import AttentionPlan
    dev = "cuda"
    return AttentionPlan(torch.from_numpy(src).to(dev), torch.from_numpy(dst).to(dev),
                         None if etype is None else torch.from_numpy(etype).to(dev), N, n_etypes=T, n_src=n_src)


def _compare(plan, transposed, params):
    from bpt_b200.attention import TilePlan
    host = TilePlan(plan, transposed=transposed, planner="host", **params)
    dev = TilePlan(plan, transposed=transposed, planner="device", **params)
    assert dev.planner == "device" and host.planner == "host"
    for f in FIELDS:
        assert getattr(dev, f) == getattr(host, f), (f, getattr(dev, f), getattr(host, f))
    used = dict(groups=host.n_groups * 8, mblocks=host.n_mblocks * 56, cols=host.n_cols, cellpos=host.n_cells,
                split=host.n_split * 4, et=None if transposed else host.n_cells * host.et_bytes)
    for name, n in used.items():
        a, b = getattr(dev, name), getattr(host, name)
        if a is None or b is None:
            assert a is None and b is None, name
            continue
        a, b = a.cpu().numpy().ravel(), b.cpu().numpy().ravel()
        if n is not None:
            a, b = a[:n], b[:n]
        assert a.shape == b.shape, (name, a.shape, b.shape)
        if not np.array_equal(a, b):
            bad = np.flatnonzero(a != b)
            raise AssertionError("%s differs at %d of %d entries, first at %d: device %s host %s" % (
                name, bad.size, a.size, bad[0], a[bad[:8]], b[bad[:8]]))


@pytest.mark.parametrize("graph", list(GRAPHS))
@pytest.mark.parametrize("params", list(PARAMS))
@pytest.mark.parametrize("transposed", [False, True])
def test_device_planner_equals_host_planner(oracle_lib, graph, params, transposed):
    g = GRAPHS[graph](oracle_lib)
    plan = _plan(g["src"], g["dst"], g["etype"], g["n_nodes"], int(g["etype"].max()) + 1)
    _compare(plan, transposed, PARAMS[params])


@pytest.mark.parametrize("params", ["forward16", "rows128", "buckets"])
def test_device_planner_cross_attention_blocks_and_empty_rows(params):
    src, dst, n0 = fully_connected_blocks(5, 30)
    plan = _plan(src, dst, None, n0 + 7, 1)
    _compare(plan, False, PARAMS[params])
    _compare(plan, True, PARAMS[params])


def test_device_planner_many_edge_types_and_no_edges(oracle_lib):
    g = oracle_lib.binary_partition(700, False, 64, 10)  # > 255 edge types: 16-bit cells
    T = int(g["etype"].max()) + 1
    assert T > 255
    plan = _plan(g["src"], g["dst"], g["etype"], g["n_nodes"], T)
    _compare(plan, False, PARAMS["forward16"])
    _compare(plan, True, PARAMS["source16"])
    empty = _plan(np.zeros(0, np.int64), np.zeros(0, np.int64), np.zeros(0, np.int64), 40, 1)
    _compare(empty, False, PARAMS["forward16"])
    _compare(empty, True, PARAMS["rows128"])


def test_device_planner_headline_graph_and_attention_result(oracle_lib):
    """Two sequences of the headline size: identical plans, and the tensor-core forward and backward give
    bitwise the same result on either."""
    from bpt_b200 import attention as A
    g = oracle_lib.batch_graphs([oracle_lib.binary_partition(8192, False, 4, 10)] * 2)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    plan = _plan(g["src"], g["dst"], g["etype"], N, T)
    _compare(plan, False, PARAMS["forward16"])
    _compare(plan, True, PARAMS["source16"])
    gen = torch.Generator().manual_seed(5)
    q, k, v, d_o = [(torch.randn(N, 8, 64, generator=gen) * 0.125).to(torch.bfloat16).cuda() for _ in range(4)]
    ak = (torch.randn(T, 64, generator=gen) * 0.125).to(torch.bfloat16).cuda()
    outs = []
    for planner in ("host", "device"):
        p = _plan(g["src"], g["dst"], g["etype"], N, T)
        p.tiles = A.TilePlan(p, planner=planner)
        p.tiles_t = A.TilePlan(p, transposed=True, min_density=0.15, planner=planner)
        o, lse = A.attention_forward_tc(p, q, k, v, ak, 0.125)
        grads = A.attention_backward(p, q, k, v, ak, 0.125, lse, d_o, o=o, tensor_cores=True)
        outs.append((o, lse) + tuple(grads))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def _batch_with_offsets(oracle_lib, specs):
    parts = [oracle_lib.binary_partition(*s) for s in specs]
    g = oracle_lib.batch_graphs(parts)
    offsets = np.concatenate([[0], np.cumsum([p["n_nodes"] for p in parts])]).tolist()
    return g, offsets


@pytest.mark.parametrize("params", ["forward16", "rows128", "buckets"])
@pytest.mark.parametrize("transposed", [False, True])
def test_device_planner_equals_host_planner_with_column_segments(oracle_lib, params, transposed):
    """Column blocks counted from each graph's first node (the graphs of a block-diagonal batch)."""
    from bpt_b200.attention import TilePlan
    g, offsets = _batch_with_offsets(oracle_lib, [(513, False, 4, 10), (100, True, 2, 3), (2048, False, 4, 10), (37, False, 1, 2)])
    plan = _plan(g["src"], g["dst"], g["etype"], g["n_nodes"], int(g["etype"].max()) + 1)
    host = TilePlan(plan, transposed=transposed, planner="host", col_segments=offsets, **PARAMS[params])
    dev = TilePlan(plan, transposed=transposed, planner="device", col_segments=offsets, **PARAMS[params])
    for f in FIELDS:
        assert getattr(dev, f) == getattr(host, f), (f, getattr(dev, f), getattr(host, f))
    for name, n in dict(groups=host.n_groups * 8, mblocks=host.n_mblocks * 56, cols=host.n_cols, cellpos=host.n_cells,
                        split=host.n_split * 4).items():
        a, b = getattr(dev, name).cpu().numpy().ravel()[:n], getattr(host, name).cpu().numpy().ravel()[:n]
        assert np.array_equal(a, b), name
    cols = dev.cols.cpu().numpy()[:dev.n_cols]
    assert cols.min() >= 0 and cols.max() < g["n_nodes"]


def test_column_segments_keep_a_batch_cut_like_its_graphs_and_the_result(oracle_lib):
    """Two sequences of the headline size: with the graphs' offsets the forward plan spreads as many rows over
    several tiles as two single-sequence plans do (63 each); attention results match the unaligned plan's at the
    dtype's tolerance and the oracle's (fp32)."""
    from bpt_b200 import attention as A
    from helpers import rel_err
    g, offsets = _batch_with_offsets(oracle_lib, [(8192, False, 4, 10)] * 2)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    plain = _plan(g["src"], g["dst"], g["etype"], N, T)
    aligned = _plan(g["src"], g["dst"], g["etype"], N, T)
    aligned.segments = offsets
    assert plain.tile_plan().n_split > 4 * 63
    assert aligned.tile_plan().n_split <= 2 * 63 + 16
    gen = torch.Generator().manual_seed(9)
    q, k, v, d_o = [(torch.randn(N, 8, 64, generator=gen) * 0.125) for _ in range(4)]
    ak = torch.randn(T, 64, generator=gen) * 0.125
    for dtype, tol in ((torch.bfloat16, 2e-2), (torch.float32, 1e-5)):
        args = [t.to(dtype).cuda() for t in (q, k, v, ak)]
        outs = []
        for p in (plain, aligned):
            o, lse = A.attention_forward(p, args[0], args[1], args[2], args[3], 0.125)
            grads = A.attention_backward(p, args[0], args[1], args[2], args[3], 0.125, lse, d_o.to(dtype).cuda(), o=o)
            outs.append((o, lse) + tuple(grads))
        for a, b in zip(*outs):
            assert rel_err(a.float().cpu(), b.float().cpu()) < tol
