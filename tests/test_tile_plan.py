"""The host-side tile planner of the tensor-core path: every edge lands in exactly one cell of
one m-block, rows marked complete really are, split rows' slots are contiguous, and span rows
of binary-partition graphs join the leaf group that stages their sources. Runs without a GPU."""
import ctypes

import numpy as np
import pytest


def _cell_pos_index(r, c):
    """Place of cell (r, c) of a 16 x 64 chunk in the exported payload array (tile_plan.cuh)."""
    return (((c // 32) * 4 + (c % 32) // 8) * 32 + (r % 8) * 4 + (c % 8) // 2) * 4 + (r // 8) * 2 + (c & 1)


FRAG_ORDER = np.array([_cell_pos_index(r, c) for r in range(16) for c in range(64)])
assert len(set(FRAG_ORDER.tolist())) == 1024


def _plan(oracle_lib, g, min_density=0.05, max_cols=384, group_rows=64, col_block=64, simt_max_degree=0, et_bytes=2,
          max_mblocks=8, join_dense=1):
    from bpt_b200 import _lib, build
    build.build()
    L = _lib.lib()
    indptr, src, eid = oracle_lib.coo_to_csr(g["dst"], g["src"], g["n_nodes"])
    et = g["etype"][eid]
    ip32, s32, e32 = indptr.astype(np.int32), src.astype(np.int32), et.astype(np.int32)
    h = L.bpt_tile_plan_create(ip32.ctypes.data, s32.ctypes.data, e32.ctypes.data, None, g["n_nodes"], len(src),
                               min_density, max_cols, group_rows, col_block, simt_max_degree, max_mblocks,
                               join_dense)
    assert h
    sizes = (ctypes.c_int64 * 12)()
    assert L.bpt_tile_plan_sizes(h, ctypes.addressof(sizes)) == 0
    (n_groups, n_mb, n_cols, n_cells, n_split, n_slots, t_max, mcp, max_mb, max_qr, n_items, n_dense) = \
        [int(x) for x in sizes]
    groups = np.empty(max(n_groups * 8, 1), np.int32)
    mblocks = np.empty(max(n_mb * 56, 1), np.int32)
    cols = np.empty(max(n_cols, 1), np.int32)
    etm = np.empty(max(n_cells, 1), np.uint8 if et_bytes == 1 else np.uint16)
    cellpos = np.empty(max(n_cells, 1), np.int32)
    split = np.empty(max(n_split * 4, 1), np.int32)
    items = np.empty(max(n_items * 4, 1), np.int32)
    assert L.bpt_tile_plan_export(h, groups.ctypes.data, mblocks.ctypes.data, cols.ctypes.data, etm.ctypes.data,
                                  et_bytes, cellpos.ctypes.data, split.ctypes.data, items.ctypes.data) == 0
    L.bpt_tile_plan_destroy(h)
    return dict(groups=groups[:n_groups * 8].reshape(n_groups, 8), mblocks=mblocks[:n_mb * 56].reshape(n_mb, 56),
                cols=cols, et=etm, cellpos=cellpos, split=split[:n_split * 4].reshape(n_split, 4),
                items=items[:n_items * 4].reshape(n_items, 4), n_slots=n_slots, t_max=t_max, mcp=mcp,
                max_mb=max_mb, max_qr=max_qr, n_dense=n_dense, csr=(indptr, src, et))


@pytest.mark.parametrize("spec,kw", [
    ([(512, False, 4, 10)], {}),
    ([(513, False, 4, 10), (100, True, 2, 3), (1, False, 1, 10)], {}),
    ([(3000, True, 8, 6)], {"et_bytes": 1}),
    ([(37, False, 1, 0)], {"simt_max_degree": 4}),
    ([(700, False, 4, 10)], {"group_rows": 32, "col_block": 32}),
    ([(2000, False, 4, 10)], {"group_rows": 128, "col_block": 128, "max_mblocks": 8, "join_dense": 0, "max_cols": 512}),
])
def test_plan_covers_every_edge_once(oracle_lib, spec, kw):
    g = oracle_lib.batch_graphs([oracle_lib.binary_partition(*s) for s in spec])
    p = _plan(oracle_lib, g, **kw)
    none = 0xFF if kw.get("et_bytes") == 1 else 0xFFFF
    indptr, src, et = p["csr"]
    N = g["n_nodes"]
    got = []
    rows_seen = np.zeros(N, np.int64)
    complete = np.zeros(N, bool)
    slots = {}
    uniform = np.array([len(set(et[indptr[r]:indptr[r + 1]])) <= 1 for r in range(N)])
    mb_seen = 0
    for grp in p["groups"]:
        coff, ncp, mb_first, mb_count, ncols = grp[:5]
        assert ncp % 64 == 0 and ncols <= ncp <= p["mcp"] and 1 <= mb_count <= min(kw.get("max_mblocks", 8), p["max_mb"])
        assert mb_first == mb_seen          # m-blocks of a group are contiguous, groups in order
        mb_seen += mb_count
        cols = p["cols"][coff:coff + ncp]
        assert np.all(np.diff(cols[:ncols]) >= 0)
        n_qr = 0
        for m in p["mblocks"][mb_first:mb_first + mb_count]:
            rows, slot, row_et, eoff, mask, tq, qr = m[0:16], m[16:32], m[32:48], m[48], m[49], m[50], m[51]
            cells = p["et"][eoff:eoff + 16 * ncp].reshape(ncp // 64, 16, 64)
            # positions are exported per chunk in mma-fragment order: undo it
            cpos = p["cellpos"][eoff:eoff + 16 * ncp].reshape(ncp // 64, 1024)[:, FRAG_ORDER].reshape(ncp // 64, 16, 64)
            assert np.array_equal(cpos >= 0, cells != none)
            valid = rows[rows >= 0]
            assert np.all(np.diff(valid) > 0)
            if qr >= 0:
                assert qr == n_qr and tq <= p["t_max"] and not all(uniform[valid])
                n_qr += 1
            else:
                assert all(uniform[valid])
            for st in range(ncp // 32):     # one activity bit per 32 columns
                assert bool((int(mask) >> st) & 1) == bool(np.any(cells[st // 2][:, 32 * (st % 2):32 * (st % 2) + 32] != none))
            for i in range(16):
                row_cells = cells[:, i, :].reshape(-1)
                if rows[i] < 0:
                    assert np.all(row_cells == none)
                    continue
                rows_seen[rows[i]] += 1
                cs = np.nonzero(row_cells != none)[0]
                assert np.all(cs < ncols)
                got += [(int(rows[i]), int(cols[c]), int(row_cells[c])) for c in cs]
                row_pos = cpos[:, i, :].reshape(-1)[cs]
                assert np.all((row_pos >= indptr[rows[i]]) & (row_pos < indptr[rows[i] + 1]))
                assert np.array_equal(src[row_pos], cols[cs]) and np.array_equal(et[row_pos], row_cells[cs])
                if qr < 0 and len(cs):
                    assert np.all(row_cells[cs] == row_et[i])
                if slot[i] < 0:
                    assert not complete[rows[i]]
                    complete[rows[i]] = True
                    assert len(cs) == indptr[rows[i] + 1] - indptr[rows[i]]
                else:
                    slots.setdefault(int(rows[i]), []).append(int(slot[i]))
        assert n_qr <= p["max_qr"]
    assert mb_seen == len(p["mblocks"])
    for row, beg, end, slot in p["items"]:      # short rows handed to the CUDA-core kernel, whole
        assert slot == -1 and beg == indptr[row] and end == indptr[row + 1] and not complete[row]
        complete[row] = True
        rows_seen[row] += 1
        got += [(int(row), int(src[j]), int(et[j])) for j in range(beg, end)]
    want = sorted((int(r), int(src[j]), int(et[j])) for r in range(N) for j in range(indptr[r], indptr[r + 1]))
    assert sorted(got) == want
    assert np.all(rows_seen >= 1)                       # rows without edges are covered too
    assert not any(complete[r] for r in slots)          # a row is either complete or split
    assert np.all(complete | np.isin(np.arange(N), list(slots)))
    assert sorted(s for v in slots.values() for s in v) == list(range(p["n_slots"]))
    assert len(p["split"]) == len(slots)
    for row, first, count, _ in p["split"]:
        assert slots[int(row)] == list(range(first, first + count))   # in m-block order


def test_leaf_blocks_become_dense_groups(oracle_lib):
    """Production parameters on the headline graph: 128 consecutive leaves share one group of 8
    m-blocks; span rows are grouped by the 128 leaves they cover; only leaf m-blocks need the
    relative-position table (span rows have a single edge type each)."""
    g = oracle_lib.binary_partition(8192, False, 4, 10)
    p = _plan(oracle_lib, g, min_density=0.04, max_cols=512, group_rows=128, col_block=128, max_mblocks=8, join_dense=0)
    assert p["n_dense"] == 64
    leaf_groups = p["groups"][:64]
    assert np.all(leaf_groups[:, 3] == 8)
    assert 330 < leaf_groups[:, 4].mean() < 420 and leaf_groups[:, 1].max() <= 512
    assert p["max_qr"] == 8 and p["max_mb"] == 8
    span_groups = p["groups"][64:]
    assert np.all(span_groups[:, 4] <= 128)
    qr = p["mblocks"][:, 51]
    first_span_mb = span_groups[0][2]
    assert np.all(qr[first_span_mb:] == -1)
