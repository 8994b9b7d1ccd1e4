"""The host-side tile planner of the tensor-core path: every edge lands in exactly one tile
cell, rows marked complete really are, and split rows' slots are contiguous. Runs without a GPU."""
import ctypes

import numpy as np
import pytest


def _plan(oracle_lib, g, min_density=0.25, max_cols=384, col_block=64, simt_max_degree=8):
    from bpt_b200 import _lib, build
    build.build()
    L = _lib.lib()
    indptr, src, eid = oracle_lib.coo_to_csr(g["dst"], g["src"], g["n_nodes"])
    et = g["etype"][eid]
    ip32, s32, e32 = indptr.astype(np.int32), src.astype(np.int32), et.astype(np.int32)
    h = L.bpt_tile_plan_create(ip32.ctypes.data, s32.ctypes.data, e32.ctypes.data, g["n_nodes"], len(src),
                               min_density, max_cols, col_block, simt_max_degree)
    assert h
    sizes = (ctypes.c_int64 * 10)()
    assert L.bpt_tile_plan_sizes(h, ctypes.addressof(sizes)) == 0
    n_tiles, n_cols, n_et, n_split, n_slots, t_max, mcp, n_row_tiles, n_items, _ = [int(x) for x in sizes]
    tiles = np.empty(n_tiles * 40, np.int32)
    cols = np.empty(max(n_cols, 1), np.int32)
    etm = np.empty(max(n_et, 1), np.uint16)
    split = np.empty(max(n_split * 4, 1), np.int32)
    items = np.empty(max(n_items * 4, 1), np.int32)
    assert L.bpt_tile_plan_export(h, tiles.ctypes.data, cols.ctypes.data, etm.ctypes.data, split.ctypes.data,
                                  items.ctypes.data) == 0
    L.bpt_tile_plan_destroy(h)
    return dict(tiles=tiles.reshape(n_tiles, 40), cols=cols, et=etm, split=split[:n_split * 4].reshape(n_split, 4),
                items=items[:n_items * 4].reshape(n_items, 4), n_slots=n_slots, t_max=t_max, mcp=mcp, n_row_tiles=n_row_tiles, csr=(indptr, src, et))


@pytest.mark.parametrize("spec", [[(512, False, 4, 10)], [(513, False, 4, 10), (100, True, 2, 3), (1, False, 1, 10)],
                                  [(3000, True, 8, 6)], [(37, False, 1, 0)]])
def test_tiles_cover_every_edge_once(oracle_lib, spec):
    g = oracle_lib.batch_graphs([oracle_lib.binary_partition(*s) for s in spec])
    p = _plan(oracle_lib, g)
    indptr, src, et = p["csr"]
    N = g["n_nodes"]
    got = []          # (row, src, etype) per cell
    rows_seen = np.zeros(N, np.int64)
    complete = np.zeros(N, bool)
    slots = {}
    for t in p["tiles"]:
        rows, slot, ncp, coff, eoff, tq, ncols = t[0:16], t[16:32], t[32], t[33], t[34], t[35], t[36]
        assert ncp % 64 == 0 and ncols <= ncp <= p["mcp"] and tq % 8 == 0 and tq <= p["t_max"]
        cols = p["cols"][coff:coff + ncp]
        m = p["et"][eoff:eoff + 16 * ncp].reshape(16, ncp)
        assert np.all(m[:, ncols:] == 0xFFFF)
        for i in range(16):
            if rows[i] < 0:
                assert np.all(m[i] == 0xFFFF)
                continue
            rows_seen[rows[i]] += 1
            cs = np.nonzero(m[i] != 0xFFFF)[0]
            assert np.all(m[i][cs] < max(tq, 1))
            got += [(int(rows[i]), int(cols[c]), int(m[i][c])) for c in cs]
            if slot[i] < 0:
                assert not complete[rows[i]]
                complete[rows[i]] = True
                assert len(cs) == indptr[rows[i] + 1] - indptr[rows[i]]
            else:
                slots.setdefault(int(rows[i]), []).append(int(slot[i]))
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
    all_slots = sorted(s for v in slots.values() for s in v)
    assert all_slots == list(range(p["n_slots"]))
    assert len(p["split"]) == len(slots)
    for row, first, count, _ in p["split"]:
        assert sorted(slots[int(row)]) == list(range(first, first + count))


def test_leaf_blocks_become_row_tiles(oracle_lib):
    g = oracle_lib.binary_partition(8192, False, 4, 10)
    p = _plan(oracle_lib, g)
    assert p["n_row_tiles"] >= 512           # the 512 blocks of 16 leaves
    leaf_tiles = [t for t in p["tiles"] if 0 <= t[0] < 8192 and t[15] < 8192 and t[15] >= 0]
    ncols = np.array([t[36] for t in leaf_tiles[:512]])
    assert ncols.max() <= 192 and 100 < ncols.mean() < 140
