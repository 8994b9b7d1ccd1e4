"""The C oracle against the golden vectors made from the reference's own builder, and
against the compiled reference itself when oracle/_ref/ is present."""
import numpy as np
import pytest

from helpers import digest


def test_oracle_matches_golden_digests(oracle_lib, golden):
    for rec in golden["cases"]:
        g = oracle_lib.binary_partition(rec["length"], rec["triu"], rec["step"], rec["clip_dist"])
        key = (rec["length"], rec["triu"], rec["step"], rec["clip_dist"])
        assert g["n_nodes"] == rec["n_nodes"], key
        assert g["n_edges"] == rec["n_edges"], key
        assert g["n_levels"] == rec["n_levels"], key
        assert digest(g["src"], g["dst"], g["etype"], g["pos"]) == rec["sha256"], key
        if "arrays" in rec:
            for name in ("src", "dst", "etype", "pos"):
                assert g[name].tolist() == rec["arrays"][name], (key, name)


def test_oracle_partition_csr_matches_golden(oracle_lib, golden):
    for rec in golden["partition_csr"]:
        row, ip = oracle_lib.partition_csr(np.array(rec["indptr"], np.int64), rec["chunk_size"])
        assert row.tolist() == rec["row"]
        assert ip.tolist() == rec["indptr_out"]


def test_oracle_matches_compiled_reference(oracle_lib):
    import build_ref
    ref = build_ref.load()
    if ref is None:
        pytest.skip("oracle/_ref not built (reference checkout absent)")
    rng = np.random.default_rng(11)
    for _ in range(150):
        n = int(rng.integers(1, 700))
        step = int(rng.choice([1, 2, 3, 4, 5, 8, 16, 64]))
        triu = bool(rng.integers(0, 2))
        clip = int(rng.choice([0, 1, 3, 6, 10, 30]))
        g = ref.BinaryPartition(n, triu, step, clip)
        s, d, t = g.get_edges(3)
        o = oracle_lib.binary_partition(n, triu, step, clip)
        assert np.array_equal(s, o["src"] + 3) and np.array_equal(d, o["dst"] + 3)
        assert np.array_equal(t, o["etype"]) and np.array_equal(g.get_pos(), o["pos"])
        assert g.number_of_nodes == o["n_nodes"] and g.number_of_levels == o["n_levels"]


def test_known_structure(oracle_lib):
    """Facts about the graph that follow from builder.pyx:64-116: power-of-two lengths give
    2n-1 nodes; every span node receives one edge from each leaf it covers, all of one type."""
    g = oracle_lib.binary_partition(512, False, 4, 10)
    assert g["n_nodes"] == 1023 and g["n_levels"] == 10 and g["n_edges"] == 28378
    g = oracle_lib.binary_partition(8192, False, 4, 10)
    assert g["n_nodes"] == 16383 and g["n_edges"] == 745786 and int(g["etype"].max()) == 98
    span = g["dst"] >= 8192
    assert int(span.sum()) == 13 * 8192
    assert oracle_lib.binary_partition(8192, True, 4, 10)["n_edges"] == 430237


def test_csr_order_and_chunks(oracle_lib):
    g = oracle_lib.binary_partition(37, False, 2, 10)
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = oracle_lib.get_csrs(g["src"], g["dst"], g["n_nodes"])
    for (indptr, indices, eid), key, other in ((out_csr, g["src"], g["dst"]), (in_csr, g["dst"], g["src"])):
        assert indptr[-1] == g["n_edges"]
        for r in range(g["n_nodes"]):
            seg = eid[indptr[r]:indptr[r + 1]]
            assert np.all(np.diff(seg) > 0)
            assert np.all(key[seg] == r)
            assert np.array_equal(indices[indptr[r]:indptr[r + 1]], other[seg])
    assert np.all(np.diff(INDPTR_C) <= 32) and np.all(np.diff(INDPTR_C) > 0)
    assert np.all(np.diff(COL) >= 0)


def test_oracle_baseline_graphs_match_golden(oracle_lib, golden):
    """FullyConnected / OpenAISparse (graph_builder/builder.pyx:154-303) against digests made
    from the compiled reference."""
    for r in golden["baselines"]:
        g = oracle_lib.fully_connected(r["length"], r["triu"], r["window"]) if r["kind"] == "fc" else \
            oracle_lib.openai_sparse(r["length"], r["stride"], r["c"])
        assert g["n_edges"] == r["n_edges"], r
        assert digest(g["src"], g["dst"], g["etype"], g["pos"]) == r["sha256"], r
