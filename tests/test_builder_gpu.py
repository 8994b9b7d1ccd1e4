"""GPU graph construction through the C ABI: bit-exact with the oracle and the golden
digests of the reference's builder."""
import pickle

import numpy as np
import pytest
import torch

from helpers import digest

pytestmark = pytest.mark.gpu


def _gb():
    from bpt_b200 import graphbuilder
    return graphbuilder


def test_gpu_builder_matches_golden_digests(golden):
    gb = _gb()
    for rec in golden["cases"]:
        g = gb.BinaryPartition(rec["length"], rec["triu"], rec["step"], rec["clip_dist"])
        key = (rec["length"], rec["triu"], rec["step"], rec["clip_dist"])
        assert g.number_of_nodes == rec["n_nodes"], key
        assert g.number_of_edges == rec["n_edges"], key
        assert g.number_of_levels == rec["n_levels"], key
        s, d, t = g.get_edges()
        assert s.dtype == np.int64
        assert digest(s, d, t, g.get_pos()) == rec["sha256"], key


def test_gpu_builder_matches_oracle_random(oracle_lib):
    gb = _gb()
    rng = np.random.default_rng(5)
    for _ in range(120):
        n = int(rng.integers(1, 3000))
        step = int(rng.choice([1, 2, 3, 4, 5, 8, 16, 64]))
        triu = bool(rng.integers(0, 2))
        clip = int(rng.choice([0, 1, 3, 6, 10, 30]))
        v_shift = int(rng.integers(0, 1000))
        g = gb.BinaryPartition(n, triu, step, clip)
        o = oracle_lib.binary_partition(n, triu, step, clip)
        s, d, t = g.get_edges(v_shift)
        assert np.array_equal(s, o["src"] + v_shift) and np.array_equal(d, o["dst"] + v_shift)
        assert np.array_equal(t, o["etype"]) and np.array_equal(g.get_pos(), o["pos"])
        assert np.array_equal(g.leaf_ids(v_shift), np.arange(v_shift, v_shift + n))
        assert g.root_id(v_shift) == v_shift + o["n_nodes"] - 1
        assert [g.number_of_nodes_at_lvl(i) for i in range(g.number_of_levels)] == o["n_nodes_arr"].tolist()
        assert len(g.internal_ids()) == o["n_nodes"] - n


def test_accessors_and_pickle():
    gb = _gb()
    g = gb.BinaryPartition(100, True, 2, 5)
    assert g.is_triu
    g2 = pickle.loads(pickle.dumps(g))
    for a, b in zip(g.get_edges(), g2.get_edges()):
        assert np.array_equal(a, b)
    with pytest.raises(ValueError):
        gb.BinaryPartition(0)


def test_partition_csr_matches_golden_and_oracle(golden, oracle_lib):
    gb = _gb()
    for rec in golden["partition_csr"]:
        row, ip = gb.partition_csr(np.array(rec["indptr"], np.int64), rec["chunk_size"])
        assert row.tolist() == rec["row"] and ip.tolist() == rec["indptr_out"]
    # empty rows only, and a device-resident call
    row, ip = gb.partition_csr(np.zeros(5, np.int64))
    assert row.size == 0 and ip.tolist() == [0]
    indptr = torch.tensor([0, 70, 70, 71, 200], device="cuda")
    row, ip = gb.partition_csr(indptr, 32)
    r2, p2 = oracle_lib.partition_csr(indptr.cpu().numpy(), 32)
    assert row.is_cuda and row.cpu().numpy().tolist() == r2.tolist() and ip.cpu().numpy().tolist() == p2.tolist()


def test_get_csrs_and_batching_match_oracle(oracle_lib):
    from bpt_b200 import csr
    gb = _gb()
    specs = [(513, False, 4, 10), (37, False, 2, 3), (513, False, 4, 10), (5, False, 1, 10), (1, False, 4, 10)]
    cache = {}
    graphs = []
    for sp in specs:
        if sp not in cache:
            cache[sp] = gb.BinaryPartition(*sp)
        graphs.append(cache[sp])
    batch = csr.batch_graphs(graphs, dtype=torch.int64)
    ob = oracle_lib.batch_graphs([oracle_lib.binary_partition(*sp) for sp in specs])
    assert batch.n_nodes == ob["n_nodes"] and batch.n_edges == ob["n_edges"]
    for mine, ref in ((batch.src, ob["src"]), (batch.dst, ob["dst"]), (batch.etype, ob["etype"]),
                      (batch.pos, ob["pos"])):
        assert np.array_equal(mine.cpu().numpy(), ref)
    # n=513 with triu=False has duplicate (src, dst) pairs: the CSR must keep them apart
    got = csr.get_csrs(batch.src, batch.dst, batch.n_nodes)
    want = oracle_lib.get_csrs(ob["src"], ob["dst"], ob["n_nodes"])
    for i in range(2):
        for j in range(3):
            assert got[i][j].dtype == torch.int64
            assert np.array_equal(got[i][j].cpu().numpy(), want[i][j]), (i, j)
    for j in range(2, 6):
        assert np.array_equal(got[j].cpu().numpy(), want[j]), j
    # int32 flavour used by the fused path
    ip, idx, eid = csr.coo_to_csr(batch.dst.int(), batch.src.int(), batch.n_nodes)
    assert ip.dtype == torch.int32 and np.array_equal(idx.cpu().numpy(), want[1][1])


def test_large_graph_digest(golden):
    """n = 65536, k = 8: 13.2 M edges, the largest size the sweep uses."""
    gb = _gb()
    rec = [r for r in golden["cases"] if r["length"] == 65536 and r["step"] == 8][0]
    g = gb.BinaryPartition(65536, False, 8, 10)
    assert g.number_of_edges == rec["n_edges"] == 13239926
    s, d, t = g.get_edges()
    assert digest(s, d, t, g.get_pos()) == rec["sha256"]


def test_baseline_graphs_match_golden_and_oracle(golden, oracle_lib):
    """FullyConnected / OpenAISparse on the GPU: golden digests of the reference's builder, then
    seeded parameter sweeps against the oracle, with v_shift and pickling."""
    gb = _gb()
    for r in golden["baselines"]:
        g = gb.FullyConnected(r["length"], r["triu"], r["window"]) if r["kind"] == "fc" else \
            gb.OpenAISparse(r["length"], r["stride"], r["c"])
        s, d, t = g.get_edges()
        assert g.number_of_edges == r["n_edges"] and g.number_of_nodes == r["length"] + 1, r
        assert digest(s, d, t, g.get_pos()) == r["sha256"], r
    rng = np.random.default_rng(9)
    for _ in range(40):
        n, w, triu = int(rng.integers(1, 400)), int(rng.integers(0, 500)), bool(rng.integers(0, 2))
        g, o = gb.FullyConnected(n, triu, w), oracle_lib.fully_connected(n, triu, w)
        s, d, t = g.get_edges(5)
        assert np.array_equal(s, o["src"] + 5) and np.array_equal(d, o["dst"] + 5) and np.array_equal(t, o["etype"])
        assert np.array_equal(g.get_pos(), o["pos"]) and g.root_id(5) == n + 5
        n, stride, c = int(rng.integers(1, 600)), int(rng.integers(1, 40)), int(rng.integers(0, 50))
        g, o = gb.OpenAISparse(n, stride, c), oracle_lib.openai_sparse(n, stride, c)
        s, d, t = g.get_edges()
        assert np.array_equal(s, o["src"]) and np.array_equal(d, o["dst"]) and np.array_equal(t, o["etype"])
        assert np.array_equal(g.get_pos(), o["pos"]) and g.is_triu
    g2 = pickle.loads(pickle.dumps(gb.OpenAISparse(50, 8, 3)))
    assert g2.number_of_edges == oracle_lib.openai_sparse(50, 8, 3)["n_edges"]
    with pytest.raises(AssertionError):
        gb.OpenAISparse(10, 4, 2, triu=False)


def test_fused_attention_on_baseline_graph(oracle_lib):
    """The dense baseline graph through the fused path (fp32 CUDA cores, bf16 tensor cores)."""
    import torch
    from bpt_b200.attention import AttentionPlan, attention_forward
    gb = _gb()
    g = gb.FullyConnected(150, True, 64)
    s, d, t = g.get_edges()
    N, T = g.number_of_nodes, int(t.max()) + 1
    csr = oracle_lib.get_csrs(s, d, N)
    gen = torch.Generator().manual_seed(0)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        q, k, v = [(torch.randn(N, 8, 64, generator=gen) * 0.125).to(dtype) for _ in range(3)]
        ak = (torch.randn(T, 64, generator=gen) * 0.125).to(dtype)
        want, _, _ = oracle_lib.attn_fwd(csr[1], t, q.float().numpy(), k.float().numpy(), v.float().numpy(),
                                         ak.float().numpy(), 0.125)
        src, dst, et = g.edges_device()
        plan = AttentionPlan(src, dst, et, N, n_etypes=T)
        o, _ = attention_forward(plan, q.cuda(), k.cuda(), v.cuda(), ak.cuda(), 0.125)
        err = np.abs(o.double().cpu().numpy() - want).max() / np.abs(want).max()
        assert err < tol, (dtype, err)


def test_inter_graph_matches_reference_formula(oracle_lib):
    """Dense sentence-aligned blocks (graph/mt.py:318-321): edge order and ids, int32 and int64,
    with an empty block in the middle and no blocks at all."""
    from bpt_b200 import csr as csrmod
    src_ranges = [(0, 5), (9, 0), (20, 3), (100, 17)]
    dst_ranges = [(3, 4), (7, 6), (40, 1), (41, 9)]
    want = oracle_lib.inter_graph(src_ranges, dst_ranges)
    for dtype in (torch.int32, torch.int64):
        got = csrmod.inter_graph(src_ranges, dst_ranges, dtype=dtype)
        assert got[0].dtype == dtype and np.array_equal(got[0].cpu().numpy(), want[0])
        assert np.array_equal(got[1].cpu().numpy(), want[1])
    empty = csrmod.inter_graph([], [])
    assert empty[0].numel() == 0 and empty[1].numel() == 0
