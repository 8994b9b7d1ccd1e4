"""The reference's unchanged modules/op.py + modules/attention.py (from the mounted checkout, and from
the copies compiled into oracle/_ref/ by oracle/build_ref_graphop.py) running on a CPU stand-in for
`graphop` made of the oracle's operator restatement.  Checks, without a GPU, the scaffolding of the
drop-in test (stub `dgl`, dict-framed graph, `from graphop import *` resolved to a module of our
choosing) and that BPTBlock.forward (modules/attention.py:54-81) equals the oracle's chain plus the
block's own layers."""
import os
import types

import numpy as np
import pytest
import torch

import build_ref_graphop
import ops_torch

REF_ROOT = os.environ.get("BPT_REFERENCE_ROOT", "/root/reference")


def _cpu_graphop():
    """A `graphop`-shaped module on ops_torch: forwards as they are, backwards through autograd."""
    m = types.ModuleType("graphop")

    def grads(fn, tensors, dy):
        with torch.enable_grad():  # called from inside autograd.Function.backward, where grad mode is off
            leaves = [t.detach().clone().requires_grad_(True) for t in tensors]
            return list(torch.autograd.grad(fn(*leaves), leaves, dy))

    m.maskedmm_csr_forward = lambda row, indptr, eid, indices, A, B: ops_torch.maskedmm_csr(row, indptr, eid, indices, A, B)
    m.maskedmm_csr_backward = lambda row, ip_r, eid_r, idx_r, col, ip_c, eid_c, idx_c, A, B, dy: grads(
        lambda a, b: ops_torch.maskedmm_csr(row, ip_r, eid_r, idx_r, a, b), (A, B), dy)
    m.node_mul_edge_forward = lambda row, indptr, eid, A, B: ops_torch.node_mul_edge(row, indptr, eid, A, B)
    m.node_mul_edge_backward = lambda row, indptr, eid, A, B, dy: grads(
        lambda a, b: ops_torch.node_mul_edge(row, indptr, eid, a, b), (A, B), dy)
    m.sparse_softmax_forward = lambda row, indptr, eid, x: ops_torch.sparse_softmax(row, indptr, eid, x)
    # dx = y * (dy - sum_row(y * dy))  (graphop_kernel.cu:208-230)
    m.sparse_softmax_backward = lambda row, indptr, eid, y, dy: y * dy - y * _row_sum_at_edges(row, indptr, eid, y * dy)
    m.vector_spmm_forward = lambda row, indptr, eid, indices, edata, x: ops_torch.vector_spmm(row, indptr, eid, indices, edata, x)
    m.vector_spmm_backward = lambda row, indptr, eid, indices, col, ip_t, eid_t, idx_t, edata, dy, x: grads(
        lambda w, xx: ops_torch.vector_spmm(row, indptr, eid, indices, w, xx), (edata, x), dy)
    return m


def _row_sum_at_edges(row, indptr, eid, val):
    """sum of val over each CSR row, broadcast back to the row's edges (indexed by edge id)."""
    r = ops_torch._expand_rows(row, indptr)
    sums = torch.zeros((int(r.max()) + 1,) + tuple(val.shape[1:]), dtype=val.dtype).index_add(0, r, val[eid])
    return torch.zeros_like(val).index_copy(0, eid, sums[r])


@pytest.mark.parametrize("source", ["checkout", "compiled"])
def test_reference_block_forward_equals_oracle_chain(oracle_lib, source):
    root = REF_ROOT if source == "checkout" else None
    if source == "checkout" and not os.path.isfile(os.path.join(REF_ROOT, "modules", "attention.py")):
        pytest.skip("reference checkout not mounted")
    if source == "compiled" and build_ref_graphop.modules_so_paths() is None:
        pytest.skip("compiled reference modules absent (python oracle/build_ref_graphop.py)")
    stand_in = _cpu_graphop()
    op_mod, att_mod = build_ref_graphop.load_modules(stand_in, root)[:2]
    assert op_mod.maskedmm_csr_forward is stand_in.maskedmm_csr_forward
    g = oracle_lib.batch_graphs([oracle_lib.binary_partition(40, False, 2, 10), oracle_lib.binary_partition(33, True, 3, 4)])
    N = g["n_nodes"]
    csr_np = oracle_lib.get_csrs(g["src"], g["dst"], N)
    f = torch.from_numpy
    csr = ([f(a) for a in csr_np[0]], [f(a) for a in csr_np[1]], f(csr_np[2]), f(csr_np[3]), f(csr_np[4]), f(csr_np[5]))
    torch.manual_seed(0)
    dim, h = 32, 4
    blk = att_mod.BPTBlock(dim, h, 64, rel_pos=True, drop_h=0.0, drop_a=0.0).double()
    blk.reset_parameters()
    etype = f(g["etype"])
    h0 = torch.randn(N, dim, dtype=torch.float64, requires_grad=True)
    graph = build_ref_graphop.FakeGraph(ndata={"h": h0}, edata={"etype": etype})
    blk(graph, csr)
    out = graph.ndata["h"]
    # the same arithmetic spelled with the oracle's chain
    q, k, v = [p(h0).view(-1, h, dim // h) for p in (blk.proj_q, blk.proj_k, blk.proj_v)]
    a = ops_torch.attention_chain(csr, etype, q, k, v, blk.embed_ak.weight, dim // h).reshape(N, dim)
    hh = blk.norm_in(h0 + blk.proj_o(a))
    want = blk.norm_inter(hh + blk.ffn(hh))
    assert torch.allclose(out, want, rtol=1e-10, atol=1e-12)
    # and the reference's autograd shim (modules/op.py:10-58) yields the chain's gradients
    w_loss = torch.randn(N, dim, dtype=torch.float64)  # (a sum of squares of a LayerNorm output has zero gradient)
    g1 = torch.autograd.grad((out * w_loss).sum(), [h0] + list(blk.parameters()), retain_graph=True)
    g2 = torch.autograd.grad((want * w_loss).sum(), [h0] + list(blk.parameters()))
    for x, y in zip(g1, g2):
        assert torch.allclose(x, y, rtol=1e-8, atol=1e-10)
    assert np.isfinite(out.detach().numpy()).all()


@pytest.mark.parametrize("source", ["checkout", "compiled"])
def test_reference_language_model_forward_equals_blocks_spelled_out(oracle_lib, source):
    """modules/model.py:197-280 (BinaryPartitionTransformer, rel_pos=True, dim_embed == dim_model) on the CPU
    stand-in: the graph object's `g.nodes[ids].data[key]` read / assignment behaves like a DGL frame (rows
    never assigned are zero), and the model equals embedding -> norm -> its blocks (each spelled with the
    oracle's chain) -> generator on the leaves."""
    root = REF_ROOT if source == "checkout" else None
    if source == "checkout" and not os.path.isfile(os.path.join(REF_ROOT, "modules", "model.py")):
        pytest.skip("reference checkout not mounted")
    if source == "compiled" and build_ref_graphop.modules_so_paths() is None:
        pytest.skip("compiled reference modules absent (python oracle/build_ref_graphop.py)")
    mods = build_ref_graphop.load_modules(_cpu_graphop(), root)
    model_mod = mods[3]
    g = oracle_lib.batch_graphs([oracle_lib.binary_partition(40, True, 2, 10), oracle_lib.binary_partition(21, True, 3, 4)])
    N = g["n_nodes"]
    csr_np = oracle_lib.get_csrs(g["src"], g["dst"], N)
    f = torch.from_numpy
    csr = ([f(a) for a in csr_np[0]], [f(a) for a in csr_np[1]], f(csr_np[2]), f(csr_np[3]), f(csr_np[4]), f(csr_np[5]))
    torch.manual_seed(0)
    vocab, dim, heads, layers = 17, 32, 4, 2
    lm = model_mod.make_model(vocab, dim, dim, 64, heads, vocab, layers, dropouti=0.0, dropouth=0.0, dropouta=0.0,
                              dropoutc=0.0, rel_pos=True).double()
    # leaves are the first n nodes of every sequence (graph_builder/builder.pyx:29-62)
    n0 = oracle_lib.binary_partition(40, True, 2, 10)["n_nodes"]
    leaf_ids = torch.cat([torch.arange(0, 40), torch.arange(n0, n0 + 21)])
    tokens = torch.randint(0, vocab, (leaf_ids.numel(),))
    x = torch.zeros(N, dtype=torch.long)
    x[leaf_ids] = tokens
    etype = f(g["etype"])
    graph = build_ref_graphop.FakeGraph(ndata={"x": x}, edata={"etype": etype}, n_nodes=N)
    batch = types.SimpleNamespace(g=graph, leaf_ids=leaf_ids, g_csr=csr, readout_ids=leaf_ids)
    out = lm(batch)
    h = torch.zeros(N, dim, dtype=torch.float64)
    h = h.index_put((leaf_ids,), lm.norm(lm.embed(tokens)))
    for blk in lm.layers:
        q, k, v = [p(h).view(-1, heads, dim // heads) for p in (blk.proj_q, blk.proj_k, blk.proj_v)]
        a = ops_torch.attention_chain(csr, etype, q, k, v, blk.embed_ak.weight, dim // heads).reshape(N, dim)
        hh = blk.norm_in(h + blk.proj_o(a))
        h = blk.norm_inter(hh + blk.ffn(hh))
    want = lm.generator(h[leaf_ids])
    assert out.shape == (leaf_ids.numel(), vocab)
    assert torch.allclose(out, want, rtol=1e-9, atol=1e-11)
    w_loss = torch.randn_like(out)
    g1 = torch.autograd.grad((out * w_loss).sum(), list(lm.parameters()), retain_graph=True, allow_unused=True)
    g2 = torch.autograd.grad((want * w_loss).sum(), list(lm.parameters()), allow_unused=True)
    for a_, b_ in zip(g1, g2):
        assert (a_ is None) == (b_ is None)
        if a_ is not None:
            assert torch.allclose(a_, b_, rtol=1e-7, atol=1e-9)
