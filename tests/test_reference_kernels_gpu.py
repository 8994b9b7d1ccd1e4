"""This library's operators and fused call against the reference's OWN CUDA kernels
(graph_kernel/graphop.cpp + graphop_kernel.cu, compiled unmodified by oracle/build_ref_graphop.py),
and the reference's unchanged attention block (modules/op.py + modules/attention.py) running on
this library's `graphop` through bpt_b200.install_dropin().

Same inputs to both sides, fp32, small cases.  Tolerance 1e-5 max-norm relative (the reference's
sums go through atomics, so its results move in the last bits from run to run; they stay far
inside that bar), 1e-4 for softmax gradients as graph_kernel/test.py:239 relaxes them.  The fp64
restatement (oracle/ops_torch.py) is compared with the reference kernels too, which pins the
oracle's floating-point half to reference outputs.  Skipped when the compiled reference is absent.
"""
import math
import os
import sys

import numpy as np
import pytest
import torch

import build_ref_graphop
import ops_torch
from helpers import fully_connected_blocks, rel_err

pytestmark = pytest.mark.gpu

REF_ROOT = os.environ.get("BPT_REFERENCE_ROOT", "/root/reference")


@pytest.fixture(scope="module")
def ref_graphop():
    mod = build_ref_graphop.load_graphop()
    if mod is None:
        pytest.skip("the reference's graphop is not built (python oracle/build_ref_graphop.py)")
    return mod


def _graph(oracle_lib, kind):
    """cfg1: 4 x BinaryPartition(512, bidirectional, k = 4); dense: graph_kernel/test.py:79-82's
    512 fully connected blocks of 30 nodes."""
    if kind == "cfg1":
        g = oracle_lib.batch_graphs([oracle_lib.binary_partition(512, False, 4, 10) for _ in range(4)])
        src, dst, N, etype = g["src"], g["dst"], g["n_nodes"], g["etype"]
    else:
        src, dst, N = fully_connected_blocks(512, 30)
        etype = (np.arange(len(src)) % 61).astype(np.int64)
    return src, dst, N, etype


def _csrs(src, dst, N):
    from bpt_b200 import csr as csrmod
    return csrmod.get_csrs(torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda(), N)


@pytest.mark.parametrize("kind", ["cfg1", "dense"])
def test_eight_operators_match_reference_kernels(oracle_lib, ref_graphop, kind):
    from bpt_b200 import graphop
    src, dst, N, _ = _graph(oracle_lib, kind)
    E, h, d = len(src), 8, 64
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = _csrs(src, dst, N)
    gen = torch.Generator().manual_seed(0)
    rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=gen) * s).cuda()
    A, B = rnd(N, h, d, s=0.3), rnd(N, h, d, s=0.3)
    dy_e, dy_n = rnd(E, h), rnd(N, h, d)
    Bed = rnd(E, d, s=0.3)
    x_e, w_e = rnd(E, h, s=2.0), rnd(E, h, s=0.2)
    cpu = lambda t: t.detach().cpu()

    # maskedmm_csr over the out-CSR, A = k, B = q (modules/attention.py:66-67)
    y_ref = ref_graphop.maskedmm_csr_forward(ROW, INDPTR_R, out_csr[2], out_csr[1], A, B)
    y = graphop.maskedmm_csr_forward(ROW, INDPTR_R, out_csr[2], out_csr[1], A, B)
    assert rel_err(cpu(y), cpu(y_ref)) < 1e-5
    c = [t.cpu() for t in (ROW, INDPTR_R, out_csr[2], out_csr[1])]
    assert rel_err(ops_torch.maskedmm_csr(*c, A.double().cpu(), B.double().cpu()), cpu(y_ref)) < 1e-5
    g_ref = ref_graphop.maskedmm_csr_backward(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2],
                                              in_csr[1], A, B, dy_e)
    g = graphop.maskedmm_csr_backward(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2], in_csr[1],
                                      A, B, dy_e)
    for a, b in zip(g, g_ref):
        assert rel_err(cpu(a), cpu(b)) < 1e-5

    # node_mul_edge over the in-CSR (attention.py:69-71)
    y_ref = ref_graphop.node_mul_edge_forward(COL, INDPTR_C, in_csr[2], A, Bed)
    y = graphop.node_mul_edge_forward(COL, INDPTR_C, in_csr[2], A, Bed)
    assert rel_err(cpu(y), cpu(y_ref)) < 1e-5
    g_ref = ref_graphop.node_mul_edge_backward(COL, INDPTR_C, in_csr[2], A, Bed, dy_e)
    g = graphop.node_mul_edge_backward(COL, INDPTR_C, in_csr[2], A, Bed, dy_e)
    for a, b in zip(g, g_ref):
        assert rel_err(cpu(a), cpu(b)) < 1e-5

    # sparse_softmax over the in-CSR and the out-CSR (test.py:395,422 check both)
    for rw, ip, ed in ((COL, INDPTR_C, in_csr[2]), (ROW, INDPTR_R, out_csr[2])):
        y_ref = ref_graphop.sparse_softmax_forward(rw, ip, ed, x_e)
        y = graphop.sparse_softmax_forward(rw, ip, ed, x_e)
        assert rel_err(cpu(y), cpu(y_ref)) < 1e-5
        y64 = ops_torch.sparse_softmax(rw.cpu(), ip.cpu(), ed.cpu(), x_e.double().cpu(), n_rows=N)
        assert rel_err(y64, cpu(y_ref)) < 1e-5
        dx_ref = ref_graphop.sparse_softmax_backward(rw, ip, ed, y_ref, dy_e)
        dx = graphop.sparse_softmax_backward(rw, ip, ed, y_ref, dy_e)
        assert rel_err(cpu(dx), cpu(dx_ref)) < 1e-4

    # vector_spmm over the in-CSR with the out-CSR as its transpose (attention.py:74-77)
    y_ref = ref_graphop.vector_spmm_forward(COL, INDPTR_C, in_csr[2], in_csr[1], w_e, A)
    y = graphop.vector_spmm_forward(COL, INDPTR_C, in_csr[2], in_csr[1], w_e, A)
    assert rel_err(cpu(y), cpu(y_ref)) < 1e-5
    c = [t.cpu() for t in (COL, INDPTR_C, in_csr[2], in_csr[1])]
    assert rel_err(ops_torch.vector_spmm(*c, w_e.double().cpu(), A.double().cpu()), cpu(y_ref)) < 1e-5
    g_ref = ref_graphop.vector_spmm_backward(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2],
                                             out_csr[1], w_e, dy_n, A)
    g = graphop.vector_spmm_backward(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2], out_csr[1],
                                     w_e, dy_n, A)
    for a, b in zip(g, g_ref):
        assert rel_err(cpu(a), cpu(b)) < 1e-5


def _layer_through(op_mod, csr, etype, q, k, v, table, d_o):
    """The chain of modules/attention.py:56-77 (dropout off) on the given op module; returns the
    output and the gradients of q, k, v and the embed_ak table."""
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = csr
    q, k, v, table = [t.detach().clone().requires_grad_(True) for t in (q, k, v, table)]
    ak = torch.nn.functional.embedding(etype, table)
    e = op_mod.masked_mm(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2], in_csr[1], k, q)
    e_rel = op_mod.node_mul_edge(COL, INDPTR_C, in_csr[2], q, ak)
    p = op_mod.sparse_softmax(COL, INDPTR_C, in_csr[2], (e_rel + e) / np.sqrt(q.size(-1)))
    o = op_mod.vec_spmm(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2], out_csr[1], p, v)
    o.backward(d_o)
    return [o.detach(), q.grad, k.grad, v.grad, table.grad]


@pytest.mark.parametrize("kind", ["cfg1", "dense"])
def test_chained_layer_and_fused_call_match_reference_kernels(oracle_lib, ref_graphop, kind):
    """Values and gradients of the whole attention layer: the reference's kernels under the
    reference's own autograd shim (modules/op.py), against (a) this library's operators under
    the same shim and (b) the fused call, fp32 and (fused only) bf16."""
    import bpt_b200
    from bpt_b200.attention import AttentionPlan, bpt_attention
    mods = build_ref_graphop.load_modules(ref_graphop, REF_ROOT)
    if mods is None:
        pytest.skip("the reference's modules/op.py is neither mounted nor compiled")
    ref_op = mods[0]
    ours_op = build_ref_graphop.load_modules(bpt_b200.install_dropin()[0], REF_ROOT)[0]
    src, dst, N, etype = _graph(oracle_lib, kind)
    h, d, T = 8, 64, int(etype.max()) + 1
    csr = _csrs(src, dst, N)
    gen = torch.Generator().manual_seed(0)
    sigma = 1.0 / math.sqrt(64)
    q, k, v = [(torch.randn(N, h, d, generator=gen) * sigma).cuda() for _ in range(3)]
    table = (torch.randn(T, d, generator=gen) * sigma).cuda()
    d_o = torch.randn(N, h, d, generator=gen).cuda()
    et = torch.from_numpy(etype).cuda()
    want = _layer_through(ref_op, csr, et, q, k, v, table, d_o)
    got = _layer_through(ours_op, csr, et, q, k, v, table, d_o)
    for a, b in zip(got, want):
        assert rel_err(a.cpu(), b.cpu()) < 1e-5
    plan = AttentionPlan(torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda(), et, N, n_etypes=T)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        if dtype == torch.bfloat16:
            # the reference kernels have no bf16; feed them the rounded inputs in fp32
            qr, kr, vr, tr, dor = [t.to(dtype).float() for t in (q, k, v, table, d_o)]
            want_d = _layer_through(ref_op, csr, et, qr, kr, vr, tr, dor)
        else:
            want_d = want
        qq, kk, vv, tt = [t.to(dtype).detach().clone().requires_grad_(True) for t in (q, k, v, table)]
        o = bpt_attention(plan, qq, kk, vv, tt, 1.0 / math.sqrt(d))
        o.backward(d_o.to(dtype))
        for a, b in zip([o.detach(), qq.grad, kk.grad, vv.grad, tt.grad], want_d):
            assert rel_err(a.float().cpu(), b.cpu()) < tol


@pytest.mark.parametrize("binding", ["extension", "ctypes"])
def test_reference_block_runs_unchanged_on_this_library(oracle_lib, ref_graphop, binding):
    """modules/attention.py:54-81 -- the reference's BPTBlock.forward(g, csr), its file unchanged --
    with `graphop` resolved to this library (bpt_b200.install_dropin: the torch C++ extension or the
    ctypes module), against the same block on the reference's own kernels and against the re-hosted
    bpt_b200.model.BPTBlock with the same weights."""
    import bpt_b200
    import bpt_b200.graphop
    from bpt_b200 import csr as csrmod, graphbuilder
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTBlock
    installed = bpt_b200.install_dropin(binding)[0]
    assert sys.modules["graphop"] is installed
    assert installed is (bpt_b200.graphop_extension() if binding == "extension" else bpt_b200.graphop)
    ours = build_ref_graphop.load_modules(installed, REF_ROOT)
    theirs = build_ref_graphop.load_modules(ref_graphop, REF_ROOT)
    if ours is None:
        pytest.skip("the reference's modules/attention.py is neither mounted nor compiled")
    # the module objects really are bound to different graphop implementations
    assert ours[0].sparse_softmax_forward is installed.sparse_softmax_forward
    assert theirs[0].sparse_softmax_forward is ref_graphop.sparse_softmax_forward
    torch.manual_seed(0)
    graphs = [graphbuilder.BinaryPartition(n, False, 4, 10) for n in (512, 300, 513)]
    batch = csrmod.batch_graphs(graphs)
    csr = csrmod.get_csrs(batch.src, batch.dst, batch.n_nodes)
    dim, heads, ff = 512, 8, 1024
    blk_ours = ours[1].BPTBlock(dim, heads, ff, rel_pos=True, drop_h=0.0, drop_a=0.0).cuda()
    blk_ours.reset_parameters()
    blk_theirs = theirs[1].BPTBlock(dim, heads, ff, rel_pos=True, drop_h=0.0, drop_a=0.0).cuda()
    blk_theirs.load_state_dict(blk_ours.state_dict())
    mine = BPTBlock(dim, heads, ff, rel_pos=True, drop_h=0.0).cuda()
    mine.load_state_dict(blk_ours.state_dict())       # the reference block's state dict loads as it is
    h0 = torch.randn(batch.n_nodes, dim, device="cuda")
    # loss = <output, fixed random tensor> (a sum of squares of a LayerNorm output is constant: zero gradient)
    w_loss = torch.randn(batch.n_nodes, dim, device="cuda")
    outs, grads = [], []
    for blk in (blk_ours, blk_theirs):
        g = build_ref_graphop.FakeGraph(ndata={"h": h0.clone().requires_grad_(True)},
                                        edata={"etype": batch.etype.long()})
        h_in = g.ndata["h"]
        blk(g, csr)
        (g.ndata["h"] * w_loss).sum().backward()
        outs.append(g.ndata["h"].detach())
        grads.append([h_in.grad] + [p.grad for p in blk.parameters()])
    assert rel_err(outs[0].cpu(), outs[1].cpu()) < 1e-5
    for a, b in zip(grads[0], grads[1]):
        assert rel_err(a.cpu(), b.cpu()) < 1e-4
    plan = AttentionPlan.from_batch(batch, n_etypes=1000)
    h_in = h0.clone().requires_grad_(True)
    out = mine(h_in, plan)
    (out * w_loss).sum().backward()
    assert rel_err(out.detach().cpu(), outs[1].cpu()) < 1e-5
    for a, b in zip([h_in.grad] + [p.grad for p in mine.parameters()], grads[1]):
        assert rel_err(a.cpu(), b.cpu()) < 1e-4
    assert "graphop" in sys.modules and sys.modules["graphop"] is installed


@pytest.mark.parametrize("ours_on", ["reference_kernels", "this_library"])
def test_reference_language_model_equals_rehosted_model(oracle_lib, ref_graphop, ours_on):
    """modules/model.py:197-280 -- the reference's BinaryPartitionTransformer, its file unchanged (rel_pos=True,
    dim_embed == dim_model, dropouts 0: the character-LM configuration) -- run over a causal batch with a graph
    object that has dict node/edge frames, against bpt_b200.model.BPTLanguageModel loaded from the reference
    model's state dict (strict).  ours_on=reference_kernels: the reference model runs on the reference's own
    compiled CUDA operators; this_library: the same reference model runs on this library's `graphop`.
    Log-probabilities within 1e-5, every parameter gradient within 1e-4 (max-norm relative)."""
    import types
    import bpt_b200
    import bpt_b200.graphop
    from bpt_b200 import csr as csrmod, graphbuilder
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTLanguageModel
    backend = ref_graphop if ours_on == "reference_kernels" else bpt_b200.install_dropin()[0]
    mods = build_ref_graphop.load_modules(backend, REF_ROOT)
    if mods is None:
        pytest.skip("the reference's modules/model.py is neither mounted nor compiled")
    ref_model = mods[3]
    torch.manual_seed(3)
    graphs = [graphbuilder.BinaryPartition(n, True, 4, 10) for n in (200, 77, 129)]
    batch = csrmod.batch_graphs(graphs)
    csr = csrmod.get_csrs(batch.src, batch.dst, batch.n_nodes)
    N = batch.n_nodes
    vocab, dim, ff, heads, layers = 50, 128, 256, 4, 2
    theirs = ref_model.make_model(vocab, dim, dim, ff, heads, vocab, layers, dropouti=0.0, dropouth=0.0,
                                  dropouta=0.0, dropoutc=0.0, rel_pos=True).cuda()
    mine = BPTLanguageModel(vocab, dim, ff, heads, layers).cuda()
    mine.load_state_dict(theirs.state_dict(), strict=True)
    leaf_ids = batch.leaf_ids().long()
    tokens = torch.randint(0, vocab, (leaf_ids.numel(),), device="cuda")
    w_loss = torch.randn(leaf_ids.numel(), vocab, device="cuda")
    x = torch.zeros(N, dtype=torch.long, device="cuda")
    x[leaf_ids] = tokens
    g = build_ref_graphop.FakeGraph(ndata={"x": x}, edata={"etype": batch.etype.long()}, n_nodes=N)
    ref_batch = types.SimpleNamespace(g=g, leaf_ids=leaf_ids, g_csr=csr, readout_ids=leaf_ids)
    want = theirs(ref_batch)
    (want * w_loss).sum().backward()
    plan = AttentionPlan.from_batch(batch, n_etypes=1000)
    got = mine(tokens, leaf_ids, plan)
    (got * w_loss).sum().backward()
    assert want.shape == got.shape == (leaf_ids.numel(), vocab)
    assert rel_err(got.detach().cpu(), want.detach().cpu()) < 1e-5
    theirs_grads = dict(theirs.named_parameters())
    checked = 0
    for name, p in mine.named_parameters():
        q = theirs_grads[name]
        if q.grad is None:
            assert p.grad is None or float(p.grad.abs().max()) == 0.0, name
            continue
        assert rel_err(p.grad.cpu(), q.grad.cpu()) < 1e-4, name
        checked += 1
    assert checked >= 20


@pytest.mark.parametrize("ours_on", ["reference_kernels", "this_library"])
def test_reference_encoder_decoder_equals_rehosted_model(oracle_lib, ref_graphop, ours_on):
    """modules/model.py:22-106 -- the reference's BinaryPartitionEncoderDecoder, its file unchanged (rel_pos=True,
    dropouts 0): encoder blocks over a bidirectional batch, memory blocks over a causal batch reading the
    encoder through the sentence-aligned cross graph (graph/mt.py:318-321, built over max(N_enc, N_dec) nodes
    with zero padding as the reference does), against bpt_b200.model.BPTEncoderDecoder loaded from the
    reference model's state dict (strict), which takes the two node sets as they are.
    Log-probabilities within 1e-5 with the reference model on its own compiled CUDA operators and on this
    library's `graphop`; parameter gradients within 1e-4 with the reference model on this library.  On the
    reference's own kernels the gradients that pass through the cross graph are incomplete: its
    vector_spmm_backward sizes the launch over the transposed CSR with the other CSR's chunk count
    (graph_kernel/graphop_kernel.cu:566,588), and the cross graph has more chunks by source than by
    destination, so the last source rows get no gradient there; they are not compared."""
    import types
    import bpt_b200
    from bpt_b200 import csr as csrmod, graphbuilder
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTEncoderDecoder
    backend = ref_graphop if ours_on == "reference_kernels" else bpt_b200.install_dropin()[0]
    mods = build_ref_graphop.load_modules(backend, REF_ROOT)
    if mods is None:
        pytest.skip("the reference's modules/model.py is neither mounted nor compiled")
    ref_model = mods[3]
    torch.manual_seed(4)
    enc_len, dec_len = [37, 20, 64], [12, 33, 50]
    enc = csrmod.batch_graphs([graphbuilder.BinaryPartition(n, False, 2, 3) for n in enc_len])
    dec = csrmod.batch_graphs([graphbuilder.BinaryPartition(n, True, 2, 3) for n in dec_len])
    src_ranges = [(enc.node_offsets[i], enc_len[i]) for i in range(3)]
    dst_ranges = [(dec.node_offsets[i], dec_len[i]) for i in range(3)]
    isrc, idst = csrmod.inter_graph(src_ranges, dst_ranges)
    n_inter = max(enc.n_nodes, dec.n_nodes)
    vocabs, dim, ff, heads = [40, 50], 128, 256, 4
    theirs = ref_model.BinaryPartitionEncoderDecoder(vocabs, dim, ff, heads, 2, 2, dropouti=0.0, dropouth=0.0,
                                                     dropouta=0.0, dropoutc=0.0, rel_pos=True).cuda()
    theirs.reset_parameters()
    mine = BPTEncoderDecoder(vocabs, dim, ff, heads, 2, 2).cuda()
    mine.load_state_dict(theirs.state_dict(), strict=True)
    enc_leaves, dec_leaves = enc.leaf_ids().long(), dec.leaf_ids().long()
    enc_tok = torch.randint(0, vocabs[0], (enc_leaves.numel(),), device="cuda")
    dec_tok = torch.randint(0, vocabs[1], (dec_leaves.numel(),), device="cuda")
    w_loss = torch.randn(dec_leaves.numel(), vocabs[1], device="cuda")

    def graph(batch, tokens, leaves):
        x = torch.zeros(batch.n_nodes, dtype=torch.long, device="cuda")
        x[leaves] = tokens
        return build_ref_graphop.FakeGraph(ndata={"x": x}, edata={"etype": batch.etype.long()}, n_nodes=batch.n_nodes)

    ref_batch = types.SimpleNamespace(
        g_enc=graph(enc, enc_tok, enc_leaves), g_dec=graph(dec, dec_tok, dec_leaves),
        g_inter=build_ref_graphop.FakeGraph(n_nodes=n_inter),
        g_enc_csr=csrmod.get_csrs(enc.src, enc.dst, enc.n_nodes), g_dec_csr=csrmod.get_csrs(dec.src, dec.dst, dec.n_nodes),
        g_inter_csr=csrmod.get_csrs(isrc, idst, n_inter), leaf_ids={"enc": enc_leaves, "dec": dec_leaves},
        readout_ids=dec_leaves)
    want = theirs(ref_batch)
    (want * w_loss).sum().backward()
    got = mine(enc_tok, enc_leaves, AttentionPlan.from_batch(enc, n_etypes=1000), dec_tok, dec_leaves,
               AttentionPlan.from_batch(dec, n_etypes=1000),
               AttentionPlan(isrc, idst, None, dec.n_nodes, n_src=enc.n_nodes), dec_leaves)
    (got * w_loss).sum().backward()
    assert rel_err(got.detach().cpu(), want.detach().cpu()) < 1e-5
    if ours_on == "reference_kernels":
        return
    theirs_params = dict(theirs.named_parameters())
    checked = 0
    for name, p in mine.named_parameters():
        q = theirs_params[name]
        if q.grad is None:
            assert p.grad is None or float(p.grad.abs().max()) == 0.0, name
            continue
        assert rel_err(p.grad.cpu(), q.grad.cpu()) < 1e-4, name
        checked += 1
    assert checked >= 40
