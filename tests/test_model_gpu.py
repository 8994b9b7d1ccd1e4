"""The re-hosted block (bpt_b200/model.py) against the reference's block arithmetic
(modules/attention.py:54-81) spelled out with the operator chain and torch layers."""
import numpy as np
import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu


def test_block_equals_operator_chain_block(oracle_lib):
    from bpt_b200 import csr as csrmod, graphbuilder, op
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTBlock, BPTLanguageModel
    torch.manual_seed(0)
    g = graphbuilder.BinaryPartition(200, True, 4, 6)
    batch = csrmod.batch_graphs([g, g])
    plan = AttentionPlan.from_batch(batch, n_etypes=1000)
    blk = BPTBlock(128, 4, 256, rel_pos=True, drop_h=0.0).cuda()
    blk.reset_parameters()
    h = torch.randn(batch.n_nodes, 128, device="cuda")
    out = blk(h, plan)
    # reference arithmetic: four operators over the CSR tuple of graph/base.py:71-86
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = csrmod.get_csrs(batch.src, batch.dst, batch.n_nodes)
    q = blk.proj_q(h).view(-1, 4, 32)
    k = blk.proj_k(h).view(-1, 4, 32)
    v = blk.proj_v(h).view(-1, 4, 32)
    ak = blk.embed_ak(batch.etype.long())
    e = op.masked_mm(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2], in_csr[1], k, q)
    e_rel = op.node_mul_edge(COL, INDPTR_C, in_csr[2], q, ak)
    p = op.sparse_softmax(COL, INDPTR_C, in_csr[2], (e_rel + e) / np.sqrt(32))
    a = op.vec_spmm(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2], out_csr[1], p, v).view(-1, 128)
    hh = blk.norm_in(h + blk.proj_o(a))
    want = blk.norm_inter(hh + blk.ffn(hh))
    assert rel_err(out.detach().cpu(), want.detach().cpu()) < 1e-5
    # gradients flow to every parameter
    out.sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in blk.parameters())
    # language model: log-probabilities normalise, bf16 runs on the tensor-core path
    lm = BPTLanguageModel(256, 128, 256, 2, 2).cuda().to(torch.bfloat16).eval()
    tokens = torch.randint(0, 256, (400,), device="cuda")
    with torch.no_grad():
        logp = lm(tokens, batch.leaf_ids(), plan)
    assert logp.shape == (400, 256)
    assert torch.allclose(logp.float().exp().sum(-1), torch.ones(400, device="cuda"), atol=2e-2)
    assert plan.tiles is not None


def test_mem_block_equals_operator_chain_block(oracle_lib):
    """BPTMemBlock against modules/attention.py:116-172 spelled out with the operator chain: the
    cross graph is sentence-aligned dense blocks (graph/mt.py:318-321) over max(N_dec, N_enc)
    nodes with the smaller side zero-padded, as the reference does; the re-hosted block takes the
    two node sets as they are."""
    from bpt_b200 import csr as csrmod, graphbuilder, op
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTEncoderDecoder, BPTMemBlock
    torch.manual_seed(1)
    enc_len, dec_len = [37, 20, 64], [12, 33, 50]
    enc = csrmod.batch_graphs([graphbuilder.BinaryPartition(n, False, 2, 3) for n in enc_len])
    dec = csrmod.batch_graphs([graphbuilder.BinaryPartition(n, True, 2, 3) for n in dec_len])
    # one aligned pair per sentence: all leaves of encoder sentence i -> all leaves of decoder sentence i
    src_ranges = [(enc.node_offsets[i], enc_len[i]) for i in range(3)]
    dst_ranges = [(dec.node_offsets[i], dec_len[i]) for i in range(3)]
    isrc, idst = csrmod.inter_graph(src_ranges, dst_ranges)
    want_src, want_dst = oracle_lib.inter_graph(src_ranges, dst_ranges)
    assert np.array_equal(isrc.cpu().numpy(), want_src) and np.array_equal(idst.cpu().numpy(), want_dst)
    plan = AttentionPlan.from_batch(dec, n_etypes=1000)
    plan_inter = AttentionPlan(isrc, idst, None, dec.n_nodes, n_src=enc.n_nodes)
    blk = BPTMemBlock(128, 4, 256, rel_pos=True, drop_h=0.0).cuda()
    blk.reset_parameters()
    h = torch.randn(dec.n_nodes, 128, device="cuda")
    mem = torch.randn(enc.n_nodes, 128, device="cuda")
    out = blk(h, plan, mem, plan_inter)

    def chain(csr, q, k, v, ak_edges):
        out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = csr
        e = op.masked_mm(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2], in_csr[1], k, q)
        if ak_edges is not None:
            e = e + op.node_mul_edge(COL, INDPTR_C, in_csr[2], q, ak_edges)
        p = op.sparse_softmax(COL, INDPTR_C, in_csr[2], e / np.sqrt(32))
        return op.vec_spmm(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2], out_csr[1], p, v).view(-1, 128)

    view = lambda t: t.view(-1, 4, 32)
    a = chain(csrmod.get_csrs(dec.src, dec.dst, dec.n_nodes), view(blk.proj_q[0](h)), view(blk.proj_k[0](h)),
              view(blk.proj_v[0](h)), blk.embed_ak(dec.etype.long()))
    hh = blk.norm_in[0](h + blk.proj_o[0](a))
    n_inter = max(dec.n_nodes, enc.n_nodes)
    pad = lambda t: torch.cat([t, t.new_zeros(n_inter - t.size(0), t.size(1))], 0)
    a = chain(csrmod.get_csrs(isrc, idst, n_inter), view(blk.proj_q[1](pad(hh))), view(blk.proj_k[1](pad(mem))),
              view(blk.proj_v[1](pad(mem))), None)[: dec.n_nodes]
    hh = blk.norm_in[1](hh + blk.proj_o[1](a))
    want = blk.norm_inter(hh + blk.ffn(hh))
    assert rel_err(out.detach().cpu(), want.detach().cpu()) < 1e-5
    out.sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in blk.parameters())
    # encoder-decoder forward in bf16: log-probabilities of the read-out nodes normalise
    model = BPTEncoderDecoder([100, 120], 128, 256, 2, 2, 2).cuda().to(torch.bfloat16).eval()
    enc_plan = AttentionPlan.from_batch(enc, n_etypes=1000)
    enc_tok = torch.randint(0, 100, (sum(enc_len),), device="cuda")
    dec_tok = torch.randint(0, 120, (sum(dec_len),), device="cuda")
    with torch.no_grad():
        logp = model(enc_tok, enc.leaf_ids(), enc_plan, dec_tok, dec.leaf_ids(), plan, plan_inter, dec.leaf_ids())
    assert logp.shape == (sum(dec_len), 120)
    assert torch.allclose(logp.float().exp().sum(-1), torch.ones(sum(dec_len), device="cuda"), atol=2e-2)
