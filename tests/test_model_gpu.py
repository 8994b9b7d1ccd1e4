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


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2), (torch.float16, 4e-3)])
def test_add_layer_norm_matches_torch(dtype, tol):
    """bpt_add_layer_norm against torch.nn.functional.layer_norm of the sum computed in fp32, over
    the dimension sizes the kernel's register tiling switches on, and its gradients."""
    from bpt_b200.model import add_layer_norm
    torch.manual_seed(3)
    for dim, rows in ((8, 5), (512, 1000), (520, 33), (1024, 17), (4096, 9)):
        norm = torch.nn.LayerNorm(dim).cuda()
        with torch.no_grad():
            norm.weight.normal_(1.0, 0.2)
            norm.bias.normal_(0.0, 0.2)
        norm = norm.to(dtype)
        x = (torch.randn(rows, dim, device="cuda") * 2 + 0.5).to(dtype).requires_grad_(True)
        r = torch.randn(rows, dim, device="cuda").to(dtype).requires_grad_(True)
        y = add_layer_norm(x, r, norm)
        want = torch.nn.functional.layer_norm(x.float() + r.float(), (dim,), norm.weight.float(), norm.bias.float(),
                                              norm.eps)
        assert y.dtype == dtype and rel_err(y.detach().float().cpu(), want.detach().cpu()) < tol
        gy = torch.randn(rows, dim, device="cuda").to(dtype)
        y.backward(gy)
        got = [t.grad.float().cpu() for t in (x, r, norm.weight, norm.bias)]
        xr, rr = x.detach().float().requires_grad_(True), r.detach().float().requires_grad_(True)
        w, b = norm.weight.detach().float().requires_grad_(True), norm.bias.detach().float().requires_grad_(True)
        torch.nn.functional.layer_norm(xr + rr, (dim,), w, b, norm.eps).backward(gy.float())
        for a, e in zip(got, (xr.grad, rr.grad, w.grad, b.grad)):
            assert rel_err(a, e.cpu()) < max(tol, 1e-4)
    # shapes outside the kernel's rules fall back to torch
    norm = torch.nn.LayerNorm(300).cuda().to(dtype)
    x = torch.randn(7, 300, device="cuda").to(dtype)
    assert torch.equal(add_layer_norm(x, x, norm), norm(x + x))


def test_feed_forward_epilogue_path_matches_plain_path():
    """Inference runs bias + activation in the GEMM epilogue; it must agree with the plain path."""
    from bpt_b200.model import PositionwiseFeedForward
    torch.manual_seed(4)
    for act in ("relu", "gelu_tanh"):
        ffn = PositionwiseFeedForward(128, 512, dropout=0.0, activation=act).cuda().eval()
        x = torch.randn(300, 128, device="cuda")
        plain = ffn(x)                      # grad mode on: plain path
        with torch.no_grad():
            fused = ffn(x)
        assert rel_err(fused.cpu(), plain.detach().cpu()) < 1e-5


def test_classifier_readouts():
    """Variable-length batch (D = 50 per head, fp32: the CUDA-core kernels): the root read-out takes each
    sequence's last node, the mean read-out equals the mean of the sequence's leaves; gradients flow."""
    from bpt_b200 import csr as csrmod
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTClassifier
    torch.manual_seed(5)
    lengths = [10, 57, 128, 301]
    cache = csrmod.GraphCache(triu=True, step=4, clip_dist=5)
    batch = csrmod.batch_graphs([cache.get(n) for n in lengths])
    plan = AttentionPlan.from_batch(batch, n_etypes=1000)
    tokens = torch.randint(0, 500, (sum(lengths),), device="cuda")
    lens = torch.tensor(lengths, device="cuda")
    for readout in ("root", "mean"):
        model = BPTClassifier(500, 300, 600, 6, 2, 2, readout=readout).cuda()
        logp = model(tokens, batch.leaf_ids(), plan, batch.root_ids(), lens)
        assert logp.shape == (4, 2)
        assert torch.allclose(logp.exp().sum(-1), torch.ones(4, device="cuda"), atol=1e-5)
        torch.nn.functional.nll_loss(logp, torch.tensor([0, 1, 1, 0], device="cuda")).backward()
        assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    assert batch.root_ids().tolist() == [o - 1 for o in batch.node_offsets[1:]]
