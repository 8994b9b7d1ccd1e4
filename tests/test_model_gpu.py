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
