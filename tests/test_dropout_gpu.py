"""Dropout on the attention weights inside the fused call (the reference's drop_att between sparse_softmax
and vec_spmm, modules/attention.py:73): the mask the kernels regenerate is exported once and the fused
forward + backward is compared with the operator chain using that same mask (1e-5 fp32 on the CUDA-core
kernels, 2e-2 bf16 on the tensor-core tile kernels); fixed seed = bitwise identical results."""
import numpy as np
import pytest
import torch

from helpers import rel_err
from test_fused_gpu import GRAPHS, _inputs

pytestmark = pytest.mark.gpu


def _chain_with_mask(g, N, q, k, v, ak, d_o, mask, rate):
    from bpt_b200 import csr as csrmod, op
    src, dst, et = [torch.from_numpy(g[n]).cuda() for n in ("src", "dst", "etype")]
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = csrmod.get_csrs(src, dst, N)
    qc, kc, vc, akc = [t.float().cuda().clone().requires_grad_(True) for t in (q, k, v, ak)]
    e = op.masked_mm(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2], in_csr[1], kc, qc)
    e_rel = op.node_mul_edge(COL, INDPTR_C, in_csr[2], qc, akc[et])
    p = op.sparse_softmax(COL, INDPTR_C, in_csr[2], (e_rel + e) / np.sqrt(q.size(-1)))
    p = p * mask.float() / (1.0 - rate)                                    # attention.py:73, drop_att
    o = op.vec_spmm(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2], out_csr[1], p, vc)
    o.backward(d_o.float().cuda())
    return [o.detach(), qc.grad, kc.grad, vc.grad, akc.grad]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("graph", ["bpt_batch", "long_rows"])
def test_fused_dropout_equals_chain_with_the_same_mask(oracle_lib, dtype, graph):
    from bpt_b200.attention import AttentionPlan, bpt_attention, dropout_mask
    g = GRAPHS[graph](oracle_lib)
    N, T, H, D = g["n_nodes"], int(g["etype"].max()) + 1, 8, 64
    q, k, v, ak, d_o = _inputs(N, H, D, T, dtype, 5)
    rate, seed = 0.25, 1234567
    src, dst, et = [torch.from_numpy(g[n]).cuda() for n in ("src", "dst", "etype")]
    mask = dropout_mask(src, dst, H, rate, seed)
    kept = mask.float().mean().item()
    assert abs(kept - (1 - rate)) < 0.01
    want = _chain_with_mask(g, N, q, k, v, ak, d_o, mask, rate)
    plan = AttentionPlan(src, dst, et, N, n_etypes=T)
    runs = []
    for _ in range(2):
        qg, kg, vg, akg = [t.cuda().clone().requires_grad_(True) for t in (q, k, v, ak)]
        o = bpt_attention(plan, qg, kg, vg, akg, 1.0 / np.sqrt(D), dropout_p=rate, seed=seed)
        o.backward(d_o.cuda())
        runs.append([o.detach(), qg.grad, kg.grad, vg.grad, akg.grad])
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for a, b in zip(runs[0], want):
        assert rel_err(a.float().cpu(), b.cpu()) < tol
    for a, b in zip(runs[0], runs[1]):
        assert torch.equal(a, b)
    if dtype == torch.bfloat16:
        assert plan.tiles is not None, "the bf16 case did not take the tile kernels"
    # another seed gives another mask; rate 0 is the plain call
    qg = q.cuda().clone()
    o2 = bpt_attention(plan, qg, k.cuda(), v.cuda(), ak.cuda(), 1.0 / np.sqrt(D), dropout_p=rate, seed=seed + 1)
    assert not torch.equal(o2, runs[0][0])
    o3 = bpt_attention(plan, qg, k.cuda(), v.cuda(), ak.cuda(), 1.0 / np.sqrt(D), dropout_p=0.0)
    o4 = bpt_attention(plan, qg, k.cuda(), v.cuda(), ak.cuda(), 1.0 / np.sqrt(D))
    assert torch.equal(o3, o4)


def test_block_with_attention_dropout_trains_and_evaluates():
    """BPTBlock(drop_a=0.1), the setting of the reference's training configurations, runs through the fused
    call; in eval mode dropout is off and the block equals one built without it."""
    from bpt_b200 import csr as csrmod, graphbuilder
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTBlock
    torch.manual_seed(0)
    batch = csrmod.batch_graphs([graphbuilder.BinaryPartition(200, True, 4, 6)] * 2)
    plan = AttentionPlan.from_batch(batch, n_etypes=1000)
    blk = BPTBlock(128, 4, 256, rel_pos=True, drop_h=0.0, drop_a=0.1).cuda()
    ref = BPTBlock(128, 4, 256, rel_pos=True, drop_h=0.0, drop_a=0.0).cuda()
    ref.load_state_dict(blk.state_dict())
    h = torch.randn(batch.n_nodes, 128, device="cuda")
    blk.train()
    out = blk(h, plan)
    out.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in blk.parameters())
    assert not torch.equal(out, ref(h, plan))
    blk.eval()
    assert torch.equal(blk(h, plan), ref(h, plan))
    with pytest.raises(RuntimeError, match="dropout rate"):
        from bpt_b200.attention import bpt_attention
        q = torch.randn(batch.n_nodes, 4, 32, device="cuda")
        bpt_attention(plan, q, q, q, None, 0.1, dropout_p=1.0, seed=1)
