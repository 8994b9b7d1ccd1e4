"""The tcgen05 forward (bpt_attn_forward_tc5) against the fp64 oracle (2e-2 max-norm relative, the bf16
bar) and against the mma.sync tile forward, on binary-partition batches incl. non-power-of-two lengths
with duplicate edges, cross-attention shapes without a relative term, empty rows, and the headline size."""
import numpy as np
import pytest
import torch

from helpers import fully_connected_blocks, rel_err
from test_fused_gpu import GRAPHS, _inputs, _oracle

pytestmark = pytest.mark.gpu


def _forward_tc5(src, dst, etype, N, T, q, k, v, ak, scale, n_src=None):
    from bpt_b200.attention import AttentionPlan, attention_forward_tc, attention_forward_tc5, tc5_eligible, tc5_status
    dev = "cuda"
    plan = AttentionPlan(torch.from_numpy(src).to(dev), torch.from_numpy(dst).to(dev),
                         None if etype is None else torch.from_numpy(etype).to(dev), N, n_etypes=T, n_src=n_src)
    qg, kg, vg = [t.to(dev) for t in (q, k, v)]
    akg = None if ak is None else ak.to(dev)
    assert tc5_eligible(qg, akg, plan)
    o, lse = attention_forward_tc5(plan, qg, kg, vg, akg, scale)
    assert tc5_status(plan, q.size(1)) == 0, "a bounded wait of the tcgen05 kernel ran out"
    o2, lse2 = attention_forward_tc5(plan, qg, kg, vg, akg, scale)
    assert torch.equal(o, o2) and torch.equal(lse, lse2), "the tcgen05 forward is not bitwise reproducible"
    o_t, lse_t = attention_forward_tc(plan, qg, kg, vg, akg, scale)
    return o, lse, o_t, lse_t


@pytest.mark.parametrize("graph", list(GRAPHS))
@pytest.mark.parametrize("heads", [8, 3])
def test_tc5_forward_matches_oracle(oracle_lib, graph, heads):
    g = GRAPHS[graph](oracle_lib)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, heads, 64, T, torch.bfloat16, 0)
    scale = 0.125
    want = _oracle(oracle_lib, g["src"], g["dst"], g["etype"], N, q, k, v, ak, d_o, scale)
    o, lse, o_t, lse_t = _forward_tc5(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, scale)
    assert rel_err(o.float().cpu(), want[0]) < 2e-2
    finite = np.isfinite(want[1])
    assert np.array_equal(np.isfinite(lse.cpu().numpy()), finite)
    assert rel_err(lse.cpu().numpy()[finite], want[1][finite]) < 1e-3
    assert rel_err(o.float().cpu(), o_t.float().cpu()) < 2e-2


def test_tc5_forward_without_relative_term_and_with_empty_rows(oracle_lib):
    src, dst, N0 = fully_connected_blocks(5, 30)
    N = N0 + 7
    q, k, v, _, d_o = _inputs(N, 8, 64, 1, torch.bfloat16, 1, sigma=0.5)
    want = _oracle(oracle_lib, src, dst, None, N, q, k, v, None, d_o, 0.125)
    o, lse, _, _ = _forward_tc5(src, dst, None, N, 1, q, k, v, None, 0.125)
    assert rel_err(o.float().cpu(), want[0]) < 2e-2
    assert torch.all(o[N0:] == 0) and torch.all(torch.isinf(lse[N0:]))


def test_tc5_forward_headline_size(oracle_lib):
    g = oracle_lib.binary_partition(8192, False, 4, 10)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, 8, 64, T, torch.bfloat16, 3, sigma=0.125)
    csr = oracle_lib.get_csrs(g["src"], g["dst"], N)
    f = lambda t: t.float().numpy()
    want_o, want_lse, _ = oracle_lib.attn_fwd(csr[1], g["etype"], f(q), f(k), f(v), f(ak), 0.125)
    o, lse, o_t, _ = _forward_tc5(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, 0.125)
    assert rel_err(o.float().cpu(), want_o) < 2e-2
    assert rel_err(lse.cpu().numpy(), want_lse) < 1e-3
