"""The fp32 forward on tensor cores (bpt_attn_forward_tc32: tile plan, every product as three TF32
products) against the fp64 oracle at the fp32 bar (1e-5 max-norm relative) and against the CUDA-core fp32
forward, on binary-partition batches incl. non-power-of-two lengths with duplicate edges and a 3000-edge
root row (rows spread over several tiles), cross-attention shapes without a relative term, empty rows, the
headline size, 16-bit cells, and with dropout (same mask as the CUDA-core kernel)."""
import numpy as np
import pytest
import torch

from helpers import fully_connected_blocks, rel_err
from test_fused_gpu import GRAPHS, _inputs, _oracle

pytestmark = pytest.mark.gpu


def _forward(src, dst, etype, N, T, q, k, v, ak, scale, dropout=None):
    from bpt_b200.attention import AttentionPlan, attention_forward, attention_forward_tc32, tc32_eligible
    dev = "cuda"
    plan = AttentionPlan(torch.from_numpy(src).to(dev), torch.from_numpy(dst).to(dev),
                         None if etype is None else torch.from_numpy(etype).to(dev), N, n_etypes=T)
    qg, kg, vg = [t.to(dev) for t in (q, k, v)]
    akg = None if ak is None else ak.to(dev)
    assert tc32_eligible(qg, akg, plan)
    o, lse = attention_forward_tc32(plan, qg, kg, vg, akg, scale, dropout)
    o2, lse2 = attention_forward_tc32(plan, qg, kg, vg, akg, scale, dropout)
    assert torch.equal(o, o2) and torch.equal(lse, lse2), "the fp32 tile forward is not bitwise reproducible"
    o_s, lse_s = attention_forward(plan, qg, kg, vg, akg, scale, tensor_cores=False, dropout=dropout)
    return o, lse, o_s, lse_s


@pytest.mark.parametrize("graph", list(GRAPHS))
@pytest.mark.parametrize("heads", [8, 3])
def test_tc32_forward_matches_oracle(oracle_lib, graph, heads):
    g = GRAPHS[graph](oracle_lib)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, heads, 64, T, torch.float32, 0)
    scale = 0.125
    want = _oracle(oracle_lib, g["src"], g["dst"], g["etype"], N, q, k, v, ak, d_o, scale)
    o, lse, o_s, lse_s = _forward(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, scale)
    assert rel_err(o.cpu(), want[0]) < 1e-5
    finite = np.isfinite(want[1])
    assert np.array_equal(np.isfinite(lse.cpu().numpy()), finite)
    assert rel_err(lse.cpu().numpy()[finite], want[1][finite]) < 1e-5
    assert rel_err(o.cpu(), o_s.cpu()) < 1e-5


def test_tc32_forward_without_relative_term_and_with_empty_rows(oracle_lib):
    src, dst, N0 = fully_connected_blocks(5, 30)
    N = N0 + 7
    q, k, v, _, d_o = _inputs(N, 8, 64, 1, torch.float32, 1, sigma=0.5)
    want = _oracle(oracle_lib, src, dst, None, N, q, k, v, None, d_o, 0.125)
    o, lse, _, _ = _forward(src, dst, None, N, 1, q, k, v, None, 0.125)
    assert rel_err(o.cpu(), want[0]) < 1e-5
    assert torch.all(o[N0:] == 0) and torch.all(torch.isinf(lse[N0:]))


def test_tc32_forward_sixteen_bit_cells(oracle_lib):
    g = oracle_lib.binary_partition(700, False, 64, 10)  # > 255 edge types
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, 2, 64, T, torch.float32, 2)
    from bpt_b200.attention import AttentionPlan, tc32_eligible
    plan = AttentionPlan(torch.from_numpy(g["src"]).cuda(), torch.from_numpy(g["dst"]).cuda(),
                         torch.from_numpy(g["etype"]).cuda(), N, n_etypes=T)
    if not tc32_eligible(q.cuda(), ak.cuda(), plan):
        pytest.skip("the tables of this many edge types do not fit in shared memory")
    want = _oracle(oracle_lib, g["src"], g["dst"], g["etype"], N, q, k, v, ak, d_o, 0.125)
    o, lse, _, _ = _forward(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, 0.125)
    assert rel_err(o.cpu(), want[0]) < 1e-5


def test_tc32_forward_headline_size(oracle_lib):
    g = oracle_lib.binary_partition(8192, False, 4, 10)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, 8, 64, T, torch.float32, 3, sigma=0.125)
    csr = oracle_lib.get_csrs(g["src"], g["dst"], N)
    f = lambda t: t.float().numpy()
    want_o, want_lse, _ = oracle_lib.attn_fwd(csr[1], g["etype"], f(q), f(k), f(v), f(ak), 0.125)
    o, lse, o_s, _ = _forward(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, 0.125)
    assert rel_err(o.cpu(), want_o) < 1e-5
    assert rel_err(lse.cpu().numpy(), want_lse) < 1e-5
    assert rel_err(o.cpu(), o_s.cpu()) < 1e-5


def test_tc32_forward_with_dropout_equals_cuda_core_forward(oracle_lib):
    g = GRAPHS["bpt_batch"](oracle_lib)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, _ = _inputs(N, 8, 64, T, torch.float32, 4)
    o, lse, o_s, lse_s = _forward(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, 0.125, dropout=(0.3, 99))
    assert rel_err(o.cpu(), o_s.cpu()) < 1e-5
    finite = torch.isfinite(lse_s)
    assert torch.equal(torch.isfinite(lse), finite)
    assert rel_err(lse[finite].cpu(), lse_s[finite].cpu()) < 1e-5
    o_plain, _, _, _ = _forward(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, 0.125)
    assert rel_err(o.cpu(), o_plain.cpu()) > 1e-3  # the mask really was applied


# ---------------------------------------------------------------- backward, destination side on tensor cores

def _backward(monkeypatch, src, dst, etype, N, T, q, k, v, ak, d_o, scale, dropout=None):
    """Gradients of the fp32 tile backward (bpt_attn_backward_tc32) and of the CUDA-core backward."""
    from bpt_b200 import attention as A
    dev = "cuda"
    plan = A.AttentionPlan(torch.from_numpy(src).to(dev), torch.from_numpy(dst).to(dev),
                           None if etype is None else torch.from_numpy(etype).to(dev), N, n_etypes=T)
    qg, kg, vg, dog = [t.to(dev) for t in (q, k, v, d_o)]
    akg = None if ak is None else ak.to(dev)
    o, lse = A.attention_forward_tc32(plan, qg, kg, vg, akg, scale, dropout)
    monkeypatch.setattr(A, "FP32_BACKWARD", "tc32")
    got = A.attention_backward(plan, qg, kg, vg, akg, scale, lse, dog, o=o, dropout=dropout)
    again = A.attention_backward(plan, qg, kg, vg, akg, scale, lse, dog, o=o, dropout=dropout)
    for a, b in zip(got, again):
        assert (a is None and b is None) or torch.equal(a, b), "the fp32 tile backward is not bitwise reproducible"
    assert ("tc32_bwd", qg.size(1)) in plan._ws, "the fp32 tile backward did not run"
    monkeypatch.setattr(A, "FP32_BACKWARD", "simt")
    ref = A.attention_backward(plan, qg, kg, vg, akg, scale, lse, dog, o=o, dropout=dropout)
    return got, ref


@pytest.mark.parametrize("graph", list(GRAPHS))
@pytest.mark.parametrize("heads", [8, 3])
def test_tc32_backward_matches_oracle(oracle_lib, monkeypatch, graph, heads):
    g = GRAPHS[graph](oracle_lib)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, heads, 64, T, torch.float32, 10)
    want = _oracle(oracle_lib, g["src"], g["dst"], g["etype"], N, q, k, v, ak, d_o, 0.125)
    got, ref = _backward(monkeypatch, g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, 0.125)
    for name, a, b, c in zip(("dq", "dk", "dv", "dak"), got, want[2:], ref):
        assert rel_err(a.cpu(), b) < 1e-5, name
        assert rel_err(a.cpu(), c.cpu()) < 1e-5, name


def test_tc32_backward_without_relative_term_and_with_empty_rows(oracle_lib, monkeypatch):
    src, dst, N0 = fully_connected_blocks(5, 30)
    N = N0 + 7
    q, k, v, _, d_o = _inputs(N, 8, 64, 1, torch.float32, 11, sigma=0.5)
    want = _oracle(oracle_lib, src, dst, None, N, q, k, v, None, d_o, 0.125)
    got, _ = _backward(monkeypatch, src, dst, None, N, 1, q, k, v, None, d_o, 0.125)
    for name, a, b in zip(("dq", "dk", "dv"), got, want[2:5]):
        assert rel_err(a.cpu(), b) < 1e-5, name
    assert got[3] is None
    assert torch.all(got[0][N0:] == 0)


def test_tc32_backward_headline_size_and_dropout(oracle_lib, monkeypatch):
    g = oracle_lib.binary_partition(8192, False, 4, 10)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, 8, 64, T, torch.float32, 12, sigma=0.125)
    got, ref = _backward(monkeypatch, g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, 0.125)
    for name, a, c in zip(("dq", "dk", "dv", "dak"), got, ref):
        assert rel_err(a.cpu(), c.cpu()) < 1e-5, name
    got, ref = _backward(monkeypatch, g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, 0.125, dropout=(0.3, 7))
    for name, a, c in zip(("dq", "dk", "dv", "dak"), got, ref):
        assert rel_err(a.cpu(), c.cpu()) < 1e-5, name


def test_tc32_backward_with_cuda_core_source_side(oracle_lib, monkeypatch):
    """The destination-side tile kernel alone (src_tiles = NULL): dK and dV from the CUDA-core kernel on its scratch."""
    from bpt_b200 import attention as A
    monkeypatch.setattr(A, "FP32_BACKWARD_SOURCE_SIDE", "simt")
    g = GRAPHS["bpt_batch"](oracle_lib)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, 8, 64, T, torch.float32, 13)
    want = _oracle(oracle_lib, g["src"], g["dst"], g["etype"], N, q, k, v, ak, d_o, 0.125)
    got, _ = _backward(monkeypatch, g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, 0.125)
    for name, a, b in zip(("dq", "dk", "dv", "dak"), got, want[2:]):
        assert rel_err(a.cpu(), b) < 1e-5, name


def test_tc32_backward_sixteen_bit_cells(oracle_lib, monkeypatch):
    g = oracle_lib.binary_partition(700, False, 64, 10)  # > 255 edge types
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, 2, 64, T, torch.float32, 14)
    from bpt_b200.attention import AttentionPlan, tc32_eligible
    plan = AttentionPlan(torch.from_numpy(g["src"]).cuda(), torch.from_numpy(g["dst"]).cuda(),
                         torch.from_numpy(g["etype"]).cuda(), N, n_etypes=T)
    if not tc32_eligible(q.cuda(), ak.cuda(), plan):
        pytest.skip("the tables of this many edge types do not fit in shared memory")
    want = _oracle(oracle_lib, g["src"], g["dst"], g["etype"], N, q, k, v, ak, d_o, 0.125)
    got, _ = _backward(monkeypatch, g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, 0.125)
    for name, a, b in zip(("dq", "dk", "dv", "dak"), got, want[2:]):
        assert rel_err(a.cpu(), b) < 1e-5, name


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_graph_without_edges_gives_zero_output_and_gradients(dtype):
    """A plan with nodes and no edge at all: o = 0, lse = -inf, every gradient zero, on the tile kernels of
    either dtype (outputs are allocated uninitialised, so every row must be written)."""
    from bpt_b200 import attention as A
    N, T = 40, 3
    z = torch.zeros(0, dtype=torch.int32, device="cuda")
    plan = A.AttentionPlan(z, z, z, N, n_etypes=T)
    gen = torch.Generator().manual_seed(3)
    q, k, v, d_o = [torch.randn(N, 8, 64, generator=gen).to(dtype).cuda() for _ in range(4)]
    ak = torch.randn(T, 64, generator=gen).to(dtype).cuda()
    o, lse = A.attention_forward(plan, q, k, v, ak, 0.125)
    assert torch.all(o == 0) and torch.all(torch.isinf(lse) & (lse < 0))
    dq, dk, dv, dak = A.attention_backward(plan, q, k, v, ak, 0.125, lse, d_o, o=o)
    for g in (dq, dk, dv, dak):
        assert torch.all(g == 0)
