"""Fused attention forward/backward through the C ABI against the fp64 CPU oracle.

Tolerances (max-norm relative error, ||a-b||_inf / ||b||_inf per tensor): 1e-5 for fp32
storage, 2e-2 for bf16 storage (inputs are rounded to bf16 first, so the oracle sees the same
numbers), as the parity bar for this path states."""
import numpy as np
import pytest
import torch

from helpers import fully_connected_blocks, rel_err

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 4e-3}


def _inputs(N, H, D, T, dtype, seed, sigma=None):
    g = torch.Generator().manual_seed(seed)
    sigma = sigma if sigma is not None else 1.0 / np.sqrt(D)
    mk = lambda *s: (torch.randn(*s, generator=g) * sigma).to(dtype)
    q, k, v, ak = mk(N, H, D), mk(N, H, D), mk(N, H, D), mk(T, D)
    d_o = torch.randn(N, H, D, generator=g).to(dtype)
    return q, k, v, ak, d_o


def _oracle(oracle_lib, src, dst, etype, N, q, k, v, ak, d_o, scale):
    csr = oracle_lib.get_csrs(src, dst, N)
    f = lambda t: None if t is None else t.float().numpy()
    o, lse, p = oracle_lib.attn_fwd(csr[1], etype, f(q), f(k), f(v), f(ak), scale)
    dq, dk, dv, dak = oracle_lib.attn_bwd(csr[1], csr[0], etype, f(q), f(k), f(v), f(ak), scale, o, p, f(d_o))
    return o, lse, dq, dk, dv, dak


def _run_gpu(src, dst, etype, N, T, q, k, v, ak, d_o, scale):
    from bpt_b200.attention import AttentionPlan, bpt_attention, attention_forward
    dev = "cuda"
    plan = AttentionPlan(torch.from_numpy(src).to(dev), torch.from_numpy(dst).to(dev),
                         None if etype is None else torch.from_numpy(etype).to(dev), N, n_etypes=T)
    qg, kg, vg = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
    akg = None if ak is None else ak.to(dev).requires_grad_(True)
    o = bpt_attention(plan, qg, kg, vg, akg, scale)
    o.backward(d_o.to(dev))
    _, lse = attention_forward(plan, qg.detach(), kg.detach(), vg.detach(), None if ak is None else akg.detach(), scale)
    return plan, o.detach(), lse, qg.grad, kg.grad, vg.grad, None if ak is None else akg.grad


def _compare(got, want, tol):
    names = ("o", "lse", "dq", "dk", "dv", "dak")
    for name, a, b in zip(names, got, want):
        if b is None:
            assert a is None
            continue
        a = a.double().cpu().numpy()
        if name == "lse":
            finite = np.isfinite(b)
            assert np.array_equal(np.isfinite(a), finite)
            assert rel_err(a[finite], b[finite]) < max(tol, 1e-5), name
        else:
            assert rel_err(a, b) < tol, (name, rel_err(a, b))


GRAPHS = {
    # three sequences incl. a non-power-of-two bidirectional one (duplicate (src,dst) pairs)
    "bpt_batch": lambda o: o.batch_graphs([o.binary_partition(300, False, 4, 10), o.binary_partition(77, True, 2, 3),
                                           o.binary_partition(513, False, 4, 10), o.binary_partition(1, False, 4, 10)]),
    # config 1 of the baseline: 4 x (n=512, k=4)
    "cfg1": lambda o: o.batch_graphs([o.binary_partition(512, False, 4, 10)] * 4),
    # a root with 3000 incoming edges: rows split over many work items
    "long_rows": lambda o: o.binary_partition(3000, True, 8, 6),
}


@pytest.mark.parametrize("graph", list(GRAPHS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd", [(8, 64), (12, 64), (6, 50), (3, 32), (2, 128), (20, 16)])
def test_fused_matches_oracle(oracle_lib, graph, dtype, hd):
    H, D = hd
    if graph != "bpt_batch" and hd not in ((8, 64), (6, 50)):
        pytest.skip("shape sweep runs on one graph")
    g = GRAPHS[graph](oracle_lib)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, H, D, T, dtype, 0)
    scale = 1.0 / np.sqrt(D)
    want = _oracle(oracle_lib, g["src"], g["dst"], g["etype"], N, q, k, v, ak, d_o, scale)
    got = _run_gpu(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, scale)[1:]
    _compare(got, want, TOL[dtype])


def test_no_relative_term_empty_rows_and_dense_blocks(oracle_lib):
    """No embed_ak (cross-attention use, modules/attention.py:156-162), destinations without
    incoming edges, and the fully connected blocks of graph_kernel/test.py."""
    src, dst, N0 = fully_connected_blocks(5, 30)
    N = N0 + 7  # seven isolated nodes at the end
    q, k, v, _, d_o = _inputs(N, 8, 64, 1, torch.float32, 1, sigma=0.5)
    want = _oracle(oracle_lib, src, dst, None, N, q, k, v, None, d_o, 0.125)
    plan, *got = _run_gpu(src, dst, None, N, 1, q, k, v, None, d_o, 0.125)
    _compare(got, want, 1e-5)
    assert torch.all(got[0][N0:] == 0) and torch.all(torch.isinf(got[1][N0:]))
    # dense check, as test.py:364,395,459 do
    B, L, H, D = 5, 30, 8, 64
    qd, kd, vd = [t[:N0].double().view(B, L, H, D).transpose(1, 2) for t in (q, k, v)]
    dense = (torch.softmax(qd @ kd.transpose(-1, -2) * 0.125, -1) @ vd).transpose(1, 2).reshape(N0, H, D)
    assert rel_err(got[0][:N0].double().cpu(), dense) < 1e-5


def test_fused_equals_operator_chain(oracle_lib):
    """The fused call and the reference-shaped chain of four operators agree."""
    from bpt_b200 import csr as csrmod, op
    from bpt_b200.attention import AttentionPlan, bpt_attention
    g = GRAPHS["cfg1"](oracle_lib)
    N, T, H, D = g["n_nodes"], int(g["etype"].max()) + 1, 8, 64
    q, k, v, ak, d_o = [t.cuda() for t in _inputs(N, H, D, T, torch.float32, 2)]
    src, dst, et = [torch.from_numpy(g[n]).cuda() for n in ("src", "dst", "etype")]
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = csrmod.get_csrs(src, dst, N)
    chain_in = [t.clone().requires_grad_(True) for t in (q, k, v, ak)]
    qc, kc, vc, akc = chain_in
    e = op.masked_mm(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2], in_csr[1], kc, qc)
    e_rel = op.node_mul_edge(COL, INDPTR_C, in_csr[2], qc, akc[et])
    p = op.sparse_softmax(COL, INDPTR_C, in_csr[2], (e_rel + e) / np.sqrt(D))
    a = op.vec_spmm(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2], out_csr[1], p, vc)
    a.backward(d_o)
    fused_in = [t.clone().requires_grad_(True) for t in (q, k, v, ak)]
    plan = AttentionPlan(src, dst, et, N, n_etypes=T)
    o = bpt_attention(plan, *fused_in)
    o.backward(d_o)
    assert rel_err(o.detach().cpu(), a.detach().cpu()) < 1e-5
    for f, c in zip(fused_in, chain_in):
        assert rel_err(f.grad.cpu(), c.grad.cpu()) < 2e-5


def test_fused_is_bitwise_reproducible(oracle_lib):
    g = GRAPHS["long_rows"](oracle_lib)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = _inputs(N, 8, 64, T, torch.float32, 3)
    a = _run_gpu(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, 0.125)[1:]
    b = _run_gpu(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, 0.125)[1:]
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_headline_size(oracle_lib, dtype):
    """n = 8192, k = 4, 8 heads x 64 (N = 16383, E = 745786): the size the headline metric is
    quoted on, inputs N(0, 1/8) as the sweep configuration draws them."""
    from bpt_b200 import graphbuilder
    gb = graphbuilder.BinaryPartition(8192, False, 4, 10)
    s, d, t = gb.get_edges()
    N, T = gb.number_of_nodes, int(t.max()) + 1
    q, k, v, ak, d_o = _inputs(N, 8, 64, T, dtype, 4, sigma=0.125)
    want = _oracle(oracle_lib, s, d, t, N, q, k, v, ak, d_o, 0.125)
    got = _run_gpu(s, d, t, N, T, q, k, v, ak, d_o, 0.125)[1:]
    _compare(got, want, TOL[dtype])
    # size-independent property: attention weights of a row sum to one, so with v = 1 the output is 1
    ones = torch.ones_like(v)
    o1 = _run_gpu(s, d, t, N, T, q, k, ones, ak, d_o, 0.125)[1]
    assert rel_err(o1.float().cpu(), torch.ones(N, 8, 64)) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_tensor_core_forward_is_used_and_matches_cuda_core_forward(oracle_lib):
    """bf16 x head dim 64 goes through bpt_attn_forward_tc; it must agree with the CUDA-core
    kernel on the same inputs (both see the same bf16 numbers) and be reproducible."""
    from bpt_b200.attention import AttentionPlan, attention_forward
    g = GRAPHS["bpt_batch"](oracle_lib)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, _ = [t.cuda() for t in _inputs(N, 8, 64, T, torch.bfloat16, 7)]
    plan = AttentionPlan(torch.from_numpy(g["src"]).cuda(), torch.from_numpy(g["dst"]).cuda(),
                         torch.from_numpy(g["etype"]).cuda(), N, n_etypes=T)
    o_tc, lse_tc = attention_forward(plan, q, k, v, ak, 0.125)
    assert plan.tiles is not None and plan.tiles.n_groups > 0
    o_cc, lse_cc = attention_forward(plan, q, k, v, ak, 0.125, tensor_cores=False)
    assert rel_err(o_tc.float().cpu(), o_cc.float().cpu()) < 2e-2
    assert rel_err(lse_tc.cpu(), lse_cc.cpu()) < 2e-3
    o2, lse2 = attention_forward(plan, q, k, v, ak, 0.125)
    assert torch.equal(o_tc, o2) and torch.equal(lse_tc, lse2)
    # without the relative-position table, and with 3 heads (fewer heads than warps)
    o_tc, lse_tc = attention_forward(plan, q[:, :3].contiguous(), k[:, :3].contiguous(), v[:, :3].contiguous(), None, 0.125)
    o_cc, lse_cc = attention_forward(plan, q[:, :3].contiguous(), k[:, :3].contiguous(), v[:, :3].contiguous(), None,
                                     0.125, tensor_cores=False)
    assert rel_err(o_tc.float().cpu(), o_cc.float().cpu()) < 2e-2 and rel_err(lse_tc.cpu(), lse_cc.cpu()) < 2e-3


def test_tensor_core_backward_matches_cuda_core_backward(oracle_lib):
    """The tensor-core backward (destination-side tiles, source-side transposed tiles) against
    the CUDA-core segment reductions on the same bf16 inputs, and run to run."""
    from bpt_b200.attention import AttentionPlan, attention_backward, attention_forward
    g = GRAPHS["bpt_batch"](oracle_lib)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    q, k, v, ak, d_o = [t.cuda() for t in _inputs(N, 8, 64, T, torch.bfloat16, 11)]
    plan = AttentionPlan(torch.from_numpy(g["src"]).cuda(), torch.from_numpy(g["dst"]).cuda(),
                         torch.from_numpy(g["etype"]).cuda(), N, n_etypes=T)
    o, lse = attention_forward(plan, q, k, v, ak, 0.125)
    a = attention_backward(plan, q, k, v, ak, 0.125, lse, d_o, o=o)
    b = attention_backward(plan, q, k, v, ak, 0.125, lse, d_o, tensor_cores=False)
    assert plan.tiles_t is not None and plan.tiles_t.n_groups > 0
    for name, x, y in zip(("dq", "dk", "dv", "dak"), a, b):
        assert rel_err(x.float().cpu(), y.float().cpu()) < 1e-2, name
    a2 = attention_backward(plan, q, k, v, ak, 0.125, lse, d_o, o=o)
    for x, y in zip(a, a2):
        assert torch.equal(x, y)
    # no relative-position table, three heads
    q3, k3, v3, d3 = [x[:, :3].contiguous() for x in (q, k, v, d_o)]
    o3, lse3 = attention_forward(plan, q3, k3, v3, None, 0.125)
    a = attention_backward(plan, q3, k3, v3, None, 0.125, lse3, d3, o=o3)
    b = attention_backward(plan, q3, k3, v3, None, 0.125, lse3, d3, tensor_cores=False)
    for x, y in zip(a[:3], b[:3]):
        assert rel_err(x.float().cpu(), y.float().cpu()) < 1e-2


def test_tensor_core_path_with_more_than_255_edge_types(oracle_lib):
    """step = 14 gives edge types up to 318: 16-bit cells in the tile plan, and the gradients of
    the relative-position table leave the per-row type table for the per-edge CUDA-core kernels.
    Checked against the fp64 oracle, with 12 heads (more heads than warps in a block)."""
    g = oracle_lib.batch_graphs([oracle_lib.binary_partition(600, False, 14, 10),
                                 oracle_lib.binary_partition(130, True, 14, 10)])
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    assert T > 256
    q, k, v, ak, d_o = _inputs(N, 12, 64, T, torch.bfloat16, 13)
    want = _oracle(oracle_lib, g["src"], g["dst"], g["etype"], N, q, k, v, ak, d_o, 0.125)
    plan, *got = _run_gpu(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, 0.125)
    assert plan.tiles is not None and plan.tiles.et_bytes == 2
    _compare(got, want, TOL[torch.bfloat16])


def test_many_edge_types_fall_back_to_cuda_cores(oracle_lib):
    """step = 64, clip 6 (the reference's configs/enwik8-8192.yml) gives ~900 edge types: the tile
    kernels' per-head tables no longer fit in shared memory, so bf16 x 64 runs on the CUDA-core
    kernels instead of failing, and still matches the oracle."""
    from bpt_b200.attention import AttentionPlan, tensor_core_eligible
    g = oracle_lib.binary_partition(700, True, 64, 6)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    assert T > 700
    q, k, v, ak, d_o = _inputs(N, 8, 64, T, torch.bfloat16, 17)
    want = _oracle(oracle_lib, g["src"], g["dst"], g["etype"], N, q, k, v, ak, d_o, 0.125)
    plan, *got = _run_gpu(g["src"], g["dst"], g["etype"], N, T, q, k, v, ak, d_o, 0.125)
    assert not tensor_core_eligible(q.cuda(), ak.cuda(), plan)
    assert tensor_core_eligible(q.cuda(), None, plan)      # without the relative-position tables it fits
    _compare(got, want, TOL[torch.bfloat16])


def test_largest_sweep_size_properties():
    """n = 65536, k = 8 (N = 131071, E = 13,239,926), bf16 x 8 x 64: the largest cell of the scaling sweep,
    too big for the CPU oracle in a test, checked through identities that hold at any size:
      - attention weights of a row sum to one: with v = 1 the output is 1;
      - O is linear in V with the weights the backward uses:  <dO, O> = <V, dV>;
      - scores are bilinear:  <Q, dQ> = <K, dK> + <embed_ak, d embed_ak>."""
    from bpt_b200 import graphbuilder
    from bpt_b200.attention import AttentionPlan, attention_backward, attention_forward
    gb = graphbuilder.BinaryPartition(65536, False, 8, 10)
    assert gb.number_of_nodes == 131071 and gb.number_of_edges == 13239926
    src, dst, et = gb.edges_device()
    N, T = gb.number_of_nodes, 1000
    plan = AttentionPlan(src, dst, et, N, n_etypes=T)
    gen = torch.Generator().manual_seed(2)
    q, k, v = [(torch.randn(N, 8, 64, generator=gen) * 0.125).bfloat16().cuda() for _ in range(3)]
    ak = (torch.randn(T, 64, generator=gen) * 0.125).bfloat16().cuda()
    d_o = torch.randn(N, 8, 64, generator=gen).bfloat16().cuda()
    o, lse = attention_forward(plan, q, k, v, ak, 0.125)
    assert plan.tiles is not None and torch.isfinite(lse).all()
    dq, dk, dv, dak = attention_backward(plan, q, k, v, ak, 0.125, lse, d_o, o=o)
    o1, _ = attention_forward(plan, q, k, torch.ones_like(v), ak, 0.125)
    assert rel_err(o1.float().cpu(), torch.ones(N, 8, 64)) < 1e-2

    def inner(a, b):
        return (a.double() * b.double()).sum().item()

    def scale_of(a, b):
        return (a.double() * b.double()).abs().sum().item()

    lhs, rhs = inner(d_o, o), inner(v, dv)
    assert abs(lhs - rhs) < 1e-2 * scale_of(d_o, o), (lhs, rhs)
    lhs, rhs = inner(q, dq), inner(k, dk) + inner(ak, dak)
    assert abs(lhs - rhs) < 1e-2 * (scale_of(q, dq) + scale_of(k, dk)), (lhs, rhs)


def test_input_checks_run_before_the_path_is_chosen(oracle_lib):
    """embed_ak of another dtype (nn.Embedding weights under autocast), a table shorter than the plan's
    n_etypes, and an edge type beyond n_etypes must raise on every path, the tensor-core one included."""
    from bpt_b200.attention import AttentionPlan, attention_backward, attention_forward
    g = oracle_lib.binary_partition(64, False, 2, 10)
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    src, dst, et = [torch.from_numpy(g[n]).cuda() for n in ("src", "dst", "etype")]
    plan = AttentionPlan(src, dst, et, N, n_etypes=T)
    q = torch.randn(N, 8, 64, device="cuda").to(torch.bfloat16)
    ak32 = torch.randn(T, 64, device="cuda")
    with pytest.raises(RuntimeError, match="embed_ak"):
        attention_forward(plan, q, q, q, ak32, 0.125)
    with pytest.raises(RuntimeError, match="embed_ak"):
        attention_forward(plan, q, q, q, ak32.to(torch.bfloat16)[: T - 1].contiguous(), 0.125)
    o, lse = attention_forward(plan, q, q, q, ak32.to(torch.bfloat16), 0.125)
    with pytest.raises(RuntimeError, match="embed_ak"):
        attention_backward(plan, q, q, q, ak32, 0.125, lse, q, o=o)
    with pytest.raises(RuntimeError, match="embed_ak"):
        attention_backward(plan, q, q, q, ak32.to(torch.bfloat16)[: T - 1].contiguous(), 0.125, lse, q, o=o)
    with pytest.raises(RuntimeError, match="out of range"):
        AttentionPlan(src, dst, et, N, n_etypes=T - 1)
    with pytest.raises(RuntimeError, match="out of range"):
        AttentionPlan(src, dst, et, N - 1, n_etypes=T)
