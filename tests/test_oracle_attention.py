"""The floating-point oracle: C restatement (analytic backward) vs the torch op-by-op
restatement (autograd), and both vs dense attention on fully connected blocks, which is the
relation the reference's own graph_kernel/test.py asserts (dense bmm :185,364; dense softmax
:218,245,395,422; sparse.mm :274,459)."""
import numpy as np
import torch

import ops_torch
from helpers import fully_connected_blocks, rel_err


def _tensors(N, H, D, T, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(N, H, D, generator=g) * 0.5
    k = torch.randn(N, H, D, generator=g) * 0.5
    v = torch.randn(N, H, D, generator=g)
    ak = torch.randn(T, D, generator=g) * 0.5
    d_o = torch.randn(N, H, D, generator=g)
    return q, k, v, ak, d_o


def _torch_csr(csr):
    return [[torch.from_numpy(a) for a in csr[0]], [torch.from_numpy(a) for a in csr[1]]] + \
        [torch.from_numpy(a) for a in csr[2:]]


def test_c_oracle_equals_torch_chain(oracle_lib):
    g = oracle_lib.batch_graphs([oracle_lib.binary_partition(37, False, 2, 3),
                                 oracle_lib.binary_partition(64, True, 4, 10),
                                 oracle_lib.binary_partition(5, False, 1, 10)])
    N = g["n_nodes"]
    csr = oracle_lib.get_csrs(g["src"], g["dst"], N)
    H, D, T = 4, 16, 120
    q, k, v, ak, d_o = _tensors(N, H, D, T, 0)
    scale = 1.0 / np.sqrt(D)
    o, lse, p = oracle_lib.attn_fwd(csr[1], g["etype"], q.numpy(), k.numpy(), v.numpy(), ak.numpy(), scale)
    dq, dk, dv, dak = oracle_lib.attn_bwd(csr[1], csr[0], g["etype"], q.numpy(), k.numpy(), v.numpy(),
                                          ak.numpy(), scale, o, p, d_o.numpy())
    qd, kd, vd, akd = [t.double().requires_grad_(True) for t in (q, k, v, ak)]
    o2 = ops_torch.attention_chain(_torch_csr(csr), torch.from_numpy(g["etype"]), qd, kd, vd, akd, D)
    o2.backward(d_o.double())
    assert rel_err(o, o2.detach().numpy()) < 1e-13
    assert rel_err(dq, qd.grad.numpy()) < 1e-12
    assert rel_err(dk, kd.grad.numpy()) < 1e-12
    assert rel_err(dv, vd.grad.numpy()) < 1e-12
    assert rel_err(dak, akd.grad.numpy()) < 1e-12
    # rows of p sum to one over incoming edges
    sums = np.zeros((N, H))
    np.add.at(sums, g["dst"], p)
    assert np.allclose(sums, 1.0, atol=1e-12)
    # fp32 variant (the timed CPU baseline) agrees with fp64 to fp32 accuracy
    of, _, _ = oracle_lib.attn_fwd(csr[1], g["etype"], q.numpy(), k.numpy(), v.numpy(), ak.numpy(), scale,
                                   precision="f32")
    assert rel_err(of, o) < 1e-5


def test_oracle_equals_dense_attention(oracle_lib):
    B, L, H, D = 3, 11, 2, 8
    src, dst, N = fully_connected_blocks(B, L)
    csr = oracle_lib.get_csrs(src, dst, N)
    q, k, v, _, d_o = _tensors(N, H, D, 1, 1)
    scale = 1.0 / np.sqrt(D)
    o, lse, p = oracle_lib.attn_fwd(csr[1], None, q.numpy(), k.numpy(), v.numpy(), None, scale)
    qd, kd, vd = [t.double().view(B, L, H, D).transpose(1, 2).requires_grad_(True) for t in (q, k, v)]
    att = torch.softmax(qd @ kd.transpose(-1, -2) * scale, -1)
    od = (att @ vd).transpose(1, 2).reshape(N, H, D)
    assert rel_err(o, od.detach().numpy()) < 1e-13
    od.backward(d_o.double())
    dq, dk, dv, _ = oracle_lib.attn_bwd(csr[1], csr[0], None, q.numpy(), k.numpy(), v.numpy(), None, scale,
                                        o, p, d_o.numpy())
    for mine, ref in ((dq, qd.grad), (dk, kd.grad), (dv, vd.grad)):
        assert rel_err(mine, ref.transpose(1, 2).reshape(N, H, D).numpy()) < 1e-12


def test_span_rows_ignore_relative_term(oracle_lib):
    """Every incoming edge of a span node has the same type (builder.pyx:110-112), so the
    relative-position term shifts all its scores equally and leaves its output unchanged."""
    g = oracle_lib.binary_partition(64, False, 4, 10)
    N = g["n_nodes"]
    csr = oracle_lib.get_csrs(g["src"], g["dst"], N)
    q, k, v, ak, _ = _tensors(N, 2, 8, 100, 2)
    o1, _, _ = oracle_lib.attn_fwd(csr[1], g["etype"], q.numpy(), k.numpy(), v.numpy(), ak.numpy(), 0.3)
    o2, _, _ = oracle_lib.attn_fwd(csr[1], None, q.numpy(), k.numpy(), v.numpy(), None, 0.3)
    assert rel_err(o1[64:], o2[64:]) < 1e-12
    assert rel_err(o1[:64], o2[:64]) > 1e-3
