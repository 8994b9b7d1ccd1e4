"""The eight graph operators through the C ABI against the CPU restatement, on
binary-partition graphs and on the fully connected blocks of graph_kernel/test.py.
Tolerance: 1e-5 max-norm relative for fp32 (the bar set for this path), 1e-12 for fp64,
2e-2 for bf16."""
import numpy as np
import pytest
import torch

import ops_torch
from helpers import fully_connected_blocks, rel_err

pytestmark = pytest.mark.gpu

TOL = {torch.float64: 1e-12, torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 4e-3}


def _graph(oracle_lib, kind):
    if kind == "bpt":
        g = oracle_lib.batch_graphs([oracle_lib.binary_partition(300, False, 4, 10),
                                     oracle_lib.binary_partition(77, True, 2, 3),
                                     oracle_lib.binary_partition(513, False, 4, 10)])
        src, dst, N, etype = g["src"], g["dst"], g["n_nodes"], g["etype"]
    else:
        src, dst, N = fully_connected_blocks(6, 30)
        etype = (np.arange(len(src)) % 17).astype(np.int64)
    csr = oracle_lib.get_csrs(src, dst, N)
    return csr, N, len(src), etype


def _to(csr, device):
    f = lambda a: torch.from_numpy(a).to(device)
    return [[f(a) for a in csr[0]], [f(a) for a in csr[1]], f(csr[2]), f(csr[3]), f(csr[4]), f(csr[5])]


def _softmax_longdouble(row, indptr, eid, x, n_rows):
    """Edge softmax over the CSR rows in numpy long double (80-bit on x86): the tie-breaker between the
    fp64 kernel and the fp64 torch restatement."""
    r = ops_torch._expand_rows(row, indptr).numpy()
    e = eid.numpy()
    xs = x[e].astype(np.longdouble)
    m = np.full((n_rows,) + xs.shape[1:], -np.inf, dtype=np.longdouble)
    np.maximum.at(m, r, xs)
    ex = np.exp(xs - m[r])
    ssum = np.zeros_like(m)
    np.add.at(ssum, r, ex)
    y = np.zeros(x.shape, dtype=np.longdouble)
    y[e] = ex / ssum[r]
    return y.astype(np.float64)


def _rand(shape, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype)


@pytest.mark.parametrize("kind", ["bpt", "dense"])
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd", [(8, 64), (1, 40), (6, 50)])
def test_operators_forward_backward(oracle_lib, kind, dtype, hd):
    from bpt_b200 import op
    h, d = hd
    csr, N, E, _ = _graph(oracle_lib, kind)
    c = _to(csr, "cpu")
    g = _to(csr, "cuda")
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = g
    nshape = (N, d) if h == 1 else (N, h, d)
    eshape = (E,) if h == 1 else (E, h)
    tol = TOL[dtype]

    def pair(shape, seed, scale=1.0):
        t = _rand(shape, seed, dtype) * scale
        return t.double().clone().requires_grad_(True), t.clone().cuda().requires_grad_(True)

    # masked_mm (SDDMM), called as attention.py:66-67 does: A = k, B = q over the out-CSR
    (a_ref, a_gpu), (b_ref, b_gpu) = pair(nshape, 1, 0.3), pair(nshape, 2, 0.3)
    dy = _rand(eshape, 3, dtype)
    y_ref = ops_torch.maskedmm_csr(c[2], c[3], c[0][2], c[0][1], a_ref, b_ref)
    y_gpu = op.masked_mm(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2], in_csr[1], a_gpu, b_gpu)
    assert y_gpu.shape == eshape and y_gpu.dtype == dtype
    assert rel_err(y_gpu.detach().double().cpu(), y_ref.detach()) < tol
    y_ref.backward(dy.double())
    y_gpu.backward(dy.cuda())
    assert rel_err(a_gpu.grad.double().cpu(), a_ref.grad) < tol
    assert rel_err(b_gpu.grad.double().cpu(), b_ref.grad) < tol

    # node_mul_edge over the in-CSR (attention.py:69-71)
    (a_ref, a_gpu), (b_ref, b_gpu) = pair(nshape, 4, 0.3), pair((E, d), 5, 0.3)
    y_ref = ops_torch.node_mul_edge(c[4], c[5], c[1][2], a_ref, b_ref)
    y_gpu = op.node_mul_edge(COL, INDPTR_C, in_csr[2], a_gpu, b_gpu)
    assert rel_err(y_gpu.detach().double().cpu(), y_ref.detach()) < tol
    y_ref.backward(dy.double())
    y_gpu.backward(dy.cuda())
    assert rel_err(a_gpu.grad.double().cpu(), a_ref.grad) < tol
    assert rel_err(b_gpu.grad.double().cpu(), b_ref.grad) < tol

    # sparse_softmax over the in-CSR and over the out-CSR (test.py:218 and :245 check both)
    for (rw, ip, ed, crw, cip, ced) in ((COL, INDPTR_C, in_csr[2], c[4], c[5], c[1][2]),
                                        (ROW, INDPTR_R, out_csr[2], c[2], c[3], c[0][2])):
        x_ref, x_gpu = pair(eshape, 6, 2.0)
        y_ref = ops_torch.sparse_softmax(crw, cip, ced, x_ref, n_rows=N)
        y_gpu = op.sparse_softmax(rw, ip, ed, x_gpu)
        err = rel_err(y_gpu.detach().double().cpu(), y_ref.detach())
        restatement_moved = False
        if dtype == torch.float64 and not err < tol:
            # The torch restatement runs on whatever vector math library the host's torch build picks;
            # an isolated 5e-10 between it and the kernel was seen in some first processes on a
            # machine, with both sides bitwise stable when rerun.  A third opinion in extended
            # precision (numpy long double, exp and sums) decides: the kernel must be within 1e-12 of it.
            truth = _softmax_longdouble(crw, cip, ced, x_ref.detach().numpy(), N)
            err_gpu = rel_err(y_gpu.detach().double().cpu().numpy(), truth)
            err_cpu = rel_err(y_ref.detach().numpy(), truth)
            print("sparse_softmax fp64: kernel vs torch restatement %.3e; kernel vs long double %.3e; "
                  "torch restatement vs long double %.3e (CPU threads %d)" % (err, err_gpu, err_cpu,
                                                                              torch.get_num_threads()))
            err, restatement_moved = err_gpu, err_cpu > tol
        assert err < tol
        y_ref.backward(dy.double())
        y_gpu.backward(dy.cuda())
        # graph_kernel/test.py:239 relaxes softmax gradients to rtol 1e-3 in fp32; we keep 10x the forward bar
        # (when the restatement's forward was the side that moved, its gradient carries that error)
        assert rel_err(x_gpu.grad.double().cpu(), x_ref.grad) < (1e-8 if restatement_moved else 10 * tol)

    # vec_spmm over the in-CSR with the out-CSR as its transpose (attention.py:74-77)
    (w_ref, w_gpu), (x_ref, x_gpu) = pair(eshape, 7, 0.2), pair(nshape, 8)
    dyn = _rand(nshape, 9, dtype)
    y_ref = ops_torch.vector_spmm(c[4], c[5], c[1][2], c[1][1], w_ref, x_ref)
    y_gpu = op.vec_spmm(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2], out_csr[1], w_gpu, x_gpu)
    assert rel_err(y_gpu.detach().double().cpu(), y_ref.detach()) < tol
    y_ref.backward(dyn.double())
    y_gpu.backward(dyn.cuda())
    assert rel_err(w_gpu.grad.double().cpu(), w_ref.grad) < tol
    assert rel_err(x_gpu.grad.double().cpu(), x_ref.grad) < tol


def test_dense_equivalences_of_reference_test_script():
    """graph_kernel/test.py:364,395,459 in miniature: on fully connected blocks the operators
    equal batched matmul, dense softmax and dense matmul."""
    from bpt_b200 import csr as csrmod, op
    B, L, h, d = 16, 30, 8, 64
    src, dst, N = fully_connected_blocks(B, L)
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = csrmod.get_csrs(
        torch.from_numpy(src).cuda(), torch.from_numpy(dst).cuda(), N)
    torch.manual_seed(0)
    A = torch.rand(N, h, d, device="cuda")
    Bm = torch.rand(N, h, d, device="cuda")
    y = op.masked_mm(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2], in_csr[1], A, Bm)
    dense = (A.view(B, L, h, d).transpose(1, 2) @ Bm.view(B, L, h, d).permute(0, 2, 3, 1)).permute(0, 2, 3, 1)
    assert torch.allclose(y, dense.reshape(-1, h), rtol=1e-5, atol=1e-5)
    x = torch.rand(B * L * L, h, device="cuda")
    assert torch.allclose(op.sparse_softmax(ROW, INDPTR_R, out_csr[2], x),
                          torch.softmax(x.view(B, L, L, h), -2).view(-1, h), rtol=1e-5, atol=1e-7)
    assert torch.allclose(op.sparse_softmax(COL, INDPTR_C, in_csr[2], x),
                          torch.softmax(x.view(B, L, L, h), -3).view(-1, h), rtol=1e-5, atol=1e-7)
    w = torch.rand(B * L * L, h, device="cuda")
    yv = op.vec_spmm(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2], out_csr[1], w, A)
    dense = torch.einsum("bsth,bshd->bthd", w.view(B, L, L, h), A.view(B, L, h, d)).reshape(N, h, d)
    assert torch.allclose(yv, dense, rtol=1e-5, atol=1e-5)


def test_operators_are_bitwise_reproducible(oracle_lib):
    """The reference's sums go through atomics and differ run to run; these must not."""
    from bpt_b200 import graphop
    csr, N, E, _ = _graph(oracle_lib, "bpt")
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = _to(csr, "cuda")
    torch.manual_seed(1)
    w = torch.rand(E, 8, device="cuda")
    x = torch.randn(N, 8, 64, device="cuda")
    dy = torch.randn(E, 8, device="cuda")
    runs = []
    for _ in range(3):
        y = graphop.vector_spmm_forward(COL, INDPTR_C, in_csr[2], in_csr[1], w, x)
        dA, dB = graphop.maskedmm_csr_backward(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C,
                                               in_csr[2], in_csr[1], x, x, dy)
        runs.append((y.clone(), dA.clone(), dB.clone()))
    for r in runs[1:]:
        for a, b in zip(runs[0], r):
            assert torch.equal(a, b)


def test_input_checks_raise():
    from bpt_b200 import graphop
    idx = torch.zeros(1, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="CUDA"):
        graphop.sparse_softmax_forward(idx, idx, idx, torch.zeros(1, 8))
    x = torch.zeros(4, 8, device="cuda").t()
    c = idx.cuda()
    with pytest.raises(RuntimeError, match="contiguous"):
        graphop.sparse_softmax_forward(c, c, c, x)
