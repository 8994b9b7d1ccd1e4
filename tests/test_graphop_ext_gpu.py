"""The thin torch C++ extension (bpt_b200._graphop_ext, the reference's `graphop` module over the C-ABI
library) against the ctypes module bpt_b200.graphop: the same kernels behind both, so every one of the
eight functions must return bitwise the same tensors, in fp32 and bf16, on a binary-partition batch with
duplicate edges; and wrong inputs raise RuntimeError as CHECK_INPUT does (graph_kernel/graphop.cpp:4-6)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _csr(oracle_lib):
    g = oracle_lib.batch_graphs([oracle_lib.binary_partition(300, False, 4, 10), oracle_lib.binary_partition(513, False, 4, 10)])
    N = g["n_nodes"]
    csr = oracle_lib.get_csrs(g["src"], g["dst"], N)
    parts = []
    for indptr, indices, eid in (csr[1], csr[0]):  # in-CSR (rows = destinations), out-CSR (rows = sources)
        row, ptr = oracle_lib.partition_csr(indptr, 32)
        parts.append([torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (row, ptr, eid, indices)])
    return N, g["n_edges"], parts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_extension_equals_ctypes_module(oracle_lib, dtype):
    import bpt_b200
    import bpt_b200.graphop
    ext, ref = bpt_b200.graphop_extension(), bpt_b200.graphop
    N, E, ((row, ptr, eid, idx), (col, ptr_t, eid_t, idx_t)) = _csr(oracle_lib)
    gen = torch.Generator().manual_seed(0)
    rnd = lambda *shape: (torch.randn(*shape, generator=gen) * 0.3).to(dtype).cuda()
    A, B, x, dyn = rnd(N, 4, 32), rnd(N, 4, 32), rnd(N, 4, 32), rnd(N, 4, 32)
    Be, w, dye = rnd(E, 32), rnd(E, 4), rnd(E, 4)
    calls = [
        ("maskedmm_csr_forward", (row, ptr, eid, idx, A, B)),
        ("maskedmm_csr_backward", (row, ptr, eid, idx, col, ptr_t, eid_t, idx_t, A, B, dye)),
        ("node_mul_edge_forward", (row, ptr, eid, A, Be)),
        ("node_mul_edge_backward", (row, ptr, eid, A, Be, dye)),
        ("sparse_softmax_forward", (row, ptr, eid, w)),
        ("sparse_softmax_backward", (row, ptr, eid, torch.rand(E, 4, generator=gen).to(dtype).cuda(), dye)),
        ("vector_spmm_forward", (row, ptr, eid, idx, w, x)),
        ("vector_spmm_backward", (row, ptr, eid, idx, col, ptr_t, eid_t, idx_t, w, dyn, x)),
    ]
    for name, args in calls:
        got, want = getattr(ext, name)(*args), getattr(ref, name)(*args)
        got, want = (got, want) if isinstance(want, (list, tuple)) else ([got], [want])
        assert len(got) == len(want), name
        for a, b in zip(got, want):
            assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b), name


def test_extension_rejects_what_check_input_rejects(oracle_lib):
    import bpt_b200
    ext = bpt_b200.graphop_extension()
    N, E, ((row, ptr, eid, idx), _) = _csr(oracle_lib)
    w = torch.randn(E, 4).cuda()
    with pytest.raises(RuntimeError):
        ext.sparse_softmax_forward(row, ptr, eid, w.cpu())
    with pytest.raises(RuntimeError):
        ext.sparse_softmax_forward(row, ptr, eid, w.t())
    with pytest.raises(RuntimeError):
        ext.sparse_softmax_forward(row.int(), ptr, eid, w)
