"""Op-by-op CPU restatement of the reference's eight graph operators in plain torch.
TEST INFRASTRUCTURE ONLY (never imported by the shipped package).

Each function computes what the corresponding kernel of graph_kernel/graphop_kernel.cu
computes, from the chunked-CSR arguments the reference passes (`row`/`indptr` are the chunk
arrays of partition_csr, graph_builder/builder.pyx:305-321).  Gradients come from torch
autograd through these functions, which makes them independent of the analytic backward
in bpt_oracle_attn.inc.
"""
import torch


def _expand_rows(row, indptr):
    """Row id of every CSR position, from the chunk arrays."""
    counts = indptr[1:] - indptr[:-1]
    return torch.repeat_interleave(row, counts)


def maskedmm_csr(row, indptr, eid, indices, A, B):
    """graphop_kernel.cu:40-55: y[eid[j]] = sum_d A[row_of(j)] * B[indices[j]] per head."""
    r = _expand_rows(row, indptr)
    y = (A[r] * B[indices]).sum(-1)
    out = torch.zeros((eid.numel(),) + tuple(y.shape[1:]), dtype=y.dtype)
    return out.index_copy(0, eid, y)


def node_mul_edge(row, indptr, eid, A, B):
    """graphop_kernel.cu:19-34: y[eid[j],h] = sum_d A[row_of(j),h,d] * B[eid[j],d]."""
    r = _expand_rows(row, indptr)
    a = A[r]
    b = B[eid]
    y = (a * b.unsqueeze(1)).sum(-1) if a.dim() == 3 else (a * b).sum(-1)
    out = torch.zeros((eid.numel(),) + tuple(y.shape[1:]), dtype=y.dtype)
    return out.index_copy(0, eid, y)


def sparse_softmax(row, indptr, eid, x, n_rows=None):
    """graphop_kernel.cu:170-202: softmax over the CSR positions of each row, per head."""
    r = _expand_rows(row, indptr)
    n = int(r.max()) + 1 if n_rows is None else n_rows
    xs = x[eid]
    shape = (n,) + tuple(xs.shape[1:])
    idx = r.view(-1, *([1] * (xs.dim() - 1))).expand_as(xs)
    m = torch.full(shape, -float("inf"), dtype=x.dtype).scatter_reduce(0, idx, xs.detach(), "amax")
    ex = torch.exp(xs - m[r])
    s = torch.zeros(shape, dtype=x.dtype).index_add(0, r, ex)
    y = ex / s[r]
    return torch.zeros_like(x).index_copy(0, eid, y)


def vector_spmm(row, indptr, eid, indices, edata, x):
    """graphop_kernel.cu:118-130: y[row_of(k)] += edata[eid[k]] * x[indices[k]] per head."""
    r = _expand_rows(row, indptr)
    w = edata[eid]
    xs = x[indices]
    contrib = w.unsqueeze(-1) * xs
    return torch.zeros_like(x).index_add(0, r, contrib)


def attention_chain(csr, etype, q, k, v, embed_ak, d_k):
    """modules/attention.py:54-77 with dropout off: the four operators chained the way
    BPTBlock.forward chains them.  csr is the 6-tuple of graph/base.py:71-86."""
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = csr
    e = maskedmm_csr(ROW, INDPTR_R, out_csr[2], out_csr[1], k, q)
    e_rel = 0
    if embed_ak is not None:
        ak = embed_ak[etype]
        e_rel = node_mul_edge(COL, INDPTR_C, in_csr[2], q, ak)
    p = sparse_softmax(COL, INDPTR_C, in_csr[2], (e_rel + e) / (d_k ** 0.5), n_rows=q.shape[0])
    return vector_spmm(COL, INDPTR_C, in_csr[2], in_csr[1], p, v)
