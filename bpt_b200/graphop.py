"""GPU counterpart of the reference's `graphop` extension module.

The eight functions have the names, argument order, argument meaning and return values of
the ones exported at graph_kernel/graphop.cpp:216-225, so `from graphop import *` in the
reference's modules/op.py:2 resolves against this module (see `bpt_b200.install_dropin`).
Inputs must be contiguous CUDA tensors, as CHECK_INPUT demands at graphop.cpp:4-6; a
violation raises RuntimeError like AT_ASSERTM does.  Index tensors are int64.  Feature
tensors may be float32/float64 as in the reference, or bfloat16/float16 (fp32 accumulation).
Each call launches on the current stream of the tensors' device and does not synchronise.
"""
import torch

from . import _lib


def _check(*tensors):
    _lib.require_cuda(*tensors)


def _hd(t):
    """(h, d) of a node feature tensor: (N, d) is single-head (graphop_kernel.cu:247)."""
    return (1, t.size(-1)) if t.dim() == 2 else (t.size(1), t.size(-1))


def _edge_out(e, h, like):
    return torch.zeros((e,) if h == 1 else (e, h), dtype=like.dtype, device=like.device)


def maskedmm_csr_forward(row, indptr, eid, indices, A, B):
    """graphop.cpp:16-30: y[eid[j]] = <A[row of j], B[indices[j]]> per head; y is (E,) or (E,h)."""
    _check(row, indptr, eid, indices, A, B)
    h, d = _hd(A)
    y = _edge_out(eid.size(0), h, A)
    with torch.cuda.device(A.device):
        _lib.check(_lib.lib().bpt_maskedmm_csr_forward(
            row.data_ptr(), indptr.data_ptr(), eid.data_ptr(), indices.data_ptr(), row.size(0),
            A.data_ptr(), B.data_ptr(), y.data_ptr(), h, d, _lib.dtype_code(A.dtype), _lib.stream()))
    return y


def maskedmm_csr_backward(row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B, dy):
    """graphop.cpp:104-131: returns [dA, dB]."""
    dy = dy.contiguous()  # the reference does not check dy (graphop.cpp:120-130)
    _check(row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B, dy)
    h, d = _hd(A)
    dA = torch.empty_like(A)
    dB = torch.empty_like(B)
    with torch.cuda.device(A.device):
        _lib.check(_lib.lib().bpt_maskedmm_csr_backward(
            row.data_ptr(), indptr_r.data_ptr(), eid_r.data_ptr(), indices_r.data_ptr(), row.size(0),
            col.data_ptr(), indptr_c.data_ptr(), eid_c.data_ptr(), indices_c.data_ptr(), col.size(0),
            A.data_ptr(), B.data_ptr(), dy.data_ptr(), dA.data_ptr(), dB.data_ptr(),
            A.size(0), B.size(0), h, d, _lib.dtype_code(A.dtype), _lib.stream()))
    return [dA, dB]


def node_mul_edge_forward(row, indptr, eid, A, B):
    """graphop.cpp:38-51: y[eid[j],h] = <A[row of j,h], B[eid[j]]>."""
    _check(row, indptr, eid, A, B)
    h, d = _hd(A)
    y = _edge_out(eid.size(0), h, A)
    with torch.cuda.device(A.device):
        _lib.check(_lib.lib().bpt_node_mul_edge_forward(
            row.data_ptr(), indptr.data_ptr(), eid.data_ptr(), row.size(0),
            A.data_ptr(), B.data_ptr(), y.data_ptr(), h, d, _lib.dtype_code(A.dtype), _lib.stream()))
    return y


def node_mul_edge_backward(row, indptr, eid, A, B, dy):
    """graphop.cpp:133-154: returns [dA, dB]."""
    dy = dy.contiguous()
    _check(row, indptr, eid, A, B, dy)
    h, d = _hd(A)
    dA = torch.empty_like(A)
    dB = torch.zeros_like(B)
    with torch.cuda.device(A.device):
        _lib.check(_lib.lib().bpt_node_mul_edge_backward(
            row.data_ptr(), indptr.data_ptr(), eid.data_ptr(), row.size(0),
            A.data_ptr(), B.data_ptr(), dy.data_ptr(), dA.data_ptr(), dB.data_ptr(), A.size(0),
            h, d, _lib.dtype_code(A.dtype), _lib.stream()))
    return [dA, dB]


def sparse_softmax_forward(row, indptr, eid, x):
    """graphop.cpp:59-70: softmax over each CSR row's entries, per head."""
    _check(row, indptr, eid, x)
    h = 1 if x.dim() == 1 else x.size(1)
    y = torch.zeros_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().bpt_sparse_softmax_forward(
            row.data_ptr(), indptr.data_ptr(), eid.data_ptr(), row.size(0),
            x.data_ptr(), y.data_ptr(), h, _lib.dtype_code(x.dtype), _lib.stream()))
    return y


def sparse_softmax_backward(row, indptr, eid, y, dy):
    """graphop.cpp:156-171: dx = y * (dy - sum_row(dy * y))."""
    dy = dy.contiguous()
    _check(row, indptr, eid, y, dy)
    h = 1 if y.dim() == 1 else y.size(1)
    dx = torch.zeros_like(y)
    with torch.cuda.device(y.device):
        _lib.check(_lib.lib().bpt_sparse_softmax_backward(
            row.data_ptr(), indptr.data_ptr(), eid.data_ptr(), row.size(0),
            y.data_ptr(), dy.data_ptr(), dx.data_ptr(), h, _lib.dtype_code(y.dtype), _lib.stream()))
    return dx


def vector_spmm_forward(row, indptr, eid, indices, edata, x):
    """graphop.cpp:80-95: y[r] = sum_j edata[eid[j]] * x[indices[j]] per head."""
    _check(row, indptr, eid, indices, edata, x)
    h, d = _hd(x)
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().bpt_vector_spmm_forward(
            row.data_ptr(), indptr.data_ptr(), eid.data_ptr(), indices.data_ptr(), row.size(0),
            edata.data_ptr(), x.data_ptr(), y.data_ptr(), x.size(0), h, d,
            _lib.dtype_code(x.dtype), _lib.stream()))
    return y


def vector_spmm_backward(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, edata, dy, x):
    """graphop.cpp:173-214: returns [dedata, dx]."""
    dy = dy.contiguous()
    _check(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, edata, dy, x)
    h, d = _hd(x)
    dedata = torch.zeros_like(edata)
    dx = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().bpt_vector_spmm_backward(
            row.data_ptr(), indptr.data_ptr(), eid.data_ptr(), indices.data_ptr(), row.size(0),
            col.data_ptr(), indptr_t.data_ptr(), eid_t.data_ptr(), indices_t.data_ptr(), col.size(0),
            edata.data_ptr(), dy.data_ptr(), x.data_ptr(), dedata.data_ptr(), dx.data_ptr(),
            x.size(0), h, d, _lib.dtype_code(x.dtype), _lib.stream()))
    return [dedata, dx]


__all__ = [
    "maskedmm_csr_forward", "maskedmm_csr_backward", "node_mul_edge_forward", "node_mul_edge_backward",
    "sparse_softmax_forward", "sparse_softmax_backward", "vector_spmm_forward", "vector_spmm_backward",
]
