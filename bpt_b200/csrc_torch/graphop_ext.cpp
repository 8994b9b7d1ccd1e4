// Thin torch C++ extension over the C-ABI library: the reference's `graphop` module
// (graph_kernel/graphop.cpp:216-225) with the same eight functions, argument order and return
// values, so `from graphop import *` in modules/op.py:2 binds to compiled code as it does in the
// reference.  Nothing is computed here: every function checks its tensors the way CHECK_INPUT does
// (graphop.cpp:4-6: CUDA and contiguous, else an error), allocates the outputs as torch tensors and
// hands plain pointers, sizes and the current stream to libbpt_b200.so (include/bpt_b200.h).
// Index tensors are int64; features float32/float64 as in the reference, or bfloat16/float16.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <vector>

#include "../../include/bpt_b200.h"

namespace {

void check_input(const at::Tensor &t, const char *name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
void check_index(const at::Tensor &t, const char *name) {
    check_input(t, name);
    TORCH_CHECK(t.scalar_type() == at::kLong, name, " must be int64");
}
#define CHECK_INPUT(x) check_input(x, #x)
#define CHECK_INDEX(x) check_index(x, #x)

int dtype_code(const at::Tensor &t) {
    switch (t.scalar_type()) {
        case at::kFloat: return BPT_F32;
        case at::kDouble: return BPT_F64;
        case at::kBFloat16: return BPT_BF16;
        case at::kHalf: return BPT_F16;
        default: TORCH_CHECK(false, "graphop: unsupported dtype ", t.scalar_type());
    }
    return -1;
}
void check_rc(int rc) { TORCH_CHECK(rc == BPT_OK, bpt_last_error()); }
bpt_stream_t stream_of(const at::Tensor &t) {
    return reinterpret_cast<bpt_stream_t>(c10::cuda::getCurrentCUDAStream(t.get_device()).stream());
}
const int64_t *idx(const at::Tensor &t) { return t.data_ptr<int64_t>(); }
// (h, d) of a node feature tensor: (N, d) is single-head (graphop_kernel.cu:247)
int heads(const at::Tensor &t) { return t.dim() == 2 ? 1 : static_cast<int>(t.size(1)); }
int width(const at::Tensor &t) { return static_cast<int>(t.size(-1)); }
at::Tensor edge_out(int64_t e, int h, const at::Tensor &like) {
    return h == 1 ? at::zeros({e}, like.options()) : at::zeros({e, h}, like.options());
}

}  // namespace

// graphop.cpp:16-30
at::Tensor maskedmm_csr_forward(const at::Tensor &row, const at::Tensor &indptr, const at::Tensor &eid,
                                const at::Tensor &indices, const at::Tensor &A, const at::Tensor &B) {
    CHECK_INDEX(row); CHECK_INDEX(indptr); CHECK_INDEX(eid); CHECK_INDEX(indices); CHECK_INPUT(A); CHECK_INPUT(B);
    const c10::cuda::CUDAGuard guard(A.device());
    const int h = heads(A), d = width(A);
    at::Tensor y = edge_out(eid.size(0), h, A);
    check_rc(bpt_maskedmm_csr_forward(idx(row), idx(indptr), idx(eid), idx(indices), row.size(0), A.data_ptr(),
                                      B.data_ptr(), y.data_ptr(), h, d, dtype_code(A), stream_of(A)));
    return y;
}

// graphop.cpp:108-131
std::vector<at::Tensor> maskedmm_csr_backward(const at::Tensor &row, const at::Tensor &indptr_r, const at::Tensor &eid_r,
                                              const at::Tensor &indices_r, const at::Tensor &col,
                                              const at::Tensor &indptr_c, const at::Tensor &eid_c,
                                              const at::Tensor &indices_c, const at::Tensor &A, const at::Tensor &B,
                                              const at::Tensor &dy_) {
    const at::Tensor dy = dy_.contiguous();  // the reference does not check dy (graphop.cpp:120-130)
    CHECK_INDEX(row); CHECK_INDEX(indptr_r); CHECK_INDEX(eid_r); CHECK_INDEX(indices_r);
    CHECK_INDEX(col); CHECK_INDEX(indptr_c); CHECK_INDEX(eid_c); CHECK_INDEX(indices_c);
    CHECK_INPUT(A); CHECK_INPUT(B); CHECK_INPUT(dy);
    const c10::cuda::CUDAGuard guard(A.device());
    const int h = heads(A), d = width(A);
    at::Tensor dA = at::empty_like(A), dB = at::empty_like(B);
    check_rc(bpt_maskedmm_csr_backward(idx(row), idx(indptr_r), idx(eid_r), idx(indices_r), row.size(0), idx(col),
                                       idx(indptr_c), idx(eid_c), idx(indices_c), col.size(0), A.data_ptr(),
                                       B.data_ptr(), dy.data_ptr(), dA.data_ptr(), dB.data_ptr(), A.size(0), B.size(0),
                                       h, d, dtype_code(A), stream_of(A)));
    return {dA, dB};
}

// graphop.cpp:39-51
at::Tensor node_mul_edge_forward(const at::Tensor &row, const at::Tensor &indptr, const at::Tensor &eid,
                                 const at::Tensor &A, const at::Tensor &B) {
    CHECK_INDEX(row); CHECK_INDEX(indptr); CHECK_INDEX(eid); CHECK_INPUT(A); CHECK_INPUT(B);
    const c10::cuda::CUDAGuard guard(A.device());
    const int h = heads(A), d = width(A);
    at::Tensor y = edge_out(eid.size(0), h, A);
    check_rc(bpt_node_mul_edge_forward(idx(row), idx(indptr), idx(eid), row.size(0), A.data_ptr(), B.data_ptr(),
                                       y.data_ptr(), h, d, dtype_code(A), stream_of(A)));
    return y;
}

// graphop.cpp:141-154
std::vector<at::Tensor> node_mul_edge_backward(const at::Tensor &row, const at::Tensor &indptr, const at::Tensor &eid,
                                               const at::Tensor &A, const at::Tensor &B, const at::Tensor &dy_) {
    const at::Tensor dy = dy_.contiguous();
    CHECK_INDEX(row); CHECK_INDEX(indptr); CHECK_INDEX(eid); CHECK_INPUT(A); CHECK_INPUT(B); CHECK_INPUT(dy);
    const c10::cuda::CUDAGuard guard(A.device());
    const int h = heads(A), d = width(A);
    at::Tensor dA = at::empty_like(A), dB = at::zeros_like(B);
    check_rc(bpt_node_mul_edge_backward(idx(row), idx(indptr), idx(eid), row.size(0), A.data_ptr(), B.data_ptr(),
                                        dy.data_ptr(), dA.data_ptr(), dB.data_ptr(), A.size(0), h, d, dtype_code(A),
                                        stream_of(A)));
    return {dA, dB};
}

// graphop.cpp:59-70
at::Tensor sparse_softmax_forward(const at::Tensor &row, const at::Tensor &indptr, const at::Tensor &eid,
                                  const at::Tensor &x) {
    CHECK_INDEX(row); CHECK_INDEX(indptr); CHECK_INDEX(eid); CHECK_INPUT(x);
    const c10::cuda::CUDAGuard guard(x.device());
    const int h = x.dim() == 1 ? 1 : static_cast<int>(x.size(1));
    at::Tensor y = at::zeros_like(x);
    check_rc(bpt_sparse_softmax_forward(idx(row), idx(indptr), idx(eid), row.size(0), x.data_ptr(), y.data_ptr(), h,
                                        dtype_code(x), stream_of(x)));
    return y;
}

// graphop.cpp:163-171
at::Tensor sparse_softmax_backward(const at::Tensor &row, const at::Tensor &indptr, const at::Tensor &eid,
                                   const at::Tensor &y, const at::Tensor &dy_) {
    const at::Tensor dy = dy_.contiguous();
    CHECK_INDEX(row); CHECK_INDEX(indptr); CHECK_INDEX(eid); CHECK_INPUT(y); CHECK_INPUT(dy);
    const c10::cuda::CUDAGuard guard(y.device());
    const int h = y.dim() == 1 ? 1 : static_cast<int>(y.size(1));
    at::Tensor dx = at::zeros_like(y);
    check_rc(bpt_sparse_softmax_backward(idx(row), idx(indptr), idx(eid), row.size(0), y.data_ptr(), dy.data_ptr(),
                                         dx.data_ptr(), h, dtype_code(y), stream_of(y)));
    return dx;
}

// graphop.cpp:79-93
at::Tensor vector_spmm_forward(const at::Tensor &row, const at::Tensor &indptr, const at::Tensor &eid,
                               const at::Tensor &indices, const at::Tensor &edata, const at::Tensor &x) {
    CHECK_INDEX(row); CHECK_INDEX(indptr); CHECK_INDEX(eid); CHECK_INDEX(indices); CHECK_INPUT(edata); CHECK_INPUT(x);
    const c10::cuda::CUDAGuard guard(x.device());
    const int h = heads(x), d = width(x);
    at::Tensor y = at::empty_like(x);
    check_rc(bpt_vector_spmm_forward(idx(row), idx(indptr), idx(eid), idx(indices), row.size(0), edata.data_ptr(),
                                     x.data_ptr(), y.data_ptr(), x.size(0), h, d, dtype_code(x), stream_of(x)));
    return y;
}

// graphop.cpp:190-214
std::vector<at::Tensor> vector_spmm_backward(const at::Tensor &row, const at::Tensor &indptr, const at::Tensor &eid,
                                             const at::Tensor &indices, const at::Tensor &col,
                                             const at::Tensor &indptr_t, const at::Tensor &eid_t,
                                             const at::Tensor &indices_t, const at::Tensor &edata,
                                             const at::Tensor &dy_, const at::Tensor &x) {
    const at::Tensor dy = dy_.contiguous();
    CHECK_INDEX(row); CHECK_INDEX(indptr); CHECK_INDEX(eid); CHECK_INDEX(indices);
    CHECK_INDEX(col); CHECK_INDEX(indptr_t); CHECK_INDEX(eid_t); CHECK_INDEX(indices_t);
    CHECK_INPUT(edata); CHECK_INPUT(dy); CHECK_INPUT(x);
    const c10::cuda::CUDAGuard guard(x.device());
    const int h = heads(x), d = width(x);
    at::Tensor dedata = at::zeros_like(edata), dx = at::empty_like(x);
    check_rc(bpt_vector_spmm_backward(idx(row), idx(indptr), idx(eid), idx(indices), row.size(0), idx(col),
                                      idx(indptr_t), idx(eid_t), idx(indices_t), col.size(0), edata.data_ptr(),
                                      dy.data_ptr(), x.data_ptr(), dedata.data_ptr(), dx.data_ptr(), x.size(0), h, d,
                                      dtype_code(x), stream_of(x)));
    return {dedata, dx};
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "The reference's graphop module on libbpt_b200.so";
    m.def("maskedmm_csr_forward", &maskedmm_csr_forward, "y[e] = <A[dst(e)], B[src(e)]> per head over the chunked CSR");
    m.def("maskedmm_csr_backward", &maskedmm_csr_backward, "[dA, dB] of maskedmm_csr_forward (CSR and its transpose)");
    m.def("node_mul_edge_forward", &node_mul_edge_forward, "y[e, h] = <A[dst(e), h], B[e]>");
    m.def("node_mul_edge_backward", &node_mul_edge_backward, "[dA, dB] of node_mul_edge_forward");
    m.def("sparse_softmax_forward", &sparse_softmax_forward, "softmax over the entries of each CSR row, per head");
    m.def("sparse_softmax_backward", &sparse_softmax_backward, "dx = y * (dy - sum over the row of dy * y)");
    m.def("vector_spmm_forward", &vector_spmm_forward, "y[r] = sum over the row of edata[e] * x[src(e)], per head");
    m.def("vector_spmm_backward", &vector_spmm_backward, "[dedata, dx] of vector_spmm_forward (CSR and its transpose)");
}
