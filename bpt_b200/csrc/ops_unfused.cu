// The eight graph operators of the reference's `graphop` module as deterministic kernels.
//
// The reference (graph_kernel/graphop_kernel.cu) gives every <=32-edge chunk its own block and
// lets chunks of the same row meet in floating-point atomics.  Here the chunk arrays are read
// only to find where a row starts and ends: the block of a row's first chunk owns the whole
// row, every output element has one writer and a fixed summation order, and blocks of the
// row's other chunks return at once.  Per-edge outputs (the SDDMM-type operators) have no
// cross-chunk reduction and keep one block per chunk.
#include "common.cuh"

namespace bpt {
namespace {

// True when chunk c is the first chunk of its row; then [beg, end) is the row's CSR range.
// Requires the chunk arrays of partition_csr: rows non-decreasing.
__device__ __forceinline__ bool row_range(const int64_t *__restrict__ row, const int64_t *__restrict__ indptr,
                                          int64_t n_chunks, int64_t c, int64_t &r, int64_t &beg,
                                          int64_t &end) {
    r = row[c];
    if (c > 0 && row[c - 1] == r) return false;
    int64_t lo = c + 1, hi = n_chunks;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (row[mid] > r) hi = mid; else lo = mid + 1;
    }
    beg = indptr[c];
    end = indptr[lo];
    return true;
}

constexpr int kGroup = 8;  // lanes that share one (edge, head) dot product

// ---------------------------------------------------------------- per-edge dot products
// y[eid[j], hh] = sum_d A[row[c], hh, d] * X[...]:
//   kPerHead:  X = B[indices[j], hh, d]   (maskedmm_csr_forward, vector_spmm_backward's dedata)
//   !kPerHead: X = B[eid[j], d]           (node_mul_edge_forward)
template <typename T, bool kPerHead>
__global__ void edge_dot_kernel(const int64_t *__restrict__ row, const int64_t *__restrict__ indptr,
                                const int64_t *__restrict__ eid, const int64_t *__restrict__ indices,
                                int64_t n_chunks, const T *__restrict__ A, const T *__restrict__ B,
                                T *__restrict__ y, int h, int d) {
    using acc_t = typename Acc<T>::type;
    const int warps_per_block = blockDim.x >> 5;
    const int64_t c = blockIdx.x * static_cast<int64_t>(warps_per_block) + (threadIdx.x >> 5);
    if (c >= n_chunks) return;
    const int lane = threadIdx.x & 31;
    const int g = lane / kGroup, gl = lane % kGroup;
    const int64_t beg = indptr[c], end = indptr[c + 1];
    const T *a_row = A + row[c] * h * static_cast<int64_t>(d);
    const int64_t pairs = (end - beg) * h;
    for (int64_t p0 = 0; p0 < pairs; p0 += 32 / kGroup) {
        const int64_t p = p0 + g;
        acc_t sum = 0;
        int64_t e = 0;
        int hh = 0;
        if (p < pairs) {
            const int64_t j = beg + p / h;
            hh = static_cast<int>(p % h);
            e = eid[j];
            const T *a = a_row + static_cast<int64_t>(hh) * d;
            const T *x = kPerHead ? B + (indices[j] * h + hh) * static_cast<int64_t>(d)
                                  : B + e * static_cast<int64_t>(d);
            for (int i = gl; i < d; i += kGroup) sum += to_acc(a[i]) * to_acc(x[i]);
        }
#pragma unroll
        for (int off = kGroup / 2; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (p < pairs && gl == 0) y[e * h + hh] = from_acc<T>(sum);
    }
}

// ---------------------------------------------------------------- row sums, one writer per column
// out[r, j] = sum_k W[eid[k], j / d] * X[...], k over the whole row, j in [0, h*d):
//   kEdgeX == false: X = Xn[indices[k], j]      (vector_spmm fwd, its dx, maskedmm_csr bwd)
//   kEdgeX == true:  X = Xe[eid[k], j % d]      (node_mul_edge bwd, dA)
// The block of the row's first chunk owns the row.  Its kRowWarps warps take the row's entries
// round-robin (warp w: entries w, w + kRowWarps, ...), each lane summing kRowCols columns 32 apart,
// so a row of thousands of entries (a span node near the root) is walked by eight warps with
// several independent loads in flight instead of one thread per column walking it alone.  The
// warps' partial sums meet in shared memory and are added in warp order: one writer per output
// element, fixed order.  Rows wider than 32 * kRowCols columns take several passes.
constexpr int kRowWarps = 8;
constexpr int kRowCols = 8;

template <typename T, bool kEdgeX>
__global__ void __launch_bounds__(kRowWarps * 32)
row_sum_kernel(const int64_t *__restrict__ row, const int64_t *__restrict__ indptr,
               const int64_t *__restrict__ eid, const int64_t *__restrict__ indices,
               int64_t n_chunks, const T *__restrict__ W, const T *__restrict__ X,
               T *__restrict__ out, int h, int d) {
    using acc_t = typename Acc<T>::type;
    __shared__ acc_t s_part[kRowWarps][32 * kRowCols];
    int64_t r, beg, end;
    if (!row_range(row, indptr, n_chunks, blockIdx.x, r, beg, end)) return;
    const int hd = h * d;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int col0 = 0; col0 < hd; col0 += 32 * kRowCols) {
        acc_t acc[kRowCols];
        int hh[kRowCols];
#pragma unroll
        for (int u = 0; u < kRowCols; ++u) {
            acc[u] = 0;
            const int j = col0 + lane + 32 * u;
            hh[u] = j < hd ? j / d : -1;
        }
#pragma unroll 4
        for (int64_t k = beg + warp; k < end; k += kRowWarps) {
            const int64_t e = eid[k];
            const T *w_row = W + e * h;
            const T *x_row = kEdgeX ? X + e * d : X + indices[k] * hd;
#pragma unroll
            for (int u = 0; u < kRowCols; ++u) {
                if (hh[u] < 0) continue;
                const int j = col0 + lane + 32 * u;
                const acc_t x = kEdgeX ? to_acc(x_row[j - hh[u] * d]) : to_acc(x_row[j]);
                acc[u] += to_acc(w_row[hh[u]]) * x;
            }
        }
#pragma unroll
        for (int u = 0; u < kRowCols; ++u) s_part[warp][lane + 32 * u] = acc[u];
        __syncthreads();
        {
            const int j = col0 + threadIdx.x;  // kRowWarps * 32 threads = 32 * kRowCols columns
            if (j < hd) {
                acc_t sum = 0;
#pragma unroll
                for (int w = 0; w < kRowWarps; ++w) sum += s_part[w][threadIdx.x];
                out[r * hd + j] = from_acc<T>(sum);
            }
        }
        __syncthreads();
    }
}
static_assert(kRowWarps * 32 == 32 * kRowCols, "one thread per column of a pass in the final sum");

// node_mul_edge backward, dB[eid[k], dd] = sum_hh dy[eid[k], hh] * A[row, hh, dd]
template <typename T>
__global__ void nme_backward_edge_kernel(const int64_t *__restrict__ row, const int64_t *__restrict__ indptr,
                                         const int64_t *__restrict__ eid, int64_t n_chunks,
                                         const T *__restrict__ A, const T *__restrict__ dy,
                                         T *__restrict__ dB, int h, int d) {
    using acc_t = typename Acc<T>::type;
    const int64_t c = blockIdx.x;
    const int64_t beg = indptr[c], end = indptr[c + 1];
    const T *a_row = A + row[c] * h * static_cast<int64_t>(d);
    const int64_t work = (end - beg) * d;
    for (int64_t idx = threadIdx.x; idx < work; idx += blockDim.x) {
        const int64_t k = beg + idx / d;
        const int dd = static_cast<int>(idx % d);
        const int64_t e = eid[k];
        acc_t sum = 0;
        for (int hh = 0; hh < h; ++hh) sum += to_acc(dy[e * h + hh]) * to_acc(a_row[hh * d + dd]);
        dB[e * d + dd] = from_acc<T>(sum);
    }
}

// ---------------------------------------------------------------- edge softmax
template <typename acc_t>
__device__ __forceinline__ acc_t warp_max(acc_t v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const acc_t o = __shfl_xor_sync(0xffffffffu, v, off);
        v = o > v ? o : v;
    }
    return v;
}
template <typename acc_t>
__device__ __forceinline__ acc_t warp_sum(acc_t v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// One block per row, one warp per head (strided); lanes stride over the row's entries.
template <typename T>
__global__ void softmax_forward_kernel(const int64_t *__restrict__ row, const int64_t *__restrict__ indptr,
                                       const int64_t *__restrict__ eid, int64_t n_chunks,
                                       const T *__restrict__ x, T *__restrict__ y, int h) {
    using acc_t = typename Acc<T>::type;
    int64_t r, beg, end;
    if (!row_range(row, indptr, n_chunks, blockIdx.x, r, beg, end)) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int hh = warp; hh < h; hh += n_warps) {
        acc_t m = -INFINITY;
        for (int64_t k = beg + lane; k < end; k += 32) {
            const acc_t v = to_acc(x[eid[k] * h + hh]);
            m = v > m ? v : m;
        }
        m = warp_max(m);
        acc_t s = 0;
        for (int64_t k = beg + lane; k < end; k += 32) s += acc_exp(to_acc(x[eid[k] * h + hh]) - m);
        s = warp_sum(s);
        const acc_t inv = acc_t(1) / s;
        for (int64_t k = beg + lane; k < end; k += 32) {
            const int64_t e = eid[k];
            y[e * h + hh] = from_acc<T>(acc_exp(to_acc(x[e * h + hh]) - m) * inv);
        }
    }
}

template <typename T>
__global__ void softmax_backward_kernel(const int64_t *__restrict__ row, const int64_t *__restrict__ indptr,
                                        const int64_t *__restrict__ eid, int64_t n_chunks,
                                        const T *__restrict__ y, const T *__restrict__ dy,
                                        T *__restrict__ dx, int h) {
    using acc_t = typename Acc<T>::type;
    int64_t r, beg, end;
    if (!row_range(row, indptr, n_chunks, blockIdx.x, r, beg, end)) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int hh = warp; hh < h; hh += n_warps) {
        acc_t s = 0;
        for (int64_t k = beg + lane; k < end; k += 32) {
            const int64_t e = eid[k];
            s += to_acc(dy[e * h + hh]) * to_acc(y[e * h + hh]);
        }
        s = warp_sum(s);
        for (int64_t k = beg + lane; k < end; k += 32) {
            const int64_t e = eid[k];
            const acc_t yy = to_acc(y[e * h + hh]);
            dx[e * h + hh] = from_acc<T>(to_acc(dy[e * h + hh]) * yy - s * yy);
        }
    }
}

// ---------------------------------------------------------------- launch helpers

int check_common(const char *name, const void *row, const void *indptr, int64_t n_chunks, int h, int d) {
    BPT_CHECK_ARG(n_chunks >= 0, "%s: negative chunk count", name);
    BPT_CHECK_ARG(n_chunks < (int64_t(1) << 31), "%s: more than 2^31-1 chunks", name);
    BPT_CHECK_ARG(h >= 1 && d >= 1, "%s: h and d must be positive", name);
    BPT_CHECK_ARG(n_chunks == 0 || (row && indptr), "%s: null chunk arrays", name);
    return BPT_OK;
}

template <typename T, bool kPerHead>
int launch_edge_dot(const int64_t *row, const int64_t *indptr, const int64_t *eid, const int64_t *indices,
                    int64_t n_chunks, const void *A, const void *B, void *y, int h, int d,
                    cudaStream_t stream) {
    if (n_chunks == 0) return BPT_OK;
    const int warps = 4;
    const unsigned blocks = static_cast<unsigned>((n_chunks + warps - 1) / warps);
    edge_dot_kernel<T, kPerHead><<<blocks, warps * 32, 0, stream>>>(
        row, indptr, eid, indices, n_chunks, static_cast<const T *>(A), static_cast<const T *>(B),
        static_cast<T *>(y), h, d);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

template <typename T, bool kEdgeX>
int launch_row_sum(const int64_t *row, const int64_t *indptr, const int64_t *eid, const int64_t *indices,
                   int64_t n_chunks, const void *W, const void *X, void *out, int64_t n_rows_out, int h,
                   int d, cudaStream_t stream) {
    BPT_CUDA(cudaMemsetAsync(out, 0, sizeof(T) * static_cast<size_t>(n_rows_out) * h * d, stream));
    if (n_chunks == 0) return BPT_OK;
    row_sum_kernel<T, kEdgeX><<<static_cast<unsigned>(n_chunks), kRowWarps * 32, 0, stream>>>(
        row, indptr, eid, indices, n_chunks, static_cast<const T *>(W), static_cast<const T *>(X),
        static_cast<T *>(out), h, d);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" int bpt_maskedmm_csr_forward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                                        const int64_t *indices, int64_t n_chunks, const void *A,
                                        const void *B, void *y, int h, int d, int dtype,
                                        bpt_stream_t stream) {
    if (int rc = check_common("maskedmm_csr_forward", row, indptr, n_chunks, h, d)) return rc;
    BPT_CHECK_ARG(n_chunks == 0 || (eid && indices && A && B && y), "maskedmm_csr_forward: null array");
    BPT_DISPATCH_DTYPE(dtype, return (launch_edge_dot<scalar_t, true>(row, indptr, eid, indices, n_chunks, A,
                                                                      B, y, h, d, as_stream(stream))));
    return BPT_OK;
}

extern "C" int bpt_maskedmm_csr_backward(const int64_t *row, const int64_t *indptr_r, const int64_t *eid_r,
                                         const int64_t *indices_r, int64_t n_chunks_r, const int64_t *col,
                                         const int64_t *indptr_c, const int64_t *eid_c,
                                         const int64_t *indices_c, int64_t n_chunks_c, const void *A,
                                         const void *B, const void *dy, void *dA, void *dB,
                                         int64_t n_rows_a, int64_t n_rows_b, int h, int d, int dtype,
                                         bpt_stream_t stream) {
    if (int rc = check_common("maskedmm_csr_backward", row, indptr_r, n_chunks_r, h, d)) return rc;
    if (int rc = check_common("maskedmm_csr_backward", col, indptr_c, n_chunks_c, h, d)) return rc;
    BPT_CHECK_ARG(dA && dB && n_rows_a >= 0 && n_rows_b >= 0, "maskedmm_csr_backward: null output");
    BPT_CHECK_ARG((n_chunks_r == 0 && n_chunks_c == 0) || (A && B && dy), "maskedmm_csr_backward: null array");
    BPT_DISPATCH_DTYPE(dtype, {
        // graphop_kernel.cu:383: rows of the first CSR own dA and gather B; :398: rows of the
        // second CSR own dB and gather A.
        if (int rc = launch_row_sum<scalar_t, false>(row, indptr_r, eid_r, indices_r, n_chunks_r, dy, B, dA,
                                                     n_rows_a, h, d, as_stream(stream)))
            return rc;
        return (launch_row_sum<scalar_t, false>(col, indptr_c, eid_c, indices_c, n_chunks_c, dy, A, dB,
                                                n_rows_b, h, d, as_stream(stream)));
    });
    return BPT_OK;
}

extern "C" int bpt_node_mul_edge_forward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                                         int64_t n_chunks, const void *A, const void *B, void *y, int h,
                                         int d, int dtype, bpt_stream_t stream) {
    if (int rc = check_common("node_mul_edge_forward", row, indptr, n_chunks, h, d)) return rc;
    BPT_CHECK_ARG(n_chunks == 0 || (eid && A && B && y), "node_mul_edge_forward: null array");
    BPT_DISPATCH_DTYPE(dtype, return (launch_edge_dot<scalar_t, false>(row, indptr, eid, nullptr, n_chunks, A,
                                                                       B, y, h, d, as_stream(stream))));
    return BPT_OK;
}

extern "C" int bpt_node_mul_edge_backward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                                          int64_t n_chunks, const void *A, const void *B, const void *dy,
                                          void *dA, void *dB, int64_t n_rows_a, int h, int d, int dtype,
                                          bpt_stream_t stream_) {
    if (int rc = check_common("node_mul_edge_backward", row, indptr, n_chunks, h, d)) return rc;
    BPT_CHECK_ARG(dA && n_rows_a >= 0, "node_mul_edge_backward: null output");
    BPT_CHECK_ARG(n_chunks == 0 || (eid && A && B && dy && dB), "node_mul_edge_backward: null array");
    cudaStream_t stream = as_stream(stream_);
    BPT_DISPATCH_DTYPE(dtype, {
        if (int rc = launch_row_sum<scalar_t, true>(row, indptr, eid, nullptr, n_chunks, dy, B, dA, n_rows_a,
                                                    h, d, stream))
            return rc;
        if (n_chunks > 0) {
            nme_backward_edge_kernel<scalar_t><<<static_cast<unsigned>(n_chunks), 128, 0, stream>>>(
                row, indptr, eid, n_chunks, static_cast<const scalar_t *>(A),
                static_cast<const scalar_t *>(dy), static_cast<scalar_t *>(dB), h, d);
            BPT_LAUNCH_CHECK();
        }
    });
    return BPT_OK;
}

extern "C" int bpt_sparse_softmax_forward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                                          int64_t n_chunks, const void *x, void *y, int h, int dtype,
                                          bpt_stream_t stream) {
    if (int rc = check_common("sparse_softmax_forward", row, indptr, n_chunks, h, 1)) return rc;
    BPT_CHECK_ARG(n_chunks == 0 || (eid && x && y), "sparse_softmax_forward: null array");
    if (n_chunks == 0) return BPT_OK;
    const int threads = 32 * (h < 8 ? h : 8);
    BPT_DISPATCH_DTYPE(dtype, {
        softmax_forward_kernel<scalar_t><<<static_cast<unsigned>(n_chunks), threads, 0, as_stream(stream)>>>(
            row, indptr, eid, n_chunks, static_cast<const scalar_t *>(x), static_cast<scalar_t *>(y), h);
    });
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

extern "C" int bpt_sparse_softmax_backward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                                           int64_t n_chunks, const void *y, const void *dy, void *dx, int h,
                                           int dtype, bpt_stream_t stream) {
    if (int rc = check_common("sparse_softmax_backward", row, indptr, n_chunks, h, 1)) return rc;
    BPT_CHECK_ARG(n_chunks == 0 || (eid && y && dy && dx), "sparse_softmax_backward: null array");
    if (n_chunks == 0) return BPT_OK;
    const int threads = 32 * (h < 8 ? h : 8);
    BPT_DISPATCH_DTYPE(dtype, {
        softmax_backward_kernel<scalar_t><<<static_cast<unsigned>(n_chunks), threads, 0, as_stream(stream)>>>(
            row, indptr, eid, n_chunks, static_cast<const scalar_t *>(y), static_cast<const scalar_t *>(dy),
            static_cast<scalar_t *>(dx), h);
    });
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

extern "C" int bpt_vector_spmm_forward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                                       const int64_t *indices, int64_t n_chunks, const void *edata,
                                       const void *x, void *y, int64_t n_rows_y, int h, int d, int dtype,
                                       bpt_stream_t stream) {
    if (int rc = check_common("vector_spmm_forward", row, indptr, n_chunks, h, d)) return rc;
    BPT_CHECK_ARG(y && n_rows_y >= 0, "vector_spmm_forward: null output");
    BPT_CHECK_ARG(n_chunks == 0 || (eid && indices && edata && x), "vector_spmm_forward: null array");
    BPT_DISPATCH_DTYPE(dtype, return (launch_row_sum<scalar_t, false>(row, indptr, eid, indices, n_chunks, edata,
                                                                      x, y, n_rows_y, h, d, as_stream(stream))));
    return BPT_OK;
}

extern "C" int bpt_vector_spmm_backward(const int64_t *row, const int64_t *indptr, const int64_t *eid,
                                        const int64_t *indices, int64_t n_chunks, const int64_t *col,
                                        const int64_t *indptr_t, const int64_t *eid_t,
                                        const int64_t *indices_t, int64_t n_chunks_t, const void *edata,
                                        const void *dy, const void *x, void *dedata, void *dx,
                                        int64_t n_rows_x, int h, int d, int dtype, bpt_stream_t stream) {
    if (int rc = check_common("vector_spmm_backward", row, indptr, n_chunks, h, d)) return rc;
    if (int rc = check_common("vector_spmm_backward", col, indptr_t, n_chunks_t, h, d)) return rc;
    BPT_CHECK_ARG(dx && n_rows_x >= 0, "vector_spmm_backward: null output");
    BPT_CHECK_ARG((n_chunks == 0 && n_chunks_t == 0) || (edata && dy && x && dedata),
                  "vector_spmm_backward: null array");
    BPT_DISPATCH_DTYPE(dtype, {
        // graphop_kernel.cu:571: dedata is an SDDMM of dy rows with x rows over the first CSR.
        if (int rc = launch_edge_dot<scalar_t, true>(row, indptr, eid, indices, n_chunks, dy, x, dedata, h, d,
                                                     as_stream(stream)))
            return rc;
        // graphop_kernel.cu:590: dx sums edata * dy over the transposed CSR.
        return (launch_row_sum<scalar_t, false>(col, indptr_t, eid_t, indices_t, n_chunks_t, edata, dy, dx,
                                                n_rows_x, h, d, as_stream(stream)));
    });
    return BPT_OK;
}
