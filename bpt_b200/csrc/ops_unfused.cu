// The eight graph operators of the reference's `graphop` module as deterministic kernels.
//
// The reference (graph_kernel/graphop_kernel.cu) gives every <=32-edge chunk its own block and
// lets chunks of the same row meet in floating-point atomics.  Here the chunk arrays are read
// only to find where a row starts and ends: the block of a row's first chunk owns the whole
// row, every output element has one writer and a fixed summation order, and blocks of the
// row's other chunks return at once.  Per-edge outputs (the SDDMM-type operators) have no
// cross-chunk reduction and keep one block per chunk.
#include <algorithm>
#include <type_traits>

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

// The same row sums for fp32 rows of 128, 256, 384 or 512 columns (head width a multiple of 4), the shapes
// of the attention layers.  One block per SM-sized share of the chunk list; its 16 warps take the rows
// that start in that share round-robin, so at any time the block works on ~16 neighbouring rows, whose
// gathered rows overlap heavily on binary-partition graphs and are then served by the L1 instead of the
// L2 (the generic kernel gives every row its own block, and neighbouring rows land on different SMs).
// A warp owns a whole row: lane l holds columns 4 l + 128 u as float4 accumulators (kVec = columns / 128
// of them), every gathered row is read with 16-byte loads, two entries are in flight per step, and
// nothing is combined across warps.  One writer per output element; a row's entries are added in CSR
// order, even and odd entries in two partial sums.
constexpr int kWideWarps = 16;
constexpr int kWideLongRow = 256;  // rows with more entries are summed by the whole block

// acc0/acc1 += W[e] * X-row for the entries [beg, end) taken `step` apart (two in flight)
template <int kVec, bool kEdgeX>
__device__ __forceinline__ void wide_accumulate(const int64_t *__restrict__ eid, const int64_t *__restrict__ indices,
                                                int64_t beg, int64_t end, const float *__restrict__ W,
                                                const float *__restrict__ X, int h, int d, int hd,
                                                const int (&head)[kVec], const int (&xpiece)[kVec],
                                                float4 (&acc0)[kVec], float4 (&acc1)[kVec]) {
    int64_t k = beg;
    for (; k + 1 < end; k += 2) {
        const int64_t e0 = eid[k], e1 = eid[k + 1];
        const float4 *x0 = reinterpret_cast<const float4 *>(kEdgeX ? X + e0 * d : X + indices[k] * hd);
        const float4 *x1 = reinterpret_cast<const float4 *>(kEdgeX ? X + e1 * d : X + indices[k + 1] * hd);
        float4 v0[kVec], v1[kVec];
        float w0[kVec], w1[kVec];
#pragma unroll
        for (int u = 0; u < kVec; ++u) {
            v0[u] = __ldg(x0 + xpiece[u]);
            v1[u] = __ldg(x1 + xpiece[u]);
            w0[u] = __ldg(W + e0 * h + head[u]);
            w1[u] = __ldg(W + e1 * h + head[u]);
        }
#pragma unroll
        for (int u = 0; u < kVec; ++u) {
            acc0[u].x = fmaf(w0[u], v0[u].x, acc0[u].x); acc0[u].y = fmaf(w0[u], v0[u].y, acc0[u].y);
            acc0[u].z = fmaf(w0[u], v0[u].z, acc0[u].z); acc0[u].w = fmaf(w0[u], v0[u].w, acc0[u].w);
            acc1[u].x = fmaf(w1[u], v1[u].x, acc1[u].x); acc1[u].y = fmaf(w1[u], v1[u].y, acc1[u].y);
            acc1[u].z = fmaf(w1[u], v1[u].z, acc1[u].z); acc1[u].w = fmaf(w1[u], v1[u].w, acc1[u].w);
        }
    }
    if (k < end) {
        const int64_t e0 = eid[k];
        const float4 *x0 = reinterpret_cast<const float4 *>(kEdgeX ? X + e0 * d : X + indices[k] * hd);
#pragma unroll
        for (int u = 0; u < kVec; ++u) {
            const float4 v = __ldg(x0 + xpiece[u]);
            const float w = __ldg(W + e0 * h + head[u]);
            acc0[u].x = fmaf(w, v.x, acc0[u].x); acc0[u].y = fmaf(w, v.y, acc0[u].y);
            acc0[u].z = fmaf(w, v.z, acc0[u].z); acc0[u].w = fmaf(w, v.w, acc0[u].w);
        }
    }
}

template <int kVec, bool kEdgeX>
__global__ void __launch_bounds__(kWideWarps * 32)
row_sum_wide_kernel(const int64_t *__restrict__ row, const int64_t *__restrict__ indptr,
                    const int64_t *__restrict__ eid, const int64_t *__restrict__ indices, int64_t n_chunks,
                    const float *__restrict__ W, const float *__restrict__ X, float *__restrict__ out, int h,
                    int d) {
    __shared__ float4 s_part[kWideWarps][32 * kVec];  // partial sums of a long row, one slice per warp
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hd = h * d;
    const int64_t c0 = n_chunks * blockIdx.x / gridDim.x, c1 = n_chunks * (blockIdx.x + 1) / gridDim.x;
    int head[kVec], xpiece[kVec];  // head of this lane's u-th column group; its float4 inside a gathered row
#pragma unroll
    for (int u = 0; u < kVec; ++u) {
        const int col = lane * 4 + 128 * u;
        head[u] = col / d;
        xpiece[u] = kEdgeX ? (col % d) / 4 : col / 4;
    }
    int ordinal = 0;  // short rows that started in this block's share so far (the same count in every warp)
    for (int64_t base = c0; base < c1; base += 32) {
        const int64_t cl = base + lane;
        const bool starts = cl < c1 && (cl == 0 || row[cl - 1] != row[cl]);
        unsigned mask = __ballot_sync(0xffffffffu, starts);
        while (mask) {
            const int bit = __ffs(mask) - 1;
            mask &= mask - 1;
            const int64_t c = base + bit;
            const int64_t r = row[c];
            // a short row ends within a few chunks; every warp walks them (the block agrees on long / short)
            int64_t ce = c + 1;
            while (ce < n_chunks && row[ce] == r) ++ce;
            const int64_t beg = indptr[c], end = indptr[ce];
            const bool is_long = end - beg > kWideLongRow;
            if (!is_long && ordinal++ % kWideWarps != warp) continue;
            float4 acc0[kVec], acc1[kVec];
#pragma unroll
            for (int u = 0; u < kVec; ++u) {
                acc0[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                acc1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float4 *o = reinterpret_cast<float4 *>(out + r * hd);
            if (!is_long) {
                wide_accumulate<kVec, kEdgeX>(eid, indices, beg, end, W, X, h, d, hd, head, xpiece, acc0, acc1);
#pragma unroll
                for (int u = 0; u < kVec; ++u)
                    o[lane + 32 * u] = make_float4(acc0[u].x + acc1[u].x, acc0[u].y + acc1[u].y,
                                                   acc0[u].z + acc1[u].z, acc0[u].w + acc1[u].w);
                continue;
            }
            // long row: warp w sums its contiguous sixteenth of the entries, the slices meet in warp order
            const int64_t len = end - beg;
            wide_accumulate<kVec, kEdgeX>(eid, indices, beg + len * warp / kWideWarps,
                                          beg + len * (warp + 1) / kWideWarps, W, X, h, d, hd, head, xpiece, acc0, acc1);
#pragma unroll
            for (int u = 0; u < kVec; ++u)
                s_part[warp][lane + 32 * u] = make_float4(acc0[u].x + acc1[u].x, acc0[u].y + acc1[u].y,
                                                          acc0[u].z + acc1[u].z, acc0[u].w + acc1[u].w);
            __syncthreads();
            for (int i = threadIdx.x; i < 32 * kVec; i += blockDim.x) {
                float4 sum = s_part[0][i];
#pragma unroll
                for (int w = 1; w < kWideWarps; ++w) {
                    const float4 p = s_part[w][i];
                    sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
                }
                o[i] = sum;
            }
            __syncthreads();
        }
    }
}

// Per-edge dot products and the per-edge gradient of node_mul_edge for the same fp32 shapes (rows of 128..512
// columns, head width 16, 32, 64 or 128).  One block per SM-sized share of the chunk list, its warps take
// the chunks round-robin (16 neighbouring chunks in flight per block, so gathered rows are shared through
// the L1); a warp keeps the chunk's A row in registers (lane l: columns 4 l + 128 u), reads every gathered
// row with 16-byte loads, two entries in flight, and reduces inside the d / 4 lanes that hold one head.
template <int kVec, bool kPerHead>
__global__ void __launch_bounds__(kWideWarps * 32)
edge_dot_wide_kernel(const int64_t *__restrict__ row, const int64_t *__restrict__ indptr,
                     const int64_t *__restrict__ eid, const int64_t *__restrict__ indices, int64_t n_chunks,
                     const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ y, int h, int d) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hd = h * d, lanes_per_head = d / 4;
    const int64_t c0 = n_chunks * blockIdx.x / gridDim.x, c1 = n_chunks * (blockIdx.x + 1) / gridDim.x;
    int head[kVec];
#pragma unroll
    for (int u = 0; u < kVec; ++u) head[u] = (lane * 4 + 128 * u) / d;
    const int bpiece = (lane * 4 % d) / 4;  // !kPerHead: this lane's float4 of the shared d-wide row
    const bool writer = lane % lanes_per_head == 0;
    for (int64_t c = c0 + warp; c < c1; c += kWideWarps) {
        const float4 *a_row = reinterpret_cast<const float4 *>(A + row[c] * hd);
        float4 a[kVec];
#pragma unroll
        for (int u = 0; u < kVec; ++u) a[u] = __ldg(a_row + lane + 32 * u);
        const int64_t beg = indptr[c], end = indptr[c + 1];
        for (int64_t k = beg; k < end; k += 2) {
            const bool two = k + 1 < end;
            const int64_t e0 = eid[k], e1 = two ? eid[k + 1] : e0;
            const float4 *b0 = reinterpret_cast<const float4 *>(kPerHead ? B + indices[k] * hd : B + e0 * d);
            const float4 *b1 = reinterpret_cast<const float4 *>(kPerHead ? B + indices[two ? k + 1 : k] * hd : B + e1 * d);
            float p0[kVec], p1[kVec];
            if (kPerHead) {
                float4 v0[kVec], v1[kVec];
#pragma unroll
                for (int u = 0; u < kVec; ++u) {
                    v0[u] = __ldg(b0 + lane + 32 * u);
                    v1[u] = __ldg(b1 + lane + 32 * u);
                }
#pragma unroll
                for (int u = 0; u < kVec; ++u) {
                    p0[u] = fmaf(a[u].x, v0[u].x, fmaf(a[u].y, v0[u].y, fmaf(a[u].z, v0[u].z, a[u].w * v0[u].w)));
                    p1[u] = fmaf(a[u].x, v1[u].x, fmaf(a[u].y, v1[u].y, fmaf(a[u].z, v1[u].z, a[u].w * v1[u].w)));
                }
            } else {
                const float4 v0 = __ldg(b0 + bpiece), v1 = __ldg(b1 + bpiece);
#pragma unroll
                for (int u = 0; u < kVec; ++u) {
                    p0[u] = fmaf(a[u].x, v0.x, fmaf(a[u].y, v0.y, fmaf(a[u].z, v0.z, a[u].w * v0.w)));
                    p1[u] = fmaf(a[u].x, v1.x, fmaf(a[u].y, v1.y, fmaf(a[u].z, v1.z, a[u].w * v1.w)));
                }
            }
            for (int off = lanes_per_head >> 1; off > 0; off >>= 1) {
#pragma unroll
                for (int u = 0; u < kVec; ++u) {
                    p0[u] += __shfl_xor_sync(0xffffffffu, p0[u], off);
                    p1[u] += __shfl_xor_sync(0xffffffffu, p1[u], off);
                }
            }
            if (writer) {
#pragma unroll
                for (int u = 0; u < kVec; ++u) {
                    y[e0 * h + head[u]] = p0[u];
                    if (two) y[e1 * h + head[u]] = p1[u];
                }
            }
        }
    }
}

template <int kVec>
__global__ void __launch_bounds__(kWideWarps * 32)
nme_backward_edge_wide_kernel(const int64_t *__restrict__ row, const int64_t *__restrict__ indptr,
                              const int64_t *__restrict__ eid, int64_t n_chunks, const float *__restrict__ A,
                              const float *__restrict__ dy, float *__restrict__ dB, int h, int d) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hd = h * d, lanes_per_head = d / 4;
    const int64_t c0 = n_chunks * blockIdx.x / gridDim.x, c1 = n_chunks * (blockIdx.x + 1) / gridDim.x;
    int head[kVec];
#pragma unroll
    for (int u = 0; u < kVec; ++u) head[u] = (lane * 4 + 128 * u) / d;
    for (int64_t c = c0 + warp; c < c1; c += kWideWarps) {
        const float4 *a_row = reinterpret_cast<const float4 *>(A + row[c] * hd);
        float4 a[kVec];
#pragma unroll
        for (int u = 0; u < kVec; ++u) a[u] = __ldg(a_row + lane + 32 * u);
        const int64_t beg = indptr[c], end = indptr[c + 1];
        for (int64_t k = beg; k < end; ++k) {
            const int64_t e = eid[k];
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);  // heads in ascending order within the lane, then across lanes
#pragma unroll
            for (int u = 0; u < kVec; ++u) {
                const float g = __ldg(dy + e * h + head[u]);
                t.x = fmaf(g, a[u].x, t.x); t.y = fmaf(g, a[u].y, t.y);
                t.z = fmaf(g, a[u].z, t.z); t.w = fmaf(g, a[u].w, t.w);
            }
            for (int off = lanes_per_head; off < 32; off <<= 1) {
                t.x += __shfl_xor_sync(0xffffffffu, t.x, off); t.y += __shfl_xor_sync(0xffffffffu, t.y, off);
                t.z += __shfl_xor_sync(0xffffffffu, t.z, off); t.w += __shfl_xor_sync(0xffffffffu, t.w, off);
            }
            if (lane < lanes_per_head) reinterpret_cast<float4 *>(dB + e * d)[lane] = t;
        }
    }
}

// True when the fp32 wide kernels apply: rows of 128, 256, 384 or 512 columns, 16-byte aligned.
inline bool wide_shape(int h, int d, bool need_head_pow2, const void *p0, const void *p1, const void *p2) {
    const int hd = h * d;
    if (hd % 128 != 0 || hd > 512 || d % 4 != 0) return false;
    if (need_head_pow2 && d != 16 && d != 32 && d != 64 && d != 128) return false;
    return reinterpret_cast<uintptr_t>(p0) % 16 == 0 && reinterpret_cast<uintptr_t>(p1) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(p2) % 16 == 0;
}
// blocks_per_sm: 1 for the kernels whose gathered rows fill the registers and the L1, more for the ones that
// move little per entry and wait on chains of dependent loads instead.
inline int wide_grid(int64_t n_chunks, unsigned &grid, int blocks_per_sm = 1) {
    int dev = 0, sms = 0;
    BPT_CUDA(cudaGetDevice(&dev));
    BPT_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    grid = static_cast<unsigned>(std::min<int64_t>(n_chunks, static_cast<int64_t>(sms) * blocks_per_sm));
    return BPT_OK;
}

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
    if (std::is_same<T, float>::value && wide_shape(h, d, true, A, B, A)) {
        unsigned grid = 1;
        if (int rc = wide_grid(n_chunks, grid, kPerHead ? 1 : 3)) return rc;
        const float *a = static_cast<const float *>(A), *b = static_cast<const float *>(B);
        float *o = static_cast<float *>(y);
        switch (h * d / 128) {
            case 1: edge_dot_wide_kernel<1, kPerHead><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, indices, n_chunks, a, b, o, h, d); break;
            case 2: edge_dot_wide_kernel<2, kPerHead><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, indices, n_chunks, a, b, o, h, d); break;
            case 3: edge_dot_wide_kernel<3, kPerHead><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, indices, n_chunks, a, b, o, h, d); break;
            default: edge_dot_wide_kernel<4, kPerHead><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, indices, n_chunks, a, b, o, h, d); break;
        }
        BPT_LAUNCH_CHECK();
        return BPT_OK;
    }
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
    const int hd = h * d;
    if (std::is_same<T, float>::value && wide_shape(h, d, false, X, out, X)) {
        unsigned grid = 1;
        if (int rc = wide_grid(n_chunks, grid)) return rc;
        const float *w = static_cast<const float *>(W), *x = static_cast<const float *>(X);
        float *o = static_cast<float *>(out);
        switch (hd / 128) {
            case 1: row_sum_wide_kernel<1, kEdgeX><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, indices, n_chunks, w, x, o, h, d); break;
            case 2: row_sum_wide_kernel<2, kEdgeX><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, indices, n_chunks, w, x, o, h, d); break;
            case 3: row_sum_wide_kernel<3, kEdgeX><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, indices, n_chunks, w, x, o, h, d); break;
            default: row_sum_wide_kernel<4, kEdgeX><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, indices, n_chunks, w, x, o, h, d); break;
        }
        BPT_LAUNCH_CHECK();
        return BPT_OK;
    }
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
        if (n_chunks > 0 && std::is_same<scalar_t, float>::value && wide_shape(h, d, true, A, dB, A)) {
            unsigned grid = 1;
            if (int rc = wide_grid(n_chunks, grid, 3)) return rc;
            const float *a = static_cast<const float *>(A), *g = static_cast<const float *>(dy);
            float *o = static_cast<float *>(dB);
            switch (h * d / 128) {
                case 1: nme_backward_edge_wide_kernel<1><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, n_chunks, a, g, o, h, d); break;
                case 2: nme_backward_edge_wide_kernel<2><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, n_chunks, a, g, o, h, d); break;
                case 3: nme_backward_edge_wide_kernel<3><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, n_chunks, a, g, o, h, d); break;
                default: nme_backward_edge_wide_kernel<4><<<grid, kWideWarps * 32, 0, stream>>>(row, indptr, eid, n_chunks, a, g, o, h, d); break;
            }
            BPT_LAUNCH_CHECK();
        } else if (n_chunks > 0) {
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
