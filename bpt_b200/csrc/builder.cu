// Binary-partition graph construction, COO->CSR and partition_csr as integer kernels.
//
// What is computed is fixed by the reference's host code (graph_builder/builder.pyx:29-116,
// :305-321 and graph/base.py:71-86) and must match it bit for bit; how it is computed is
// not: every leaf's edge run is independent once its first edge id is known, so the
// builder is a count pass, a device-wide exclusive scan and a fill pass.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "common.cuh"

namespace bpt {
namespace {

constexpr int kMaxLevels = 40;

struct LevelTable {
    uint32_t nn[kMaxLevels];  // nodes per level
    uint32_t sh[kMaxLevels];  // first node id of the level
    int n_lvl;
    int64_t n_nodes;
};

// builder.pyx:41-56
int make_levels(int64_t length, LevelTable *t) {
    int64_t n = length, total = 0;
    int lvl = 0;
    while (n >= 2) {
        if (lvl >= kMaxLevels - 1) return -1;
        t->nn[lvl] = static_cast<uint32_t>(n);
        t->sh[lvl] = static_cast<uint32_t>(total);
        total += n;
        ++lvl;
        n = (n + 1) >> 1;
    }
    t->nn[lvl] = 1;
    t->sh[lvl] = static_cast<uint32_t>(total);
    total += 1;
    ++lvl;
    t->n_lvl = lvl;
    t->n_nodes = total;
    return 0;
}

// One leaf's walk up the tree (builder.pyx:67-116).  Emit(src, dst, etype) is called once
// per edge, in the reference's order: per level, per k: right then left; then the
// bottom-up edge of that level.
template <typename Emit>
__device__ __forceinline__ void walk_leaf(const LevelTable &t, int i, bool triu, int step,
                                          int clip, Emit emit) {
    int v = i;
    uint32_t shift = 0;
    int l_ptr = i - 1, r_ptr = i + 1;
    bool l_ov = false, r_ov = false;
    const uint32_t per_lvl = 2u * static_cast<uint32_t>(step) + 1u;
    for (int j = 0; j < t.n_lvl; ++j) {
        const uint32_t base = per_lvl * static_cast<uint32_t>(j < clip ? j : clip);
        const uint32_t nn_j = t.nn[j];
        for (int k = 0; k < step; ++k) {
            if (!triu && static_cast<uint32_t>(r_ptr) < nn_j) {
                // The bound is checked at level j but an overlap substitutes the level j-1
                // child 2r+1, which may lie past that level's end: kept as the reference has it.
                const uint32_t s = r_ov ? t.sh[j - 1] + ((static_cast<uint32_t>(r_ptr) << 1) + 1u)
                                        : t.sh[j] + static_cast<uint32_t>(r_ptr);
                emit(s, static_cast<uint32_t>(i), base + 2u * (static_cast<uint32_t>(k) + 1u));
                r_ov = false;
            }
            ++r_ptr;
            if (l_ptr >= 0) {
                const uint32_t s = l_ov ? t.sh[j - 1] + (static_cast<uint32_t>(l_ptr) << 1)
                                        : t.sh[j] + static_cast<uint32_t>(l_ptr);
                emit(s, static_cast<uint32_t>(i), base + 2u * static_cast<uint32_t>(k) + 1u);
                l_ov = false;
            }
            --l_ptr;
        }
        if ((l_ptr & 1) == 0) l_ov = true;
        if ((r_ptr & 1) == 1) r_ov = true;
        r_ptr >>= 1;
        l_ptr >>= 1;  // arithmetic shift: -1 stays -1
        emit(static_cast<uint32_t>(i), shift + static_cast<uint32_t>(v), base);
        shift += nn_j;
        v >>= 1;
    }
}

__global__ void bp_count_kernel(LevelTable t, int64_t length, bool triu, int step, int clip,
                                int64_t *__restrict__ counts) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i > length) return;
    int64_t c = 0;
    if (i < length)
        walk_leaf(t, static_cast<int>(i), triu, step, clip,
                  [&](uint32_t, uint32_t, uint32_t) { ++c; });
    counts[i] = c;  // counts[length] = 0 closes the exclusive scan
}

template <typename I>
__global__ void bp_fill_kernel(LevelTable t, int64_t length, bool triu, int step, int clip,
                               const int64_t *__restrict__ leaf_offsets, int64_t v_shift,
                               I *__restrict__ src, I *__restrict__ dst, I *__restrict__ etype) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= length) return;
    int64_t e = leaf_offsets[i];
    walk_leaf(t, static_cast<int>(i), triu, step, clip, [&](uint32_t s, uint32_t d, uint32_t ty) {
        if (src) src[e] = static_cast<I>(static_cast<int64_t>(s) + v_shift);
        if (dst) dst[e] = static_cast<I>(static_cast<int64_t>(d) + v_shift);
        if (etype) etype[e] = static_cast<I>(ty);
        ++e;
    });
}

// builder.pyx:46-47,57-62: pos = min((idx+1)*2^level - 1, length-1); root = length-1.
template <typename I>
__global__ void bp_pos_kernel(LevelTable t, int64_t length, I *__restrict__ pos) {
    const int64_t node = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (node >= t.n_nodes) return;
    int j = 0;
    while (j + 1 < t.n_lvl && node >= static_cast<int64_t>(t.sh[j + 1])) ++j;
    int64_t p;
    if (j == t.n_lvl - 1) {
        p = length - 1;
    } else {
        const int64_t idx = node - t.sh[j];
        p = ((idx + 1) << j) - 1;
        if (p >= length) p = length - 1;
    }
    pos[node] = static_cast<I>(p);
}

// ------------------------------------------------------------------ COO -> CSR

template <typename I>
__global__ void csr_prepare_kernel(const I *__restrict__ key, int64_t n_edges,
                                   uint32_t *__restrict__ keys, uint32_t *__restrict__ vals) {
    const int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (e >= n_edges) return;
    keys[e] = static_cast<uint32_t>(key[e]);
    vals[e] = static_cast<uint32_t>(e);
}

// indptr[r] = number of sorted keys < r (lower bound); r in [0, n_rows].
template <typename I>
__global__ void csr_indptr_kernel(const uint32_t *__restrict__ sorted_keys, int64_t n_edges,
                                  int64_t n_rows, I *__restrict__ indptr) {
    const int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (r > n_rows) return;
    int64_t lo = 0, hi = n_edges;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (static_cast<int64_t>(sorted_keys[mid]) < r) lo = mid + 1; else hi = mid;
    }
    indptr[r] = static_cast<I>(lo);
}

template <typename I>
__global__ void csr_gather_kernel(const uint32_t *__restrict__ sorted_eid, const I *__restrict__ other,
                                  int64_t n_edges, I *__restrict__ indices, I *__restrict__ eid) {
    const int64_t p = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (p >= n_edges) return;
    const uint32_t e = sorted_eid[p];
    indices[p] = other[e];
    eid[p] = static_cast<I>(e);
}

int key_bits(int64_t n_rows) {
    int bits = 1;
    while ((int64_t(1) << bits) < n_rows && bits < 32) ++bits;
    return bits;
}

size_t sort_temp_bytes(int64_t n_edges, int bits) {
    size_t bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, bytes, static_cast<const uint32_t *>(nullptr),
                                    static_cast<uint32_t *>(nullptr),
                                    static_cast<const uint32_t *>(nullptr),
                                    static_cast<uint32_t *>(nullptr), n_edges, 0, bits);
    return bytes;
}

size_t scan_temp_bytes(int64_t n) {
    size_t bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, bytes, static_cast<const int64_t *>(nullptr),
                                  static_cast<int64_t *>(nullptr), n);
    return bytes;
}

template <typename I>
int coo_to_csr_impl(const I *key, const I *other, int64_t n_edges, int64_t n_rows, I *indptr,
                    I *indices, I *eid, void *ws_ptr, size_t ws_bytes, cudaStream_t stream) {
    const int bits = key_bits(n_rows);
    Workspace ws(ws_ptr, ws_bytes);
    const size_t ne = static_cast<size_t>(n_edges > 0 ? n_edges : 1);
    uint32_t *k_in = ws.take<uint32_t>(ne), *k_out = ws.take<uint32_t>(ne);
    uint32_t *v_in = ws.take<uint32_t>(ne), *v_out = ws.take<uint32_t>(ne);
    size_t temp_bytes = sort_temp_bytes(n_edges, bits);
    char *temp = ws.take<char>(temp_bytes > 0 ? temp_bytes : 1);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "coo_to_csr: workspace of %zu bytes is too small", ws_bytes);
    const int threads = 256;
    if (n_edges > 0) {
        const unsigned blocks = static_cast<unsigned>((n_edges + threads - 1) / threads);
        csr_prepare_kernel<I><<<blocks, threads, 0, stream>>>(key, n_edges, k_in, v_in);
        BPT_LAUNCH_CHECK();
        BPT_CUDA(cub::DeviceRadixSort::SortPairs(temp, temp_bytes, k_in, k_out, v_in, v_out, n_edges, 0,
                                                 bits, stream));
        csr_gather_kernel<I><<<blocks, threads, 0, stream>>>(v_out, other, n_edges, indices, eid);
        BPT_LAUNCH_CHECK();
    }
    const unsigned rblocks = static_cast<unsigned>((n_rows + 1 + threads - 1) / threads);
    csr_indptr_kernel<I><<<rblocks, threads, 0, stream>>>(k_out, n_edges, n_rows, indptr);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

// ------------------------------------------------------------------ partition_csr

__global__ void chunk_count_kernel(const int64_t *__restrict__ indptr, int64_t n_rows, int chunk,
                                   int64_t *__restrict__ counts) {
    const int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (r > n_rows) return;
    counts[r] = (r < n_rows) ? (indptr[r + 1] - indptr[r] + chunk - 1) / chunk : 0;
}

// One thread per chunk: its row is the last row whose first chunk id is <= c.
__global__ void chunk_fill_kernel(const int64_t *__restrict__ indptr, int64_t n_rows, int chunk,
                                  const int64_t *__restrict__ chunk_offsets,
                                  int64_t *__restrict__ row, int64_t *__restrict__ indptr_out) {
    const int64_t n_chunks = chunk_offsets[n_rows];
    const int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (c == n_chunks) indptr_out[c] = indptr[n_rows];
    if (c >= n_chunks) return;
    int64_t lo = 0, hi = n_rows;  // find the first row with chunk_offsets[row + 1] > c
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (chunk_offsets[mid + 1] > c) hi = mid; else lo = mid + 1;
    }
    row[c] = lo;
    indptr_out[c] = indptr[lo] + (c - chunk_offsets[lo]) * chunk;
}

// ------------------------------------------------------------------ baseline graphs
// FullyConnected (graph_builder/builder.pyx:228-274) and OpenAISparse (:154-196): token nodes
// [0, length) plus one root node `length`.  Each leaf's edge run has a closed-form length and
// every edge a closed-form position inside the run, so one block fills one leaf's run.

// builder.pyx:243-265: self edge, then for j = 1 .. min(length, window+1)-1: left (i >= j, type
// 2j-1), right (!triu and i+j < length, type 2j); then the edge to the root.
__device__ __host__ inline int64_t fc_leaf_count(int64_t i, int64_t length, int64_t jmax, bool triu) {
    const int64_t left = i < jmax ? i : jmax;
    const int64_t right = triu ? 0 : ((length - 1 - i) < jmax ? (length - 1 - i) : jmax);
    return 2 + left + right;
}

__global__ void fc_count_kernel(int64_t length, int64_t jmax, bool triu, int64_t *__restrict__ counts) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i > length) return;
    counts[i] = i < length ? fc_leaf_count(i, length, jmax, triu) : 0;
}

template <typename I>
__global__ void fc_fill_kernel(int64_t length, int64_t jmax, bool triu, const int64_t *__restrict__ leaf_offsets,
                               int64_t v_shift, I *__restrict__ src, I *__restrict__ dst, I *__restrict__ etype) {
    const int64_t i = blockIdx.x;
    const int64_t base = leaf_offsets[i];
    const int64_t right_max = length - 1 - i;
    auto put = [&](int64_t e, int64_t s, int64_t d, int64_t t) {
        if (src) src[e] = static_cast<I>(s + v_shift);
        if (dst) dst[e] = static_cast<I>(d + v_shift);
        if (etype) etype[e] = static_cast<I>(t);
    };
    if (threadIdx.x == 0) {
        put(base, i, i, 0);
        put(base + fc_leaf_count(i, length, jmax, triu) - 1, i, length, 0);
    }
    for (int64_t j = 1 + threadIdx.x; j <= jmax; j += blockDim.x) {
        // edges emitted by iterations j' < j: one left each while j' <= i, one right each while j' <= right_max
        int64_t e = base + 1 + ((j - 1) < i ? (j - 1) : i);
        if (!triu) e += (j - 1) < right_max ? (j - 1) : right_max;
        if (i >= j) { put(e, i - j, i, 2 * j - 1); ++e; }
        if (!triu && j <= right_max) put(e, i + j, i, 2 * j);
    }
}

// builder.pyx:171-194: sources of leaf i: its stride block up to itself, then the last c
// positions of every earlier block boundary j*stride (skipped when c > j*stride: the unsigned
// start of the reference's range wraps and the range is empty), then the edge to the root.
__device__ __host__ inline int64_t oas_first_j(int64_t stride, int64_t c) {
    const int64_t j = (c + stride - 1) / stride;
    return j < 1 ? 1 : j;
}
__device__ __host__ inline int64_t oas_leaf_count(int64_t i, int64_t stride, int64_t c) {
    const int64_t nb = i / stride, j0 = oas_first_j(stride, c);
    return (i - nb * stride + 1) + (nb >= j0 ? (nb - j0 + 1) * c : 0) + 1;
}

__global__ void oas_count_kernel(int64_t length, int64_t stride, int64_t c, int64_t *__restrict__ counts) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i > length) return;
    counts[i] = i < length ? oas_leaf_count(i, stride, c) : 0;
}

template <typename I>
__global__ void oas_fill_kernel(int64_t length, int64_t stride, int64_t c, const int64_t *__restrict__ leaf_offsets,
                                int64_t v_shift, I *__restrict__ src, I *__restrict__ dst, I *__restrict__ etype) {
    const int64_t i = blockIdx.x;
    const int64_t base = leaf_offsets[i];
    const int64_t nb = i / stride, j0 = oas_first_j(stride, c);
    const int64_t inside = i - nb * stride + 1;
    const int64_t total = oas_leaf_count(i, stride, c);
    for (int64_t e = threadIdx.x; e < total; e += blockDim.x) {
        int64_t s, d = i;
        if (e < inside) {
            s = nb * stride + e;
        } else if (e < total - 1) {
            const int64_t r = e - inside;
            const int64_t j = j0 + r / c;
            s = stride * j - c + r % c;
        } else {
            s = i;
            d = length;
        }
        if (src) src[base + e] = static_cast<I>(s + v_shift);
        if (dst) dst[base + e] = static_cast<I>(d + v_shift);
        if (etype) etype[base + e] = 0;
    }
}

// pos of the baseline graphs: leaves i, root `root_pos` (builder.pyx:173,196 / :245,267).
template <typename I>
__global__ void baseline_pos_kernel(int64_t length, int64_t root_pos, I *__restrict__ pos) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i > length) return;
    pos[i] = static_cast<I>(i < length ? i : root_pos);
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" int bpt_bp_levels(int64_t length, uint32_t *n_nodes_arr, uint32_t *shift,
                             int64_t *n_nodes, int *n_levels) {
    BPT_CHECK_ARG(length >= 1 && length <= (int64_t(1) << 30), "bp_levels: length %lld out of range [1, 2^30]",
                  static_cast<long long>(length));
    LevelTable t;
    if (make_levels(length, &t) != 0) return fail(BPT_ERR_INVALID, "bp_levels: too many levels");
    for (int j = 0; j < t.n_lvl; ++j) {
        if (n_nodes_arr) n_nodes_arr[j] = t.nn[j];
        if (shift) shift[j] = t.sh[j];
    }
    if (n_nodes) *n_nodes = t.n_nodes;
    if (n_levels) *n_levels = t.n_lvl;
    return BPT_OK;
}

extern "C" size_t bpt_bp_count_workspace_bytes(int64_t length) {
    if (length < 1) return 0;
    return align_up(static_cast<size_t>(length + 1) * sizeof(int64_t), 256) +
           align_up(scan_temp_bytes(length + 1), 256) + 256;
}

extern "C" int bpt_bp_count(int64_t length, int triu, int step, int clip_dist,
                            int64_t *leaf_offsets, void *workspace, size_t workspace_bytes,
                            int64_t *n_edges_host, bpt_stream_t stream_) {
    BPT_CHECK_ARG(length >= 1 && length <= (int64_t(1) << 30), "bp_count: length %lld out of range [1, 2^30]",
                  static_cast<long long>(length));
    BPT_CHECK_ARG(step >= 1 && clip_dist >= 0, "bp_count: step must be >= 1 and clip_dist >= 0");
    BPT_CHECK_ARG(leaf_offsets != nullptr, "bp_count: leaf_offsets is null");
    LevelTable t;
    if (make_levels(length, &t) != 0) return fail(BPT_ERR_INVALID, "bp_count: too many levels");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    int64_t *counts = ws.take<int64_t>(static_cast<size_t>(length + 1));
    size_t temp_bytes = scan_temp_bytes(length + 1);
    char *temp = ws.take<char>(temp_bytes > 0 ? temp_bytes : 1);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "bp_count: workspace of %zu bytes is too small", workspace_bytes);
    const int threads = 128;
    const unsigned blocks = static_cast<unsigned>((length + 1 + threads - 1) / threads);
    bp_count_kernel<<<blocks, threads, 0, stream>>>(t, length, triu != 0, step, clip_dist, counts);
    BPT_LAUNCH_CHECK();
    BPT_CUDA(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, counts, leaf_offsets, length + 1, stream));
    if (n_edges_host) {
        BPT_CUDA(cudaMemcpyAsync(n_edges_host, leaf_offsets + length, sizeof(int64_t),
                                 cudaMemcpyDeviceToHost, stream));
        BPT_CUDA(cudaStreamSynchronize(stream));
    }
    return BPT_OK;
}

extern "C" int bpt_bp_fill(int64_t length, int triu, int step, int clip_dist,
                           const int64_t *leaf_offsets, int64_t v_shift, int index_bytes,
                           void *src, void *dst, void *etype, void *pos, bpt_stream_t stream_) {
    BPT_CHECK_ARG(length >= 1 && length <= (int64_t(1) << 30), "bp_fill: length %lld out of range [1, 2^30]",
                  static_cast<long long>(length));
    BPT_CHECK_ARG(step >= 1 && clip_dist >= 0, "bp_fill: step must be >= 1 and clip_dist >= 0");
    BPT_CHECK_ARG(index_bytes == 4 || index_bytes == 8, "bp_fill: index_bytes must be 4 or 8");
    BPT_CHECK_ARG(leaf_offsets != nullptr, "bp_fill: leaf_offsets is null");
    LevelTable t;
    if (make_levels(length, &t) != 0) return fail(BPT_ERR_INVALID, "bp_fill: too many levels");
    if (index_bytes == 4)
        BPT_CHECK_ARG(t.n_nodes + v_shift < (int64_t(1) << 31), "bp_fill: node ids exceed int32");
    cudaStream_t stream = as_stream(stream_);
    const int threads = 128;
    if (src || dst || etype) {
        const unsigned blocks = static_cast<unsigned>((length + threads - 1) / threads);
        if (index_bytes == 4)
            bp_fill_kernel<int32_t><<<blocks, threads, 0, stream>>>(
                t, length, triu != 0, step, clip_dist, leaf_offsets, v_shift,
                static_cast<int32_t *>(src), static_cast<int32_t *>(dst), static_cast<int32_t *>(etype));
        else
            bp_fill_kernel<int64_t><<<blocks, threads, 0, stream>>>(
                t, length, triu != 0, step, clip_dist, leaf_offsets, v_shift,
                static_cast<int64_t *>(src), static_cast<int64_t *>(dst), static_cast<int64_t *>(etype));
        BPT_LAUNCH_CHECK();
    }
    if (pos) {
        const unsigned blocks = static_cast<unsigned>((t.n_nodes + 255) / 256);
        if (index_bytes == 4)
            bp_pos_kernel<int32_t><<<blocks, 256, 0, stream>>>(t, length, static_cast<int32_t *>(pos));
        else
            bp_pos_kernel<int64_t><<<blocks, 256, 0, stream>>>(t, length, static_cast<int64_t *>(pos));
        BPT_LAUNCH_CHECK();
    }
    return BPT_OK;
}

extern "C" size_t bpt_coo_to_csr_workspace_bytes(int64_t n_edges, int64_t n_rows) {
    if (n_edges < 0 || n_rows < 0) return 0;
    const size_t ne = static_cast<size_t>(n_edges > 0 ? n_edges : 1);
    return 4 * align_up(ne * sizeof(uint32_t), 256) +
           align_up(sort_temp_bytes(n_edges, key_bits(n_rows)), 256) + 512;
}

extern "C" int bpt_coo_to_csr(const void *key, const void *other, int64_t n_edges, int64_t n_rows,
                              int index_bytes, void *indptr, void *indices, void *eid,
                              void *workspace, size_t workspace_bytes, bpt_stream_t stream) {
    BPT_CHECK_ARG(n_edges >= 0 && n_rows >= 0, "coo_to_csr: negative size");
    BPT_CHECK_ARG(n_edges < (int64_t(1) << 31) && n_rows < (int64_t(1) << 31),
                  "coo_to_csr: more than 2^31-1 edges or rows");
    BPT_CHECK_ARG(index_bytes == 4 || index_bytes == 8, "coo_to_csr: index_bytes must be 4 or 8");
    BPT_CHECK_ARG(indptr != nullptr, "coo_to_csr: indptr is null");
    BPT_CHECK_ARG(n_edges == 0 || (key && other && indices && eid), "coo_to_csr: null array");
    if (index_bytes == 4)
        return coo_to_csr_impl<int32_t>(static_cast<const int32_t *>(key), static_cast<const int32_t *>(other),
                                        n_edges, n_rows, static_cast<int32_t *>(indptr),
                                        static_cast<int32_t *>(indices), static_cast<int32_t *>(eid),
                                        workspace, workspace_bytes, as_stream(stream));
    return coo_to_csr_impl<int64_t>(static_cast<const int64_t *>(key), static_cast<const int64_t *>(other),
                                    n_edges, n_rows, static_cast<int64_t *>(indptr),
                                    static_cast<int64_t *>(indices), static_cast<int64_t *>(eid),
                                    workspace, workspace_bytes, as_stream(stream));
}

extern "C" size_t bpt_partition_csr_workspace_bytes(int64_t n_rows) {
    if (n_rows < 0) return 0;
    return align_up(static_cast<size_t>(n_rows + 1) * sizeof(int64_t), 256) +
           align_up(scan_temp_bytes(n_rows + 1), 256) + 256;
}

extern "C" int bpt_partition_csr_count(const int64_t *indptr, int64_t n_rows, int chunk_size,
                                       int64_t *chunk_offsets, void *workspace, size_t workspace_bytes,
                                       int64_t *n_chunks_host, bpt_stream_t stream_) {
    BPT_CHECK_ARG(n_rows >= 0 && chunk_size >= 1, "partition_csr: bad n_rows or chunk_size");
    BPT_CHECK_ARG(indptr && chunk_offsets, "partition_csr: null array");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    int64_t *counts = ws.take<int64_t>(static_cast<size_t>(n_rows + 1));
    size_t temp_bytes = scan_temp_bytes(n_rows + 1);
    char *temp = ws.take<char>(temp_bytes > 0 ? temp_bytes : 1);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "partition_csr: workspace of %zu bytes is too small", workspace_bytes);
    const unsigned blocks = static_cast<unsigned>((n_rows + 1 + 255) / 256);
    chunk_count_kernel<<<blocks, 256, 0, stream>>>(indptr, n_rows, chunk_size, counts);
    BPT_LAUNCH_CHECK();
    BPT_CUDA(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, counts, chunk_offsets, n_rows + 1, stream));
    if (n_chunks_host) {
        BPT_CUDA(cudaMemcpyAsync(n_chunks_host, chunk_offsets + n_rows, sizeof(int64_t),
                                 cudaMemcpyDeviceToHost, stream));
        BPT_CUDA(cudaStreamSynchronize(stream));
    }
    return BPT_OK;
}

extern "C" int bpt_partition_csr_fill(const int64_t *indptr, int64_t n_rows, int chunk_size,
                                      const int64_t *chunk_offsets, int64_t n_chunks, int64_t *row,
                                      int64_t *indptr_out, bpt_stream_t stream_) {
    BPT_CHECK_ARG(n_rows >= 0 && chunk_size >= 1 && n_chunks >= 0, "partition_csr: bad size");
    BPT_CHECK_ARG(indptr && chunk_offsets && indptr_out, "partition_csr: null array");
    BPT_CHECK_ARG(n_chunks == 0 || row, "partition_csr: row is null");
    const unsigned blocks = static_cast<unsigned>((n_chunks + 1 + 255) / 256);
    chunk_fill_kernel<<<blocks, 256, 0, as_stream(stream_)>>>(indptr, n_rows, chunk_size, chunk_offsets,
                                                             row, indptr_out);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

// ---- baseline graphs -------------------------------------------------------------------

namespace {
// Exclusive scan of the per-leaf counts (carved first from `ws` by the caller) into leaf_offsets.
int baseline_scan(int64_t length, const int64_t *counts, int64_t *leaf_offsets, Workspace &ws,
                  int64_t *n_edges_host, cudaStream_t stream) {
    size_t temp_bytes = scan_temp_bytes(length + 1);
    char *temp = ws.take<char>(temp_bytes > 0 ? temp_bytes : 1);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "baseline graph: workspace of %zu bytes is too small", ws.size);
    BPT_CUDA(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, counts, leaf_offsets, length + 1, stream));
    if (n_edges_host) {
        BPT_CUDA(cudaMemcpyAsync(n_edges_host, leaf_offsets + length, sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
        BPT_CUDA(cudaStreamSynchronize(stream));
    }
    return BPT_OK;
}
}  // namespace

extern "C" int bpt_fc_count(int64_t length, int triu, int64_t window, int64_t *leaf_offsets, void *workspace,
                            size_t workspace_bytes, int64_t *n_edges_host, bpt_stream_t stream_) {
    BPT_CHECK_ARG(length >= 1 && length <= (int64_t(1) << 30) && window >= 0, "fc_count: bad length or window");
    BPT_CHECK_ARG(leaf_offsets != nullptr, "fc_count: leaf_offsets is null");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    int64_t *counts = ws.take<int64_t>(static_cast<size_t>(length + 1));
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "fc_count: workspace of %zu bytes is too small", workspace_bytes);
    const int64_t jmax = (length < window + 1 ? length : window + 1) - 1;  // builder.pyx:251
    fc_count_kernel<<<static_cast<unsigned>((length + 1 + 255) / 256), 256, 0, stream>>>(length, jmax, triu != 0, counts);
    BPT_LAUNCH_CHECK();
    return baseline_scan(length, counts, leaf_offsets, ws, n_edges_host, stream);
}

extern "C" int bpt_fc_fill(int64_t length, int triu, int64_t window, const int64_t *leaf_offsets, int64_t v_shift,
                           int index_bytes, void *src, void *dst, void *etype, void *pos, bpt_stream_t stream_) {
    BPT_CHECK_ARG(length >= 1 && length <= (int64_t(1) << 30) && window >= 0, "fc_fill: bad length or window");
    BPT_CHECK_ARG(index_bytes == 4 || index_bytes == 8, "fc_fill: index_bytes must be 4 or 8");
    BPT_CHECK_ARG(leaf_offsets != nullptr, "fc_fill: leaf_offsets is null");
    if (index_bytes == 4) BPT_CHECK_ARG(length + 1 + v_shift < (int64_t(1) << 31), "fc_fill: node ids exceed int32");
    cudaStream_t stream = as_stream(stream_);
    const int64_t jmax = (length < window + 1 ? length : window + 1) - 1;
    const unsigned pb = static_cast<unsigned>((length + 1 + 255) / 256);
    if (index_bytes == 4) {
        if (src || dst || etype)
            fc_fill_kernel<int32_t><<<static_cast<unsigned>(length), 128, 0, stream>>>(
                length, jmax, triu != 0, leaf_offsets, v_shift, static_cast<int32_t *>(src),
                static_cast<int32_t *>(dst), static_cast<int32_t *>(etype));
        if (pos) baseline_pos_kernel<int32_t><<<pb, 256, 0, stream>>>(length, length, static_cast<int32_t *>(pos));
    } else {
        if (src || dst || etype)
            fc_fill_kernel<int64_t><<<static_cast<unsigned>(length), 128, 0, stream>>>(
                length, jmax, triu != 0, leaf_offsets, v_shift, static_cast<int64_t *>(src),
                static_cast<int64_t *>(dst), static_cast<int64_t *>(etype));
        if (pos) baseline_pos_kernel<int64_t><<<pb, 256, 0, stream>>>(length, length, static_cast<int64_t *>(pos));
    }
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

extern "C" int bpt_oas_count(int64_t length, int64_t stride, int64_t c, int64_t *leaf_offsets, void *workspace,
                             size_t workspace_bytes, int64_t *n_edges_host, bpt_stream_t stream_) {
    BPT_CHECK_ARG(length >= 1 && length <= (int64_t(1) << 30) && stride >= 1 && c >= 0, "oas_count: bad arguments");
    BPT_CHECK_ARG(leaf_offsets != nullptr, "oas_count: leaf_offsets is null");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    int64_t *counts = ws.take<int64_t>(static_cast<size_t>(length + 1));
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "oas_count: workspace of %zu bytes is too small", workspace_bytes);
    oas_count_kernel<<<static_cast<unsigned>((length + 1 + 255) / 256), 256, 0, stream>>>(length, stride, c, counts);
    BPT_LAUNCH_CHECK();
    return baseline_scan(length, counts, leaf_offsets, ws, n_edges_host, stream);
}

extern "C" int bpt_oas_fill(int64_t length, int64_t stride, int64_t c, const int64_t *leaf_offsets, int64_t v_shift,
                            int index_bytes, void *src, void *dst, void *etype, void *pos, bpt_stream_t stream_) {
    BPT_CHECK_ARG(length >= 1 && length <= (int64_t(1) << 30) && stride >= 1 && c >= 0, "oas_fill: bad arguments");
    BPT_CHECK_ARG(index_bytes == 4 || index_bytes == 8, "oas_fill: index_bytes must be 4 or 8");
    BPT_CHECK_ARG(leaf_offsets != nullptr, "oas_fill: leaf_offsets is null");
    if (index_bytes == 4) BPT_CHECK_ARG(length + 1 + v_shift < (int64_t(1) << 31), "oas_fill: node ids exceed int32");
    cudaStream_t stream = as_stream(stream_);
    const unsigned pb = static_cast<unsigned>((length + 1 + 255) / 256);
    if (index_bytes == 4) {
        if (src || dst || etype)
            oas_fill_kernel<int32_t><<<static_cast<unsigned>(length), 128, 0, stream>>>(
                length, stride, c, leaf_offsets, v_shift, static_cast<int32_t *>(src), static_cast<int32_t *>(dst),
                static_cast<int32_t *>(etype));
        if (pos) baseline_pos_kernel<int32_t><<<pb, 256, 0, stream>>>(length, length - 1, static_cast<int32_t *>(pos));
    } else {
        if (src || dst || etype)
            oas_fill_kernel<int64_t><<<static_cast<unsigned>(length), 128, 0, stream>>>(
                length, stride, c, leaf_offsets, v_shift, static_cast<int64_t *>(src), static_cast<int64_t *>(dst),
                static_cast<int64_t *>(etype));
        if (pos) baseline_pos_kernel<int64_t><<<pb, 256, 0, stream>>>(length, length - 1, static_cast<int64_t *>(pos));
    }
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

// ---- sentence-aligned cross graph ----
namespace bpt {
namespace {
// Edge e lies in the block b with edge_offsets[b] <= e < edge_offsets[b+1]; inside the block the
// source is the slow index: (e - offset) / n_dst-th source, (e - offset) % n_dst-th destination,
// which is np.repeat(src_ids, n_dst) against np.tile(dst_ids, n_src) of graph/mt.py:318-321.
template <typename IT>
__global__ void dense_blocks_fill_kernel(const int64_t *__restrict__ blocks, const int64_t *__restrict__ edge_offsets,
                                         int64_t n_blocks, int64_t n_edges, IT *__restrict__ src, IT *__restrict__ dst) {
    const int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (e >= n_edges) return;
    int64_t lo = 0, hi = n_blocks;  // last block whose offset is <= e
    while (hi - lo > 1) {
        const int64_t mid = (lo + hi) >> 1;
        if (edge_offsets[mid] <= e) lo = mid; else hi = mid;
    }
    const int64_t *b = blocks + lo * 4;
    const int64_t local = e - edge_offsets[lo], n_dst = b[3];
    src[e] = static_cast<IT>(b[0] + local / n_dst);
    dst[e] = static_cast<IT>(b[2] + local % n_dst);
}
}  // namespace
}  // namespace bpt

extern "C" int bpt_dense_blocks_fill(const int64_t *blocks, const int64_t *edge_offsets, int64_t n_blocks,
                                     int64_t n_edges, int index_bytes, void *src, void *dst, bpt_stream_t stream_) {
    BPT_CHECK_ARG(n_blocks >= 0 && n_edges >= 0, "dense_blocks_fill: negative size");
    BPT_CHECK_ARG(index_bytes == 4 || index_bytes == 8, "dense_blocks_fill: index_bytes must be 4 or 8");
    if (n_edges == 0) return BPT_OK;
    BPT_CHECK_ARG(n_blocks >= 1 && blocks && edge_offsets && src && dst, "dense_blocks_fill: null argument");
    cudaStream_t stream = as_stream(stream_);
    const unsigned grid = static_cast<unsigned>((n_edges + 255) / 256);
    if (index_bytes == 4)
        dense_blocks_fill_kernel<int32_t><<<grid, 256, 0, stream>>>(blocks, edge_offsets, n_blocks, n_edges,
                                                                    static_cast<int32_t *>(src), static_cast<int32_t *>(dst));
    else
        dense_blocks_fill_kernel<int64_t><<<grid, 256, 0, stream>>>(blocks, edge_offsets, n_blocks, n_edges,
                                                                    static_cast<int64_t *>(src), static_cast<int64_t *>(dst));
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}
