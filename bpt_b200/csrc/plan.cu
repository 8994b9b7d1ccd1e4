// Builds the fused-attention plan on the device: the in-CSR the forward walks, the out-CSR
// and the by-type buckets the backward's segment reductions walk, and warp-sized work lists
// for each.  All of it is integer work derived from the COO edge list; none of it exists in
// the reference, which hands int64 CSRs and 32-edge chunk arrays (graph/base.py:71-86) to
// one kernel per operator.
#include <cub/device/device_scan.cuh>

#include "plan.cuh"

namespace bpt {
namespace {

// in_rank[p] = rank in the by-source order of the edge at in-CSR position p; eid_by_src maps that
// rank to the edge id.
__global__ void permute_in_kernel(const int32_t *__restrict__ in_rank, const int32_t *__restrict__ eid_by_src,
                                  const int32_t *__restrict__ etype, int64_t n_edges,
                                  int32_t *__restrict__ in_etype, int32_t *__restrict__ inpos_of_eid) {
    const int64_t p = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (p >= n_edges) return;
    const int32_t e = eid_by_src[in_rank[p]];
    in_etype[p] = etype ? etype[e] : 0;
    inpos_of_eid[e] = static_cast<int32_t>(p);
}

// flags[0..2] = 1 when some src is outside [0, n_src), some dst outside [0, n_nodes), some etype
// outside [0, n_etypes).  Everything downstream indexes with these values.
__global__ void range_check_kernel(const int32_t *__restrict__ src, const int32_t *__restrict__ dst,
                                   const int32_t *__restrict__ etype, int64_t n_edges, int64_t n_src,
                                   int64_t n_nodes, int n_etypes, int32_t *__restrict__ flags) {
    const int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (e >= n_edges) return;
    if (src[e] < 0 || src[e] >= n_src) flags[0] = 1;
    if (dst[e] < 0 || dst[e] >= n_nodes) flags[1] = 1;
    if (etype && (etype[e] < 0 || etype[e] >= n_etypes)) flags[2] = 1;
}

__global__ void gather_kernel(const int32_t *__restrict__ idx, const int32_t *__restrict__ table,
                              int64_t n, int32_t *__restrict__ out) {
    const int64_t p = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (p < n) out[p] = table[idx[p]];
}

// row_uniform[r] = 1 when the row's incoming edges all have one type (or it has none).
// One warp per row; the lanes stride over the row's edges.
__global__ void row_uniform_kernel(const int32_t *__restrict__ indptr, const int32_t *__restrict__ in_etype,
                                   int64_t n_rows, int32_t *__restrict__ row_uniform) {
    const int64_t r = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    const int beg = indptr[r], end = indptr[r + 1];
    const int first = beg < end ? in_etype[beg] : 0;
    bool same = true;
    for (int j0 = beg; j0 < end && same; j0 += 32) {
        const int j = j0 + lane;
        same = __all_sync(0xffffffffu, j >= end || in_etype[j] == first);
    }
    if (lane == 0) row_uniform[r] = same ? 1 : 0;
}

// Bucket key of every edge (edge-id order): its type, or n_etypes when its destination row is uniform.
__global__ void bucket_keys_kernel(const int32_t *__restrict__ etype, const int32_t *__restrict__ dst,
                                   const int32_t *__restrict__ row_uniform, int64_t n_edges, int n_etypes,
                                   int32_t *__restrict__ keys) {
    const int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (e >= n_edges) return;
    keys[e] = row_uniform[dst[e]] ? n_etypes : (etype ? etype[e] : 0);
}

// Per row: how many items, slots and split-row records it contributes.
__global__ void work_count_kernel(const int32_t *__restrict__ indptr, int64_t n_rows,
                                  int32_t *__restrict__ n_items, int32_t *__restrict__ n_slots,
                                  int32_t *__restrict__ n_split) {
    const int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (r > n_rows) return;
    int items = 0;
    if (r < n_rows) {
        const int deg = indptr[r + 1] - indptr[r];
        items = deg <= kSegEdges ? 1 : (deg + kSegEdges - 1) / kSegEdges;
    }
    n_items[r] = items;
    n_slots[r] = items > 1 ? items : 0;
    n_split[r] = items > 1 ? 1 : 0;
}

__global__ void work_fill_kernel(const int32_t *__restrict__ indptr, int64_t n_rows,
                                 const int32_t *__restrict__ item_off, const int32_t *__restrict__ slot_off,
                                 const int32_t *__restrict__ split_off, WorkList w) {
    const int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (r == n_rows) {
        w.counters[0] = item_off[n_rows];
        w.counters[1] = slot_off[n_rows];
        w.counters[2] = split_off[n_rows];
    }
    if (r >= n_rows) return;
    const int beg = indptr[r], end = indptr[r + 1];
    const int items = item_off[r + 1] - item_off[r];
    if (items == 1) {
        w.items[item_off[r]] = make_int4(static_cast<int>(r), beg, end, -1);
        return;
    }
    // Split evenly so no item is nearly empty.
    const int deg = end - beg;
    const int per = (deg + items - 1) / items;
    for (int i = 0; i < items; ++i) {
        const int b = beg + i * per;
        int e = b + per;
        if (e > end) e = end;
        w.items[item_off[r] + i] = make_int4(static_cast<int>(r), b, e, slot_off[r] + i);
    }
    w.split_rows[split_off[r]] = make_int4(static_cast<int>(r), slot_off[r], items, 0);
}

size_t scan_i32_temp_bytes(int64_t n) {
    size_t bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, bytes, static_cast<const int32_t *>(nullptr),
                                  static_cast<int32_t *>(nullptr), n);
    return bytes;
}

int build_work(const int32_t *indptr, int64_t n_rows, WorkList w, Workspace &ws, cudaStream_t stream) {
    const size_t n1 = static_cast<size_t>(n_rows + 1);
    int32_t *cnt = ws.take<int32_t>(3 * n1);
    int32_t *off = ws.take<int32_t>(3 * n1);
    size_t temp_bytes = scan_i32_temp_bytes(n_rows + 1);
    char *temp = ws.take<char>(temp_bytes > 0 ? temp_bytes : 1);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_plan_build: workspace too small");
    const unsigned blocks = static_cast<unsigned>((n_rows + 1 + 255) / 256);
    work_count_kernel<<<blocks, 256, 0, stream>>>(indptr, n_rows, cnt, cnt + n1, cnt + 2 * n1);
    BPT_LAUNCH_CHECK();
    for (int i = 0; i < 3; ++i)
        BPT_CUDA(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, cnt + i * n1, off + i * n1, n_rows + 1, stream));
    work_fill_kernel<<<blocks, 256, 0, stream>>>(indptr, n_rows, off, off + n1, off + 2 * n1, w);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

size_t work_ws_bytes(int64_t n_rows) {
    const size_t n1 = static_cast<size_t>(n_rows + 1);
    return 2 * align_up(3 * n1 * 4, 256) + align_up(scan_i32_temp_bytes(n_rows + 1), 256) + 256;
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" size_t bpt_attn_plan_bytes(int64_t n_nodes, int64_t n_src, int64_t n_edges, int n_etypes) {
    if (n_nodes < 0 || n_src < 0 || n_edges < 0 || n_etypes < 1) return 0;
    return plan_view(nullptr, n_nodes, n_src, n_edges, n_etypes).bytes;
}

extern "C" size_t bpt_attn_plan_workspace_bytes(int64_t n_nodes, int64_t n_src, int64_t n_edges, int n_etypes) {
    if (n_nodes < 0 || n_src < 0 || n_edges < 0 || n_etypes < 1) return 0;
    int64_t rows = n_nodes > n_etypes + 1 ? n_nodes : n_etypes + 1;
    rows = rows > n_src ? rows : n_src;
    const size_t e = static_cast<size_t>(n_edges > 0 ? n_edges : 1);
    return 5 * align_up(e * 4, 256) + bpt_coo_to_csr_workspace_bytes(n_edges, rows) + 256 + 3 * work_ws_bytes(rows) + 1024;
}

extern "C" int bpt_attn_plan_build(const int32_t *src, const int32_t *dst, const int32_t *etype,
                                   int64_t n_edges, int64_t n_nodes, int64_t n_src, int n_etypes, void *plan,
                                   size_t plan_bytes, void *workspace, size_t workspace_bytes,
                                   int32_t *counts_host, bpt_stream_t stream_) {
    BPT_CHECK_ARG(n_nodes >= 0 && n_src >= 0 && n_edges >= 0 && n_etypes >= 1, "attn_plan_build: bad sizes");
    if (n_nodes >= (int64_t(1) << 31) - 1 || n_src >= (int64_t(1) << 31) - 1 || n_edges >= (int64_t(1) << 31) - 1)
        return fail(BPT_ERR_OVERFLOW, "attn_plan_build: nodes or edges exceed 32-bit indices");
    BPT_CHECK_ARG(plan != nullptr && counts_host != nullptr, "attn_plan_build: null output");
    BPT_CHECK_ARG(n_edges == 0 || (src && dst), "attn_plan_build: null edge arrays");
    PlanView p = plan_view(plan, n_nodes, n_src, n_edges, n_etypes);
    if (plan_bytes < p.bytes) return fail(BPT_ERR_WORKSPACE, "attn_plan_build: plan buffer too small");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    const size_t e = static_cast<size_t>(n_edges > 0 ? n_edges : 1);
    int32_t *tmp_eid = ws.take<int32_t>(e);
    int32_t *inpos_of_eid = ws.take<int32_t>(e);
    int32_t *bucket_keys = ws.take<int32_t>(e);
    int32_t *eid_by_src = ws.take<int32_t>(e);
    int32_t *src_by_src = ws.take<int32_t>(e);
    int64_t rows = n_nodes > n_etypes + 1 ? n_nodes : n_etypes + 1;
    rows = rows > n_src ? rows : n_src;
    const size_t csr_ws_bytes = bpt_coo_to_csr_workspace_bytes(n_edges, rows);
    char *csr_ws = ws.take<char>(csr_ws_bytes);
    int32_t *range_flags = ws.take<int32_t>(4);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_plan_build: workspace too small");
    const unsigned eb = static_cast<unsigned>((n_edges + 255) / 256);

    // Every later kernel indexes with src, dst and etype, so an id out of range is refused here (the
    // reference's nn.Embedding raises on an edge type beyond its table, modules/attention.py:57).
    if (n_edges > 0) {
        int32_t bad[4] = {0, 0, 0, 0};
        BPT_CUDA(cudaMemsetAsync(range_flags, 0, 4 * sizeof(int32_t), stream));
        range_check_kernel<<<eb, 256, 0, stream>>>(src, dst, etype, n_edges, n_src, n_nodes, n_etypes, range_flags);
        BPT_LAUNCH_CHECK();
        BPT_CUDA(cudaMemcpyAsync(bad, range_flags, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
        BPT_CUDA(cudaStreamSynchronize(stream));
        if (bad[0] || bad[1] || bad[2])
            return fail(BPT_ERR_INVALID, "attn_plan_build: %s%s%sout of range (n_src %lld, n_nodes %lld, n_etypes %d)",
                        bad[0] ? "a source id, " : "", bad[1] ? "a destination id, " : "",
                        bad[2] ? "an edge type, " : "", static_cast<long long>(n_src),
                        static_cast<long long>(n_nodes), n_etypes);
    }

    // out-CSR (rows = sources, edge-id order inside a row)
    if (int rc = bpt_coo_to_csr(src, dst, n_edges, n_src, 4, p.out_indptr, p.out_dst, eid_by_src, csr_ws,
                                csr_ws_bytes, stream_))
        return rc;
    // in-CSR (rows = destinations), a row's edges ordered by source and then by edge id: the stable
    // sort by destination of the by-source order.  Neighbouring cells of a row of the tile plans
    // (whose columns are sorted sources) are then neighbours in every per-edge array.
    if (n_edges > 0) {
        gather_kernel<<<eb, 256, 0, stream>>>(eid_by_src, src, n_edges, src_by_src);
        BPT_LAUNCH_CHECK();
    }
    if (int rc = bpt_coo_to_csr(p.out_dst, src_by_src, n_edges, n_nodes, 4, p.in_indptr, p.in_src, tmp_eid, csr_ws,
                                csr_ws_bytes, stream_))
        return rc;
    if (n_edges > 0) {
        permute_in_kernel<<<eb, 256, 0, stream>>>(tmp_eid, eid_by_src, etype, n_edges, p.in_etype, inpos_of_eid);
        BPT_LAUNCH_CHECK();
        gather_kernel<<<eb, 256, 0, stream>>>(eid_by_src, inpos_of_eid, n_edges, p.out_inpos);
        BPT_LAUNCH_CHECK();
    }
    // buckets by edge type; edges into uniform rows (zero gradient of the type table) go last
    if (n_nodes > 0) {
        row_uniform_kernel<<<static_cast<unsigned>((n_nodes * 32 + 255) / 256), 256, 0, stream>>>(
            p.in_indptr, p.in_etype, n_nodes, p.row_uniform);
        BPT_LAUNCH_CHECK();
    }
    if (n_edges > 0) {
        bucket_keys_kernel<<<eb, 256, 0, stream>>>(etype, dst, p.row_uniform, n_edges, n_etypes, bucket_keys);
        BPT_LAUNCH_CHECK();
    }
    if (int rc = bpt_coo_to_csr(bucket_keys, dst, n_edges, n_etypes + 1, 4, p.et_indptr, p.et_dst, tmp_eid, csr_ws,
                                csr_ws_bytes, stream_))
        return rc;
    if (n_edges > 0) {
        gather_kernel<<<eb, 256, 0, stream>>>(tmp_eid, inpos_of_eid, n_edges, p.et_inpos);
        BPT_LAUNCH_CHECK();
    }
    // work lists
    if (int rc = build_work(p.in_indptr, n_nodes, p.in_work, ws, stream)) return rc;
    if (int rc = build_work(p.out_indptr, n_src, p.out_work, ws, stream)) return rc;
    if (int rc = build_work(p.et_indptr, n_etypes, p.et_work, ws, stream)) return rc;
    BPT_CUDA(cudaMemcpyAsync(counts_host + 0, p.in_work.counters, 3 * sizeof(int), cudaMemcpyDeviceToHost, stream));
    BPT_CUDA(cudaMemcpyAsync(counts_host + 3, p.out_work.counters, 3 * sizeof(int), cudaMemcpyDeviceToHost, stream));
    BPT_CUDA(cudaMemcpyAsync(counts_host + 6, p.et_work.counters, 3 * sizeof(int), cudaMemcpyDeviceToHost, stream));
    BPT_CUDA(cudaStreamSynchronize(stream));
    counts_host[kCountsNSrc] = static_cast<int32_t>(n_src);
    counts_host[10] = 0;
    counts_host[11] = 0;
    return BPT_OK;
}

extern "C" int bpt_export_in_csr(const void *plan, const int32_t *counts_host, int64_t n_nodes, int64_t n_edges,
                                 int n_etypes,
                                 int32_t *in_indptr_host, int32_t *in_src_host, int32_t *in_etype_host,
                                 bpt_stream_t stream_) {
    BPT_CHECK_ARG(plan && counts_host && in_indptr_host, "export_in_csr: null argument");
    BPT_CHECK_ARG(n_edges == 0 || (in_src_host && in_etype_host), "export_in_csr: null argument");
    const PlanView p = plan_view(const_cast<void *>(plan), n_nodes, counts_host[kCountsNSrc], n_edges, n_etypes);
    cudaStream_t stream = as_stream(stream_);
    BPT_CUDA(cudaMemcpyAsync(in_indptr_host, p.in_indptr, sizeof(int32_t) * static_cast<size_t>(n_nodes + 1),
                             cudaMemcpyDeviceToHost, stream));
    if (n_edges > 0) {
        BPT_CUDA(cudaMemcpyAsync(in_src_host, p.in_src, sizeof(int32_t) * static_cast<size_t>(n_edges),
                                 cudaMemcpyDeviceToHost, stream));
        BPT_CUDA(cudaMemcpyAsync(in_etype_host, p.in_etype, sizeof(int32_t) * static_cast<size_t>(n_edges),
                                 cudaMemcpyDeviceToHost, stream));
    }
    BPT_CUDA(cudaStreamSynchronize(stream));
    return BPT_OK;
}

extern "C" int bpt_export_out_csr(const void *plan, const int32_t *counts_host, int64_t n_nodes, int64_t n_edges,
                                  int n_etypes, int32_t *out_indptr_host, int32_t *out_dst_host,
                                  int32_t *out_inpos_host, bpt_stream_t stream_) {
    BPT_CHECK_ARG(plan && counts_host && out_indptr_host, "export_out_csr: null argument");
    BPT_CHECK_ARG(n_edges == 0 || (out_dst_host && out_inpos_host), "export_out_csr: null argument");
    const PlanView p = plan_view(const_cast<void *>(plan), n_nodes, counts_host[kCountsNSrc], n_edges, n_etypes);
    cudaStream_t stream = as_stream(stream_);
    BPT_CUDA(cudaMemcpyAsync(out_indptr_host, p.out_indptr, sizeof(int32_t) * static_cast<size_t>(p.n_src + 1),
                             cudaMemcpyDeviceToHost, stream));
    if (n_edges > 0) {
        BPT_CUDA(cudaMemcpyAsync(out_dst_host, p.out_dst, sizeof(int32_t) * static_cast<size_t>(n_edges),
                                 cudaMemcpyDeviceToHost, stream));
        BPT_CUDA(cudaMemcpyAsync(out_inpos_host, p.out_inpos, sizeof(int32_t) * static_cast<size_t>(n_edges),
                                 cudaMemcpyDeviceToHost, stream));
    }
    BPT_CUDA(cudaStreamSynchronize(stream));
    return BPT_OK;
}
