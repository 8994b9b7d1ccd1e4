// Layout of the fused-attention plan: one device blob of int32 arrays derived from a COO
// edge list.  Build (plan.cu) and the kernels that consume it share this description.
#pragma once

#include "common.cuh"

namespace bpt {

// Edges of one CSR row handled by one warp-sized work item; longer rows are split into
// several items whose partial results are merged in item order.
constexpr int kSegEdges = 128;

// counts_host layout: [0..2] in-CSR items/slots/split rows, [3..5] out-CSR, [6..8] type buckets,
// [9] number of source rows (k, v), [10..11] reserved.
constexpr int kCountsLen = 12;
constexpr int kCountsNSrc = 9;

struct WorkList {
    int4 *items;       // {row, begin, end, slot}; slot = -1 when the item covers its whole row
    int4 *split_rows;  // {row, first_slot, n_slots, 0} for rows covered by more than one item
    int *counters;     // [0] = items, [1] = slots, [2] = split rows (device-resident counts)
    int64_t max_items, max_split;
};

struct PlanView {
    int64_t n_nodes;  // destination rows (rows of the in-CSR; q, o, lse)
    int64_t n_src;    // source rows (rows of the out-CSR; k, v)
    int64_t n_edges;
    int n_etypes;
    // in-CSR: rows are destinations; a row's entries are ordered by source, then by edge id
    int32_t *in_indptr, *in_src, *in_etype;
    // 1 where all incoming edges of the row have one type (or there are none): the relative-position
    // term is then a per-row constant, cancels in the softmax and has zero gradient
    int32_t *row_uniform;
    // out-CSR: rows are sources; out_inpos = position of the same edge in the in-CSR
    int32_t *out_indptr, *out_dst, *out_inpos;
    // edges bucketed by type: et_dst = destination, et_inpos = position in the in-CSR; edges into
    // uniform rows sit in an extra last bucket (n_etypes) that nothing reads
    int32_t *et_indptr, *et_dst, *et_inpos;
    WorkList in_work, out_work, et_work;
    size_t bytes;
};

inline int64_t max_items_for(int64_t rows, int64_t edges) { return rows + edges / kSegEdges + 1; }
inline int64_t max_split_for(int64_t rows, int64_t edges) {
    const int64_t by_edges = edges / kSegEdges + 1;
    return (rows < by_edges ? rows : by_edges) + 1;
}

// Carves the blob. base may be null to compute only the size.
inline PlanView plan_view(void *base, int64_t n_nodes, int64_t n_src, int64_t n_edges, int n_etypes) {
    PlanView p;
    p.n_nodes = n_nodes;
    p.n_src = n_src;
    p.n_edges = n_edges;
    p.n_etypes = n_etypes;
    char *b = static_cast<char *>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        char *ptr = b ? b + off : nullptr;
        off += align_up(bytes > 0 ? bytes : 4, 256);
        return ptr;
    };
    const size_t e = static_cast<size_t>(n_edges), n1 = static_cast<size_t>(n_nodes + 1);
    const size_t s1 = static_cast<size_t>(n_src + 1);
    p.in_indptr = reinterpret_cast<int32_t *>(take(n1 * 4));
    p.in_src = reinterpret_cast<int32_t *>(take(e * 4));
    p.in_etype = reinterpret_cast<int32_t *>(take(e * 4));
    p.row_uniform = reinterpret_cast<int32_t *>(take(n1 * 4));
    p.out_indptr = reinterpret_cast<int32_t *>(take(s1 * 4));
    p.out_dst = reinterpret_cast<int32_t *>(take(e * 4));
    p.out_inpos = reinterpret_cast<int32_t *>(take(e * 4));
    p.et_indptr = reinterpret_cast<int32_t *>(take(static_cast<size_t>(n_etypes + 2) * 4));
    p.et_dst = reinterpret_cast<int32_t *>(take(e * 4));
    p.et_inpos = reinterpret_cast<int32_t *>(take(e * 4));
    auto work = [&](int64_t rows) {
        WorkList w;
        w.max_items = max_items_for(rows, n_edges);
        w.max_split = max_split_for(rows, n_edges);
        w.items = reinterpret_cast<int4 *>(take(static_cast<size_t>(w.max_items) * sizeof(int4)));
        w.split_rows = reinterpret_cast<int4 *>(take(static_cast<size_t>(w.max_split) * sizeof(int4)));
        w.counters = reinterpret_cast<int *>(take(4 * sizeof(int)));
        return w;
    };
    p.in_work = work(n_nodes);
    p.out_work = work(n_src);
    p.et_work = work(n_etypes);
    p.bytes = off;
    return p;
}

}  // namespace bpt
