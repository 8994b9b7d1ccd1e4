// The tile planner of the tensor-core attention path on the device.
//
// Same plan as the host planner (tile_plan.cu), array for array: dense groups of `group_rows`
// consecutive rows whose union of columns is small and reasonably filled, every other row's entries
// bucketed by block of `col_block` consecutive columns and cut into m-blocks of 16 rows, rows spread
// over several m-blocks given contiguous slots in m-block order.  Where the host walks rows and sorts
// small vectors, this file sorts composite keys once:
//   * (row group, column, parallel-edge rank) orders every row group's entries by column; the number
//     of distinct keys of a group is its column count and a running count of distinct keys gives each
//     entry its column index;
//   * a stable sort of the remaining entries by column block keeps (row, column) order inside each
//     bucket, so an entry's row ordinal inside its bucket (m-block = ordinal / 16, tile row =
//     ordinal % 16) is a running count of row changes; the bucket's columns come from a second sort by
//     (bucket, column, rank);
//   * rows split over several buckets become slots through a stable sort of the partial pieces by row.
// Everything the host needs (array sizes) crosses in three small device-to-host copies.  Takes the
// CSR arrays where bpt_attn_plan_build left them, so a new batch shape costs no export, no host
// planning and no upload.  join_dense and CUDA-core row items are not offered here (the callers that
// want them use the host planner).
#include <cub/cub.cuh>

#include <algorithm>
#include <climits>
#include <vector>

#include "common.cuh"
#include "plan.cuh"
#include "tile_plan.cuh"

namespace bpt {
namespace {

constexpr int kThreads = 256;
constexpr int kGroupShift = 40;  // composite keys: (row group or bucket) << 40 | column << 8 | rank
constexpr uint64_t kLowMask = (1ull << kGroupShift) - 1;
constexpr uint32_t kNoBucket = 0xFFFFFFFFu;

inline unsigned blocks_for(int64_t n) { return static_cast<unsigned>(std::max<int64_t>(1, (n + kThreads - 1) / kThreads)); }
inline int bits_for(uint64_t max_value) {
    int b = 1;
    while (b < 64 && (max_value >> b) != 0) ++b;
    return b;
}

// Counters and error flags kept on the device while the plan is built.
struct Counts {
    int n_left;       // entries of rows outside dense groups
    int n_buckets;    // column blocks those entries fall into
    int n_pieces;     // (bucket, row) pairs
    int n_zero_rows;  // rows without entries outside dense groups
    int n_partial;    // pieces that do not hold their row's whole entry list
    int n_split;      // rows with partial pieces
    int t_max, max_cols_pad, max_mblocks, max_qr;
    int max_etype;
    int err_rank;     // more than 256 parallel edges between two nodes
    int err_etype;    // an edge type outside [0, 65535), or (on export) one that does not fit 8 bits
};

// ---- stage 0: entries in (row, column, edge id) order with their parallel-edge rank ----
__global__ void entry_rows_kernel(const int32_t *__restrict__ indptr, int64_t n_rows, int64_t n_entries,
                                  int32_t *__restrict__ erow) {
    const int64_t j = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (j >= n_entries) return;
    int64_t lo = 0, hi = n_rows;  // last row with indptr[row] <= j
    while (hi - lo > 1) {
        const int64_t mid = (lo + hi) >> 1;
        if (indptr[mid] <= j) lo = mid; else hi = mid;
    }
    erow[j] = static_cast<int32_t>(lo);
}
__global__ void row_col_key_kernel(const int32_t *__restrict__ erow, const int32_t *__restrict__ col,
                                   int64_t n_entries, uint64_t *__restrict__ key, int32_t *__restrict__ iota) {
    const int64_t j = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (j >= n_entries) return;
    key[j] = (static_cast<uint64_t>(static_cast<uint32_t>(erow[j])) << 32) | static_cast<uint32_t>(col[j]);
    iota[j] = static_cast<int32_t>(j);
}
// Column segments (the graphs of a block-diagonal batch): segment s holds the columns [start[s], start[s + 1])
// and is planned as if it began at start[s] + shift[s], a multiple of the column block, so that the blocks of
// `col_block` consecutive columns fall in every graph where they fall when it is planned alone.  n_segs == 0:
// no shift.  The plan's column lists are shifted back once they are written.
struct ColSegments {
    const int32_t *start;  // n_segs + 1 ascending real column ids (the last one past the end)
    const int32_t *shift;  // n_segs non-decreasing shifts
    int n_segs;
};
__device__ __forceinline__ int32_t shifted_col(const ColSegments &cs, int32_t c) {
    if (cs.n_segs == 0) return c;
    int lo = 0, hi = cs.n_segs - 1;  // last segment whose start is <= c
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (cs.start[mid] <= c) lo = mid; else hi = mid - 1;
    }
    return c + cs.shift[lo];
}
__global__ void unshift_cols_kernel(int32_t *__restrict__ cols, int64_t n, ColSegments cs) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    const int32_t v = cols[i];
    int lo = 0, hi = cs.n_segs - 1;  // last segment whose shifted start is <= v
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (cs.start[mid] + cs.shift[mid] <= v) lo = mid; else hi = mid - 1;
    }
    cols[i] = v - cs.shift[lo];
}
// perm == nullptr: entry i is CSR entry i.
__global__ void gather_entries_kernel(const int32_t *__restrict__ perm, const int32_t *__restrict__ col,
                                      const int32_t *__restrict__ etype, const int32_t *__restrict__ payload,
                                      int64_t n_entries, int32_t *__restrict__ scol, int32_t *__restrict__ set,
                                      int32_t *__restrict__ spos, Counts *__restrict__ counts, ColSegments cs) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n_entries) return;
    const int32_t j = perm ? perm[i] : static_cast<int32_t>(i);
    scol[i] = shifted_col(cs, col[j]);
    const int32_t e = etype ? etype[j] : 0;
    if (e < 0 || e >= kNoEdge) atomicOr(&counts->err_etype, 1);
    set[i] = e;
    spos[i] = payload ? payload[j] : j;
}
__global__ void rank_key_kernel(const int32_t *__restrict__ indptr, const int32_t *__restrict__ erow,
                                const int32_t *__restrict__ scol, const int32_t *__restrict__ set, int64_t n_entries,
                                int group_rows, uint64_t *__restrict__ gkey, int32_t *__restrict__ iota,
                                Counts *__restrict__ counts) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n_entries) return;
    const int32_t row = erow[i], c = scol[i];
    const int64_t start = indptr[row];
    int rank = 0;
    for (int64_t k = i; k > start && scol[k - 1] == c; --k)
        if (++rank > 255) break;
    if (rank > 255) {
        atomicOr(&counts->err_rank, 1);
        rank = 255;
    }
    gkey[i] = (static_cast<uint64_t>(row / group_rows) << kGroupShift) | (static_cast<uint64_t>(static_cast<uint32_t>(c)) << 8) |
              static_cast<uint64_t>(rank);
    iota[i] = static_cast<int32_t>(i);
}
// The single edge type of each row, or -1 if its entries differ (rows without entries: 0); one warp per
// row.  Also the largest edge type of the graph (one atomic per warp).
__global__ void row_uniform_et_kernel(const int32_t *__restrict__ indptr, int64_t n_rows,
                                      const int32_t *__restrict__ set, int32_t *__restrict__ runi,
                                      Counts *__restrict__ counts) {
    const int64_t r = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    const int beg = indptr[r], end = indptr[r + 1];
    int lo = INT_MAX, hi = -1;
    for (int j = beg + lane; j < end; j += 32) {
        const int e = set ? set[j] : 0;
        lo = min(lo, e);
        hi = max(hi, e);
    }
    lo = __reduce_min_sync(0xffffffffu, lo);
    hi = __reduce_max_sync(0xffffffffu, hi);
    if (lane == 0) {
        runi[r] = end == beg ? 0 : (lo == hi ? lo : -1);
        if (hi >= 0) atomicMax(&counts->max_etype, hi);
    }
}

// ---- distinct keys of a sorted key array: flag[s] = 1 where a new key starts (s < *n_valid) ----
__global__ void distinct_flag_kernel(const uint64_t *__restrict__ sorted, int64_t n, const int *__restrict__ n_valid,
                                     int32_t *__restrict__ flag) {
    const int64_t s = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (s >= n) return;
    const int64_t valid = n_valid ? *n_valid : n;
    flag[s] = s < valid && (s == 0 || sorted[s] != sorted[s - 1]) ? 1 : 0;
}

// ---- stage 1: which row groups are dense, and the column index of their entries ----
__global__ void group_decide_kernel(const int32_t *__restrict__ indptr, int64_t n_rows, int64_t n_groups,
                                    int group_rows, const int32_t *__restrict__ ucnt, int max_cols,
                                    double min_density, int32_t *__restrict__ accept, int32_t *__restrict__ ncols_g) {
    const int64_t gi = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (gi >= n_groups) {
        if (gi == n_groups) accept[gi] = 0;  // closes the exclusive sum that numbers the dense groups
        return;
    }
    const int64_t r0 = gi * group_rows;
    const int nr = static_cast<int>(min(static_cast<int64_t>(group_rows), n_rows - r0));
    const int64_t gs = indptr[r0], ge = indptr[r0 + nr], ne = ge - gs;
    const int64_t ncols = ne > 0 ? ucnt[ge - 1] - ucnt[gs] + 1 : 0;
    const bool ok = ne == 0 || (ne <= static_cast<int64_t>(nr) * max_cols && ncols <= max_cols &&
                                static_cast<double>(ne) >= min_density * nr * ncols);
    accept[gi] = ok ? 1 : 0;
    ncols_g[gi] = ok ? static_cast<int32_t>(ncols) : 0;
}
__global__ void dense_col_kernel(const uint64_t *__restrict__ gk_sorted, const int32_t *__restrict__ gidx,
                                 const int32_t *__restrict__ ucnt, const int32_t *__restrict__ indptr,
                                 int64_t n_entries, int group_rows, const int32_t *__restrict__ accept,
                                 int32_t *__restrict__ ecol) {
    const int64_t s = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (s >= n_entries) return;
    const int64_t gi = static_cast<int64_t>(gk_sorted[s] >> kGroupShift);
    if (!accept[gi]) return;
    ecol[gidx[s]] = ucnt[s] - ucnt[indptr[gi * group_rows]];
}

// ---- stage 2: the other rows ----
__global__ void zero_row_flag_kernel(const int32_t *__restrict__ indptr, int64_t n_rows, int group_rows,
                                     const int32_t *__restrict__ accept, int32_t *__restrict__ zflag,
                                     int32_t *__restrict__ iota) {
    const int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (r >= n_rows) return;
    zflag[r] = !accept[r / group_rows] && indptr[r + 1] == indptr[r] ? 1 : 0;
    iota[r] = static_cast<int32_t>(r);
}
__global__ void left_key_kernel(const int32_t *__restrict__ erow, const int32_t *__restrict__ scol,
                                const uint64_t *__restrict__ gkey, int64_t n_entries, int group_rows, int col_block,
                                const int32_t *__restrict__ accept, uint32_t *__restrict__ sbkey,
                                uint64_t *__restrict__ bkey, int32_t *__restrict__ iota, int32_t *__restrict__ iota2,
                                Counts *__restrict__ counts) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    bool left = false;
    if (i < n_entries) {
        left = !accept[erow[i] / group_rows];
        const uint32_t sb = static_cast<uint32_t>(scol[i] / col_block);
        sbkey[i] = left ? sb : kNoBucket;
        bkey[i] = left ? (static_cast<uint64_t>(sb) << kGroupShift) | (gkey[i] & kLowMask) : ~0ull;
        iota[i] = static_cast<int32_t>(i);
        iota2[i] = static_cast<int32_t>(i);
    }
    const int n = __syncthreads_count(left);
    if (threadIdx.x == 0 && n) atomicAdd(&counts->n_left, n);
}
// On the entries sorted by bucket (stable: (row, column) order inside a bucket): where buckets and
// (bucket, row) pieces start.
__global__ void piece_flag_kernel(const uint32_t *__restrict__ sb_sorted, const int32_t *__restrict__ le,
                                  const int32_t *__restrict__ erow, int64_t n_entries,
                                  const Counts *__restrict__ counts, int32_t *__restrict__ pflag,
                                  int32_t *__restrict__ bflag) {
    const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (t >= n_entries) return;
    int p = 0, b = 0;
    if (t < counts->n_left) {
        b = t == 0 || sb_sorted[t] != sb_sorted[t - 1];
        p = b || erow[le[t]] != erow[le[t - 1]];
    }
    pflag[t] = p;
    bflag[t] = b;
}
__global__ void piece_scatter_kernel(const int32_t *__restrict__ pflag, const int32_t *__restrict__ bflag,
                                     const int32_t *__restrict__ pscan, const int32_t *__restrict__ bscan,
                                     const int32_t *__restrict__ le, const int32_t *__restrict__ erow,
                                     int64_t n_entries, Counts *__restrict__ counts, int32_t *__restrict__ bstart,
                                     int32_t *__restrict__ pb0, int32_t *__restrict__ piece_row,
                                     int32_t *__restrict__ piece_t0) {
    const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (t >= n_entries || t >= counts->n_left) return;
    const int b = bscan[t] - 1, p = pscan[t] - 1;
    if (bflag[t]) {
        bstart[b] = static_cast<int32_t>(t);
        pb0[b] = p;
    }
    if (pflag[t]) {
        piece_row[p] = erow[le[t]];
        piece_t0[p] = static_cast<int32_t>(t);
    }
    if (t == counts->n_left - 1) {
        counts->n_buckets = b + 1;
        counts->n_pieces = p + 1;
    }
}
// Per bucket: m-blocks and group copies; per entry (in bucket order): its bucket and row ordinal.
__global__ void bucket_kernel(const int32_t *__restrict__ pb0, int64_t n_max, const Counts *__restrict__ counts,
                              int max_mblocks, int32_t *__restrict__ nmb_b, int32_t *__restrict__ ncopies_b) {
    const int64_t b = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (b > n_max) return;
    int nmb = 0;
    if (b < counts->n_buckets) {
        const int nrows = (b + 1 < counts->n_buckets ? pb0[b + 1] : counts->n_pieces) - pb0[b];
        nmb = (nrows + kTileRows - 1) / kTileRows;
    }
    nmb_b[b] = nmb;
    ncopies_b[b] = (nmb + max_mblocks - 1) / max_mblocks;
}
__global__ void entry_piece_kernel(const int32_t *__restrict__ pscan, const int32_t *__restrict__ bscan,
                                   const int32_t *__restrict__ pb0, const int32_t *__restrict__ le,
                                   int64_t n_entries, const Counts *__restrict__ counts, int32_t *__restrict__ e_bucket,
                                   int32_t *__restrict__ e_ord) {
    const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (t >= n_entries || t >= counts->n_left) return;
    const int b = bscan[t] - 1;
    e_bucket[le[t]] = b;
    e_ord[le[t]] = pscan[t] - 1 - pb0[b];
}
__global__ void piece_partial_kernel(const int32_t *__restrict__ piece_row, const int32_t *__restrict__ piece_t0,
                                     const int32_t *__restrict__ indptr, int64_t n_max, Counts *__restrict__ counts,
                                     uint32_t *__restrict__ part_key, int32_t *__restrict__ iota) {
    const int64_t p = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    bool partial = false;
    if (p < n_max) {
        uint32_t key = kNoBucket;
        if (p < counts->n_pieces) {
            const int cnt = (p + 1 < counts->n_pieces ? piece_t0[p + 1] : counts->n_left) - piece_t0[p];
            const int row = piece_row[p];
            partial = cnt != indptr[row + 1] - indptr[row];
            if (partial) key = static_cast<uint32_t>(row);
        }
        part_key[p] = key;
        iota[p] = static_cast<int32_t>(p);
    }
    const int n = __syncthreads_count(partial);
    if (threadIdx.x == 0 && n) atomicAdd(&counts->n_partial, n);
}
// On the leftover entries sorted by (bucket, column, rank): column index inside the bucket, bucket widths.
__global__ void left_col_kernel(const int32_t *__restrict__ gidx2, const int32_t *__restrict__ ucnt2,
                                const int32_t *__restrict__ bflag, const int32_t *__restrict__ bscan,
                                const int32_t *__restrict__ bstart, int64_t n_entries,
                                const Counts *__restrict__ counts, int32_t *__restrict__ ecol,
                                int32_t *__restrict__ ncols_b) {
    const int64_t s = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (s >= n_entries || s >= counts->n_left) return;
    const int b = bscan[s] - 1;
    const int c = ucnt2[s] - ucnt2[bstart[b]];
    ecol[gidx2[s]] = c;
    if (s + 1 == counts->n_left || bflag[s + 1]) ncols_b[b] = c + 1;
}

// ---- stage 3: emitted groups ----
struct GroupArrays {
    int32_t *ncols, *pad, *mbc, *cells;       // per emitted group (+1 closing element for the scans)
    int32_t *col_off, *mb_first;              // exclusive sums of pad, mbc
    int64_t *cells_off;                       // exclusive sum of cells (64-bit: the total is checked against 2^31)
};
__device__ __forceinline__ void set_group(const GroupArrays &g, int64_t gr, int ncols, int mbc) {
    const int pad = (ncols + kTileChunk - 1) / kTileChunk * kTileChunk;
    g.ncols[gr] = ncols;
    g.pad[gr] = pad;
    g.mbc[gr] = mbc;
    g.cells[gr] = mbc * (pad / kTileChunk) * kTileRows * kTileChunk;
}
__global__ void emit_groups_kernel(GroupArrays g, int64_t n_row_groups, int64_t n_rows, int group_rows,
                                   const int32_t *__restrict__ accept, const int32_t *__restrict__ dpos,
                                   const int32_t *__restrict__ ncols_g, int n_dense, int n_buckets,
                                   const int32_t *__restrict__ cbase, const int32_t *__restrict__ ncopies_b,
                                   const int32_t *__restrict__ nmb_b, const int32_t *__restrict__ ncols_b,
                                   int max_mblocks, int n_copies, int n_zero_groups) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i < n_row_groups) {
        if (accept[i]) {
            const int nr = static_cast<int>(min(static_cast<int64_t>(group_rows), n_rows - i * group_rows));
            set_group(g, dpos[i], ncols_g[i], (nr + kTileRows - 1) / kTileRows);
        }
    } else if (i < n_row_groups + n_buckets) {
        const int64_t b = i - n_row_groups;
        for (int c = 0; c < ncopies_b[b]; ++c)
            set_group(g, n_dense + cbase[b] + c, ncols_b[b], min(max_mblocks, nmb_b[b] - c * max_mblocks));
    } else if (i < n_row_groups + n_buckets + n_zero_groups) {
        set_group(g, n_dense + n_copies + (i - n_row_groups - n_buckets), 0, 1);
    } else if (i == n_row_groups + n_buckets + n_zero_groups) {
        const int64_t last = static_cast<int64_t>(n_dense) + n_copies + n_zero_groups;
        g.ncols[last] = 0; g.pad[last] = 0; g.mbc[last] = 0; g.cells[last] = 0;
    }
}

// Group records, m-block records (rows, row types, edge-type matrix offset, table slot), one thread per group.
struct PieceArrays {
    const int32_t *pb0, *piece_row;
    int32_t *piece_mb, *piece_local;
};
__global__ void write_groups_kernel(GroupArrays g, int64_t n_emitted, int n_dense, int n_copies,
                                    const int32_t *__restrict__ dense_gi, int64_t n_rows, int group_rows,
                                    const int32_t *__restrict__ copy_bucket, const int32_t *__restrict__ cbase,
                                    PieceArrays pc, int n_buckets, int n_pieces, int n_zero_rows, int max_mblocks,
                                    const int32_t *__restrict__ zrows, const int32_t *__restrict__ runi,
                                    int32_t *__restrict__ groups, int32_t *__restrict__ mblocks,
                                    int32_t *__restrict__ mb_group, Counts *__restrict__ counts) {
    const int64_t gr = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (gr >= n_emitted) return;
    int32_t *rec = groups + gr * kGroupInts;
    rec[kGroupColOff] = g.col_off[gr];
    rec[kGroupNcolsPad] = g.pad[gr];
    rec[kGroupMbFirst] = g.mb_first[gr];
    rec[kGroupMbCount] = g.mbc[gr];
    rec[kGroupNcols] = g.ncols[gr];
    rec[5] = 0; rec[6] = 0; rec[7] = 0;
    atomicMax(&counts->max_cols_pad, g.pad[gr]);
    atomicMax(&counts->max_mblocks, g.mbc[gr]);
    const int chunk_cells = (g.pad[gr] / kTileChunk) * kTileRows * kTileChunk;
    int n_qr = 0;
    for (int k = 0; k < g.mbc[gr]; ++k) {
        const int64_t m = g.mb_first[gr] + k;
        int32_t *mb = mblocks + m * kMbInts;
        mb_group[m] = static_cast<int32_t>(gr);
        bool uniform = true;
        for (int i = 0; i < kTileRows; ++i) {
            int32_t row = -1;
            if (gr < n_dense) {
                const int64_t r = static_cast<int64_t>(dense_gi[gr]) * group_rows + k * kTileRows + i;
                const int64_t end = min(n_rows, (static_cast<int64_t>(dense_gi[gr]) + 1) * group_rows);
                if (r < end) row = static_cast<int32_t>(r);
            } else if (gr < n_dense + n_copies) {
                const int b = copy_bucket[gr - n_dense];
                const int copy = static_cast<int>(gr - n_dense) - cbase[b];
                const int ord = (copy * max_mblocks + k) * kTileRows + i;
                const int nrows = (b + 1 < n_buckets ? pc.pb0[b + 1] : n_pieces) - pc.pb0[b];
                if (ord < nrows) {
                    const int p = pc.pb0[b] + ord;
                    row = pc.piece_row[p];
                    pc.piece_mb[p] = static_cast<int32_t>(m);
                    pc.piece_local[p] = i;
                }
            } else {
                const int64_t z = (gr - n_dense - n_copies) * kTileRows + i;
                if (z < n_zero_rows) row = zrows[z];
            }
            mb[kMbRowOff + i] = row;
            mb[kMbSlotOff + i] = -1;
            mb[kMbRowEtOff + i] = row >= 0 ? runi[row] : 0;
            if (row >= 0 && runi[row] < 0) uniform = false;
        }
        mb[kMbEtOff] = static_cast<int32_t>(g.cells_off[gr]) + k * chunk_cells;
        mb[kMbChunkMask] = 0;
        mb[kMbTq] = -1;  // holds the largest edge type until finish_mblocks_kernel
        mb[kMbQrSlot] = uniform ? -1 : n_qr++;
        mb[kMbFineMask] = 0;
        mb[53] = 0; mb[54] = 0; mb[55] = 0;
    }
    atomicMax(&counts->max_qr, n_qr);
}
__global__ void dense_gi_kernel(const int32_t *__restrict__ accept, const int32_t *__restrict__ dpos,
                                int64_t n_row_groups, int32_t *__restrict__ dense_gi) {
    const int64_t gi = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (gi < n_row_groups && accept[gi]) dense_gi[dpos[gi]] = static_cast<int32_t>(gi);
}
__global__ void copy_bucket_kernel(const int32_t *__restrict__ cbase, const int32_t *__restrict__ ncopies_b,
                                   int n_buckets, int32_t *__restrict__ copy_bucket) {
    const int64_t b = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (b >= n_buckets) return;
    for (int c = 0; c < ncopies_b[b]; ++c) copy_bucket[cbase[b] + c] = static_cast<int32_t>(b);
}

// Column lists: every distinct key writes its column (the first one also the padding columns).
__global__ void write_dense_cols_kernel(const uint64_t *__restrict__ gk_sorted, const int32_t *__restrict__ uflag,
                                        const int32_t *__restrict__ ucnt, const int32_t *__restrict__ indptr,
                                        int64_t n_entries, int group_rows, const int32_t *__restrict__ accept,
                                        const int32_t *__restrict__ dpos, GroupArrays g, int32_t *__restrict__ cols) {
    const int64_t s = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (s >= n_entries || !uflag[s]) return;
    const int64_t gi = static_cast<int64_t>(gk_sorted[s] >> kGroupShift);
    if (!accept[gi]) return;
    const int64_t gr = dpos[gi];
    const int c = ucnt[s] - ucnt[indptr[gi * group_rows]];
    const int32_t col = static_cast<int32_t>((gk_sorted[s] & kLowMask) >> 8);
    int32_t *out = cols + g.col_off[gr];
    out[c] = col;
    if (c == 0)
        for (int pc = g.ncols[gr]; pc < g.pad[gr]; ++pc) out[pc] = col;
}
__global__ void write_bucket_cols_kernel(const uint64_t *__restrict__ bk_sorted, const int32_t *__restrict__ uflag2,
                                         const int32_t *__restrict__ ucnt2, const int32_t *__restrict__ bscan,
                                         const int32_t *__restrict__ bstart, int64_t n_entries,
                                         const Counts *__restrict__ counts, int n_dense,
                                         const int32_t *__restrict__ cbase, const int32_t *__restrict__ ncopies_b,
                                         GroupArrays g, int32_t *__restrict__ cols) {
    const int64_t s = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (s >= n_entries || s >= counts->n_left || !uflag2[s]) return;
    const int b = bscan[s] - 1;
    const int c = ucnt2[s] - ucnt2[bstart[b]];
    const int32_t col = static_cast<int32_t>((bk_sorted[s] & kLowMask) >> 8);
    for (int copy = 0; copy < ncopies_b[b]; ++copy) {
        const int64_t gr = static_cast<int64_t>(n_dense) + cbase[b] + copy;
        int32_t *out = cols + g.col_off[gr];
        out[c] = col;
        if (c == 0)
            for (int pc = g.ncols[gr]; pc < g.pad[gr]; ++pc) out[pc] = col;
    }
}

// Every entry into its cell: edge type, payload (in the order the mma lanes read), activity masks.
__global__ void scatter_entries_kernel(const int32_t *__restrict__ erow, const int32_t *__restrict__ ecol,
                                       const int32_t *__restrict__ set, const int32_t *__restrict__ spos,
                                       int64_t n_entries, int group_rows, const int32_t *__restrict__ accept,
                                       const int32_t *__restrict__ dpos, int n_dense,
                                       const int32_t *__restrict__ e_bucket, const int32_t *__restrict__ e_ord,
                                       const int32_t *__restrict__ cbase, int max_mblocks, GroupArrays g,
                                       int32_t *__restrict__ mblocks, uint16_t *__restrict__ et,
                                       int32_t *__restrict__ cellpos) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n_entries) return;
    const int32_t row = erow[i];
    const int64_t gi = row / group_rows;
    int64_t gr;
    int k, r;
    if (accept[gi]) {
        gr = dpos[gi];
        const int local = static_cast<int>(row - gi * group_rows);
        k = local / kTileRows;
        r = local % kTileRows;
    } else {
        const int mbk = e_ord[i] / kTileRows;
        r = e_ord[i] % kTileRows;
        gr = static_cast<int64_t>(n_dense) + cbase[e_bucket[i]] + mbk / max_mblocks;
        k = mbk % max_mblocks;
    }
    const int c = ecol[i];
    const int64_t m = g.mb_first[gr] + k;
    int32_t *mb = mblocks + m * kMbInts;
    const int64_t base = mb[kMbEtOff];
    const int chunk = c / kTileChunk, cc = c % kTileChunk;
    et[base + (static_cast<int64_t>(chunk) * kTileRows + r) * kTileChunk + cc] = static_cast<uint16_t>(set[i]);
    cellpos[base + static_cast<int64_t>(chunk) * kTileRows * kTileChunk + cell_pos_index(r, cc)] = spos[i];
    atomicOr(reinterpret_cast<unsigned int *>(mb + kMbChunkMask), 1u << (c / kMaskCols));
    if (c < 512) atomicOr(reinterpret_cast<unsigned int *>(mb + kMbFineMask), 1u << (c / 16));
    atomicMax(mb + kMbTq, set[i]);
}
__global__ void finish_mblocks_kernel(int64_t n_mblocks, const int32_t *__restrict__ mb_group, GroupArrays g,
                                      int32_t *__restrict__ mblocks, Counts *__restrict__ counts) {
    const int64_t m = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (m >= n_mblocks) return;
    int32_t *mb = mblocks + m * kMbInts;
    const int tq = (mb[kMbTq] + 1 + 7) / 8 * 8;
    mb[kMbTq] = tq;
    if (g.pad[mb_group[m]] > 512) mb[kMbFineMask] = 0;
    if (mb[kMbQrSlot] >= 0) atomicMax(&counts->t_max, tq);
}

// ---- slots of the rows that are spread over several m-blocks ----
__global__ void slot_kernel(const uint32_t *__restrict__ prow_sorted, const int32_t *__restrict__ pidx_sorted,
                            int64_t n_max, const Counts *__restrict__ counts, const int32_t *__restrict__ piece_mb,
                            const int32_t *__restrict__ piece_local, int32_t *__restrict__ mblocks,
                            int32_t *__restrict__ sflag) {
    const int64_t q = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (q >= n_max) return;
    int f = 0;
    if (q < counts->n_partial) {
        const int p = pidx_sorted[q];
        mblocks[static_cast<int64_t>(piece_mb[p]) * kMbInts + kMbSlotOff + piece_local[p]] = static_cast<int32_t>(q);
        f = q == 0 || prow_sorted[q] != prow_sorted[q - 1];
    }
    sflag[q] = f;
}
__global__ void split_first_kernel(const uint32_t *__restrict__ prow_sorted, const int32_t *__restrict__ sflag,
                                   const int32_t *__restrict__ sscan, int64_t n_max, Counts *__restrict__ counts,
                                   int32_t *__restrict__ split) {
    const int64_t q = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (q >= n_max || q >= counts->n_partial) return;
    if (sflag[q]) {
        int32_t *rec = split + static_cast<int64_t>(sscan[q] - 1) * 4;
        rec[0] = static_cast<int32_t>(prow_sorted[q]);
        rec[1] = static_cast<int32_t>(q);
        rec[3] = 0;
    }
    if (q == counts->n_partial - 1) counts->n_split = sscan[q];
}
__global__ void split_count_kernel(int64_t n_max, const Counts *__restrict__ counts, int32_t *__restrict__ split) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n_max || i >= counts->n_split) return;
    const int next = i + 1 < counts->n_split ? split[(i + 1) * 4 + 1] : counts->n_partial;
    split[i * 4 + 2] = next - split[i * 4 + 1];
}

__global__ void narrow_et_kernel(const uint16_t *__restrict__ et, int64_t n, uint8_t *__restrict__ out,
                                 Counts *__restrict__ counts) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    const uint16_t e = et[i];
    if (e != kNoEdge && e >= kNoEdge8) atomicOr(&counts->err_etype, 2);
    out[i] = e == kNoEdge ? kNoEdge8 : static_cast<uint8_t>(e);
}

// Device memory of one build, released together.
struct Arena {
    std::vector<void *> blocks;
    char *pool = nullptr;  // one reservation that the first takes are carved from
    size_t pool_bytes = 0, pool_used = 0;
    bool ok = true;
    void reserve(size_t bytes) {
        void *p = nullptr;
        if (pool == nullptr && cudaMalloc(&p, bytes) == cudaSuccess) {
            blocks.push_back(p);
            pool = static_cast<char *>(p);
            pool_bytes = bytes;
        } else {
            cudaGetLastError();  // a reservation that does not fit is not an error: takes allocate one by one
        }
    }
    template <typename T>
    T *take(int64_t count) {
        const size_t bytes = align_up(static_cast<size_t>(std::max<int64_t>(count, 1)) * sizeof(T), 256);
        if (pool_used + bytes <= pool_bytes) {
            T *p = reinterpret_cast<T *>(pool + pool_used);
            pool_used += bytes;
            return p;
        }
        void *p = nullptr;
        if (cudaMalloc(&p, bytes) != cudaSuccess) {
            ok = false;
            return nullptr;
        }
        blocks.push_back(p);
        return static_cast<T *>(p);
    }
    void release() {
        for (void *p : blocks) cudaFree(p);
        blocks.clear();
    }
    ~Arena() { release(); }
};

struct DeviceTilePlan {
    Arena mem;  // the plan's arrays
    int32_t *groups = nullptr, *mblocks = nullptr, *cols = nullptr, *cellpos = nullptr, *split = nullptr;
    uint16_t *et = nullptr;
    Counts *counts = nullptr;
    int64_t sizes[13] = {0};
};

#define PLAN_CUDA(call)                                                                                   \
    do {                                                                                                  \
        cudaError_t err__ = (call);                                                                       \
        if (err__ != cudaSuccess) {                                                                       \
            fail(BPT_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(err__), __FILE__, __LINE__); \
            return false;                                                                                 \
        }                                                                                                 \
    } while (0)

struct Sorter {
    Arena &tmp;
    void *buf = nullptr;
    size_t bytes = 0;
    explicit Sorter(Arena &a) : tmp(a) {}
    bool reserve(size_t need) {
        if (need <= bytes) return true;
        buf = tmp.take<char>(static_cast<int64_t>(need));
        bytes = need;
        return buf != nullptr;
    }
    template <typename K>
    bool sort_pairs(const K *kin, K *kout, const int32_t *vin, int32_t *vout, int64_t n, int end_bit, cudaStream_t s) {
        size_t need = 0;
        PLAN_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, need, kin, kout, vin, vout, n, 0, end_bit, s));
        if (!reserve(need)) return false;
        PLAN_CUDA(cub::DeviceRadixSort::SortPairs(buf, need, kin, kout, vin, vout, n, 0, end_bit, s));
        return true;
    }
    bool inclusive_sum(const int32_t *in, int32_t *out, int64_t n, cudaStream_t s) {
        size_t need = 0;
        PLAN_CUDA(cub::DeviceScan::InclusiveSum(nullptr, need, in, out, n, s));
        if (!reserve(need)) return false;
        PLAN_CUDA(cub::DeviceScan::InclusiveSum(buf, need, in, out, n, s));
        return true;
    }
    template <typename Out>
    bool exclusive_sum(const int32_t *in, Out *out, int64_t n, cudaStream_t s) {
        size_t need = 0;
        PLAN_CUDA(cub::DeviceScan::ExclusiveScan(nullptr, need, in, out, cub::Sum(), Out(0), n, s));
        if (!reserve(need)) return false;
        PLAN_CUDA(cub::DeviceScan::ExclusiveScan(buf, need, in, out, cub::Sum(), Out(0), n, s));
        return true;
    }
    bool select_flagged(const int32_t *in, const int32_t *flags, int32_t *out, int *n_out, int64_t n, cudaStream_t s) {
        size_t need = 0;
        PLAN_CUDA(cub::DeviceSelect::Flagged(nullptr, need, in, flags, out, n_out, n, s));
        if (!reserve(need)) return false;
        PLAN_CUDA(cub::DeviceSelect::Flagged(buf, need, in, flags, out, n_out, n, s));
        return true;
    }
};

bool build(DeviceTilePlan &plan, const int32_t *indptr, const int32_t *col, const int32_t *etype,
           const int32_t *payload, int64_t R, int64_t E, bool rows_sorted, double min_density, int max_cols,
           int group_rows, int col_block, int max_mblocks, const int64_t *seg_starts_host, int n_segs,
           cudaStream_t stream) {
    Arena tmp;
    Sorter sorter(tmp);
    const int64_t nG = (R + group_rows - 1) / group_rows;
    // all temporaries of the build: ~50 arrays of one 32-bit word per entry, the sorts' scratch, per-row arrays
    tmp.reserve(static_cast<size_t>(E) * 4 * 56 + static_cast<size_t>(R) * 4 * 8 + static_cast<size_t>(nG) * 4 * 8 + (8u << 20));
    plan.counts = plan.mem.take<Counts>(1);
    if (!plan.counts) { fail(BPT_ERR_CUDA, "tile_plan_device: out of device memory"); return false; }
    Counts *counts = plan.counts;
    Counts h{};
    h.max_etype = -1;
    PLAN_CUDA(cudaMemcpyAsync(counts, &h, sizeof(h), cudaMemcpyHostToDevice, stream));

    // stage 0
    int32_t *erow = tmp.take<int32_t>(E), *scol = tmp.take<int32_t>(E), *set = tmp.take<int32_t>(E);
    int32_t *spos = tmp.take<int32_t>(E), *iota = tmp.take<int32_t>(std::max(E, R)), *iota2 = tmp.take<int32_t>(E);
    uint64_t *gkey = tmp.take<uint64_t>(E), *gk_sorted = tmp.take<uint64_t>(E);
    int32_t *gidx = tmp.take<int32_t>(E), *uflag = tmp.take<int32_t>(E), *ucnt = tmp.take<int32_t>(E);
    int32_t *runi = tmp.take<int32_t>(R);
    int32_t *accept = tmp.take<int32_t>(nG + 1), *dpos = tmp.take<int32_t>(nG + 1), *ncols_g = tmp.take<int32_t>(nG + 1);
    int32_t *ecol = tmp.take<int32_t>(E);
    if (!tmp.ok) { fail(BPT_ERR_CUDA, "tile_plan_device: out of device memory"); return false; }
    ColSegments cs{nullptr, nullptr, 0};
    std::vector<int32_t> seg_host;  // starts, then shifts; read by the copy below before this function returns
    if (n_segs > 0) {
        seg_host.resize(2 * static_cast<size_t>(n_segs) + 1);
        int64_t vstart = 0;
        for (int i = 0; i < n_segs; ++i) {
            seg_host[i] = static_cast<int32_t>(seg_starts_host[i]);
            seg_host[n_segs + 1 + i] = static_cast<int32_t>(vstart - seg_starts_host[i]);
            vstart = (vstart + (seg_starts_host[i + 1] - seg_starts_host[i]) + col_block - 1) / col_block * col_block;
        }
        seg_host[n_segs] = static_cast<int32_t>(seg_starts_host[n_segs]);
        int32_t *seg_dev = tmp.take<int32_t>(static_cast<int64_t>(seg_host.size()));
        if (!tmp.ok) { fail(BPT_ERR_CUDA, "tile_plan_device: out of device memory"); return false; }
        PLAN_CUDA(cudaMemcpyAsync(seg_dev, seg_host.data(), sizeof(int32_t) * seg_host.size(), cudaMemcpyHostToDevice, stream));
        PLAN_CUDA(cudaStreamSynchronize(stream));
        cs = ColSegments{seg_dev, seg_dev + n_segs + 1, n_segs};
    }
    if (E > 0) {
        entry_rows_kernel<<<blocks_for(E), kThreads, 0, stream>>>(indptr, R, E, erow);
        const int32_t *perm = nullptr;
        if (!rows_sorted) {
            // a row's entries by (column, position): one sort of (row, column) keys, stable in the position
            row_col_key_kernel<<<blocks_for(E), kThreads, 0, stream>>>(erow, col, E, gkey, iota);
            if (!sorter.sort_pairs(gkey, gk_sorted, iota, gidx, E, 32 + bits_for(static_cast<uint64_t>(R)), stream)) return false;
            PLAN_CUDA(cudaMemcpyAsync(iota2, gidx, sizeof(int32_t) * E, cudaMemcpyDeviceToDevice, stream));
            perm = iota2;
        }
        gather_entries_kernel<<<blocks_for(E), kThreads, 0, stream>>>(perm, col, etype, payload, E, scol, set, spos, counts, cs);
    }
    if (E > 0) {
        rank_key_kernel<<<blocks_for(E), kThreads, 0, stream>>>(indptr, erow, scol, set, E, group_rows, gkey, iota, counts);
        // stage 1
        if (!sorter.sort_pairs(gkey, gk_sorted, iota, gidx, E, kGroupShift + bits_for(static_cast<uint64_t>(nG)), stream)) return false;
        distinct_flag_kernel<<<blocks_for(E), kThreads, 0, stream>>>(gk_sorted, E, nullptr, uflag);
        if (!sorter.inclusive_sum(uflag, ucnt, E, stream)) return false;
    }
    row_uniform_et_kernel<<<blocks_for(R * 32), kThreads, 0, stream>>>(indptr, R, E > 0 ? set : nullptr, runi, counts);
    group_decide_kernel<<<blocks_for(nG + 1), kThreads, 0, stream>>>(indptr, R, nG, group_rows, ucnt, max_cols, min_density, accept, ncols_g);
    if (!sorter.exclusive_sum(accept, dpos, nG + 1, stream)) return false;
    if (E > 0) dense_col_kernel<<<blocks_for(E), kThreads, 0, stream>>>(gk_sorted, gidx, ucnt, indptr, E, group_rows, accept, ecol);

    // stage 2
    int32_t *zflag = tmp.take<int32_t>(R), *zrows = tmp.take<int32_t>(R);
    uint32_t *sbkey = tmp.take<uint32_t>(E), *sb_sorted = tmp.take<uint32_t>(E);
    uint64_t *bkey = tmp.take<uint64_t>(E), *bk_sorted = tmp.take<uint64_t>(E);
    int32_t *le = tmp.take<int32_t>(E), *gidx2 = tmp.take<int32_t>(E);
    int32_t *pflag = tmp.take<int32_t>(E), *bflag = tmp.take<int32_t>(E + 1), *pscan = tmp.take<int32_t>(E), *bscan = tmp.take<int32_t>(E);
    int32_t *bstart = tmp.take<int32_t>(E), *pb0 = tmp.take<int32_t>(E), *piece_row = tmp.take<int32_t>(E), *piece_t0 = tmp.take<int32_t>(E);
    int32_t *nmb_b = tmp.take<int32_t>(E + 1), *ncopies_b = tmp.take<int32_t>(E + 1), *cbase = tmp.take<int32_t>(E + 1), *ncols_b = tmp.take<int32_t>(E);
    int32_t *e_bucket = tmp.take<int32_t>(E), *e_ord = tmp.take<int32_t>(E);
    int32_t *uflag2 = tmp.take<int32_t>(E), *ucnt2 = tmp.take<int32_t>(E);
    uint32_t *part_key = tmp.take<uint32_t>(E), *prow_sorted = tmp.take<uint32_t>(E);
    int32_t *pidx_sorted = tmp.take<int32_t>(E);
    if (!tmp.ok) { fail(BPT_ERR_CUDA, "tile_plan_device: out of device memory"); return false; }
    zero_row_flag_kernel<<<blocks_for(R), kThreads, 0, stream>>>(indptr, R, group_rows, accept, zflag, iota);
    if (R > 0 && !sorter.select_flagged(iota, zflag, zrows, &counts->n_zero_rows, R, stream)) return false;
    if (E > 0) {
        left_key_kernel<<<blocks_for(E), kThreads, 0, stream>>>(erow, scol, gkey, E, group_rows, col_block, accept, sbkey, bkey, iota, iota2, counts);
        if (!sorter.sort_pairs(sbkey, sb_sorted, iota, le, E, 32, stream)) return false;
        piece_flag_kernel<<<blocks_for(E), kThreads, 0, stream>>>(sb_sorted, le, erow, E, counts, pflag, bflag);
        if (!sorter.inclusive_sum(pflag, pscan, E, stream)) return false;
        if (!sorter.inclusive_sum(bflag, bscan, E, stream)) return false;
        piece_scatter_kernel<<<blocks_for(E), kThreads, 0, stream>>>(pflag, bflag, pscan, bscan, le, erow, E, counts, bstart, pb0, piece_row, piece_t0);
        entry_piece_kernel<<<blocks_for(E), kThreads, 0, stream>>>(pscan, bscan, pb0, le, E, counts, e_bucket, e_ord);
        if (!sorter.sort_pairs(bkey, bk_sorted, iota2, gidx2, E, 64, stream)) return false;
        distinct_flag_kernel<<<blocks_for(E), kThreads, 0, stream>>>(bk_sorted, E, &counts->n_left, uflag2);
        if (!sorter.inclusive_sum(uflag2, ucnt2, E, stream)) return false;
        left_col_kernel<<<blocks_for(E), kThreads, 0, stream>>>(gidx2, ucnt2, bflag, bscan, bstart, E, counts, ecol, ncols_b);
        piece_partial_kernel<<<blocks_for(E), kThreads, 0, stream>>>(piece_row, piece_t0, indptr, E, counts, part_key, iota);
    }
    bucket_kernel<<<blocks_for(E + 1), kThreads, 0, stream>>>(pb0, E, counts, max_mblocks, nmb_b, ncopies_b);
    if (!sorter.exclusive_sum(ncopies_b, cbase, E + 1, stream)) return false;

    // first crossing: how many groups of each kind
    int n_dense = 0, n_copies = 0;
    PLAN_CUDA(cudaMemcpyAsync(&h, counts, sizeof(h), cudaMemcpyDeviceToHost, stream));
    PLAN_CUDA(cudaMemcpyAsync(&n_dense, dpos + nG, sizeof(int), cudaMemcpyDeviceToHost, stream));
    PLAN_CUDA(cudaStreamSynchronize(stream));
    if (h.err_rank) { fail(BPT_ERR_UNSUPPORTED, "tile_plan_create: more than 256 parallel edges between two nodes"); return false; }
    if (h.err_etype) { fail(BPT_ERR_UNSUPPORTED, "tile_plan_create: an edge type outside [0, 65535)"); return false; }
    PLAN_CUDA(cudaMemcpyAsync(&n_copies, cbase + h.n_buckets, sizeof(int), cudaMemcpyDeviceToHost, stream));
    PLAN_CUDA(cudaStreamSynchronize(stream));
    const int n_zero_groups = (h.n_zero_rows + kTileRows - 1) / kTileRows;
    const int64_t n_emitted = static_cast<int64_t>(n_dense) + n_copies + n_zero_groups;

    // stage 3
    GroupArrays g;
    g.ncols = tmp.take<int32_t>(n_emitted + 1); g.pad = tmp.take<int32_t>(n_emitted + 1);
    g.mbc = tmp.take<int32_t>(n_emitted + 1); g.cells = tmp.take<int32_t>(n_emitted + 1);
    g.col_off = tmp.take<int32_t>(n_emitted + 1); g.mb_first = tmp.take<int32_t>(n_emitted + 1);
    g.cells_off = tmp.take<int64_t>(n_emitted + 1);
    int32_t *dense_gi = tmp.take<int32_t>(n_dense), *copy_bucket = tmp.take<int32_t>(n_copies);
    if (!tmp.ok) { fail(BPT_ERR_CUDA, "tile_plan_device: out of device memory"); return false; }
    emit_groups_kernel<<<blocks_for(nG + h.n_buckets + n_zero_groups + 1), kThreads, 0, stream>>>(
        g, nG, R, group_rows, accept, dpos, ncols_g, n_dense, h.n_buckets, cbase, ncopies_b, nmb_b, ncols_b, max_mblocks,
        n_copies, n_zero_groups);
    dense_gi_kernel<<<blocks_for(nG), kThreads, 0, stream>>>(accept, dpos, nG, dense_gi);
    copy_bucket_kernel<<<blocks_for(h.n_buckets), kThreads, 0, stream>>>(cbase, ncopies_b, h.n_buckets, copy_bucket);
    if (!sorter.exclusive_sum(g.pad, g.col_off, n_emitted + 1, stream)) return false;
    if (!sorter.exclusive_sum(g.mbc, g.mb_first, n_emitted + 1, stream)) return false;
    if (!sorter.exclusive_sum(g.cells, g.cells_off, n_emitted + 1, stream)) return false;
    // second crossing: array sizes.  Cell offsets are 32-bit in the m-block records; check the 64-bit total.
    int totals[2] = {0, 0};
    int64_t total_cells = 0;
    PLAN_CUDA(cudaMemcpyAsync(&totals[0], g.col_off + n_emitted, sizeof(int), cudaMemcpyDeviceToHost, stream));
    PLAN_CUDA(cudaMemcpyAsync(&totals[1], g.mb_first + n_emitted, sizeof(int), cudaMemcpyDeviceToHost, stream));
    PLAN_CUDA(cudaMemcpyAsync(&total_cells, g.cells_off + n_emitted, sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
    PLAN_CUDA(cudaStreamSynchronize(stream));
    const int64_t n_cols = totals[0], n_mblocks = totals[1], n_cells = total_cells;
    if (n_cols < 0 || n_mblocks < 0 || n_cells >= (1ll << 31)) {
        fail(BPT_ERR_UNSUPPORTED, "tile_plan_create: the plan has more than 2^31 cells");
        return false;
    }
    plan.groups = plan.mem.take<int32_t>(n_emitted * kGroupInts);
    plan.mblocks = plan.mem.take<int32_t>(n_mblocks * kMbInts);
    plan.cols = plan.mem.take<int32_t>(n_cols);
    plan.et = plan.mem.take<uint16_t>(n_cells);
    plan.cellpos = plan.mem.take<int32_t>(n_cells);
    plan.split = plan.mem.take<int32_t>(static_cast<int64_t>(h.n_partial) * 4);
    int32_t *mb_group = tmp.take<int32_t>(n_mblocks);
    int32_t *piece_mb = tmp.take<int32_t>(h.n_pieces), *piece_local = tmp.take<int32_t>(h.n_pieces);
    int32_t *sflag = tmp.take<int32_t>(h.n_pieces), *sscan = tmp.take<int32_t>(h.n_pieces);
    if (!tmp.ok || !plan.mem.ok) { fail(BPT_ERR_CUDA, "tile_plan_device: out of device memory"); return false; }
    PLAN_CUDA(cudaMemsetAsync(plan.et, 0xff, sizeof(uint16_t) * std::max<int64_t>(n_cells, 1), stream));
    PLAN_CUDA(cudaMemsetAsync(plan.cellpos, 0xff, sizeof(int32_t) * std::max<int64_t>(n_cells, 1), stream));
    PieceArrays pc{pb0, piece_row, piece_mb, piece_local};
    write_groups_kernel<<<blocks_for(n_emitted), kThreads, 0, stream>>>(
        g, n_emitted, n_dense, n_copies, dense_gi, R, group_rows, copy_bucket, cbase, pc, h.n_buckets, h.n_pieces,
        h.n_zero_rows, max_mblocks, zrows, runi, plan.groups, plan.mblocks, mb_group, counts);
    if (E > 0) {
        write_dense_cols_kernel<<<blocks_for(E), kThreads, 0, stream>>>(gk_sorted, uflag, ucnt, indptr, E, group_rows, accept, dpos, g, plan.cols);
        write_bucket_cols_kernel<<<blocks_for(E), kThreads, 0, stream>>>(bk_sorted, uflag2, ucnt2, bscan, bstart, E, counts, n_dense, cbase, ncopies_b, g, plan.cols);
        scatter_entries_kernel<<<blocks_for(E), kThreads, 0, stream>>>(erow, ecol, set, spos, E, group_rows, accept, dpos, n_dense, e_bucket, e_ord, cbase, max_mblocks, g, plan.mblocks, plan.et, plan.cellpos);
        if (cs.n_segs > 0 && n_cols > 0) unshift_cols_kernel<<<blocks_for(n_cols), kThreads, 0, stream>>>(plan.cols, n_cols, cs);
    }
    finish_mblocks_kernel<<<blocks_for(n_mblocks), kThreads, 0, stream>>>(n_mblocks, mb_group, g, plan.mblocks, counts);
    if (h.n_partial > 0) {
        if (!sorter.sort_pairs(part_key, prow_sorted, iota, pidx_sorted, h.n_pieces, 32, stream)) return false;
        slot_kernel<<<blocks_for(h.n_pieces), kThreads, 0, stream>>>(prow_sorted, pidx_sorted, h.n_pieces, counts, piece_mb, piece_local, plan.mblocks, sflag);
        if (!sorter.inclusive_sum(sflag, sscan, h.n_pieces, stream)) return false;
        split_first_kernel<<<blocks_for(h.n_pieces), kThreads, 0, stream>>>(prow_sorted, sflag, sscan, h.n_pieces, counts, plan.split);
        split_count_kernel<<<blocks_for(h.n_partial), kThreads, 0, stream>>>(h.n_partial, counts, plan.split);
    }
    // third crossing: the maxima and the number of split rows
    PLAN_CUDA(cudaGetLastError());
    PLAN_CUDA(cudaMemcpyAsync(&h, counts, sizeof(h), cudaMemcpyDeviceToHost, stream));
    PLAN_CUDA(cudaStreamSynchronize(stream));
    plan.sizes[0] = n_emitted;
    plan.sizes[1] = n_mblocks;
    plan.sizes[2] = n_cols;
    plan.sizes[3] = n_cells;
    plan.sizes[4] = h.n_split;
    plan.sizes[5] = h.n_partial;
    plan.sizes[6] = h.t_max;
    plan.sizes[7] = h.max_cols_pad;
    plan.sizes[8] = h.max_mblocks;
    plan.sizes[9] = h.max_qr;
    plan.sizes[10] = 0;
    plan.sizes[11] = n_dense;
    plan.sizes[12] = h.max_etype;
    return true;
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" void *bpt_tile_plan_create_device_aligned(const void *attn_plan, const int32_t *counts_host,
                                                     int64_t n_nodes, int64_t n_edges, int n_etypes, int transposed,
                                                     const int64_t *col_seg_starts_host, int n_segs,
                                                     double min_density, int max_cols, int group_rows, int col_block,
                                                     int max_mblocks, bpt_stream_t stream_) {
    if (!attn_plan || !counts_host || n_nodes < 0 || n_edges < 0 || n_edges > INT_MAX || max_cols < kTileChunk ||
        max_cols > kMaxMaskBits * kMaskCols || col_block < 1 || group_rows < kTileRows ||
        group_rows % kTileRows != 0 || max_mblocks < 1 || max_mblocks > kMaxMBlocks ||
        group_rows / kTileRows > max_mblocks) {
        fail(BPT_ERR_INVALID, "tile_plan_create_device: bad arguments");
        return nullptr;
    }
    const PlanView p = plan_view(const_cast<void *>(attn_plan), n_nodes, counts_host[kCountsNSrc], n_edges, n_etypes);
    const int64_t n_rows = transposed ? p.n_src : p.n_nodes;
    int64_t n_col_space = transposed ? p.n_nodes : p.n_src;
    if (n_segs < 0 || (n_segs > 0 && !col_seg_starts_host)) {
        fail(BPT_ERR_INVALID, "tile_plan_create_device: bad column segments");
        return nullptr;
    }
    if (n_segs > 0) {
        // segments must tile [0, columns) in ascending order; the planner then sees every segment start at a
        // multiple of col_block
        int64_t vend = 0;
        bool ok_segs = col_seg_starts_host[0] == 0 && col_seg_starts_host[n_segs] == n_col_space;
        for (int i = 0; i < n_segs && ok_segs; ++i) {
            ok_segs = col_seg_starts_host[i + 1] >= col_seg_starts_host[i];
            vend = (vend + (col_seg_starts_host[i + 1] - col_seg_starts_host[i]) + col_block - 1) / col_block * col_block;
        }
        if (!ok_segs) {
            fail(BPT_ERR_INVALID, "tile_plan_create_device: column segments must ascend from 0 to the number of columns");
            return nullptr;
        }
        n_col_space = vend;
    }
    if ((n_rows + group_rows - 1) / group_rows >= (1ll << 22) || n_rows >= (1ll << 31) - 1 ||
        n_col_space / col_block >= (1ll << 22) || n_col_space >= (1ll << 31) - 1) {
        fail(BPT_ERR_UNSUPPORTED, "tile_plan_create_device: too many rows or column blocks for the composite sort keys");
        return nullptr;
    }
    DeviceTilePlan *plan = new DeviceTilePlan();
    const bool ok = transposed
                        ? build(*plan, p.out_indptr, p.out_dst, nullptr, p.out_inpos, n_rows, n_edges, false, min_density,
                                max_cols, group_rows, col_block, max_mblocks, col_seg_starts_host, n_segs,
                                as_stream(stream_))
                        : build(*plan, p.in_indptr, p.in_src, p.in_etype, nullptr, n_rows, n_edges, true, min_density,
                                max_cols, group_rows, col_block, max_mblocks, col_seg_starts_host, n_segs,
                                as_stream(stream_));
    if (!ok) {
        cudaStreamSynchronize(as_stream(stream_));
        delete plan;
        return nullptr;
    }
    return plan;
}

extern "C" void *bpt_tile_plan_create_device(const void *attn_plan, const int32_t *counts_host, int64_t n_nodes,
                                             int64_t n_edges, int n_etypes, int transposed, double min_density,
                                             int max_cols, int group_rows, int col_block, int max_mblocks,
                                             bpt_stream_t stream_) {
    return bpt_tile_plan_create_device_aligned(attn_plan, counts_host, n_nodes, n_edges, n_etypes, transposed, nullptr, 0,
                                               min_density, max_cols, group_rows, col_block, max_mblocks, stream_);
}

extern "C" int bpt_tile_plan_device_sizes(const void *handle, int64_t *sizes) {
    BPT_CHECK_ARG(handle && sizes, "tile_plan_device_sizes: null argument");
    const DeviceTilePlan *p = static_cast<const DeviceTilePlan *>(handle);
    for (int i = 0; i < 13; ++i) sizes[i] = p->sizes[i];
    return BPT_OK;
}

extern "C" int bpt_tile_plan_device_export(const void *handle, int32_t *groups, int32_t *mblocks, int32_t *cols,
                                           void *et, int et_bytes, int32_t *cell_pos, int32_t *split_rows,
                                           bpt_stream_t stream_) {
    BPT_CHECK_ARG(handle, "tile_plan_device_export: null handle");
    BPT_CHECK_ARG(et_bytes == 1 || et_bytes == 2, "tile_plan_device_export: et_bytes must be 1 or 2");
    const DeviceTilePlan *p = static_cast<const DeviceTilePlan *>(handle);
    cudaStream_t stream = as_stream(stream_);
    const int64_t *n = p->sizes;
    if (groups && n[0] > 0)
        BPT_CUDA(cudaMemcpyAsync(groups, p->groups, sizeof(int32_t) * n[0] * kGroupInts, cudaMemcpyDeviceToDevice, stream));
    if (mblocks && n[1] > 0)
        BPT_CUDA(cudaMemcpyAsync(mblocks, p->mblocks, sizeof(int32_t) * n[1] * kMbInts, cudaMemcpyDeviceToDevice, stream));
    if (cols && n[2] > 0) BPT_CUDA(cudaMemcpyAsync(cols, p->cols, sizeof(int32_t) * n[2], cudaMemcpyDeviceToDevice, stream));
    if (cell_pos && n[3] > 0)
        BPT_CUDA(cudaMemcpyAsync(cell_pos, p->cellpos, sizeof(int32_t) * n[3], cudaMemcpyDeviceToDevice, stream));
    if (split_rows && n[4] > 0)
        BPT_CUDA(cudaMemcpyAsync(split_rows, p->split, sizeof(int32_t) * n[4] * 4, cudaMemcpyDeviceToDevice, stream));
    if (et && n[3] > 0) {
        if (et_bytes == 2) {
            BPT_CUDA(cudaMemcpyAsync(et, p->et, sizeof(uint16_t) * n[3], cudaMemcpyDeviceToDevice, stream));
        } else {
            narrow_et_kernel<<<blocks_for(n[3]), kThreads, 0, stream>>>(p->et, n[3], static_cast<uint8_t *>(et), p->counts);
            BPT_LAUNCH_CHECK();
            Counts h;
            BPT_CUDA(cudaMemcpyAsync(&h, p->counts, sizeof(h), cudaMemcpyDeviceToHost, stream));
            BPT_CUDA(cudaStreamSynchronize(stream));
            if (h.err_etype & 2) return fail(BPT_ERR_UNSUPPORTED, "tile_plan_device_export: an edge type does not fit 8 bits");
        }
    }
    BPT_CUDA(cudaStreamSynchronize(stream));
    return BPT_OK;
}

extern "C" void bpt_tile_plan_device_destroy(void *handle) { delete static_cast<DeviceTilePlan *>(handle); }
