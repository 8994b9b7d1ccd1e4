// Host-side planner of the tensor-core attention path.
//
// The sparse attention matrix (rows = destinations, columns = sources) is covered by groups:
// a group is a sorted list of source columns shared by several m-blocks of <=16 destination
// rows each (tile_plan.cuh).  The kernel stages a group's K/V rows once per head and lets all
// its m-blocks attend over them, so the planner's job is to put rows with overlapping sources
// into one group:
//   1. `group_rows` consecutive rows whose union of sources is small and reasonably filled
//      become a dense group (binary-partition graphs: 64 consecutive leaves share ~230-260
//      sources, against ~120-145 per 16 leaves);
//   2. the edges of all other rows are bucketed by block of `col_block` consecutive sources and
//      the rows of a bucket cut into m-blocks of 16.  If the dense group made of the rows with
//      those same ids holds all of the bucket's sources as columns, the m-blocks join it and
//      reuse its staged K/V (binary-partition graphs: the span nodes above a block of leaves
//      attend exactly to those leaves); otherwise they form a group of their own;
//   3. a row spread over several m-blocks gets one partial result ("slot") per m-block; slots
//      of a row are contiguous and in m-block order, and are combined afterwards in that order.
// Parallel edges (the reference's builder emits duplicate (src, dst) pairs for some lengths,
// graph_builder/builder.pyx:77-85) get separate columns, so a cell holds at most one edge.
// Pure integer host code: no CUDA calls, usable and testable without a GPU.
#include <algorithm>
#include <cstring>
#include <vector>

#include "tile_plan.cuh"

namespace bpt {
namespace {

struct HostTilePlan {
    std::vector<int32_t> groups, mblocks, cols, split, simt;
    std::vector<uint16_t> et;
    std::vector<int32_t> cellpos;  // per cell, parallel to et: the edge's payload (CSR position), -1 = no edge
    int64_t n_slots = 0, t_max = 0, max_cols_pad = 0, max_mblocks = 0, max_qr_slots = 0, n_dense_groups = 0;
};

struct EdgeRec {
    int64_t key;  // (src << 8) | rank among parallel edges of the same (row, src)
    int32_t row, etype, pos;
};

// An m-block before it is laid out: sorted rows and their edges (grouped by row, row order).
struct MBlockBuild {
    std::vector<int32_t> rows;
    std::vector<EdgeRec> edges;
};

struct GroupBuild {
    std::vector<int64_t> keys;  // sorted unique column keys
    std::vector<MBlockBuild> mblocks;
    bool dense = false;
};

// One record per edge of `rows`, with the parallel-edge rank inside each row.
bool collect_edges(const int32_t *indptr, const int32_t *src, const int32_t *etype, const int32_t *payload,
                   const int32_t *rows, int64_t n_rows, std::vector<EdgeRec> &out,
                   std::vector<std::pair<int32_t, int32_t>> &tmp) {
    bool ok = true;
    for (int64_t i = 0; i < n_rows; ++i) {
        const int32_t r = rows[i];
        tmp.clear();
        for (int32_t j = indptr[r]; j < indptr[r + 1]; ++j) tmp.emplace_back(src[j], j);
        std::sort(tmp.begin(), tmp.end());
        int rank = 0;
        for (size_t p = 0; p < tmp.size(); ++p) {
            rank = (p > 0 && tmp[p].first == tmp[p - 1].first) ? rank + 1 : 0;
            if (rank > 255) ok = false;  // more than 256 parallel edges between one pair of nodes
            EdgeRec rec;
            rec.key = (static_cast<int64_t>(tmp[p].first) << 8) | (rank & 255);
            rec.row = r;
            rec.etype = etype ? etype[tmp[p].second] : 0;
            rec.pos = payload ? payload[tmp[p].second] : tmp[p].second;
            out.push_back(rec);
        }
    }
    return ok;
}

struct Partial {
    int32_t row, mblock, local;
};

// Lays a group out into the plan arrays; m-blocks beyond max_mblocks spill into copies of the
// group (same columns).  Rows whose edges are not all inside their m-block are reported as
// partial.
void emit_group(HostTilePlan &plan, const GroupBuild &gb, const int32_t *indptr, const int32_t *row_uniform_et,
                std::vector<Partial> &partials, int max_mblocks) {
    const int ncols = static_cast<int>(gb.keys.size());
    const int ncols_pad = (ncols + kTileChunk - 1) / kTileChunk * kTileChunk;
    const int n_chunks = ncols_pad / kTileChunk;
    if (ncols_pad > plan.max_cols_pad) plan.max_cols_pad = ncols_pad;
    for (size_t first = 0; first < gb.mblocks.size() || first == 0; first += max_mblocks) {
        const size_t count = std::min<size_t>(max_mblocks, gb.mblocks.size() - first);
        const size_t gidx = plan.groups.size();
        plan.groups.resize(gidx + kGroupInts, 0);
        plan.groups[gidx + kGroupColOff] = static_cast<int32_t>(plan.cols.size());
        plan.groups[gidx + kGroupNcolsPad] = ncols_pad;
        plan.groups[gidx + kGroupMbFirst] = static_cast<int32_t>(plan.mblocks.size() / kMbInts);
        plan.groups[gidx + kGroupMbCount] = static_cast<int32_t>(count);
        plan.groups[gidx + kGroupNcols] = ncols;
        for (int c = 0; c < ncols_pad; ++c)
            plan.cols.push_back(static_cast<int32_t>((c < ncols ? gb.keys[c] : gb.keys[0]) >> 8));
        if (static_cast<int64_t>(count) > plan.max_mblocks) plan.max_mblocks = static_cast<int64_t>(count);
        int n_qr = 0;
        for (size_t b = first; b < first + count; ++b) {
            const MBlockBuild &mb = gb.mblocks[b];
            const int nr = static_cast<int>(mb.rows.size());
            const int32_t midx = static_cast<int32_t>(plan.mblocks.size() / kMbInts);
            plan.mblocks.resize(plan.mblocks.size() + kMbInts, 0);
            int32_t *m = &plan.mblocks[static_cast<size_t>(midx) * kMbInts];
            bool uniform = true;
            for (int i = 0; i < kTileRows; ++i) {
                m[kMbRowOff + i] = i < nr ? mb.rows[i] : -1;
                m[kMbSlotOff + i] = -1;
                m[kMbRowEtOff + i] = i < nr ? row_uniform_et[mb.rows[i]] : 0;
                if (i < nr && row_uniform_et[mb.rows[i]] < 0) uniform = false;
            }
            m[kMbEtOff] = static_cast<int32_t>(plan.et.size());
            const size_t base = plan.et.size();
            plan.et.resize(base + static_cast<size_t>(n_chunks) * kTileRows * kTileChunk, kNoEdge);
            plan.cellpos.resize(plan.et.size(), -1);
            uint32_t mask = 0, fine = 0;
            int max_et = -1;
            size_t p = 0;
            for (int r = 0; r < nr; ++r) {
                int64_t cnt = 0;
                while (p < mb.edges.size() && mb.edges[p].row == mb.rows[r]) {
                    const EdgeRec &e = mb.edges[p];
                    const int c = static_cast<int>(std::lower_bound(gb.keys.begin(), gb.keys.end(), e.key) - gb.keys.begin());
                    const int chunk = c / kTileChunk;
                    const size_t cell = base + (static_cast<size_t>(chunk) * kTileRows + r) * kTileChunk + (c % kTileChunk);
                    plan.et[cell] = static_cast<uint16_t>(e.etype);
                    plan.cellpos[cell] = e.pos;
                    mask |= 1u << (c / kMaskCols);
                    if (c < 512) fine |= 1u << (c / 16);
                    if (e.etype > max_et) max_et = e.etype;
                    ++cnt;
                    ++p;
                }
                if (cnt != indptr[mb.rows[r] + 1] - indptr[mb.rows[r]]) partials.push_back({mb.rows[r], midx, r});
            }
            m[kMbChunkMask] = static_cast<int32_t>(mask);
            m[kMbFineMask] = ncols_pad <= 512 ? static_cast<int32_t>(fine) : 0;
            m[kMbTq] = (max_et + 1 + 7) / 8 * 8;
            m[kMbQrSlot] = uniform ? -1 : n_qr++;
            if (!uniform && m[kMbTq] > plan.t_max) plan.t_max = m[kMbTq];
        }
        if (n_qr > plan.max_qr_slots) plan.max_qr_slots = n_qr;
        if (gb.dense) ++plan.n_dense_groups;
        if (gb.mblocks.empty()) break;
    }
}

struct Leftover {
    int32_t sblock, row;
    EdgeRec rec;
};

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" void *bpt_tile_plan_create(const int32_t *in_indptr, const int32_t *in_src, const int32_t *in_etype,
                                      const int32_t *in_payload, int64_t n_nodes, int64_t n_edges, double min_density, int max_cols,
                                      int group_rows, int col_block, int simt_max_degree, int max_mblocks,
                                      int join_dense) {
    if (!in_indptr || (n_edges > 0 && !in_src) || n_nodes < 0 || n_edges < 0 || max_cols < kTileChunk ||
        max_cols > kMaxMaskBits * kMaskCols || col_block < 1 || group_rows < kTileRows ||
        group_rows % kTileRows != 0 || max_mblocks < 1 || max_mblocks > kMaxMBlocks ||
        group_rows / kTileRows > max_mblocks) {
        fail(BPT_ERR_INVALID, "tile_plan_create: bad arguments");
        return nullptr;
    }
    if (in_etype)
        for (int64_t j = 0; j < n_edges; ++j)
            if (in_etype[j] < 0 || in_etype[j] >= kNoEdge) {
                fail(BPT_ERR_UNSUPPORTED, "tile_plan_create: edge type %d outside [0, 65535)", in_etype[j]);
                return nullptr;
            }
    // the single edge type of each row, or -1 if its edges differ (rows without edges: 0)
    std::vector<int32_t> row_uniform_et(static_cast<size_t>(n_nodes), 0);
    for (int64_t r = 0; r < n_nodes; ++r)
        for (int32_t j = in_indptr[r]; j < in_indptr[r + 1]; ++j) {
            const int32_t e = in_etype ? in_etype[j] : 0;
            if (j == in_indptr[r]) row_uniform_et[r] = e;
            else if (row_uniform_et[r] != e) row_uniform_et[r] = -1;
        }

    HostTilePlan *plan = new HostTilePlan();
    std::vector<EdgeRec> edges;
    std::vector<std::pair<int32_t, int32_t>> tmp;
    std::vector<int32_t> leftover_rows, zero_rows, rows(group_rows);
    const int64_t n_row_groups = (n_nodes + group_rows - 1) / group_rows;
    std::vector<GroupBuild> dense(static_cast<size_t>(n_row_groups));
    std::vector<GroupBuild> standalone;
    const char *too_many = "tile_plan_create: more than 256 parallel edges between two nodes";

    // 1. dense groups of `group_rows` consecutive rows
    for (int64_t gi = 0; gi < n_row_groups; ++gi) {
        const int64_t r0 = gi * group_rows;
        const int nr = static_cast<int>(std::min<int64_t>(group_rows, n_nodes - r0));
        for (int i = 0; i < nr; ++i) rows[i] = static_cast<int32_t>(r0 + i);
        const int64_t ne = in_indptr[r0 + nr] - in_indptr[r0];
        GroupBuild &gb = dense[gi];
        edges.clear();
        bool accept = ne == 0;
        if (!accept && ne <= static_cast<int64_t>(nr) * max_cols) {
            if (!collect_edges(in_indptr, in_src, in_etype, in_payload, rows.data(), nr, edges, tmp)) {
                fail(BPT_ERR_UNSUPPORTED, "%s", too_many);
                delete plan;
                return nullptr;
            }
            for (const EdgeRec &e : edges) gb.keys.push_back(e.key);
            std::sort(gb.keys.begin(), gb.keys.end());
            gb.keys.erase(std::unique(gb.keys.begin(), gb.keys.end()), gb.keys.end());
            const int64_t ncols = static_cast<int64_t>(gb.keys.size());
            accept = ncols <= max_cols && static_cast<double>(ne) >= min_density * nr * ncols;
        }
        if (!accept) {
            gb.keys.clear();
            for (int i = 0; i < nr; ++i) {
                const int32_t deg = in_indptr[rows[i] + 1] - in_indptr[rows[i]];
                if (deg == 0) zero_rows.push_back(rows[i]);
                else if (deg <= simt_max_degree)
                    plan->simt.insert(plan->simt.end(), {rows[i], in_indptr[rows[i]], in_indptr[rows[i] + 1], -1});
                else leftover_rows.push_back(rows[i]);
            }
            continue;
        }
        gb.dense = true;
        size_t p = 0;  // collect_edges walks rows in order, so edges are grouped by row
        for (int b = 0; b < nr; b += kTileRows) {
            MBlockBuild mb;
            const int nb = std::min(kTileRows, nr - b);
            mb.rows.assign(rows.begin() + b, rows.begin() + b + nb);
            size_t q = p;
            while (q < edges.size() && edges[q].row < rows[b] + nb) ++q;
            mb.edges.assign(edges.begin() + p, edges.begin() + q);
            p = q;
            gb.mblocks.push_back(std::move(mb));
        }
    }

    // 2. the other rows' edges, bucketed by block of `col_block` consecutive sources
    {
        std::vector<Leftover> left;
        edges.clear();
        if (!collect_edges(in_indptr, in_src, in_etype, in_payload, leftover_rows.data(),
                           static_cast<int64_t>(leftover_rows.size()), edges, tmp)) {
            fail(BPT_ERR_UNSUPPORTED, "%s", too_many);
            delete plan;
            return nullptr;
        }
        left.reserve(edges.size());
        for (const EdgeRec &e : edges) left.push_back({static_cast<int32_t>((e.key >> 8) / col_block), e.row, e});
        std::sort(left.begin(), left.end(), [](const Leftover &a, const Leftover &b) {
            if (a.sblock != b.sblock) return a.sblock < b.sblock;
            if (a.row != b.row) return a.row < b.row;
            return a.rec.key < b.rec.key;
        });
        for (size_t i = 0; i < left.size();) {
            // all rows touching this bucket of sources: one group (their union of columns), rows cut
            // into m-blocks of 16
            const int32_t sb = left[i].sblock;
            std::vector<MBlockBuild> mbs;
            size_t j = i;
            while (j < left.size() && left[j].sblock == sb) {
                if (mbs.empty() || (left[j].row != mbs.back().rows.back() &&
                                    mbs.back().rows.size() == static_cast<size_t>(kTileRows)))
                    mbs.emplace_back();
                MBlockBuild &mb = mbs.back();
                if (mb.rows.empty() || left[j].row != mb.rows.back()) mb.rows.push_back(left[j].row);
                mb.edges.push_back(left[j].rec);
                ++j;
            }
            // the dense group whose rows carry the ids of this bucket's sources, if it has them all as columns
            const int64_t gi = static_cast<int64_t>(sb) * col_block / group_rows;
            bool join = join_dense && gi < n_row_groups && dense[gi].dense && !dense[gi].keys.empty();
            if (join)
                for (size_t e = i; e < j && join; ++e)
                    join = std::binary_search(dense[gi].keys.begin(), dense[gi].keys.end(), left[e].rec.key);
            if (join) {
                for (MBlockBuild &mb : mbs) dense[gi].mblocks.push_back(std::move(mb));
            } else {
                GroupBuild gb;
                for (size_t e = i; e < j; ++e) gb.keys.push_back(left[e].rec.key);
                std::sort(gb.keys.begin(), gb.keys.end());
                gb.keys.erase(std::unique(gb.keys.begin(), gb.keys.end()), gb.keys.end());
                gb.mblocks = std::move(mbs);
                standalone.push_back(std::move(gb));
            }
            i = j;
        }
    }
    // rows without edges that no dense group covers still need their zero output written
    for (size_t i = 0; i < zero_rows.size(); i += kTileRows) {
        GroupBuild gb;
        MBlockBuild mb;
        mb.rows.assign(zero_rows.begin() + i, zero_rows.begin() + std::min(zero_rows.size(), i + kTileRows));
        gb.mblocks.push_back(std::move(mb));
        standalone.push_back(std::move(gb));
    }

    std::vector<Partial> partials;
    for (const GroupBuild &gb : dense)
        if (gb.dense) emit_group(*plan, gb, in_indptr, row_uniform_et.data(), partials, max_mblocks);
    for (const GroupBuild &gb : standalone) emit_group(*plan, gb, in_indptr, row_uniform_et.data(), partials, max_mblocks);

    // 3. slots, contiguous per row, in m-block order
    std::stable_sort(partials.begin(), partials.end(), [](const Partial &a, const Partial &b) { return a.row < b.row; });
    for (size_t p = 0; p < partials.size();) {
        size_t q = p;
        while (q < partials.size() && partials[q].row == partials[p].row) {
            plan->mblocks[static_cast<size_t>(partials[q].mblock) * kMbInts + kMbSlotOff + partials[q].local] =
                static_cast<int32_t>(q);
            ++q;
        }
        plan->split.insert(plan->split.end(), {partials[p].row, static_cast<int32_t>(p), static_cast<int32_t>(q - p), 0});
        p = q;
    }
    plan->n_slots = static_cast<int64_t>(partials.size());
    return plan;
}

// sizes[12] = {groups, m-blocks, column entries, etype cells, split rows, slots, t_max,
//              max_cols_pad, max m-blocks per group, max QR slots per group, row items, dense groups}
extern "C" int bpt_tile_plan_sizes(const void *handle, int64_t *sizes) {
    BPT_CHECK_ARG(handle && sizes, "tile_plan_sizes: null argument");
    const HostTilePlan *p = static_cast<const HostTilePlan *>(handle);
    sizes[0] = static_cast<int64_t>(p->groups.size() / kGroupInts);
    sizes[1] = static_cast<int64_t>(p->mblocks.size() / kMbInts);
    sizes[2] = static_cast<int64_t>(p->cols.size());
    sizes[3] = static_cast<int64_t>(p->et.size());
    sizes[4] = static_cast<int64_t>(p->split.size() / 4);
    sizes[5] = p->n_slots;
    sizes[6] = p->t_max;
    sizes[7] = p->max_cols_pad;
    sizes[8] = p->max_mblocks;
    sizes[9] = p->max_qr_slots;
    sizes[10] = static_cast<int64_t>(p->simt.size() / 4);
    sizes[11] = p->n_dense_groups;
    return BPT_OK;
}

// et_bytes = 1 stores edge types as uint8 (0xFF = no edge; needs every type < 255), 2 as uint16.
extern "C" int bpt_tile_plan_export(const void *handle, int32_t *groups, int32_t *mblocks, int32_t *cols, void *et,
                                    int et_bytes, int32_t *cell_pos, int32_t *split_rows, int32_t *row_items) {
    BPT_CHECK_ARG(handle, "tile_plan_export: null handle");
    BPT_CHECK_ARG(et_bytes == 1 || et_bytes == 2, "tile_plan_export: et_bytes must be 1 or 2");
    const HostTilePlan *p = static_cast<const HostTilePlan *>(handle);
    if (groups && !p->groups.empty()) std::memcpy(groups, p->groups.data(), p->groups.size() * sizeof(int32_t));
    if (mblocks && !p->mblocks.empty()) std::memcpy(mblocks, p->mblocks.data(), p->mblocks.size() * sizeof(int32_t));
    if (cols && !p->cols.empty()) std::memcpy(cols, p->cols.data(), p->cols.size() * sizeof(int32_t));
    if (et && !p->et.empty()) {
        if (et_bytes == 2) {
            std::memcpy(et, p->et.data(), p->et.size() * sizeof(uint16_t));
        } else {
            uint8_t *out = static_cast<uint8_t *>(et);
            for (size_t i = 0; i < p->et.size(); ++i) {
                if (p->et[i] != kNoEdge && p->et[i] >= kNoEdge8)
                    return fail(BPT_ERR_UNSUPPORTED, "tile_plan_export: edge type %d does not fit 8 bits", p->et[i]);
                out[i] = p->et[i] == kNoEdge ? kNoEdge8 : static_cast<uint8_t>(p->et[i]);
            }
        }
    }
    if (cell_pos && !p->cellpos.empty()) {
        // Fragment order (kCellPosIndex): the 16 payloads an mma lane needs per 32 columns are four
        // 16-byte pieces, and a warp's pieces of one column group are 512 contiguous bytes.
        const size_t chunk_cells = static_cast<size_t>(kTileRows) * kTileChunk;
        for (size_t base = 0; base + chunk_cells <= p->cellpos.size(); base += chunk_cells)
            for (int r = 0; r < kTileRows; ++r)
                for (int c = 0; c < kTileChunk; ++c)
                    cell_pos[base + cell_pos_index(r, c)] = p->cellpos[base + static_cast<size_t>(r) * kTileChunk + c];
    }
    if (split_rows && !p->split.empty()) std::memcpy(split_rows, p->split.data(), p->split.size() * sizeof(int32_t));
    if (row_items && !p->simt.empty()) std::memcpy(row_items, p->simt.data(), p->simt.size() * sizeof(int32_t));
    return BPT_OK;
}

extern "C" void bpt_tile_plan_destroy(void *handle) { delete static_cast<HostTilePlan *>(handle); }
