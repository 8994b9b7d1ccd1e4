// Host-side planner of the tensor-core attention path.
//
// The sparse attention matrix (rows = destinations, columns = sources) is covered by tiles of
// at most 16 rows and an explicit list of source columns, chosen so that each tile is dense
// enough to be computed as a masked dense block:
//   1. every block of 16 consecutive rows whose union of sources is small and well filled
//      becomes one tile holding all edges of its rows (binary-partition graphs: 16 consecutive
//      leaves share ~120-150 sources at 60-70 % fill);
//   2. the edges of all other rows are grouped by block of 64 consecutive sources; the rows
//      touching a source block are cut into tiles of 16 (binary-partition graphs: the span
//      nodes covering a leaf block). A row spread over several tiles gets one partial result
//      per tile ("slot") and is combined afterwards in slot order.
// Parallel edges (the reference's builder emits duplicate (src, dst) pairs for some lengths,
// graph_builder/builder.pyx:77-85) get separate columns, so a tile cell holds at most one edge.
// Pure integer host code: no CUDA calls, usable and testable without a GPU.
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "tile_plan.cuh"

namespace bpt {
namespace {

struct HostTilePlan {
    std::vector<int32_t> tiles;
    std::vector<int32_t> cols;
    std::vector<uint16_t> et;
    std::vector<int32_t> split;  // int4 records {row, first_slot, n_slots, 0}
    std::vector<int32_t> simt;   // int4 records {row, begin, end, -1}: short rows left to the CUDA-core kernel
    int64_t n_slots = 0, t_max = 0, max_cols_pad = 0, n_cells = 0, n_row_tiles = 0;
};

struct EdgeRec {
    int64_t key;  // (src << 8) | rank among parallel edges of the same (row, src)
    int32_t row, etype;
};

// Assigns the parallel-edge rank inside each row and returns one record per edge of `rows`.
bool collect_edges(const int32_t *indptr, const int32_t *src, const int32_t *etype, const int32_t *rows,
                   int n_rows, std::vector<EdgeRec> &out, std::vector<std::pair<int32_t, int32_t>> &tmp) {
    bool ok = true;
    for (int i = 0; i < n_rows; ++i) {
        const int32_t r = rows[i];
        const int32_t b = indptr[r], e = indptr[r + 1];
        tmp.clear();
        for (int32_t j = b; j < e; ++j) tmp.emplace_back(src[j], j);
        std::sort(tmp.begin(), tmp.end());
        int rank = 0;
        for (size_t p = 0; p < tmp.size(); ++p) {
            rank = (p > 0 && tmp[p].first == tmp[p - 1].first) ? rank + 1 : 0;
            EdgeRec rec;
            if (rank > 255) ok = false;  // more than 256 parallel edges between one pair of nodes
            rec.key = (static_cast<int64_t>(tmp[p].first) << 8) | (rank & 255);
            rec.row = r;
            rec.etype = etype ? etype[tmp[p].second] : 0;
            out.push_back(rec);
        }
    }
    return ok;
}

// Emits one tile from edge records (all of whose rows are in `rows`).  Returns its index.
int emit_tile(HostTilePlan &plan, const int32_t *rows, int n_rows, const EdgeRec *edges, size_t n_edges,
              std::vector<int64_t> &keys) {
    keys.clear();
    for (size_t i = 0; i < n_edges; ++i) keys.push_back(edges[i].key);
    std::sort(keys.begin(), keys.end());
    keys.erase(std::unique(keys.begin(), keys.end()), keys.end());
    const int ncols = static_cast<int>(keys.size());
    const int ncols_pad = (ncols + kTileChunk - 1) / kTileChunk * kTileChunk;
    const int idx = static_cast<int>(plan.tiles.size() / kTileInts);
    plan.tiles.resize(plan.tiles.size() + kTileInts, 0);
    int32_t *t = &plan.tiles[static_cast<size_t>(idx) * kTileInts];
    for (int i = 0; i < kTileRows; ++i) {
        t[kTileRowOff + i] = i < n_rows ? rows[i] : -1;
        t[kTileSlotOff + i] = -1;
    }
    t[kTileNcolsPad] = ncols_pad;
    t[kTileColOff] = static_cast<int32_t>(plan.cols.size());
    t[kTileEtOff] = static_cast<int32_t>(plan.et.size());
    t[kTileNcols] = ncols;
    for (int c = 0; c < ncols_pad; ++c)
        plan.cols.push_back(c < ncols ? static_cast<int32_t>(keys[c] >> 8) : static_cast<int32_t>(keys[0] >> 8));
    const size_t et_base = plan.et.size();
    plan.et.resize(et_base + static_cast<size_t>(kTileRows) * ncols_pad, kNoEdge);
    int max_et = -1;
    for (size_t i = 0; i < n_edges; ++i) {
        const int local = static_cast<int>(std::lower_bound(rows, rows + n_rows, edges[i].row) - rows);
        const int c = static_cast<int>(std::lower_bound(keys.begin(), keys.end(), edges[i].key) - keys.begin());
        plan.et[et_base + static_cast<size_t>(local) * ncols_pad + c] = static_cast<uint16_t>(edges[i].etype);
        if (edges[i].etype > max_et) max_et = edges[i].etype;
    }
    t[kTileTq] = (max_et + 1 + 7) / 8 * 8;
    if (t[kTileTq] > plan.t_max) plan.t_max = t[kTileTq];
    if (ncols_pad > plan.max_cols_pad) plan.max_cols_pad = ncols_pad;
    plan.n_cells += static_cast<int64_t>(kTileRows) * ncols_pad;
    return idx;
}

struct Leftover {
    int32_t sblock, row;
    EdgeRec rec;
};

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" void *bpt_tile_plan_create(const int32_t *in_indptr, const int32_t *in_src, const int32_t *in_etype,
                                      int64_t n_nodes, int64_t n_edges, double min_density, int max_cols,
                                      int col_block, int simt_max_degree) {
    if (!in_indptr || (n_edges > 0 && !in_src) || n_nodes < 0 || n_edges < 0 || max_cols < kTileChunk ||
        col_block < 1) {
        fail(BPT_ERR_INVALID, "tile_plan_create: bad arguments");
        return nullptr;
    }
    if (in_etype)
        for (int64_t j = 0; j < n_edges; ++j)
            if (in_etype[j] < 0 || in_etype[j] >= kNoEdge) {
                fail(BPT_ERR_UNSUPPORTED, "tile_plan_create: edge type %d outside [0, 65535)", in_etype[j]);
                return nullptr;
            }
    HostTilePlan *plan = new HostTilePlan();
    std::vector<EdgeRec> edges;
    std::vector<std::pair<int32_t, int32_t>> tmp;
    std::vector<int64_t> keys;
    std::vector<int32_t> leftover_rows, zero_rows;
    std::vector<int32_t> rows(kTileRows);

    // 1. blocks of 16 consecutive rows
    for (int64_t r0 = 0; r0 < n_nodes; r0 += kTileRows) {
        const int nr = static_cast<int>(std::min<int64_t>(kTileRows, n_nodes - r0));
        for (int i = 0; i < nr; ++i) rows[i] = static_cast<int32_t>(r0 + i);
        const int64_t ne = in_indptr[r0 + nr] - in_indptr[r0];
        bool as_tile = ne == 0;
        if (!as_tile && ne <= static_cast<int64_t>(kTileRows) * max_cols) {
            edges.clear();
            if (!collect_edges(in_indptr, in_src, in_etype, rows.data(), nr, edges, tmp)) {
                fail(BPT_ERR_UNSUPPORTED, "tile_plan_create: more than 256 parallel edges between two nodes");
                delete plan;
                return nullptr;
            }
            keys.clear();
            for (const EdgeRec &e : edges) keys.push_back(e.key);
            std::sort(keys.begin(), keys.end());
            const int64_t ncols = std::unique(keys.begin(), keys.end()) - keys.begin();
            as_tile = ncols <= max_cols && static_cast<double>(ne) >= min_density * kTileRows * ncols;
        }
        if (as_tile) {
            if (ne == 0) edges.clear();
            emit_tile(*plan, rows.data(), nr, edges.data(), edges.size(), keys);
            ++plan->n_row_tiles;
        } else {
            for (int i = 0; i < nr; ++i) {
                const int32_t deg = in_indptr[rows[i] + 1] - in_indptr[rows[i]];
                if (deg <= simt_max_degree) {
                    // too few edges to be worth a tile cell row: one warp walks the row instead
                    plan->simt.push_back(rows[i]);
                    plan->simt.push_back(in_indptr[rows[i]]);
                    plan->simt.push_back(in_indptr[rows[i] + 1]);
                    plan->simt.push_back(-1);
                } else if (deg == 0) {
                    zero_rows.push_back(rows[i]);
                } else {
                    leftover_rows.push_back(rows[i]);
                }
            }
        }
    }
    // rows without edges that were not covered above still need their zero output written
    for (size_t i = 0; i < zero_rows.size(); i += kTileRows) {
        const int nr = static_cast<int>(std::min<size_t>(kTileRows, zero_rows.size() - i));
        emit_tile(*plan, &zero_rows[i], nr, nullptr, 0, keys);
    }

    // 2. remaining edges by block of `col_block` consecutive sources
    std::vector<Leftover> left;
    {
        edges.clear();
        if (!collect_edges(in_indptr, in_src, in_etype, leftover_rows.data(),
                           static_cast<int>(leftover_rows.size()), edges, tmp)) {
            fail(BPT_ERR_UNSUPPORTED, "tile_plan_create: more than 256 parallel edges between two nodes");
            delete plan;
            return nullptr;
        }
        left.reserve(edges.size());
        for (const EdgeRec &e : edges) {
            Leftover l;
            l.sblock = static_cast<int32_t>((e.key >> 8) / col_block);
            l.row = e.row;
            l.rec = e;
            left.push_back(l);
        }
        std::sort(left.begin(), left.end(), [](const Leftover &a, const Leftover &b) {
            if (a.sblock != b.sblock) return a.sblock < b.sblock;
            if (a.row != b.row) return a.row < b.row;
            return a.rec.key < b.rec.key;
        });
    }
    struct Partial { int32_t row, tile, local; };
    std::vector<Partial> partials;
    size_t i = 0;
    while (i < left.size()) {
        // one tile: up to 16 distinct rows of the same source block
        const int32_t sb = left[i].sblock;
        size_t j = i;
        int nr = 0;
        int32_t last_row = -1;
        edges.clear();
        while (j < left.size() && left[j].sblock == sb) {
            if (left[j].row != last_row) {
                if (nr == kTileRows) break;
                rows[nr++] = left[j].row;
                last_row = left[j].row;
            }
            edges.push_back(left[j].rec);
            ++j;
        }
        const int tile = emit_tile(*plan, rows.data(), nr, edges.data(), edges.size(), keys);
        // a row is complete here only if this tile holds all of its edges
        size_t p = 0;
        for (int r = 0; r < nr; ++r) {
            int64_t cnt = 0;
            while (p < edges.size() && edges[p].row == rows[r]) { ++cnt; ++p; }
            if (cnt != in_indptr[rows[r] + 1] - in_indptr[rows[r]]) partials.push_back({rows[r], tile, r});
        }
        i = j;
    }
    // 3. slots, contiguous per row, in tile order
    std::stable_sort(partials.begin(), partials.end(), [](const Partial &a, const Partial &b) { return a.row < b.row; });
    for (size_t p = 0; p < partials.size();) {
        size_t q = p;
        while (q < partials.size() && partials[q].row == partials[p].row) {
            plan->tiles[static_cast<size_t>(partials[q].tile) * kTileInts + kTileSlotOff + partials[q].local] =
                static_cast<int32_t>(q);
            ++q;
        }
        plan->split.push_back(partials[p].row);
        plan->split.push_back(static_cast<int32_t>(p));
        plan->split.push_back(static_cast<int32_t>(q - p));
        plan->split.push_back(0);
        p = q;
    }
    plan->n_slots = static_cast<int64_t>(partials.size());
    return plan;
}

extern "C" int bpt_tile_plan_sizes(const void *handle, int64_t *sizes) {
    BPT_CHECK_ARG(handle && sizes, "tile_plan_sizes: null argument");
    const HostTilePlan *p = static_cast<const HostTilePlan *>(handle);
    sizes[0] = static_cast<int64_t>(p->tiles.size() / kTileInts);
    sizes[1] = static_cast<int64_t>(p->cols.size());
    sizes[2] = static_cast<int64_t>(p->et.size());
    sizes[3] = static_cast<int64_t>(p->split.size() / 4);
    sizes[4] = p->n_slots;
    sizes[5] = p->t_max;
    sizes[6] = p->max_cols_pad;
    sizes[7] = p->n_row_tiles;
    sizes[8] = static_cast<int64_t>(p->simt.size() / 4);
    sizes[9] = p->n_cells;
    return BPT_OK;
}

extern "C" int bpt_tile_plan_export(const void *handle, int32_t *tiles, int32_t *cols, uint16_t *et,
                                    int32_t *split_rows, int32_t *simt_items) {
    BPT_CHECK_ARG(handle, "tile_plan_export: null handle");
    const HostTilePlan *p = static_cast<const HostTilePlan *>(handle);
    if (tiles && !p->tiles.empty()) std::memcpy(tiles, p->tiles.data(), p->tiles.size() * sizeof(int32_t));
    if (cols && !p->cols.empty()) std::memcpy(cols, p->cols.data(), p->cols.size() * sizeof(int32_t));
    if (et && !p->et.empty()) std::memcpy(et, p->et.data(), p->et.size() * sizeof(uint16_t));
    if (split_rows && !p->split.empty()) std::memcpy(split_rows, p->split.data(), p->split.size() * sizeof(int32_t));
    if (simt_items && !p->simt.empty()) std::memcpy(simt_items, p->simt.data(), p->simt.size() * sizeof(int32_t));
    return BPT_OK;
}

extern "C" void bpt_tile_plan_destroy(void *handle) { delete static_cast<HostTilePlan *>(handle); }
