// Fused graph attention forward on tensor cores (bf16 storage, fp32 accumulation, head dim 64).
//
// A thread block works on two groups of the tile plan (tile_plan.cuh) at once, four warps each; a
// warp takes heads w, w + 4, ... of its group.  (Two groups per block keep four independent
// chains of dependent loads in flight per SM at the same register and shared-memory budget, and
// share one copy of the embed_ak rows.)  The four warps stage the group's column ids and the
// m-block's cells (as table indices) once; the warp's first K and V rows are already travelling
// while that happens.  For
// each m-block of the group (<=16 destination rows x the group's column list) and each active
// 32-column step a warp
//   1. takes the step's K rows from its K buffer (cp.async, swizzled; ldmatrix B fragments),
//   2. S = Q K^T on tensor cores, then refills the K buffer with the next step's rows; the
//      relative-position term and the edge mask come from one table lookup per cell:
//      table[row][etype] = scale * <q[row], embed_ak[etype]> (computed on tensor cores once per
//      m-block and head, parked in shared memory as fp16 in the log2 domain) with an extra entry
//      of -inf that cells without an edge point to.  M-blocks whose rows each have a single edge
//      type use a two-entry table {0, -inf}: the term is then a per-row constant that cancels in
//      the softmax and is added to lse at the end,
//   3. online softmax in registers, P packed to bf16 A fragments in place,
//   4. O += P V from its V buffer (ldmatrix.trans), then refills the V buffer.
// So K of step j+1 travels during softmax and PV of step j, V of step j+1 during QK^T of j+1.
// Scores never leave the SM.  Rows wholly inside one m-block are written as final O / lse; rows
// spread over several m-blocks write (m, l, O) partials that a merge kernel combines in slot
// order, so results are bitwise reproducible.
#include "fused_common.cuh"
#include "plan.cuh"
#include "tile_plan.cuh"

namespace bpt {
namespace {

constexpr int kHeadDim = 64;
constexpr int kRowBytes = kHeadDim * 2;                  // one head row of K or V: 128 B = 8 pieces of 16 B
constexpr int kStep = 32;                                // source columns per pipeline step
constexpr int kStepBytes = kStep * kRowBytes;            // 4 KB: one step's K (or V) rows of one head
constexpr int kKvStageBytes = 2 * kStepBytes;            // per warp: one K buffer and one V buffer

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
}
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void *gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// A lane's share of one 64-element head row in mma operand order: for k-step s the element pairs
// at 16s + 2t and 16s + 8 + 2t (t = lane % 4) in w[2s], w[2s+1].  Q rows (A operand, rows g and
// g+8) and embed_ak rows (B operand, column g) are read this way; K comes through ldmatrix, which
// hands out the same pairs.
__device__ __forceinline__ void load_row_frag(const __nv_bfloat16 *__restrict__ row, int t, uint32_t (&w)[8]) {
    const uint32_t *r32 = reinterpret_cast<const uint32_t *>(row);
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        w[2 * s] = __ldg(r32 + 8 * s + t);
        w[2 * s + 1] = __ldg(r32 + 8 * s + 4 + t);
    }
}

template <typename ET> struct EtTraits;
template <> struct EtTraits<uint8_t> { static constexpr uint32_t kNone = kNoEdge8; };
template <> struct EtTraits<uint16_t> { static constexpr uint32_t kNone = kNoEdge; };

constexpr int kTileWarps = 4;       // warps that share one tile (group); a warp takes heads w, w + 4, ...
constexpr int kTilesPerBlock = 2;   // a block works on two tiles at once, four warps each
constexpr int kWarps = kTileWarps * kTilesPerBlock;
constexpr int kEtPad = 8;  // padding per staged index row (spreads the 8 row groups over the banks)
// Staged table indices are as wide as the plan's cells; with 8-bit cells the -inf entry's index
// (the m-block's type count, at most kMaxTypes8) still fits.
constexpr int kMaxTypes8 = 248;

// Two neighbouring staged table indices (8- or 16-bit) in one shared-memory load.
__device__ __forceinline__ void load_idx_pair(const uint8_t *p, uint32_t &a, uint32_t &b) {
    const uint32_t v = *reinterpret_cast<const uint16_t *>(p);
    a = v & 0xffu;
    b = v >> 8;
}
__device__ __forceinline__ void load_idx_pair(const uint16_t *p, uint32_t &a, uint32_t &b) {
    const uint32_t v = *reinterpret_cast<const uint32_t *>(p);
    a = v & 0xffffu;
    b = v >> 16;
}
// Barrier among the four warps of one tile (ids 1 and 2; 0 is the block's).
__device__ __forceinline__ void tile_barrier(int tile_in_block) {
    if (tile_in_block == 0)
        asm volatile("bar.sync 1, %0;\n" ::"n"(kTileWarps * 32) : "memory");
    else
        asm volatile("bar.sync 2, %0;\n" ::"n"(kTileWarps * 32) : "memory");
}

struct TcParams {
    const int32_t *groups, *mblocks, *cols;
    const void *et;
    const __nv_bfloat16 *q, *k, *v, *ak;
    __nv_bfloat16 *o;
    float *lse, *part_o, *part_ml;
    int n_etypes, H, max_cols_pad, t_max, tab_stride;
    int64_t n_groups;
    float scale;
    Dropout drop;
};

template <typename ET, bool kHasBias, bool kDrop>
__global__ void __launch_bounds__(kWarps * 32, 2)
attn_forward_tile_kernel(const TcParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: K and V buffers (one pair per warp, 8 KB) | column ids (per tile) | table indices of the
    // m-block (per tile) | tables (fp16, one per warp) | embed_ak rows (shared by both tiles)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tib = warp / kTileWarps, wl = warp % kTileWarps;  // tile in block, warp in tile
    const int tid = threadIdx.x % (kTileWarps * 32);             // thread in tile
    constexpr int kTileThreads = kTileWarps * 32;
    const int idx_stride = p.max_cols_pad + kEtPad;
    int32_t *s_cols = reinterpret_cast<int32_t *>(smem + kWarps * kKvStageBytes) + tib * p.max_cols_pad;
    ET *s_idx_all = reinterpret_cast<ET *>(reinterpret_cast<int32_t *>(smem + kWarps * kKvStageBytes) +
                                           kTilesPerBlock * p.max_cols_pad);
    ET *s_idx = s_idx_all + tib * kTileRows * idx_stride;
    __half *s_tab_all = reinterpret_cast<__half *>(s_idx_all + kTilesPerBlock * kTileRows * idx_stride);
    const int tab_stride = p.tab_stride;  // t_max types + the -inf entry, padded (table_stride(): >= 8, even)
    // embed_ak rows [0, t_max), staged once per block (16-byte aligned: every region before it is)
    const uint32_t s_ak_addr = static_cast<uint32_t>(
        __cvta_generic_to_shared(s_tab_all + static_cast<int64_t>(kWarps) * kTileRows * tab_stride));

    if (kHasBias) {
        for (int i = threadIdx.x; i < p.t_max * 8; i += blockDim.x) {
            const int r = i >> 3, piece = i & 7;
            const int type = r < p.n_etypes ? r : p.n_etypes - 1;
            cp_async16(s_ak_addr + r * kRowBytes + ((piece ^ (r & 7)) << 4),
                       p.ak + static_cast<int64_t>(type) * kHeadDim + piece * 8);
        }
    }
    cp_async_commit();
    const int64_t tile = static_cast<int64_t>(blockIdx.x) * kTilesPerBlock + tib;
    const int32_t *grp = p.groups + (tile < p.n_groups ? tile : 0) * kGroupInts;
    const int n_mblocks = tile < p.n_groups ? grp[kGroupMbCount] : 0;
    if (n_mblocks == 0) {  // no tile for this half of the block: only keep the block's one barrier
        cp_async_wait<0>();
        __syncthreads();
        return;
    }
    const int ncols_pad = grp[kGroupNcolsPad];
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H;
    const uint32_t s_k_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem + warp * kKvStageBytes));
    const uint32_t s_v_addr = s_k_addr + kStepBytes;
    const int n_steps = ncols_pad / kStep;
    __half *s_tab = s_tab_all + static_cast<int64_t>(warp) * kTileRows * tab_stride;
    const float sl2 = p.scale * kLog2e;
    const ET *et_base = static_cast<const ET *>(p.et);

    {
        const int32_t *gc = p.cols + grp[kGroupColOff];
        for (int i = tid; i < ncols_pad; i += kTileThreads) s_cols[i] = gc[i];
    }

    // 32 rows of K or V of head h for step j -> the warp's buffer (16-byte pieces, piece index XOR (row & 7)).
    // Lane l copies piece (l & 7) of rows (l >> 3) + 4 i: the swizzled offset takes two values per lane
    // (i even / odd) plus 1024 bytes per pair of i, and a row's address is one widening multiply-add.
    const int copy_row = lane >> 3, copy_piece = lane & 7;
    const uint32_t copy_even = copy_row * kRowBytes + ((copy_piece ^ copy_row) << 4);
    const uint32_t copy_odd = (copy_row + 4) * kRowBytes + ((copy_piece ^ (copy_row + 4)) << 4);
    const uint32_t row_pitch = static_cast<uint32_t>(H) * kRowBytes;  // bytes between consecutive nodes
    auto issue_rows = [&](uint32_t dst, const __nv_bfloat16 *__restrict__ base, int h, int j) {
        const char *src = reinterpret_cast<const char *>(base) + (h * kRowBytes + copy_piece * 16);
        const int32_t *cj = s_cols + j * kStep + copy_row;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            cp_async16(dst + (i >> 1) * (8 * kRowBytes) + ((i & 1) ? copy_odd : copy_even),
                       src + static_cast<uint64_t>(static_cast<uint32_t>(cj[4 * i])) * row_pitch);
    };

    for (int mbi = 0; mbi < n_mblocks; ++mbi) {
        const int32_t *mb = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + mbi) * kMbInts;
        const bool use_qr = kHasBias && mb[kMbQrSlot] >= 0;
        const int tq = use_qr ? mb[kMbTq] : 0;            // table entry tq (or 1) is the -inf entry
        const uint32_t none_idx = use_qr ? tq : 1;
        const uint32_t chunk_mask = static_cast<uint32_t>(mb[kMbChunkMask]);
        // first step after j with an edge in this m-block (one mask bit per 32 columns); n_steps if none
        static_assert(kStep == kMaskCols, "the forward's pipeline step is the mask's granularity");
        auto next_step = [&](int j) {
            ++j;
            while (j < n_steps && !((chunk_mask >> j) & 1u)) ++j;
            return j;
        };
        tile_barrier(tib);  // previous m-block's indices are no longer read; s_cols is visible
        // The warp's first K and V rows start travelling now; the cells, Q and the table follow
        // while they are in flight.
        int primed_step = -1;
        if (wl < H) primed_step = next_step(-1);
        if (primed_step >= 0 && primed_step < n_steps) issue_rows(s_k_addr, p.k, wl, primed_step);
        cp_async_commit();
        if (primed_step >= 0 && primed_step < n_steps) issue_rows(s_v_addr, p.v, wl, primed_step);
        cp_async_commit();
        const int row_lo = mb[kMbRowOff + g], row_hi = mb[kMbRowOff + g + 8];
        uint32_t q_lo[8], q_hi[8];
        if (wl < H) {
            load_row_frag(p.q + (static_cast<int64_t>(row_lo < 0 ? 0 : row_lo) * H + wl) * kHeadDim, t, q_lo);
            load_row_frag(p.q + (static_cast<int64_t>(row_hi < 0 ? 0 : row_hi) * H + wl) * kHeadDim, t, q_hi);
        }
        {
            // stage the m-block's cells as table indices: edge type, or the -inf entry; 16 bytes of
            // cells per thread and step (the matrix is [chunk][16][64], so a piece stays in one row)
            constexpr int kCellsPerPiece = 16 / static_cast<int>(sizeof(ET));
            const uint4 *ge = reinterpret_cast<const uint4 *>(et_base + mb[kMbEtOff]);
            const int pieces = kTileRows * ncols_pad / kCellsPerPiece;
            for (int i = tid; i < pieces; i += kTileThreads) {
                const int cell = i * kCellsPerPiece;
                const int chunk = cell / (kTileRows * kTileChunk), rem = cell % (kTileRows * kTileChunk);
                const int r = rem / kTileChunk, c = rem % kTileChunk;
                const uint4 raw = __ldg(ge + i);
                const ET *e = reinterpret_cast<const ET *>(&raw);
                ET *dst = s_idx + r * idx_stride + chunk * kTileChunk + c;
#pragma unroll
                for (int u = 0; u < kCellsPerPiece; ++u)
                    dst[u] = static_cast<ET>(e[u] == EtTraits<ET>::kNone ? none_idx : (use_qr ? e[u] : 0u));
            }
        }
        if (mbi == 0) {
            cp_async_wait<2>();  // embed_ak rows have landed (the two newest groups are the first K and V)
            __syncthreads();     // the block's one barrier: both tiles' threads staged embed_ak
        } else {
            tile_barrier(tib);
        }

        for (int h = wl; h < H; h += kTileWarps) {
            if (h != wl) {
                load_row_frag(p.q + (static_cast<int64_t>(row_lo < 0 ? 0 : row_lo) * H + h) * kHeadDim, t, q_lo);
                load_row_frag(p.q + (static_cast<int64_t>(row_hi < 0 ? 0 : row_hi) * H + h) * kHeadDim, t, q_hi);
            }
            // per-row constant of m-blocks without a table (log2 domain), parked in the unused table entries
            // [2, 4) of the row until the epilogue
            float *s_bias_lo = reinterpret_cast<float *>(s_tab + g * tab_stride + 2);
            float *s_bias_hi = reinterpret_cast<float *>(s_tab + (g + 8) * tab_stride + 2);
            if (use_qr) {
                // table[row][type] = scale * log2(e) * <q[row], ak[type]> for the types of this m-block
                for (int nt = 0; nt < tq; nt += 8) {
                    const int r = nt + (lane & 7), pc = lane >> 3;
                    uint32_t b0[4], b1[4];
                    ldmatrix_x4(b0, s_ak_addr + r * kRowBytes + ((pc ^ (r & 7)) << 4));
                    ldmatrix_x4(b1, s_ak_addr + r * kRowBytes + (((pc + 4) ^ (r & 7)) << 4));
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_bf16(c, q_lo[0], q_hi[0], q_lo[1], q_hi[1], b0[0], b0[1]);
                    mma_bf16(c, q_lo[2], q_hi[2], q_lo[3], q_hi[3], b0[2], b0[3]);
                    mma_bf16(c, q_lo[4], q_hi[4], q_lo[5], q_hi[5], b1[0], b1[1]);
                    mma_bf16(c, q_lo[6], q_hi[6], q_lo[7], q_hi[7], b1[2], b1[3]);
                    *reinterpret_cast<__half2 *>(s_tab + g * tab_stride + nt + 2 * t) =
                        __floats2half2_rn(c[0] * sl2, c[1] * sl2);
                    *reinterpret_cast<__half2 *>(s_tab + (g + 8) * tab_stride + nt + 2 * t) =
                        __floats2half2_rn(c[2] * sl2, c[3] * sl2);
                }
                if (t == 0) {
                    s_tab[g * tab_stride + tq] = __float2half_rn(-INFINITY);
                    s_tab[(g + 8) * tab_stride + tq] = __float2half_rn(-INFINITY);
                }
            } else {
                if (t == 0) {
                    *reinterpret_cast<__half2 *>(s_tab + g * tab_stride) = __floats2half2_rn(0.f, -INFINITY);
                    *reinterpret_cast<__half2 *>(s_tab + (g + 8) * tab_stride) = __floats2half2_rn(0.f, -INFINITY);
                }
                if (kHasBias) {
                    // every row has one edge type: <q[row], ak[type]> shifts all its scores alike
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        int type = mb[kMbRowEtOff + g + 8 * half];
                        type = type < 0 ? 0 : (type < p.n_etypes ? type : p.n_etypes - 1);
                        uint32_t a[8];
                        load_row_frag(p.ak + static_cast<int64_t>(type) * kHeadDim, t, a);
                        float sum = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float2 x = __bfloat1622float2(
                                *reinterpret_cast<const __nv_bfloat162 *>(half ? &q_hi[i] : &q_lo[i]));
                            const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&a[i]));
                            sum = fmaf(x.x, y.x, fmaf(x.y, y.y, sum));
                        }
                        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                        if (t == 0) *(half ? s_bias_hi : s_bias_lo) = sum * sl2;
                    }
                } else if (t == 0) {
                    *s_bias_lo = 0.f;
                    *s_bias_hi = 0.f;
                }
            }
            __syncwarp();

            float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
            float acc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) { acc[i][0] = 0.f; acc[i][1] = 0.f; acc[i][2] = 0.f; acc[i][3] = 0.f; }

            // Software pipeline over the active 32-column steps: K and V each have one buffer; K of
            // the next step is fetched while this step's softmax and PV run, V of the next step while
            // the next step's QK^T runs.  Every iteration commits two cp.async groups (possibly empty),
            // so "all but the newest group" is always the data the next phase needs.
            int j = primed_step;
            if (j < 0) {
                j = next_step(-1);
                if (j < n_steps) issue_rows(s_k_addr, p.k, h, j);
                cp_async_commit();
                if (j < n_steps) issue_rows(s_v_addr, p.v, h, j);
                cp_async_commit();
            }
            primed_step = -1;
            while (j < n_steps) {
                const int nj = next_step(j);
                const int c0 = j * kStep;
                cp_async_wait<1>();  // K of this step has landed
                __syncwarp();
                float s[4][4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int r = nt * 8 + (lane & 7), pc = lane >> 3;
                    uint32_t b0[4], b1[4];
                    ldmatrix_x4(b0, s_k_addr + r * kRowBytes + ((pc ^ (r & 7)) << 4));
                    ldmatrix_x4(b1, s_k_addr + r * kRowBytes + (((pc + 4) ^ (r & 7)) << 4));
                    s[nt][0] = 0.f; s[nt][1] = 0.f; s[nt][2] = 0.f; s[nt][3] = 0.f;
                    mma_bf16(s[nt], q_lo[0], q_hi[0], q_lo[1], q_hi[1], b0[0], b0[1]);
                    mma_bf16(s[nt], q_lo[2], q_hi[2], q_lo[3], q_hi[3], b0[2], b0[3]);
                    mma_bf16(s[nt], q_lo[4], q_hi[4], q_lo[5], q_hi[5], b1[0], b1[1]);
                    mma_bf16(s[nt], q_lo[6], q_hi[6], q_lo[7], q_hi[7], b1[2], b1[3]);
                }
                __syncwarp();  // every lane has read K: its buffer may be refilled
                if (nj < n_steps) issue_rows(s_k_addr, p.k, h, nj);
                cp_async_commit();
                // scale, relative-position term and mask: one table entry per cell
                float cmax_lo = -INFINITY, cmax_hi = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    uint32_t i_lo0, i_lo1, i_hi0, i_hi1;
                    load_idx_pair(s_idx + g * idx_stride + c0 + nt * 8 + 2 * t, i_lo0, i_lo1);
                    load_idx_pair(s_idx + (g + 8) * idx_stride + c0 + nt * 8 + 2 * t, i_hi0, i_hi1);
                    s[nt][0] = fmaf(s[nt][0], sl2, __half2float(s_tab[g * tab_stride + i_lo0]));
                    s[nt][1] = fmaf(s[nt][1], sl2, __half2float(s_tab[g * tab_stride + i_lo1]));
                    s[nt][2] = fmaf(s[nt][2], sl2, __half2float(s_tab[(g + 8) * tab_stride + i_hi0]));
                    s[nt][3] = fmaf(s[nt][3], sl2, __half2float(s_tab[(g + 8) * tab_stride + i_hi1]));
                    cmax_lo = fmaxf(cmax_lo, fmaxf(s[nt][0], s[nt][1]));
                    cmax_hi = fmaxf(cmax_hi, fmaxf(s[nt][2], s[nt][3]));
                }
                cmax_lo = fmaxf(cmax_lo, __shfl_xor_sync(0xffffffffu, cmax_lo, 1));
                cmax_lo = fmaxf(cmax_lo, __shfl_xor_sync(0xffffffffu, cmax_lo, 2));
                cmax_hi = fmaxf(cmax_hi, __shfl_xor_sync(0xffffffffu, cmax_hi, 1));
                cmax_hi = fmaxf(cmax_hi, __shfl_xor_sync(0xffffffffu, cmax_hi, 2));
                const float mn_lo = fmaxf(m_lo, cmax_lo), mn_hi = fmaxf(m_hi, cmax_hi);
                const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
                if (__any_sync(0xffffffffu, mn_lo != m_lo || mn_hi != m_hi)) {  // some row's maximum moved
                    const float corr_lo = ex2(m_lo - ms_lo), corr_hi = ex2(m_hi - ms_hi);
                    l_lo *= corr_lo;
                    l_hi *= corr_hi;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        acc[i][0] *= corr_lo; acc[i][1] *= corr_lo;
                        acc[i][2] *= corr_hi; acc[i][3] *= corr_hi;
                    }
                    m_lo = mn_lo;
                    m_hi = mn_hi;
                }
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    s[nt][0] = ex2(s[nt][0] - ms_lo);
                    s[nt][1] = ex2(s[nt][1] - ms_lo);
                    s[nt][2] = ex2(s[nt][2] - ms_hi);
                    s[nt][3] = ex2(s[nt][3] - ms_hi);
                    l_lo += s[nt][0] + s[nt][1];
                    l_hi += s[nt][2] + s[nt][3];
                }
                if (kDrop) {  // the row sums keep every weight; the weights that multiply V are masked and rescaled
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        const int src0 = s_cols[c0 + nt * 8 + 2 * t], src1 = s_cols[c0 + nt * 8 + 2 * t + 1];
                        s[nt][0] *= dropout_factor(p.drop, row_lo, src0, h);
                        s[nt][1] *= dropout_factor(p.drop, row_lo, src1, h);
                        s[nt][2] *= dropout_factor(p.drop, row_hi, src0, h);
                        s[nt][3] *= dropout_factor(p.drop, row_hi, src1, h);
                    }
                }
                // O += P V
                cp_async_wait<1>();  // V of this step has landed (the newest group is the next K)
                __syncwarp();
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    const uint32_t a0 = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
                    const uint32_t a1 = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
                    const uint32_t a2 = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
                    const uint32_t a3 = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
                    const int r = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
                    for (int dn = 0; dn < 8; dn += 2) {
                        const int piece = dn + (lane >> 4);
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, s_v_addr + r * kRowBytes + ((piece ^ (r & 7)) << 4));
                        mma_bf16(acc[dn], a0, a1, a2, a3, b[0], b[1]);
                        mma_bf16(acc[dn + 1], a0, a1, a2, a3, b[2], b[3]);
                    }
                }
                __syncwarp();  // every lane has read V: its buffer may be refilled
                if (nj < n_steps) issue_rows(s_v_addr, p.v, h, nj);
                cp_async_commit();
                j = nj;
            }
            cp_async_wait<0>();

            // row sums live per lane: finish them across the quad
            l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
            l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
            l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
            l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = kDrop ? (half ? row_hi : row_lo) : mb[kMbRowOff + g + 8 * half];
                if (row < 0) continue;
                const int slot = mb[kMbSlotOff + g + 8 * half];
                const float m = (half ? m_hi : m_lo) + (use_qr ? 0.f : *(half ? s_bias_hi : s_bias_lo));
                const float l = half ? l_hi : l_lo;
                if (slot < 0) {
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    __nv_bfloat16 *dst = p.o + (static_cast<int64_t>(row) * H + h) * kHeadDim + 2 * t;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn)
                        *reinterpret_cast<uint32_t *>(dst + dn * 8) =
                            pack_bf16(acc[dn][2 * half] * inv, acc[dn][2 * half + 1] * inv);
                    if (t == 0) p.lse[static_cast<int64_t>(row) * H + h] = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;
                } else {
                    float *dst = p.part_o + (static_cast<int64_t>(slot) * H + h) * kHeadDim + 2 * t;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn)
                        *reinterpret_cast<float2 *>(dst + dn * 8) = make_float2(acc[dn][2 * half], acc[dn][2 * half + 1]);
                    if (t == 0) {
                        p.part_ml[(static_cast<int64_t>(slot) * H + h) * 2] = m;
                        p.part_ml[(static_cast<int64_t>(slot) * H + h) * 2 + 1] = l;
                    }
                }
            }
            __syncwarp();  // the table is rewritten for the next head
        }
    }
}

// Shared memory of a block without the score tables, the tables' row stride, and the total.
size_t tc_other_smem_bytes(int max_cols_pad, int t_max, int et_bytes) {
    return static_cast<size_t>(kWarps) * kKvStageBytes + static_cast<size_t>(kTilesPerBlock) * max_cols_pad * 4 +
           static_cast<size_t>(kTilesPerBlock) * kTileRows * (max_cols_pad + kEtPad) * et_bytes +
           static_cast<size_t>(t_max) * kRowBytes;
}
int tc_table_stride(int max_cols_pad, int t_max, int et_bytes) {
    return table_stride(tc_other_smem_bytes(max_cols_pad, t_max, et_bytes), t_max, kWarps);
}
size_t tc_smem_bytes(int max_cols_pad, int t_max, int et_bytes) {
    return tc_other_smem_bytes(max_cols_pad, t_max, et_bytes) +
           static_cast<size_t>(kWarps) * kTileRows * tc_table_stride(max_cols_pad, t_max, et_bytes) * 2;
}

template <typename ET, bool kHasBias, bool kDrop>
int launch_tile_kernel_d(const TcParams &p, int64_t n_groups, size_t smem, cudaStream_t stream) {
    BPT_CUDA(cudaFuncSetAttribute(attn_forward_tile_kernel<ET, kHasBias, kDrop>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attn_forward_tile_kernel<ET, kHasBias, kDrop><<<static_cast<unsigned>((n_groups + kTilesPerBlock - 1) / kTilesPerBlock),
                                                    kWarps * 32, smem, stream>>>(p);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}
template <typename ET, bool kHasBias>
int launch_tile_kernel(const TcParams &p, int64_t n_groups, size_t smem, cudaStream_t stream) {
    return p.drop.threshold ? launch_tile_kernel_d<ET, kHasBias, true>(p, n_groups, smem, stream)
                            : launch_tile_kernel_d<ET, kHasBias, false>(p, n_groups, smem, stream);
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" size_t bpt_attn_tc_smem_bytes(int max_cols_pad, int t_max, int et_bytes) {
    if (max_cols_pad < 0 || t_max < 0 || (et_bytes != 1 && et_bytes != 2)) return 0;
    return tc_smem_bytes(max_cols_pad, t_max, et_bytes);
}

extern "C" size_t bpt_attn_forward_tc_workspace_bytes(int64_t n_slots, int h) {
    if (n_slots < 0 || h < 1) return 0;
    const size_t s = static_cast<size_t>(n_slots);
    return align_up(s * h * kHeadDim * 4, 256) + align_up(s * h * 2 * 4, 256) + 512;
}

extern "C" int bpt_attn_forward_tc(const int32_t *groups, int64_t n_groups, const int32_t *mblocks,
                                   const int32_t *cols, const void *et, int et_bytes, const int32_t *split_rows,
                                   int64_t n_split, int64_t n_slots, const int32_t *row_items,
                                   int64_t n_row_items, const void *attn_plan, const int32_t *counts_host,
                                   int64_t n_nodes, int64_t n_edges, int max_cols_pad, int t_max,
                                   int max_mblocks, int max_qr_slots, int n_etypes, const void *q,
                                   const void *k, const void *v, const void *ak, double scale, void *o,
                                   float *lse, int h, int d, int dtype, void *workspace,
                                   size_t workspace_bytes, const bpt_dropout_t *dropout, bpt_stream_t stream_) {
    BPT_CHECK_ARG(dropout == nullptr || (dropout->rate >= 0.0 && dropout->rate < 1.0),
                  "attn_forward_tc: dropout rate must be in [0, 1)");
    const Dropout drop = make_dropout(dropout);
    BPT_CHECK_ARG(n_groups >= 0 && n_split >= 0 && n_slots >= 0 && n_row_items >= 0 && h >= 1,
                  "attn_forward_tc: bad sizes");
    if (d != kHeadDim || dtype != BPT_BF16)
        return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc: only bf16 with head dim 64 (got dtype %d, d %d)", dtype, d);
    if (n_groups == 0 && n_row_items == 0) return BPT_OK;
    BPT_CHECK_ARG(q && k && v && o && lse, "attn_forward_tc: null tensor");
    BPT_CHECK_ARG(n_groups == 0 || (groups && mblocks), "attn_forward_tc: null plan arrays");
    BPT_CHECK_ARG(max_cols_pad == 0 || (cols && et), "attn_forward_tc: null plan arrays");
    BPT_CHECK_ARG(et_bytes == 1 || et_bytes == 2, "attn_forward_tc: et_bytes must be 1 or 2");
    BPT_CHECK_ARG(max_cols_pad % kTileChunk == 0 && max_cols_pad <= kMaxMaskBits * kMaskCols && t_max % 8 == 0 &&
                      n_etypes >= 1 && max_mblocks >= 0 && max_mblocks <= kMaxMBlocks && max_qr_slots >= 0,
                  "attn_forward_tc: bad plan sizes");
    BPT_CHECK_ARG(n_groups < (int64_t(1) << 31) && n_row_items < (int64_t(1) << 31) && h <= 65535,
                  "attn_forward_tc: too many groups, row items or heads");
    BPT_CHECK_ARG(n_row_items == 0 || (row_items && attn_plan && counts_host), "attn_forward_tc: null row-item list");
    BPT_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                    reinterpret_cast<uintptr_t>(ak) | reinterpret_cast<uintptr_t>(o)) & 15) == 0,
                  "attn_forward_tc: tensors must be 16-byte aligned");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    float *part_o = ws.take<float>(static_cast<size_t>(n_slots) * h * kHeadDim);
    float *part_ml = ws.take<float>(static_cast<size_t>(n_slots) * h * 2);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_forward_tc: workspace of %zu bytes is too small", workspace_bytes);

    if (n_row_items > 0) {
        const PlanView pv = plan_view(const_cast<void *>(attn_plan), n_nodes, counts_host[kCountsNSrc], n_edges, n_etypes);
        if (int rc = launch_forward_items_bf16(reinterpret_cast<const int4 *>(row_items), static_cast<int>(n_row_items),
                                               pv.in_src, pv.in_etype, q, k, v, ak, static_cast<float>(scale), o, lse,
                                               h, d, drop, stream))
            return rc;
    }
    if (n_groups > 0) {
        const bool bias = ak != nullptr;
        TcParams p{};
        p.groups = groups; p.mblocks = mblocks; p.cols = cols; p.et = et;
        p.q = static_cast<const __nv_bfloat16 *>(q); p.k = static_cast<const __nv_bfloat16 *>(k);
        p.v = static_cast<const __nv_bfloat16 *>(v); p.ak = static_cast<const __nv_bfloat16 *>(ak);
        p.o = static_cast<__nv_bfloat16 *>(o);
        p.lse = lse; p.part_o = part_o; p.part_ml = part_ml;
        p.n_etypes = n_etypes; p.H = h; p.max_cols_pad = max_cols_pad;
        p.t_max = bias ? t_max : 0;
        p.scale = static_cast<float>(scale);
        p.n_groups = n_groups;
        p.drop = drop;
        if (et_bytes == 1 && p.t_max > kMaxTypes8)
            return fail(BPT_ERR_INVALID, "attn_forward_tc: 8-bit cells need t_max <= %d (got %d)", kMaxTypes8, p.t_max);
        p.tab_stride = tc_table_stride(max_cols_pad, p.t_max, et_bytes);
        const size_t smem = tc_smem_bytes(max_cols_pad, p.t_max, et_bytes);
        if (smem > 227 * 1024)
            return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc: tile plan needs %zu bytes of shared memory", smem);
        int rc;
        if (et_bytes == 1)
            rc = bias ? launch_tile_kernel<uint8_t, true>(p, n_groups, smem, stream)
                      : launch_tile_kernel<uint8_t, false>(p, n_groups, smem, stream);
        else
            rc = bias ? launch_tile_kernel<uint16_t, true>(p, n_groups, smem, stream)
                      : launch_tile_kernel<uint16_t, false>(p, n_groups, smem, stream);
        if (rc) return rc;
    }
    if (n_split > 0) {
        const Geometry g{h, kHeadDim};
        attn_forward_merge_kernel<__nv_bfloat16><<<static_cast<unsigned>(n_split), merge_threads(h, kHeadDim),
                                                   merge_smem_bytes(h), stream>>>(
            reinterpret_cast<const int4 *>(split_rows), static_cast<int>(n_split), part_o, part_ml,
            static_cast<__nv_bfloat16 *>(o), lse, g);
        BPT_LAUNCH_CHECK();
    }
    return BPT_OK;
}
