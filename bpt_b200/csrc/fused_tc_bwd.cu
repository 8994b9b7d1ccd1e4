// Fused attention backward on tensor cores (bf16, head dim 64): the destination-side kernel
// (P, dP, delta, K part of dQ) on the forward's tile plan and the source-side kernel (dK, dV) on
// the transposed tile plan.
//
// ---- dK and dV ----
// Works on the transposed tile plan: an m-block is <=16 SOURCE rows, its columns are the
// destinations that attend to them, and every cell knows its edge's position in the in-CSR.
// The destination-side kernel has already left one word {bf16 p, bf16 dS} per (edge, head) in
// scratch, so a cell's two weights are one gather away:
//     dV[src] = sum_dst p * dO[dst],   dK[src] = sum_dst dS * q[dst].
// One block per m-block, one warp per head; per 16 destinations the warp stages their dO and Q
// rows in swizzled shared memory (cp.async, two buffers so that the next step's rows and
// weights travel while this step's products run), packs the gathered weights into mma A
// fragments and accumulates both products with ldmatrix.trans B fragments.  A source row wholly inside
// one m-block is written once; rows spread over several m-blocks write fp32 partials that are
// summed in slot order.  No atomics: results are bitwise reproducible.
#include <cublas_v2.h>

#include <mutex>

#include "fused_common.cuh"
#include "plan.cuh"
#include "tile_plan.cuh"

namespace bpt {
namespace {

constexpr int kHeadDim = 64;
constexpr int kWarps = 8;
constexpr int kHalf = 32;                               // destinations staged per step
constexpr int kRowBytes = kHeadDim * 2;
constexpr int kStageBytes = kHalf * kRowBytes;          // 4 KB per matrix
constexpr int kPosPad = 4;                              // int32 padding per staged position row
constexpr int kDkvStep = 16;                            // destinations per pipeline step of the dK/dV kernel
constexpr int kDkvBufBytes = 2 * kDkvStep * kRowBytes;  // one buffer: dO rows then Q rows of a step (4 KB)

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
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void *gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

struct DkvParams {
    const int32_t *groups, *mblocks, *cols, *cellpos;
    const uint32_t *PS;  // [head][in-CSR position]: {bf16 p (low half), bf16 dS (high half)}
    int64_t n_edges;
    const __nv_bfloat16 *q, *d_o;
    __nv_bfloat16 *dk, *dv;
    float *part;
    int H, max_cols_pad;
};

__global__ void __launch_bounds__(kWarps * 32, 2)
attn_backward_dkv_tile_kernel(const DkvParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: per warp {dO stage, Q stage} (8 KB) | destination ids | edge positions of the m-block
    int32_t *s_cols = reinterpret_cast<int32_t *>(smem + kWarps * 2 * kStageBytes);
    int32_t *s_pos = s_cols + p.max_cols_pad;

    const int32_t *grp = p.groups + static_cast<int64_t>(blockIdx.x) * kGroupInts;
    const int ncols_pad = grp[kGroupNcolsPad];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H;
    const uint32_t s_do = static_cast<uint32_t>(__cvta_generic_to_shared(smem + warp * 2 * kStageBytes));
    {
        const int32_t *gc = p.cols + grp[kGroupColOff];
        for (int i = threadIdx.x; i < ncols_pad; i += blockDim.x) s_cols[i] = gc[i];
    }
    const int n_steps = ncols_pad / kDkvStep;
    // dO and Q rows of head h for the 16 destinations of step j -> buffer b of the warp
    // Lane l copies piece (l & 7) of rows (l >> 3) + 4 i: two swizzled offsets per lane (i even / odd)
    // plus 1024 bytes per pair of i; a row's offset in dO and Q is one widening multiply-add.
    const int copy_row = lane >> 3, copy_piece = lane & 7;
    const uint32_t copy_even = copy_row * kRowBytes + ((copy_piece ^ copy_row) << 4);
    const uint32_t copy_odd = (copy_row + 4) * kRowBytes + ((copy_piece ^ (copy_row + 4)) << 4);
    const uint32_t row_pitch = static_cast<uint32_t>(H) * kRowBytes;  // bytes between consecutive nodes
    auto issue_rows = [&](int h, int j, int b) {
        const uint64_t head_off = static_cast<uint64_t>(h * kRowBytes + copy_piece * 16);
        const int32_t *cj = s_cols + j * kDkvStep + copy_row;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint64_t off = static_cast<uint64_t>(static_cast<uint32_t>(cj[4 * i])) * row_pitch + head_off;
            const uint32_t dst = s_do + b * kDkvBufBytes + (i >> 1) * (8 * kRowBytes) + ((i & 1) ? copy_odd : copy_even);
            cp_async16(dst, reinterpret_cast<const char *>(p.d_o) + off);
            cp_async16(dst + kDkvBufBytes / 2, reinterpret_cast<const char *>(p.q) + off);
        }
    };
    for (int mbi = 0; mbi < grp[kGroupMbCount]; ++mbi) {
        const int32_t *mb = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + mbi) * kMbInts;
        const uint32_t chunk_mask = static_cast<uint32_t>(mb[kMbChunkMask]);
        // first step after j with a cell in this m-block (one mask bit per 32 columns, two steps); n_steps if none
        static_assert(kMaskCols == 2 * kDkvStep, "two pipeline steps per mask bit");
        auto next_step = [&](int j) {
            ++j;
            while (j < n_steps && !((chunk_mask >> (j >> 1)) & 1u)) ++j;
            return j;
        };
        // packed {p, dS} words of this lane's 8 cells of step j: rows g / g+8, destinations 8nt + 2t, +1
        auto gather_weights = [&](int h, int j, uint32_t (&w)[8]) {
            const uint32_t *__restrict__ ps_h = p.PS + static_cast<int64_t>(h) * p.n_edges;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                // step j covers column groups 2j and 2j+1 (8 columns each; four groups per 32 columns)
                const int4 pos = reinterpret_cast<const int4 *>(s_pos)[(j * 2 + nt) * 32 + lane];
                w[4 * nt + 0] = pos.x >= 0 ? __ldg(ps_h + pos.x) : 0u;
                w[4 * nt + 1] = pos.y >= 0 ? __ldg(ps_h + pos.y) : 0u;
                w[4 * nt + 2] = pos.z >= 0 ? __ldg(ps_h + pos.z) : 0u;
                w[4 * nt + 3] = pos.w >= 0 ? __ldg(ps_h + pos.w) : 0u;
            }
        };
        __syncthreads();
        // the first head's first rows start travelling before the cells are staged
        int primed_step = -1;
        if (warp < H) {
            primed_step = next_step(-1);
            if (primed_step < n_steps) issue_rows(warp, primed_step, 0);
        }
        cp_async_commit();
        {
            // the cells' positions come in fragment order (cell_pos_index) and are staged as they are
            const int4 *gp = reinterpret_cast<const int4 *>(p.cellpos + mb[kMbEtOff]);
            const int pieces = kTileRows * ncols_pad / 4;
            for (int i = threadIdx.x; i < pieces; i += blockDim.x) reinterpret_cast<int4 *>(s_pos)[i] = __ldg(gp + i);
        }
        __syncthreads();
        const int row_lo = mb[kMbRowOff + g], row_hi = mb[kMbRowOff + g + 8];
        for (int h = warp; h < H; h += kWarps) {
            float dk[8][4], dv[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) { dk[i][j] = 0.f; dv[i][j] = 0.f; }
            // Two buffers: while the products of one step run, the next step's rows (cp.async) and
            // weights (registers) are in flight.  One cp.async group per iteration, possibly empty.
            int j = primed_step;
            if (j < 0) {
                j = next_step(-1);
                if (j < n_steps) issue_rows(h, j, 0);
                cp_async_commit();
            }
            primed_step = -1;
            uint32_t w[8];
            if (j < n_steps) gather_weights(h, j, w);
            int buf = 0;
            while (j < n_steps) {
                const int nj = next_step(j);
                uint32_t wn[8];
                if (nj < n_steps) {
                    issue_rows(h, nj, buf ^ 1);
                    gather_weights(h, nj, wn);
                }
                cp_async_commit();
                cp_async_wait_one();  // this step's rows have landed; the newest group is the next step's
                __syncwarp();
                {
                    // A fragments: pairs of low halves (p) / high halves (dS) of the packed words
                    const uint32_t p0 = __byte_perm(w[0], w[1], 0x5410), p1 = __byte_perm(w[2], w[3], 0x5410);
                    const uint32_t p2 = __byte_perm(w[4], w[5], 0x5410), p3 = __byte_perm(w[6], w[7], 0x5410);
                    const uint32_t s0 = __byte_perm(w[0], w[1], 0x7632), s1 = __byte_perm(w[2], w[3], 0x7632);
                    const uint32_t s2 = __byte_perm(w[4], w[5], 0x7632), s3 = __byte_perm(w[6], w[7], 0x7632);
                    const int r = ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
                    for (int dn = 0; dn < 8; dn += 2) {
                        const int piece = dn + (lane >> 4);
                        const uint32_t off = buf * kDkvBufBytes + r * kRowBytes + ((piece ^ (r & 7)) << 4);
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, s_do + off);
                        mma_bf16(dv[dn], p0, p1, p2, p3, b[0], b[1]);
                        mma_bf16(dv[dn + 1], p0, p1, p2, p3, b[2], b[3]);
                        ldmatrix_x4_trans(b, s_do + kDkvBufBytes / 2 + off);
                        mma_bf16(dk[dn], s0, s1, s2, s3, b[0], b[1]);
                        mma_bf16(dk[dn + 1], s0, s1, s2, s3, b[2], b[3]);
                    }
                }
                __syncwarp();  // this buffer is refilled by the step after next
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] = wn[i];
                j = nj;
                buf ^= 1;
            }
            cp_async_wait_all();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = half ? row_hi : row_lo;
                if (row < 0) continue;
                const int slot = mb[kMbSlotOff + g + 8 * half];
                if (slot < 0) {
                    const int64_t off = (static_cast<int64_t>(row) * H + h) * kHeadDim + 2 * t;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn) {
                        *reinterpret_cast<uint32_t *>(p.dk + off + dn * 8) = pack_bf16(dk[dn][2 * half], dk[dn][2 * half + 1]);
                        *reinterpret_cast<uint32_t *>(p.dv + off + dn * 8) = pack_bf16(dv[dn][2 * half], dv[dn][2 * half + 1]);
                    }
                } else {
                    // partial layout of the sum-merge kernel: [slot][dK (H*64) | dV (H*64)]
                    float *base = p.part + static_cast<int64_t>(slot) * 2 * H * kHeadDim + h * kHeadDim + 2 * t;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn) {
                        *reinterpret_cast<float2 *>(base + dn * 8) = make_float2(dk[dn][2 * half], dk[dn][2 * half + 1]);
                        *reinterpret_cast<float2 *>(base + H * kHeadDim + dn * 8) =
                            make_float2(dv[dn][2 * half], dv[dn][2 * half + 1]);
                    }
                }
            }
        }
    }
}

// ---- destination side ----
// One block per m-block of the forward's tile plan, one warp per head.  With lse from the forward
// and delta = <dO, O> per row, every cell's gradient is local:
//     p = exp2(s - lse),  dp = <dO[row], v[col]>,  dS = scale * p * (dp - delta).
// Per 16 columns the warp stages their K and V rows in swizzled shared memory (cp.async, two
// buffers: the next step's rows travel while this step's products run), computes
// dP = dO V^T and S = Q K^T (ldmatrix B fragments), looks the relative-position term and the
// edge mask up in the same fp16 table as the forward, scatters {p, dS} as two bf16 to the
// per-edge scratch ([head][in-CSR position], for the source-side kernel and the gradient of
// the type table) and accumulates dQ += dS K (ldmatrix.trans B fragments).  The
// relative-position part of dQ is
// added afterwards by a CUDA-core kernel.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
}

// Standard mma A-fragment words of one 64-element row for lane column t: w[2s] = elements
// (16s + 2t, +1), w[2s+1] = (16s + 8 + 2t, +1).  Also the B-fragment words of a row used as a column.
__device__ __forceinline__ void load_a_row(const __nv_bfloat16 *__restrict__ row, int t, uint32_t (&w)[8]) {
    const uint32_t *p = reinterpret_cast<const uint32_t *>(row);
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        w[2 * s] = __ldg(p + 8 * s + t);
        w[2 * s + 1] = __ldg(p + 8 * s + 4 + t);
    }
}
template <typename ET> struct EtTraits;
template <> struct EtTraits<uint8_t> { static constexpr uint32_t kNone = kNoEdge8; };
template <> struct EtTraits<uint16_t> { static constexpr uint32_t kNone = kNoEdge; };

constexpr int kIdxPad = 8;
// The destination-side kernel works on two tiles per block, four warps each (a warp takes heads
// w, w + 4, ...): four independent chains of dependent loads per SM instead of two, one copy of the
// embed_ak rows.  8-bit plans stage 8-bit table indices, which is what makes room for the second tile.
constexpr int kTileWarps = 4;
constexpr int kTilesPerBlock = 2;
constexpr int kMaxTypes8 = 248;  // with 8-bit cells the -inf entry's index (the type count) must fit a byte
static_assert(kTileWarps * kTilesPerBlock == kWarps, "two tiles of four warps fill the block");

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
constexpr int kDqStep = 16;                            // columns per pipeline step of the dQ tile kernel
constexpr int kDqBufBytes = 2 * kDqStep * kRowBytes;   // one buffer: K rows then V rows of a step (4 KB)
constexpr int kKStageBytes = 2 * kDqBufBytes;          // per warp: two buffers

struct DqParams {
    const int32_t *groups, *mblocks, *cols, *cellpos;
    const void *et;
    const __nv_bfloat16 *q, *k, *v, *ak, *o, *d_o;
    const float *lse;
    uint32_t *PS;  // [head][in-CSR position]
    int64_t n_edges;
    float *part_dq;
    __nv_bfloat16 *dq;
    int n_etypes, H, max_cols_pad, t_max, tab_stride;
    int64_t n_groups;
    float scale;
    Dropout drop;
};

template <typename ET, bool kHasBias, bool kDrop>
__global__ void __launch_bounds__(kWarps * 32, 2)
attn_backward_dq_tile_kernel(const DqParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: K/V buffers (per warp, 8 KB) | column ids (per tile) | table indices of the m-block (per tile) |
    // tables (fp16, per warp) | embed_ak rows [0, t_max) (shared by both tiles)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tib = warp / kTileWarps, wl = warp % kTileWarps;  // tile in block, warp in tile
    const int tid = threadIdx.x % (kTileWarps * 32);
    constexpr int kTileThreads = kTileWarps * 32;
    const int idx_stride = p.max_cols_pad + kIdxPad;
    int32_t *s_cols = reinterpret_cast<int32_t *>(smem + kWarps * kKStageBytes) + tib * p.max_cols_pad;
    ET *s_idx_all = reinterpret_cast<ET *>(reinterpret_cast<int32_t *>(smem + kWarps * kKStageBytes) +
                                           kTilesPerBlock * p.max_cols_pad);
    ET *s_idx = s_idx_all + tib * kTileRows * idx_stride;
    __half *s_tab_all = reinterpret_cast<__half *>(s_idx_all + kTilesPerBlock * kTileRows * idx_stride);
    const int tab_stride = p.tab_stride;
    const uint32_t s_ak = static_cast<uint32_t>(
        __cvta_generic_to_shared(s_tab_all + static_cast<int64_t>(kWarps) * kTileRows * tab_stride));
    if (kHasBias) {
        for (int i = threadIdx.x; i < p.t_max * 8; i += blockDim.x) {
            const int r = i >> 3, piece = i & 7;
            const int type = r < p.n_etypes ? r : p.n_etypes - 1;
            cp_async16(s_ak + r * kRowBytes + ((piece ^ (r & 7)) << 4), p.ak + static_cast<int64_t>(type) * kHeadDim + piece * 8);
        }
    }
    cp_async_commit();
    const int64_t tile = static_cast<int64_t>(blockIdx.x) * kTilesPerBlock + tib;
    const int32_t *grp = p.groups + (tile < p.n_groups ? tile : 0) * kGroupInts;
    const int n_mblocks = tile < p.n_groups ? grp[kGroupMbCount] : 0;
    if (n_mblocks == 0) {  // no tile for this half of the block: only keep the block's one barrier
        cp_async_wait_all();
        __syncthreads();
        return;
    }
    const int ncols_pad = grp[kGroupNcolsPad];
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H;
    const uint32_t s_k = static_cast<uint32_t>(__cvta_generic_to_shared(smem + warp * kKStageBytes));
    __half *s_tab = s_tab_all + static_cast<int64_t>(warp) * kTileRows * tab_stride;
    const float sl2 = p.scale * kLog2e;
    const ET *et_base = static_cast<const ET *>(p.et);
    {
        const int32_t *gc = p.cols + grp[kGroupColOff];
        for (int i = tid; i < ncols_pad; i += kTileThreads) s_cols[i] = gc[i];
    }
    const int n_steps = ncols_pad / kDqStep;
    // K and V rows of head h for the 16 columns of step j -> buffer b of the warp (K rows, then V rows)
    // Lane l copies piece (l & 7) of rows (l >> 3) + 4 i: two swizzled offsets per lane (i even / odd)
    // plus 1024 bytes per pair of i; a row's offset in K and V is one widening multiply-add.
    const int copy_row = lane >> 3, copy_piece = lane & 7;
    const uint32_t copy_even = copy_row * kRowBytes + ((copy_piece ^ copy_row) << 4);
    const uint32_t copy_odd = (copy_row + 4) * kRowBytes + ((copy_piece ^ (copy_row + 4)) << 4);
    const uint32_t row_pitch = static_cast<uint32_t>(H) * kRowBytes;  // bytes between consecutive nodes
    auto issue_kv = [&](int h, int j, int b) {
        const uint64_t head_off = static_cast<uint64_t>(h * kRowBytes + copy_piece * 16);
        const int32_t *cj = s_cols + j * kDqStep + copy_row;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint64_t off = static_cast<uint64_t>(static_cast<uint32_t>(cj[4 * i])) * row_pitch + head_off;
            const uint32_t dst = s_k + b * kDqBufBytes + (i >> 1) * (8 * kRowBytes) + ((i & 1) ? copy_odd : copy_even);
            cp_async16(dst, reinterpret_cast<const char *>(p.k) + off);
            cp_async16(dst + kDqBufBytes / 2, reinterpret_cast<const char *>(p.v) + off);
        }
    };
    for (int mbi = 0; mbi < n_mblocks; ++mbi) {
        const int32_t *mb = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + mbi) * kMbInts;
        const bool use_qr = kHasBias && mb[kMbQrSlot] >= 0;
        const int tq = use_qr ? mb[kMbTq] : 0;
        const uint32_t none_idx = use_qr ? tq : 1;
        const uint32_t chunk_mask = static_cast<uint32_t>(mb[kMbChunkMask]);
        const int32_t *cell_pos = p.cellpos + mb[kMbEtOff];
        const int row_lo = mb[kMbRowOff + g], row_hi = mb[kMbRowOff + g + 8];
        uint32_t q_lo[8], q_hi[8], do_lo[8], do_hi[8];
        float delta_lo = 0.f, delta_hi = 0.f, lse2_lo = 0.f, lse2_hi = 0.f;
        // a head's rows of Q and dO, delta = <dO, O> and lse (log2 domain) of the two rows of this lane
        auto load_head = [&](int h) {
            const int64_t off_lo = (static_cast<int64_t>(row_lo < 0 ? 0 : row_lo) * H + h) * kHeadDim;
            const int64_t off_hi = (static_cast<int64_t>(row_hi < 0 ? 0 : row_hi) * H + h) * kHeadDim;
            load_a_row(p.q + off_lo, t, q_lo);
            load_a_row(p.q + off_hi, t, q_hi);
            load_a_row(p.d_o + off_lo, t, do_lo);
            load_a_row(p.d_o + off_hi, t, do_hi);
            uint32_t o_lo[8], o_hi[8];
            load_a_row(p.o + off_lo, t, o_lo);
            load_a_row(p.o + off_hi, t, o_hi);
            lse2_lo = row_lo < 0 ? 0.f : p.lse[static_cast<int64_t>(row_lo) * H + h];
            lse2_hi = row_hi < 0 ? 0.f : p.lse[static_cast<int64_t>(row_hi) * H + h];
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&do_lo[i]));
                const float2 y0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&o_lo[i]));
                const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&do_hi[i]));
                const float2 y1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&o_hi[i]));
                a = fmaf(x0.x, y0.x, fmaf(x0.y, y0.y, a));
                b = fmaf(x1.x, y1.x, fmaf(x1.y, y1.y, b));
            }
            a += __shfl_xor_sync(0xffffffffu, a, 1);
            a += __shfl_xor_sync(0xffffffffu, a, 2);
            b += __shfl_xor_sync(0xffffffffu, b, 1);
            b += __shfl_xor_sync(0xffffffffu, b, 2);
            delta_lo = a;
            delta_hi = b;
            lse2_lo = lse2_lo == -INFINITY ? 0.f : lse2_lo * kLog2e;
            lse2_hi = lse2_hi == -INFINITY ? 0.f : lse2_hi * kLog2e;
        };
        tile_barrier(tib);  // previous m-block's indices are no longer read; s_cols is visible
        // first step after j with an edge in this m-block (one mask bit per 32 columns, two steps); n_steps if none
        static_assert(kMaskCols == 2 * kDqStep, "two pipeline steps per mask bit");
        auto next_step = [&](int j) {
            ++j;
            while (j < n_steps && !((chunk_mask >> (j >> 1)) & 1u)) ++j;
            return j;
        };
        // The first head's first rows and operand rows start travelling before the cells are staged.
        int primed_step = -1;
        if (wl < H) {
            primed_step = next_step(-1);
            if (primed_step < n_steps) issue_kv(wl, primed_step, 0);
        }
        cp_async_commit();
        if (wl < H) load_head(wl);
        {
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
            cp_async_wait_one();  // embed_ak rows have landed; the newest group is the first K and V
            __syncthreads();      // the block's one barrier: both tiles' threads staged embed_ak
        } else {
            tile_barrier(tib);
        }

        for (int h = wl; h < H; h += kTileWarps) {
            if (h != wl) load_head(h);
            if (use_qr) {
                for (int nt = 0; nt < tq; nt += 8) {
                    const int r = nt + (lane & 7), pc = lane >> 3;
                    uint32_t b0[4], b1[4];
                    ldmatrix_x4(b0, s_ak + r * kRowBytes + ((pc ^ (r & 7)) << 4));
                    ldmatrix_x4(b1, s_ak + r * kRowBytes + (((pc + 4) ^ (r & 7)) << 4));
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_bf16(c, q_lo[0], q_hi[0], q_lo[1], q_hi[1], b0[0], b0[1]);
                    mma_bf16(c, q_lo[2], q_hi[2], q_lo[3], q_hi[3], b0[2], b0[3]);
                    mma_bf16(c, q_lo[4], q_hi[4], q_lo[5], q_hi[5], b1[0], b1[1]);
                    mma_bf16(c, q_lo[6], q_hi[6], q_lo[7], q_hi[7], b1[2], b1[3]);
                    *reinterpret_cast<__half2 *>(s_tab + g * tab_stride + nt + 2 * t) = __floats2half2_rn(c[0] * sl2, c[1] * sl2);
                    *reinterpret_cast<__half2 *>(s_tab + (g + 8) * tab_stride + nt + 2 * t) = __floats2half2_rn(c[2] * sl2, c[3] * sl2);
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
                    // single-type rows: the forward folded scale * <q, ak[type]> into lse; take it out again
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        int type = mb[kMbRowEtOff + g + 8 * half];
                        type = type < 0 ? 0 : (type < p.n_etypes ? type : p.n_etypes - 1);
                        uint32_t a[8];
                        load_a_row(p.ak + static_cast<int64_t>(type) * kHeadDim, t, a);
                        float sum = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(half ? &q_hi[i] : &q_lo[i]));
                            const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&a[i]));
                            sum = fmaf(x.x, y.x, fmaf(x.y, y.y, sum));
                        }
                        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                        (half ? lse2_hi : lse2_lo) -= sum * sl2;
                    }
                }
            }
            __syncwarp();

            float acc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) { acc[i][0] = 0.f; acc[i][1] = 0.f; acc[i][2] = 0.f; acc[i][3] = 0.f; }
            uint32_t *__restrict__ ps_h = p.PS + static_cast<int64_t>(h) * p.n_edges;

            // Two buffers for K and two for V, 16 columns each: the next step's rows travel while
            // this step's three products run.  One cp.async group per iteration, possibly empty.
            int j = primed_step;
            if (j < 0) {
                j = next_step(-1);
                if (j < n_steps) issue_kv(h, j, 0);
                cp_async_commit();
            }
            primed_step = -1;
            int buf = 0;
            // cell positions in lane order (cell_pos_index) of column groups 2j, 2j+1; the next step's are
            // fetched as soon as this step's have been used
            const int4 *pos_base = reinterpret_cast<const int4 *>(cell_pos) + lane;
            int4 pos_cur[2] = {make_int4(-1, -1, -1, -1), make_int4(-1, -1, -1, -1)};
            if (j < n_steps) {
                pos_cur[0] = __ldg(pos_base + (j * 2) * 32);
                pos_cur[1] = __ldg(pos_base + (j * 2 + 1) * 32);
            }
            while (j < n_steps) {
                const int nj = next_step(j);
                if (nj < n_steps) issue_kv(h, nj, buf ^ 1);
                cp_async_commit();
                cp_async_wait_one();  // this step's rows have landed; the newest group is the next step's
                __syncwarp();
                const uint32_t k_buf = s_k + buf * kDqBufBytes, v_buf = k_buf + kDqBufBytes / 2;
                // dP = dO V^T and S = Q K^T for 2 column groups of 8
                float dp[2][4], s[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int r = nt * 8 + (lane & 7), pc = lane >> 3;
                    const uint32_t off0 = r * kRowBytes + ((pc ^ (r & 7)) << 4);
                    const uint32_t off1 = r * kRowBytes + (((pc + 4) ^ (r & 7)) << 4);
                    uint32_t b0[4], b1[4];
                    ldmatrix_x4(b0, v_buf + off0);
                    ldmatrix_x4(b1, v_buf + off1);
                    dp[nt][0] = 0.f; dp[nt][1] = 0.f; dp[nt][2] = 0.f; dp[nt][3] = 0.f;
                    mma_bf16(dp[nt], do_lo[0], do_hi[0], do_lo[1], do_hi[1], b0[0], b0[1]);
                    mma_bf16(dp[nt], do_lo[2], do_hi[2], do_lo[3], do_hi[3], b0[2], b0[3]);
                    mma_bf16(dp[nt], do_lo[4], do_hi[4], do_lo[5], do_hi[5], b1[0], b1[1]);
                    mma_bf16(dp[nt], do_lo[6], do_hi[6], do_lo[7], do_hi[7], b1[2], b1[3]);
                    ldmatrix_x4(b0, k_buf + off0);
                    ldmatrix_x4(b1, k_buf + off1);
                    s[nt][0] = 0.f; s[nt][1] = 0.f; s[nt][2] = 0.f; s[nt][3] = 0.f;
                    mma_bf16(s[nt], q_lo[0], q_hi[0], q_lo[1], q_hi[1], b0[0], b0[1]);
                    mma_bf16(s[nt], q_lo[2], q_hi[2], q_lo[3], q_hi[3], b0[2], b0[3]);
                    mma_bf16(s[nt], q_lo[4], q_hi[4], q_lo[5], q_hi[5], b1[0], b1[1]);
                    mma_bf16(s[nt], q_lo[6], q_hi[6], q_lo[7], q_hi[7], b1[2], b1[3]);
                    // probabilities, per-edge scratch, dS (kept in s)
                    const int c = j * kDqStep + nt * 8 + 2 * t;
                    uint32_t i_lo0, i_lo1, i_hi0, i_hi1;
                    load_idx_pair(s_idx + g * idx_stride + c, i_lo0, i_lo1);
                    load_idx_pair(s_idx + (g + 8) * idx_stride + c, i_hi0, i_hi1);
                    const int4 pos4 = pos_cur[nt];
                    const float tab[4] = {__half2float(s_tab[g * tab_stride + i_lo0]),
                                          __half2float(s_tab[g * tab_stride + i_lo1]),
                                          __half2float(s_tab[(g + 8) * tab_stride + i_hi0]),
                                          __half2float(s_tab[(g + 8) * tab_stride + i_hi1])};
                    const int pos[4] = {pos4.x, pos4.y, pos4.z, pos4.w};
                    float keep[4] = {1.f, 1.f, 1.f, 1.f};
                    if (kDrop) {  // the factor the forward multiplied this weight by before summing V
                        const int src0 = s_cols[c], src1 = s_cols[c + 1];
                        keep[0] = dropout_factor(p.drop, row_lo, src0, h);
                        keep[1] = dropout_factor(p.drop, row_lo, src1, h);
                        keep[2] = dropout_factor(p.drop, row_hi, src0, h);
                        keep[3] = dropout_factor(p.drop, row_hi, src1, h);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float pr = ex2(fmaf(s[nt][i], sl2, tab[i]) - (i < 2 ? lse2_lo : lse2_hi));
                        // dS = scale * p * (dp - delta) with dp the gradient of p, i.e. keep * <dO, v>; the source
                        // side needs the weight V was summed with, keep * p
                        s[nt][i] = p.scale * pr * (dp[nt][i] * keep[i] - (i < 2 ? delta_lo : delta_hi));
                        if (pos[i] >= 0) ps_h[pos[i]] = pack_bf16(pr * keep[i], s[nt][i]);
                    }
                }
                // the next step's cell positions travel during dQ += dS K and the next step's first products
                if (nj < n_steps) {
                    pos_cur[0] = __ldg(pos_base + (nj * 2) * 32);
                    pos_cur[1] = __ldg(pos_base + (nj * 2 + 1) * 32);
                }
                // dQ += dS K
                {
                    const uint32_t a0 = pack_bf16(s[0][0], s[0][1]), a1 = pack_bf16(s[0][2], s[0][3]);
                    const uint32_t a2 = pack_bf16(s[1][0], s[1][1]), a3 = pack_bf16(s[1][2], s[1][3]);
                    const int r = ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
                    for (int dn = 0; dn < 8; dn += 2) {
                        const int piece = dn + (lane >> 4);
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, k_buf + r * kRowBytes + ((piece ^ (r & 7)) << 4));
                        mma_bf16(acc[dn], a0, a1, a2, a3, b[0], b[1]);
                        mma_bf16(acc[dn + 1], a0, a1, a2, a3, b[2], b[3]);
                    }
                }
                __syncwarp();  // these buffers are refilled by the step after next
                j = nj;
                buf ^= 1;
            }
            cp_async_wait_all();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = half ? row_hi : row_lo;
                if (row < 0) continue;
                const int slot = mb[kMbSlotOff + g + 8 * half];
                if (slot < 0) {
                    __nv_bfloat16 *dst = p.dq + (static_cast<int64_t>(row) * H + h) * kHeadDim + 2 * t;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn)
                        *reinterpret_cast<uint32_t *>(dst + dn * 8) = pack_bf16(acc[dn][2 * half], acc[dn][2 * half + 1]);
                } else {
                    float *dst = p.part_dq + (static_cast<int64_t>(slot) * H + h) * kHeadDim + 2 * t;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn)
                        *reinterpret_cast<float2 *>(dst + dn * 8) = make_float2(acc[dn][2 * half], acc[dn][2 * half + 1]);
                }
            }
            __syncwarp();  // the table is rewritten for the next head
        }
    }
}

// ---- relative-position terms through a dense per-row table ----
// G[row, h, t] = sum of dS over the row's edges of type t (zero rows for rows whose edges share one
// type: their dS sums to zero).  With it the two relative-position gradients are plain GEMMs:
//     dQ[row, h, :] += G[row, h, :] . embed_ak          d embed_ak = G^T . Q
// One warp per destination row, 32 edges at a time (one per lane, coalesced per head).  When the
// 32 types differ (the usual case: a leaf's edges all differ in level or offset) the lanes add
// into their own bins at once; otherwise they add one after the other in lane order.  Either
// way every bin sees its edges in CSR order, so the sums have a fixed order.
// G is (n_nodes * H, tq).  kPacked: G is bf16 and PS is [head][in-CSR position] words {bf16 p, bf16 dS};
// otherwise G is fp32 and dS = scale * p * (dp - delta) comes from the fp32 scratch of the CUDA-core backward
// (P, dP in [in-CSR position][head] order, delta per (row, head)).
template <bool kPacked>
struct TableScratch {
    const uint32_t *PS;
    int64_t n_edges;
    const float *P, *dP, *delta;
    float scale;
};
__device__ __forceinline__ void store_table_pair(__nv_bfloat16 *out, float a, float b) {
    *reinterpret_cast<__nv_bfloat162 *>(out) = __floats2bfloat162_rn(a, b);
}
__device__ __forceinline__ void store_table_pair(float *out, float a, float b) {
    *reinterpret_cast<float2 *>(out) = make_float2(a, b);
}
template <bool kPacked, typename GT>
__global__ void __launch_bounds__(128)
build_type_table_kernel(const int32_t *__restrict__ in_indptr, const int32_t *__restrict__ in_etype,
                        const int32_t *__restrict__ row_uniform, int n_rows, const TableScratch<kPacked> sc,
                        GT *__restrict__ G, int H, int tq) {
    const uint32_t *__restrict__ PS = sc.PS;
    const int64_t n_edges = sc.n_edges;
    extern __shared__ float s_g[];  // [4 warps][H][tq]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row >= n_rows) return;
    float *g = s_g + static_cast<int64_t>(warp) * H * tq;
    GT *out = G + static_cast<int64_t>(row) * H * tq;
    const int cells = H * tq;
    if (row_uniform[row]) {
        for (int i = lane * 2; i < cells; i += 64) store_table_pair(out + i, 0.f, 0.f);
        return;
    }
    for (int i = lane; i < cells; i += 32) g[i] = 0.f;
    __syncwarp();
    const int beg = in_indptr[row], end = in_indptr[row + 1];
    for (int j0 = beg; j0 < end; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j < end;
        const int type = valid ? in_etype[j] : -1 - lane;  // idle lanes get distinct keys
        const bool distinct = __all_sync(0xffffffffu, __match_any_sync(0xffffffffu, type) == (1u << lane));
        for (int h0 = 0; h0 < H; h0 += 8) {
            float ds[8];  // the loads of eight heads travel together
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (kPacked) {
                    ds[u] = valid && h0 + u < H
                                ? __uint_as_float(__ldg(PS + static_cast<int64_t>(h0 + u) * n_edges + j) & 0xffff0000u)
                                : 0.f;
                } else {
                    ds[u] = 0.f;
                    if (valid && h0 + u < H) {
                        const int64_t at = static_cast<int64_t>(j) * H + h0 + u;
                        ds[u] = sc.scale * __ldg(sc.P + at) *
                                (__ldg(sc.dP + at) - __ldg(sc.delta + static_cast<int64_t>(row) * H + h0 + u));
                    }
                }
            }
            if (distinct) {
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (valid && h0 + u < H) g[(h0 + u) * tq + type] += ds[u];
            } else {
                for (int i = 0; i < 32; ++i) {
                    if (lane == i && valid) {
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            if (h0 + u < H) g[(h0 + u) * tq + type] += ds[u];
                    }
                    __syncwarp();
                }
            }
        }
        __syncwarp();
    }
    for (int i = lane * 2; i < cells; i += 64) store_table_pair(out + i, g[i], g[i + 1]);
}

// One cuBLAS handle per device, created on first use.
cublasHandle_t cublas_handle() {
    static std::mutex mu;
    static cublasHandle_t handles[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (handles[dev] == nullptr && cublasCreate(&handles[dev]) != CUBLAS_STATUS_SUCCESS) handles[dev] = nullptr;
    return handles[dev];
}

// A second stream per device, so that the relative-position step (type table + two GEMMs) and the source-side
// tile kernel, which both depend only on the destination-side kernel, can run side by side.  The caller's
// stream forks into it and joins it again inside the call (events), so the call stays stream-ordered.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
SideStream *side_stream() {
    static std::mutex mu;
    static SideStream side[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    SideStream &s = side[dev];
    if (s.stream == nullptr) {
        if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
            s.stream = nullptr;
            return nullptr;
        }
    }
    return &s;
}

// Block size of dkv_sum_merge_kernel: one column per thread where that fits.
inline int sum_merge_threads(int columns) {
    const int t = (columns + 31) / 32 * 32;
    return t < 128 ? 128 : (t > 1024 ? 1024 : t);
}

// out0[row] | out1[row] = sum over the row's slots, in slot order, of the slot's two halves.
// (out1 == nullptr: a slot holds one array of `width` values.)
__global__ void __launch_bounds__(1024, 2) dkv_sum_merge_kernel(const int4 *__restrict__ split_rows, int n_split, const float *__restrict__ part,
                                     int width, __nv_bfloat16 *__restrict__ out0, __nv_bfloat16 *__restrict__ out1) {
    const int sr = blockIdx.x;
    if (sr >= n_split) return;
    const int4 rec = split_rows[sr];
    const int row = rec.x, first = rec.y, count = rec.z;
    const int stride = out1 ? 2 * width : width;
    for (int c = threadIdx.x; c < stride; c += blockDim.x) {
        const float *src = part + static_cast<int64_t>(first) * stride + c;
        float acc = 0.f;
        int s = 0;
        for (; s + 16 <= count; s += 16) {
            float x[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) x[u] = src[static_cast<int64_t>(s + u) * stride];
#pragma unroll
            for (int u = 0; u < 16; ++u) acc += x[u];
        }
        if (s < count) {  // the last, partial batch: its loads travel together too
            float x[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) x[u] = s + u < count ? src[static_cast<int64_t>(s + u) * stride] : 0.f;
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (s + u < count) acc += x[u];
        }
        if (c < width) out0[static_cast<int64_t>(row) * width + c] = __float2bfloat16_rn(acc);
        else out1[static_cast<int64_t>(row) * width + (c - width)] = __float2bfloat16_rn(acc);
    }
}

constexpr int kMaxTableTypes = 256;  // beyond this the dense per-row type table is not used
}  // namespace

// The relative-position gradients of the fp32 backward through the dense per-row type table: G (fp32,
// n_nodes * H x tq) from the fp32 scratch, then dQ += G . embed_ak and d embed_ak = G^T . Q as fp32 library
// GEMMs (no tensor-core math: the 1e-5 bar).  type_table_f32_elems: floats of G, 0 when the table does not apply
// (no types, too many types for the kernel's shared memory) and the caller keeps its per-edge kernels.
size_t type_table_f32_elems(int tq, int64_t n_nodes, int h) {
    if (tq <= 0 || tq > kMaxTableTypes || static_cast<size_t>(4) * h * tq * sizeof(float) > 48 * 1024) return 0;
    return static_cast<size_t>(n_nodes) * h * tq;
}
int launch_type_table_terms_f32(const PlanView &pv, int tq, int n_etypes, const float *q, const float *ak,
                                const float *P, const float *dP, const float *delta, float scale, float *dq,
                                float *dak, float *G, int h, cudaStream_t stream) {
    const int64_t n_nodes = pv.n_nodes;
    if (n_nodes == 0) return BPT_OK;
    const long long nh = static_cast<long long>(n_nodes) * h;
    BPT_CHECK_ARG(nh < (1ll << 31), "attn_backward_tc32: n_nodes * h exceeds the GEMM index range");
    const int kk = tq < n_etypes ? tq : n_etypes;
    const size_t smem_g = static_cast<size_t>(4) * h * tq * sizeof(float);
    const TableScratch<false> scratch{nullptr, pv.n_edges, P, dP, delta, scale};
    build_type_table_kernel<false, float><<<static_cast<unsigned>((n_nodes + 3) / 4), 128, smem_g, stream>>>(
        pv.in_indptr, pv.in_etype, pv.row_uniform, static_cast<int>(n_nodes), scratch, G, h, tq);
    BPT_LAUNCH_CHECK();
    cublasHandle_t handle = cublas_handle();
    if (handle == nullptr) return fail(BPT_ERR_CUDA, "attn_backward_tc32: cuBLAS handle could not be created");
    if (cublasSetStream(handle, stream) != CUBLAS_STATUS_SUCCESS) return fail(BPT_ERR_CUDA, "attn_backward_tc32: cublasSetStream failed");
    const float one = 1.f, zero = 0.f;
    // row-major dQ (nh x 64) += G (nh x tq) . ak (tq x 64)   ==   column-major dQ^T = ak^T . G^T
    cublasStatus_t st = cublasGemmEx(handle, CUBLAS_OP_N, CUBLAS_OP_N, kHeadDim, static_cast<int>(nh), kk, &one, ak,
                                     CUDA_R_32F, kHeadDim, G, CUDA_R_32F, tq, &one, dq, CUDA_R_32F, kHeadDim,
                                     CUBLAS_COMPUTE_32F_PEDANTIC, CUBLAS_GEMM_DEFAULT);
    if (st != CUBLAS_STATUS_SUCCESS) return fail(BPT_ERR_CUDA, "attn_backward_tc32: cublasGemmEx (dQ) failed with %d", int(st));
    // row-major d ak (kk x 64) = G^T (kk x nh) . Q (nh x 64)   ==   column-major (d ak)^T = Q^T . G
    st = cublasGemmEx(handle, CUBLAS_OP_N, CUBLAS_OP_T, kHeadDim, kk, static_cast<int>(nh), &one, q, CUDA_R_32F,
                      kHeadDim, G, CUDA_R_32F, tq, &zero, dak, CUDA_R_32F, kHeadDim, CUBLAS_COMPUTE_32F_PEDANTIC,
                      CUBLAS_GEMM_DEFAULT);
    if (st != CUBLAS_STATUS_SUCCESS) return fail(BPT_ERR_CUDA, "attn_backward_tc32: cublasGemmEx (d ak) failed with %d", int(st));
    return BPT_OK;
}

}  // namespace bpt

using namespace bpt;

namespace {

int check_tile_plan(const char *name, const bpt_tile_plan_t *tp, bool need_et, bool need_pos) {
    BPT_CHECK_ARG(tp != nullptr, "%s: null tile plan", name);
    BPT_CHECK_ARG(tp->n_groups >= 0 && tp->n_split >= 0 && tp->n_slots >= 0 && tp->n_groups < (int64_t(1) << 31),
                  "%s: bad tile plan sizes", name);
    BPT_CHECK_ARG(tp->n_groups == 0 || (tp->groups && tp->mblocks), "%s: null tile plan arrays", name);
    BPT_CHECK_ARG(tp->max_cols_pad % kTileChunk == 0 && tp->max_cols_pad <= kMaxMaskBits * kMaskCols && tp->t_max % 8 == 0,
                  "%s: bad tile plan sizes", name);
    BPT_CHECK_ARG(tp->max_cols_pad == 0 || tp->cols, "%s: null tile plan arrays", name);
    if (need_et) BPT_CHECK_ARG(tp->max_cols_pad == 0 || (tp->et && (tp->et_bytes == 1 || tp->et_bytes == 2)), "%s: tile plan without edge types", name);
    if (need_pos) BPT_CHECK_ARG(tp->max_cols_pad == 0 || tp->cell_pos, "%s: tile plan without cell positions", name);
    BPT_CHECK_ARG(tp->n_split == 0 || tp->split_rows, "%s: null split rows", name);
    return BPT_OK;
}

int run_dkv(const bpt_tile_plan_t *tp, const uint32_t *PS, int64_t n_edges, const void *q, const void *d_o, void *dk, void *dv, int h,
            float *part, cudaStream_t stream) {
    if (tp->n_groups == 0) return BPT_OK;
    DkvParams p{};
    p.groups = tp->groups; p.mblocks = tp->mblocks; p.cols = tp->cols; p.cellpos = tp->cell_pos;
    p.PS = PS; p.n_edges = n_edges;
    p.q = static_cast<const __nv_bfloat16 *>(q); p.d_o = static_cast<const __nv_bfloat16 *>(d_o);
    p.dk = static_cast<__nv_bfloat16 *>(dk); p.dv = static_cast<__nv_bfloat16 *>(dv);
    p.part = part; p.H = h; p.max_cols_pad = tp->max_cols_pad;
    const size_t smem = static_cast<size_t>(kWarps) * 2 * kStageBytes + static_cast<size_t>(tp->max_cols_pad) * 4 +
                        static_cast<size_t>(kTileRows) * (tp->max_cols_pad + kPosPad) * 4;
    if (smem > 227 * 1024)
        return fail(BPT_ERR_UNSUPPORTED, "attn_backward_tc: transposed tile plan needs %zu bytes of shared memory", smem);
    BPT_CUDA(cudaFuncSetAttribute(attn_backward_dkv_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
    attn_backward_dkv_tile_kernel<<<static_cast<unsigned>(tp->n_groups), kWarps * 32, smem, stream>>>(p);
    BPT_LAUNCH_CHECK();
    if (tp->n_split > 0) {
        dkv_sum_merge_kernel<<<static_cast<unsigned>(tp->n_split), sum_merge_threads(2 * h * kHeadDim), 0, stream>>>(
            reinterpret_cast<const int4 *>(tp->split_rows), static_cast<int>(tp->n_split), part, h * kHeadDim, p.dk, p.dv);
        BPT_LAUNCH_CHECK();
    }
    return BPT_OK;
}

template <typename ET, bool kHasBias, bool kDrop>
int launch_dq_kernel_d(const DqParams &p, int64_t n_groups, size_t smem, cudaStream_t stream) {
    BPT_CUDA(cudaFuncSetAttribute(attn_backward_dq_tile_kernel<ET, kHasBias, kDrop>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attn_backward_dq_tile_kernel<ET, kHasBias, kDrop><<<static_cast<unsigned>((n_groups + kTilesPerBlock - 1) / kTilesPerBlock),
                                                        kWarps * 32, smem, stream>>>(p);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}
template <typename ET, bool kHasBias>
int launch_dq_kernel(const DqParams &p, int64_t n_groups, size_t smem, cudaStream_t stream) {
    return p.drop.threshold ? launch_dq_kernel_d<ET, kHasBias, true>(p, n_groups, smem, stream)
                            : launch_dq_kernel_d<ET, kHasBias, false>(p, n_groups, smem, stream);
}

}  // namespace

namespace {
size_t type_table_elems(const bpt_tile_plan_t *dst_tiles, int64_t n_nodes, int h) {
    const int tq = dst_tiles->t_max;
    return tq > 0 && tq <= kMaxTableTypes ? static_cast<size_t>(n_nodes) * h * tq : 1;
}
}  // namespace

extern "C" size_t bpt_attn_backward_tc_workspace_bytes(const bpt_tile_plan_t *dst_tiles, const bpt_tile_plan_t *src_tiles,
                                                       const int32_t *counts_host, int64_t n_nodes, int64_t n_edges,
                                                       int h) {
    if (!dst_tiles || !src_tiles || !counts_host || n_nodes < 0 || n_edges < 0 || h < 1) return 0;
    const size_t e = static_cast<size_t>(n_edges);
    return align_up(e * h * 4, 256) +
           align_up(static_cast<size_t>(dst_tiles->n_slots) * h * kHeadDim * 4, 256) +
           align_up(static_cast<size_t>(src_tiles->n_slots) * 2 * h * kHeadDim * 4, 256) +
           align_up(static_cast<size_t>(counts_host[7]) * kHeadDim * 4, 256) +
           align_up(type_table_elems(dst_tiles, n_nodes, h) * 2, 256) + 2048;
}

extern "C" int bpt_attn_backward_tc(const bpt_tile_plan_t *dst_tiles, const bpt_tile_plan_t *src_tiles,
                                    const void *attn_plan, const int32_t *counts_host, int64_t n_nodes,
                                    int64_t n_edges, int n_etypes, const void *q, const void *k, const void *v,
                                    const void *ak, double scale, const void *o, const float *lse, const void *d_o,
                                    void *dq, void *dk, void *dv, float *dak, int h, int d, int dtype,
                                    void *workspace, size_t workspace_bytes, const bpt_dropout_t *dropout,
                                    bpt_stream_t stream_) {
    BPT_CHECK_ARG(dropout == nullptr || (dropout->rate >= 0.0 && dropout->rate < 1.0),
                  "attn_backward_tc: dropout rate must be in [0, 1)");
    if (d != kHeadDim || dtype != BPT_BF16)
        return fail(BPT_ERR_UNSUPPORTED, "attn_backward_tc: only bf16 with head dim 64 (got dtype %d, d %d)", dtype, d);
    if (int rc = check_tile_plan("attn_backward_tc", dst_tiles, true, true)) return rc;
    if (int rc = check_tile_plan("attn_backward_tc", src_tiles, false, true)) return rc;
    BPT_CHECK_ARG(attn_plan && counts_host && n_nodes >= 0 && n_edges >= 0 && n_etypes >= 1 && h >= 1,
                  "attn_backward_tc: bad plan arguments");
    BPT_CHECK_ARG(dst_tiles->n_row_items == 0, "attn_backward_tc: the tile plan must not hold CUDA-core row items");
    if (n_nodes == 0) return BPT_OK;
    BPT_CHECK_ARG(q && k && v && o && lse && d_o && dq && dk && dv, "attn_backward_tc: null tensor");
    BPT_CHECK_ARG(ak == nullptr || dak != nullptr, "attn_backward_tc: ak given without dak");
    BPT_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                    reinterpret_cast<uintptr_t>(ak) | reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(d_o) |
                    reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15) == 0,
                  "attn_backward_tc: tensors must be 16-byte aligned");
    cudaStream_t stream = as_stream(stream_);
    const PlanView pv = plan_view(const_cast<void *>(attn_plan), n_nodes, counts_host[kCountsNSrc], n_edges, n_etypes);
    Workspace ws(workspace, workspace_bytes);
    const size_t e = static_cast<size_t>(n_edges);
    uint32_t *PS = ws.take<uint32_t>(e * h);
    float *part_dq = ws.take<float>(static_cast<size_t>(dst_tiles->n_slots) * h * kHeadDim);
    float *part_dkv = ws.take<float>(static_cast<size_t>(src_tiles->n_slots) * 2 * h * kHeadDim);
    float *part_dak = ws.take<float>(static_cast<size_t>(counts_host[7]) * kHeadDim);
    __nv_bfloat16 *G = ws.take<__nv_bfloat16>(type_table_elems(dst_tiles, n_nodes, h));
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_backward_tc: workspace of %zu bytes is too small", workspace_bytes);
    const float sc = static_cast<float>(scale);

    // 1. destination side: P, dP, delta, K part of dQ
    if (dst_tiles->n_groups > 0) {
        const bool bias = ak != nullptr;
        DqParams p{};
        p.groups = dst_tiles->groups; p.mblocks = dst_tiles->mblocks; p.cols = dst_tiles->cols;
        p.cellpos = dst_tiles->cell_pos; p.et = dst_tiles->et;
        p.q = static_cast<const __nv_bfloat16 *>(q); p.k = static_cast<const __nv_bfloat16 *>(k);
        p.v = static_cast<const __nv_bfloat16 *>(v); p.ak = static_cast<const __nv_bfloat16 *>(ak);
        p.o = static_cast<const __nv_bfloat16 *>(o); p.d_o = static_cast<const __nv_bfloat16 *>(d_o);
        p.lse = lse; p.PS = PS; p.n_edges = n_edges; p.part_dq = part_dq;
        p.dq = static_cast<__nv_bfloat16 *>(dq);
        p.n_etypes = n_etypes; p.H = h; p.max_cols_pad = dst_tiles->max_cols_pad;
        p.t_max = bias ? dst_tiles->t_max : 0;
        p.scale = sc;
        p.n_groups = dst_tiles->n_groups;
        p.drop = make_dropout(dropout);
        if (dst_tiles->et_bytes == 1 && p.t_max > kMaxTypes8)
            return fail(BPT_ERR_INVALID, "attn_backward_tc: 8-bit cells need t_max <= %d (got %d)", kMaxTypes8, p.t_max);
        const size_t other = static_cast<size_t>(kWarps) * kKStageBytes +
                             static_cast<size_t>(kTilesPerBlock) * p.max_cols_pad * 4 +
                             static_cast<size_t>(kTilesPerBlock) * kTileRows * (p.max_cols_pad + kIdxPad) * dst_tiles->et_bytes +
                             static_cast<size_t>(p.t_max) * kRowBytes;
        p.tab_stride = table_stride(other, p.t_max, kWarps);
        const size_t smem = other + static_cast<size_t>(kWarps) * kTileRows * p.tab_stride * 2;
        if (smem > 227 * 1024)
            return fail(BPT_ERR_UNSUPPORTED, "attn_backward_tc: tile plan needs %zu bytes of shared memory", smem);
        int rc;
        if (dst_tiles->et_bytes == 1)
            rc = bias ? launch_dq_kernel<uint8_t, true>(p, dst_tiles->n_groups, smem, stream)
                      : launch_dq_kernel<uint8_t, false>(p, dst_tiles->n_groups, smem, stream);
        else
            rc = bias ? launch_dq_kernel<uint16_t, true>(p, dst_tiles->n_groups, smem, stream)
                      : launch_dq_kernel<uint16_t, false>(p, dst_tiles->n_groups, smem, stream);
        if (rc) return rc;
        if (dst_tiles->n_split > 0) {
            dkv_sum_merge_kernel<<<static_cast<unsigned>(dst_tiles->n_split), sum_merge_threads(h * kHeadDim), 0, stream>>>(
                reinterpret_cast<const int4 *>(dst_tiles->split_rows), static_cast<int>(dst_tiles->n_split), part_dq,
                h * kHeadDim, static_cast<__nv_bfloat16 *>(dq), nullptr);
            BPT_LAUNCH_CHECK();
        }
    }
    // 2. and 3. both read the per-edge scratch the destination side has just written and touch disjoint outputs
    // (2: dQ and d embed_ak, 3: dK and dV), so 2 goes to a second stream that forks from and joins the caller's.
    SideStream *side = side_stream();
    if (side == nullptr) return fail(BPT_ERR_CUDA, "attn_backward_tc: could not create the side stream");
    BPT_CUDA(cudaEventRecord(side->fork, stream));
    BPT_CUDA(cudaStreamWaitEvent(side->stream, side->fork, 0));
    cudaStream_t main_stream = stream;
    stream = side->stream;
    // 2. relative-position part of dQ and the gradient of the type table
    const int tq = dst_tiles->t_max;
    if (ak != nullptr && dak != nullptr)
        BPT_CUDA(cudaMemsetAsync(dak, 0, sizeof(float) * static_cast<size_t>(n_etypes) * kHeadDim, stream));
    if (ak != nullptr && tq > 0 && tq <= kMaxTableTypes && static_cast<size_t>(4) * h * tq * sizeof(float) <= 48 * 1024) {
        // dense per-row type table, then two library GEMMs
        const int kk = tq < n_etypes ? tq : n_etypes;
        const size_t smem_g = static_cast<size_t>(4) * h * tq * sizeof(float);
        const TableScratch<true> scratch{PS, n_edges, nullptr, nullptr, nullptr, 1.f};
        build_type_table_kernel<true, __nv_bfloat16><<<static_cast<unsigned>((n_nodes + 3) / 4), 128, smem_g, stream>>>(
            pv.in_indptr, pv.in_etype, pv.row_uniform, static_cast<int>(n_nodes), scratch, G, h, tq);
        BPT_LAUNCH_CHECK();
        cublasHandle_t handle = cublas_handle();
        if (handle == nullptr) return fail(BPT_ERR_CUDA, "attn_backward_tc: cuBLAS handle could not be created");
        if (cublasSetStream(handle, stream) != CUBLAS_STATUS_SUCCESS) return fail(BPT_ERR_CUDA, "attn_backward_tc: cublasSetStream failed");
        const float one = 1.f, zero = 0.f;
        const long long nh = static_cast<long long>(n_nodes) * h;
        BPT_CHECK_ARG(nh < (1ll << 31), "attn_backward_tc: n_nodes * h exceeds the GEMM index range");
        // row-major dQ (nh x 64) += G (nh x tq) . ak (tq x 64)   ==   column-major dQ^T = ak^T . G^T
        cublasStatus_t st = cublasGemmEx(handle, CUBLAS_OP_N, CUBLAS_OP_N, kHeadDim, static_cast<int>(nh), kk, &one, ak,
                                         CUDA_R_16BF, kHeadDim, G, CUDA_R_16BF, tq, &one, dq, CUDA_R_16BF, kHeadDim,
                                         CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
        if (st != CUBLAS_STATUS_SUCCESS) return fail(BPT_ERR_CUDA, "attn_backward_tc: cublasGemmEx (dQ) failed with %d", int(st));
        // row-major d ak (kk x 64) = G^T (kk x nh) . Q (nh x 64)   ==   column-major (d ak)^T = Q^T . G
        st = cublasGemmEx(handle, CUBLAS_OP_N, CUBLAS_OP_T, kHeadDim, kk, static_cast<int>(nh), &one, q, CUDA_R_16BF,
                          kHeadDim, G, CUDA_R_16BF, tq, &zero, dak, CUDA_R_32F, kHeadDim, CUBLAS_COMPUTE_32F,
                          CUBLAS_GEMM_DEFAULT);
        if (st != CUBLAS_STATUS_SUCCESS) return fail(BPT_ERR_CUDA, "attn_backward_tc: cublasGemmEx (d ak) failed with %d", int(st));
    } else {
        // many edge types: per-edge CUDA-core kernels
        if (int rc = launch_backward_ak_terms_bf16(pv, counts_host, q, ak, PS, dq, dak, part_dak, h, d, stream)) return rc;
    }
    stream = main_stream;
    BPT_CUDA(cudaEventRecord(side->join, side->stream));
    // 3. source side: dK, dV
    const int rc_dkv = run_dkv(src_tiles, PS, n_edges, q, d_o, dk, dv, h, part_dkv, stream);
    BPT_CUDA(cudaStreamWaitEvent(stream, side->join, 0));
    return rc_dkv;
}
