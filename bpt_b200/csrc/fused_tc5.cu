// Fused graph attention forward on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory), bf16 storage, fp32 accumulation, head dim 64.
//
// A thread block of 128 threads owns one group of the tile plan built with 128-row groups
// (tile_plan.cuh: up to 8 m-blocks of 16 destination rows over one sorted list of source columns).
// Thread t owns destination row t of the group: it is lane t of tensor memory, so a row's scores,
// its running maximum and sum, and its output accumulator all belong to one thread and the softmax
// needs no exchange between threads.  Per head, for each active chunk of 64 source columns:
//   1. the block gathers the chunk's K and V rows into 128-byte-swizzled shared-memory tiles
//      (16-byte cp.async; the next chunk travels while this one is worked on),
//   2. one thread issues S = Q K^T (M = 128, N = 64, K = 64) into tensor memory,
//   3. every thread reads its row of S (tcgen05.ld), adds the relative-position term and the edge mask
//      with one table lookup per cell -- table[row][type] = scale * log2(e) * <q[row], embed_ak[type]>,
//      itself a tcgen05.mma (Q . embed_ak^T) parked in shared memory as fp16, with an entry of -inf
//      that cells without an edge point to --, keeps an online softmax with a lazily updated maximum
//      (the accumulator row is rescaled only when the maximum grows by more than 2^8), and writes its
//      row of P as bf16 into a swizzled tile,
//   4. one thread issues O += P V (V read as an MN-major operand straight from its gathered rows).
// Warps skip 32-column halves in which none of their 32 rows has an edge; chunks without any edge
// are skipped by the whole block.  Rows wholly inside the group are written as final O / lse; rows
// spread over several groups write (m, l, O) partials for the merge kernel, in slot order.
// Every wait on an mbarrier is bounded; a wait that runs out sets a status word and the block frees
// its tensor memory and returns.
#include "fused_common.cuh"
#include "plan.cuh"
#include "tc5.cuh"
#include "tile_plan.cuh"

namespace bpt {
namespace {

using namespace tc5;

constexpr int kHeadDim = 64;
constexpr int kRows = 128;             // destination rows per block = TMEM lanes
constexpr int kChunk = 64;             // source columns per step
constexpr int kTileBytes = kChunk * 128;  // one K or V chunk: 64 rows of 128 bytes
constexpr int kMaxTypes = 248;         // cells are bytes; 0xFF marks "no edge"

struct Tc5Params {
    const int32_t *groups, *mblocks, *cols;
    const uint8_t *et;
    const __nv_bfloat16 *q, *k, *v, *ak;
    __nv_bfloat16 *o;
    float *lse, *part_o, *part_ml;
    int32_t *status;
    int n_etypes, H, max_cols_pad, tq16;  // tq16: table width (multiple of 16; 0 without embed_ak)
    float scale;
};

struct Tc5Smem {
    uint32_t q, k, v, p, ak, tab, cols, xch, bar, total;
    int tab_stride;  // in halves
};
__host__ __device__ inline Tc5Smem tc5_smem_layout(int max_cols_pad, int tq16) {
    Tc5Smem s;
    s.q = 0;
    s.k = s.q + kRows * 128;
    s.v = s.k + 2 * kTileBytes;
    s.p = s.v + 2 * kTileBytes;
    s.ak = s.p + kRows * 128;
    s.tab = s.ak + static_cast<uint32_t>((tq16 * 128 + 1023) / 1024 * 1024);
    s.tab_stride = tq16 + 2;  // an odd number of 32-bit words per row: the rows of a warp start in 32 different banks
    s.cols = s.tab + static_cast<uint32_t>((kRows * s.tab_stride * 2 + 15) / 16 * 16);
    s.xch = s.cols + static_cast<uint32_t>(max_cols_pad) * 4;  // [2][128] floats exchanged between a row's two threads
    s.bar = s.xch + 2 * kRows * 4;
    s.bar = (s.bar + 15) / 16 * 16;
    s.total = s.bar + 64 + 1024;  // barriers, TMEM slot; slack for the 1024-byte alignment of the base
    return s;
}

__device__ __forceinline__ float lds_half(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts32f(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ float lds32f(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
// Barrier among the 64 threads (two warps) that share one quarter of the rows.
__device__ __forceinline__ void pair_barrier(int quarter) {
    switch (quarter) {  // literal ids: the kernel then reserves five barriers, not all sixteen
        case 0: asm volatile("bar.sync 1, 64;\n" ::: "memory"); break;
        case 1: asm volatile("bar.sync 2, 64;\n" ::: "memory"); break;
        case 2: asm volatile("bar.sync 3, 64;\n" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 64;\n" ::: "memory"); break;
    }
}

constexpr int kThreads = 2 * kRows;  // two threads per destination row: each takes 32 of a chunk's 64 columns

template <bool kHasBias>
__global__ void __launch_bounds__(kThreads, 2) attn_forward_tc5_kernel(const Tc5Params p) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char *sm = smem_raw + (base - raw);
    const Tc5Smem L = tc5_smem_layout(p.max_cols_pad, kHasBias ? p.tq16 : 0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quarter = warp & 3, half = warp >> 2;  // TMEM lanes 32 * quarter ..., columns 32 * half ... of a chunk
    const int trow = quarter * 32 + lane;            // this thread's row of the tile
    const int H = p.H;

    const int32_t *grp = p.groups + static_cast<int64_t>(blockIdx.x) * kGroupInts;
    const int n_mb = grp[kGroupMbCount];
    if (n_mb == 0) return;
    const int ncols_pad = grp[kGroupNcolsPad];
    const int n_chunks = ncols_pad / kChunk;
    const int my_mb = trow >> 4, r16 = trow & 15;
    const bool has_mb = my_mb < n_mb;
    const int32_t *mb = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + (has_mb ? my_mb : 0)) * kMbInts;
    const int row = has_mb ? mb[kMbRowOff + r16] : -1;
    const int slot = has_mb ? mb[kMbSlotOff + r16] : -1;
    const bool use_qr = kHasBias && has_mb && mb[kMbQrSlot] >= 0;
    const uint32_t my_fine = has_mb ? static_cast<uint32_t>(mb[kMbFineMask]) : 0u;  // bit per 16 columns
    const uint32_t warp_fine = my_fine | __shfl_xor_sync(0xffffffffu, my_fine, 16);
    uint32_t group_mask = 0;  // bit per 32 columns
    bool group_table = false;  // some m-block of the group needs the relative-position table
    for (int i = 0; i < n_mb; ++i) {
        const int32_t *mbi = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + i) * kMbInts;
        group_mask |= static_cast<uint32_t>(mbi[kMbChunkMask]);
        group_table = group_table || mbi[kMbQrSlot] >= 0;
    }
    group_table = group_table && kHasBias;
    const uint8_t *et_row = p.et + (has_mb ? mb[kMbEtOff] : 0) + r16 * kTileChunk + half * 32;  // + chunk * 16 * 64
    static_assert(kTileChunk == kChunk && kMaskCols * 2 == kChunk, "plan chunking and the kernel's step agree");

    int32_t *s_cols = reinterpret_cast<int32_t *>(sm + L.cols);
    const uint32_t tab_addr = base + L.tab + static_cast<uint32_t>(trow) * L.tab_stride * 2;
    const uint32_t xch_mine = base + L.xch + (half * kRows + trow) * 4, xch_other = base + L.xch + ((half ^ 1) * kRows + trow) * 4;
    const uint32_t bar_tab = base + L.bar, bar_s = bar_tab + 8, bar_pv = bar_tab + 16;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(sm + L.bar + 32);

    const int tq16 = kHasBias ? p.tq16 : 0;
    const uint32_t tmem_cols = tq16 == 0 ? 128u : (tq16 <= 128 ? 256u : 512u);
    const uint32_t col_s = tq16 == 0 ? 0u : (tq16 <= 128 ? 128u : 256u), col_o = col_s + kChunk;

    if (tid == 0) {
        mbar_init(bar_tab, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_pv, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(base + L.bar + 32, tmem_cols);
    {
        const int32_t *gc = p.cols + grp[kGroupColOff];
        for (int i = tid; i < ncols_pad; i += kThreads) s_cols[i] = gc[i];
    }
    if (kHasBias) {
        for (int i = tid; i < tq16 * 8; i += kThreads) {
            const int r = i >> 3, piece = i & 7;
            const int type = r < p.n_etypes ? r : p.n_etypes - 1;
            cp_async16(base + L.ak + swz(r, piece), p.ak + static_cast<int64_t>(type) * kHeadDim + piece * 8);
        }
    }
    cp_async_commit();
    cp_async_wait_all();
    fence_async_smem();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tm_tab = tmem + lane_base, tm_s = tmem + lane_base + col_s + half * 32, tm_o = tmem + lane_base + col_o + half * 32;

    const float sl2 = p.scale * kLog2e;
    const uint32_t none_idx = kHasBias ? static_cast<uint32_t>(tq16) : 1u;
    const uint32_t none4 = none_idx * 0x01010101u;
    constexpr uint32_t kIdescS = instr_desc(kRows, kChunk, 0, 0);     // S = Q K^T
    constexpr uint32_t kIdescPV = instr_desc(kRows, kHeadDim, 0, 1);  // O += P V, V MN-major
    const uint32_t idesc_tab = instr_desc(kRows, tq16 > 0 ? tq16 : 16, 0, 0);

    auto first_chunk_from = [&](int c) {
        while (c < n_chunks && !((group_mask >> (2 * c)) & 3u)) ++c;
        return c;
    };
    // K and V rows of head h for chunk c -> buffer b (2 + 2 pieces per thread)
    auto issue_kv = [&](int h, int c, int b) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int id = i * kThreads + tid;
            const int r = id >> 3, piece = id & 7;
            const int64_t off = (static_cast<int64_t>(s_cols[c * kChunk + r]) * H + h) * kHeadDim + piece * 8;
            const uint32_t dst = static_cast<uint32_t>(b) * kTileBytes + swz(r, piece);
            cp_async16(base + L.k + dst, p.k + off);
            cp_async16(base + L.v + dst, p.v + off);
        }
    };

    uint32_t n_tab_done = 0, n_s_done = 0, n_pv_done = 0;  // completions already waited for, per barrier
    bool ok = true;
    const int c_first = first_chunk_from(0);

    // Q of head h (4 pieces of the row per thread) and the K and V rows of its first chunk -> buffer b
    auto issue_head = [&](int h, int b) {
        const __nv_bfloat16 *src = p.q + (static_cast<int64_t>(row < 0 ? 0 : row) * H + h) * kHeadDim;
#pragma unroll
        for (int i = 0; i < 4; ++i) cp_async16(base + L.q + swz(trow, half * 4 + i), src + (half * 4 + i) * 8);
        if (c_first < n_chunks) issue_kv(h, c_first, b);
    };
    // the head's first MMAs: the table Q embed_ak^T and S of the first chunk (one thread)
    auto issue_head_mma = [&](int b) {
        if (group_table) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                mma_ss(tmem, desc_kmajor(base + L.q, ks), desc_kmajor(base + L.ak, ks), idesc_tab, ks > 0);
            mma_commit(bar_tab);
        }
        if (c_first < n_chunks) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                mma_ss(tmem + col_s, desc_kmajor(base + L.q, ks), desc_kmajor(base + L.k + b * kTileBytes, ks), kIdescS, ks > 0);
            mma_commit(bar_s);
        }
    };
    if (!group_table) {  // no table in this group: every row looks up {0, ..., -inf} (entry 0 and the last one)
        if (half == 0) {
            asm volatile("st.shared.u16 [%0], %1;\n" ::"r"(tab_addr), "h"(static_cast<unsigned short>(0)) : "memory");
            asm volatile("st.shared.u16 [%0], %1;\n" ::"r"(tab_addr + none_idx * 2), "h"(static_cast<unsigned short>(0xFC00)) : "memory");
        }
    }

    int buf = 0;            // K/V buffer of the chunk being worked on; carried from head to head
    bool issued_ahead = false;  // the previous head's last step already loaded this head's Q and first chunk and issued its first MMAs
    for (int h = 0; h < H; ++h) {
        if (!issued_ahead) {
            issue_head(h, buf);
            cp_async_commit();
            cp_async_wait_all();
            fence_async_smem();
            fence_before_sync();
            if (__syncthreads_or(!ok)) break;
            if (tid == 0) {
                fence_after_sync();
                issue_head_mma(buf);
            }
        }
        issued_ahead = false;
        // ---- the head's table row: scale * log2(e) * <q[row], embed_ak[type]> as fp16 (each of the row's two
        // threads converts half of it); rows whose edges share one type keep zeros: the term is then a
        // per-row constant that cancels in the softmax and is added to lse
        float bias_row = 0.f;
        if (group_table) {
            ok = ok && mbar_wait(bar_tab, n_tab_done & 1u);
            ++n_tab_done;
            fence_after_sync();
            const int n_units = tq16 / 16, u_split = (n_units + 1) / 2;
            for (int u = half ? u_split : 0; u < (half ? n_units : u_split); ++u) {
                uint32_t t[16];
                tmem_ld16(tm_tab + u * 16, t);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    const float a = use_qr ? __uint_as_float(t[i]) * sl2 : 0.f;
                    const float b = use_qr ? __uint_as_float(t[i + 1]) * sl2 : 0.f;
                    __half2 hv = __floats2half2_rn(a, b);
                    asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(tab_addr + (u * 16 + i) * 2), "r"(*reinterpret_cast<uint32_t *>(&hv)) : "memory");
                }
            }
            if (half) asm volatile("st.shared.u16 [%0], %1;\n" ::"r"(tab_addr + tq16 * 2), "h"(static_cast<unsigned short>(0xFC00)) : "memory");
        }
        if (kHasBias && !use_qr && row >= 0 && half == 0) {
            // a row whose edges share one type: <q[row], embed_ak[type]> from the staged Q tile and embed_ak rows
            int type = mb[kMbRowEtOff + r16];
            type = type < 0 ? 0 : (type < p.n_etypes ? type : p.n_etypes - 1);
            float sum = 0.f;
#pragma unroll
            for (int piece = 0; piece < 8; ++piece) {
                const uint4 x = *reinterpret_cast<const uint4 *>(sm + L.q + swz(trow, piece));
                const uint4 y = type < tq16 ? *reinterpret_cast<const uint4 *>(sm + L.ak + swz(type, piece))
                                            : __ldg(reinterpret_cast<const uint4 *>(p.ak + static_cast<int64_t>(type) * kHeadDim) + piece);
                const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xw[u]));
                    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&yw[u]));
                    sum = fmaf(a.x, b.x, fmaf(a.y, b.y, sum));
                }
            }
            bias_row = sum * sl2;
        }
        pair_barrier(quarter);  // the row's other thread wrote the other half of the table row

        float m_run = -INFINITY, l_run = 0.f;  // m_run is shared by the row's two threads, l_run is this thread's part
        int n_pv = 0;
        int c = c_first;
        bool aborted = false;
        while (c < n_chunks) {
            const int nc = first_chunk_from(c + 1);
            // this thread's 32 cells of the chunk (edge types, 0xFF = no edge), fetched while S is on its way
            uint32_t cells[8];
            if (has_mb) {
                const uint4 *cp = reinterpret_cast<const uint4 *>(et_row + c * (kTileRows * kTileChunk));
                const uint4 x = __ldg(cp), y = __ldg(cp + 1);
                cells[0] = x.x; cells[1] = x.y; cells[2] = x.z; cells[3] = x.w;
                cells[4] = y.x; cells[5] = y.y; cells[6] = y.z; cells[7] = y.w;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) cells[j] = 0xFFFFFFFFu;
            }
            if (n_pv > 0) {  // the previous chunk's O += P V is done: P, the other K/V buffer and O are free
                ok = ok && mbar_wait(bar_pv, n_pv_done & 1u);
                ++n_pv_done;
            }
            if (nc < n_chunks) issue_kv(h, nc, buf ^ 1);
            cp_async_commit();
            ok = ok && mbar_wait(bar_s, n_s_done & 1u);
            ++n_s_done;
            fence_after_sync();
            // last step of the head: S, the last MMA that reads Q, is done, so the next head's Q and first chunk
            // travel while this step's softmax runs
            const bool ahead = nc >= n_chunks && h + 1 < H;
            if (ahead) {
                issue_head(h + 1, buf ^ 1);
                cp_async_commit();
            }

            // scores of the two 16-column units of this thread, in the log2 domain, mask applied
            const uint32_t act = (warp_fine >> (4 * c + 2 * half)) & 3u;  // uniform over the warp
            float x[32];
            float cmax = -INFINITY;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if ((act >> u) & 1u) {
                    uint32_t s[16];
                    tmem_ld16(tm_s + u * 16, s);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t w = cells[4 * u + j];
                        const uint32_t none = __vcmpeq4(w, 0xFFFFFFFFu);
                        const uint32_t idx4 = ((use_qr ? w : 0u) & ~none) | (none4 & none);
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            const uint32_t idx2 = (idx4 >> (8 * b) << 1) & 0x1FEu;  // byte offset of the table entry
                            const float v = fmaf(__uint_as_float(s[4 * j + b]), sl2, lds_half(tab_addr + idx2));
                            x[16 * u + 4 * j + b] = v;
                            cmax = fmaxf(cmax, v);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) x[16 * u + i] = -INFINITY;
                }
            }
            // one maximum per row: exchange with the row's other thread; it moves (and the sums are rescaled)
            // only when it grows by more than 8
            sts32f(xch_mine, cmax);
            pair_barrier(quarter);
            cmax = fmaxf(cmax, lds32f(xch_other));
            pair_barrier(quarter);  // both have read before the next chunk's exchange overwrites
            const bool need = cmax > m_run + 8.f || (m_run == -INFINITY && cmax > -INFINITY);
            if (__any_sync(0xffffffffu, need)) {
                const float f = need ? ex2(m_run - cmax) : 1.f;
                if (need) {
                    m_run = cmax;
                    l_run *= f;
                }
                if (n_pv > 0) {  // this thread rescales its 32 of the row's 64 accumulator columns
                    uint32_t o[32];
                    tmem_ld32(tm_o, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                    tmem_st32(tm_o, o);
                    tmem_st_wait();
                }
            }
            const float ms = m_run == -INFINITY ? 0.f : m_run;
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float e0 = ex2(x[i] - ms), e1 = ex2(x[i + 1] - ms);
                l_run += e0 + e1;
                __nv_bfloat162 v2 = __floats2bfloat162_rn(e0, e1);
                pk[i >> 1] = *reinterpret_cast<uint32_t *>(&v2);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                sts128(base + L.p + swz(trow, half * 4 + j), pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            cp_async_wait_all();  // the next chunk's K and V have landed
            fence_async_smem();
            fence_before_sync();
            if (__syncthreads_or(!ok)) {
                aborted = true;
                break;
            }
            if (tid == 0) {
                fence_after_sync();
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_ss(tmem + col_o, desc_kmajor(base + L.p, ks), desc_mnmajor(base + L.v + buf * kTileBytes, ks), kIdescPV,
                           (n_pv > 0 || ks > 0) ? 1u : 0u);
                mma_commit(bar_pv);
                if (nc < n_chunks) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        mma_ss(tmem + col_s, desc_kmajor(base + L.q, ks), desc_kmajor(base + L.k + (buf ^ 1) * kTileBytes, ks),
                               kIdescS, ks > 0);
                    mma_commit(bar_s);
                } else if (ahead) {
                    issue_head_mma(buf ^ 1);
                }
            }
            issued_ahead = ahead;
            ++n_pv;
            c = nc;
            buf ^= 1;
        }
        if (aborted) break;

        // ---- the head's result: each of the row's two threads finishes 32 of the 64 output columns
        sts32f(xch_mine, l_run);
        float acc[32];
        if (n_pv > 0) {
            ok = ok && mbar_wait(bar_pv, n_pv_done & 1u);
            ++n_pv_done;
            fence_after_sync();
            uint32_t o[32];
            tmem_ld32(tm_o, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(o[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.f;
        }
        pair_barrier(quarter);
        const float l_row = l_run + lds32f(xch_other);
        pair_barrier(quarter);
        if (row >= 0 && ok) {
            const float m_out = m_run + bias_row;  // bias_row is known to the first of the two threads, which writes lse
            if (slot < 0) {
                const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
                uint4 *dst = reinterpret_cast<uint4 *>(p.o + (static_cast<int64_t>(row) * H + h) * kHeadDim + half * 32);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t w[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        __nv_bfloat162 v2 = __floats2bfloat162_rn(acc[8 * j + 2 * u] * inv, acc[8 * j + 2 * u + 1] * inv);
                        w[u] = *reinterpret_cast<uint32_t *>(&v2);
                    }
                    dst[j] = make_uint4(w[0], w[1], w[2], w[3]);
                }
                if (half == 0)
                    p.lse[static_cast<int64_t>(row) * H + h] = l_row > 0.f ? (m_out + log2f(l_row)) * kLn2 : -INFINITY;
            } else {
                float4 *dst = reinterpret_cast<float4 *>(p.part_o + (static_cast<int64_t>(slot) * H + h) * kHeadDim + half * 32);
#pragma unroll
                for (int j = 0; j < 8; ++j) dst[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
                if (half == 0)
                    *reinterpret_cast<float2 *>(p.part_ml + (static_cast<int64_t>(slot) * H + h) * 2) = make_float2(m_out, l_row);
            }
        }
    }
    if (!ok) atomicExch(p.status, 1);
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_free(tmem, tmem_cols);
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" size_t bpt_attn_forward_tc5_smem_bytes(int max_cols_pad, int t_max) {
    if (max_cols_pad < 0 || t_max < 0) return 0;
    return tc5_smem_layout(max_cols_pad, (t_max + 15) / 16 * 16).total;
}

extern "C" size_t bpt_attn_forward_tc5_workspace_bytes(int64_t n_slots, int h) {
    if (n_slots < 0 || h < 1) return 0;
    const size_t s = static_cast<size_t>(n_slots);
    return 256 + align_up(s * h * kHeadDim * 4, 256) + align_up(s * h * 2 * 4, 256) + 512;
}

extern "C" int bpt_attn_forward_tc5(const bpt_tile_plan_t *tiles, int64_t n_nodes, int n_etypes, const void *q,
                                    const void *k, const void *v, const void *ak, double scale, void *o, float *lse,
                                    int h, int d, int dtype, void *workspace, size_t workspace_bytes,
                                    bpt_stream_t stream_) {
    BPT_CHECK_ARG(tiles != nullptr && n_nodes >= 0 && n_etypes >= 1 && h >= 1, "attn_forward_tc5: bad arguments");
    if (d != kHeadDim || dtype != BPT_BF16)
        return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc5: only bf16 with head dim 64 (got dtype %d, d %d)", dtype, d);
    BPT_CHECK_ARG(tiles->n_groups >= 0 && tiles->n_groups < (int64_t(1) << 31) && tiles->n_split >= 0 && tiles->n_slots >= 0,
                  "attn_forward_tc5: bad tile plan sizes");
    BPT_CHECK_ARG(tiles->n_row_items == 0, "attn_forward_tc5: the tile plan must not hold CUDA-core row items");
    if (tiles->n_groups == 0) return BPT_OK;
    BPT_CHECK_ARG(tiles->groups && tiles->mblocks && q && k && v && o && lse, "attn_forward_tc5: null array");
    BPT_CHECK_ARG(tiles->max_cols_pad == 0 || (tiles->cols && tiles->et), "attn_forward_tc5: null tile plan arrays");
    BPT_CHECK_ARG(tiles->max_cols_pad % kTileChunk == 0 && tiles->max_cols_pad <= 512 && tiles->t_max % 8 == 0,
                  "attn_forward_tc5: bad tile plan sizes (groups of at most 512 columns)");
    if (tiles->et_bytes != 1 || (ak != nullptr && tiles->t_max > kMaxTypes))
        return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc5: needs 8-bit cells and at most %d edge types", kMaxTypes);
    BPT_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                    reinterpret_cast<uintptr_t>(ak) | reinterpret_cast<uintptr_t>(o)) & 15) == 0,
                  "attn_forward_tc5: tensors must be 16-byte aligned");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    int32_t *status = ws.take<int32_t>(4);
    float *part_o = ws.take<float>(static_cast<size_t>(tiles->n_slots) * h * kHeadDim);
    float *part_ml = ws.take<float>(static_cast<size_t>(tiles->n_slots) * h * 2);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_forward_tc5: workspace of %zu bytes is too small", workspace_bytes);

    Tc5Params p{};
    p.groups = tiles->groups; p.mblocks = tiles->mblocks; p.cols = tiles->cols;
    p.et = static_cast<const uint8_t *>(tiles->et);
    p.q = static_cast<const __nv_bfloat16 *>(q); p.k = static_cast<const __nv_bfloat16 *>(k);
    p.v = static_cast<const __nv_bfloat16 *>(v); p.ak = static_cast<const __nv_bfloat16 *>(ak);
    p.o = static_cast<__nv_bfloat16 *>(o);
    p.lse = lse; p.part_o = part_o; p.part_ml = part_ml; p.status = status;
    p.n_etypes = n_etypes; p.H = h; p.max_cols_pad = tiles->max_cols_pad;
    const bool bias = ak != nullptr;
    // at least one table column group even when no m-block needs the table, so that the layout is one
    p.tq16 = bias ? ((tiles->t_max > 0 ? tiles->t_max : 8) + 15) / 16 * 16 : 0;
    p.scale = static_cast<float>(scale);
    const size_t smem = tc5_smem_layout(p.max_cols_pad, p.tq16).total;
    if (smem > 227 * 1024)
        return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc5: tile plan needs %zu bytes of shared memory", smem);
    if (bias) {
        BPT_CUDA(cudaFuncSetAttribute(attn_forward_tc5_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
        attn_forward_tc5_kernel<true><<<static_cast<unsigned>(tiles->n_groups), kThreads, smem, stream>>>(p);
    } else {
        BPT_CUDA(cudaFuncSetAttribute(attn_forward_tc5_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
        attn_forward_tc5_kernel<false><<<static_cast<unsigned>(tiles->n_groups), kThreads, smem, stream>>>(p);
    }
    BPT_LAUNCH_CHECK();
    if (tiles->n_split > 0) {
        const Geometry g{h, kHeadDim};
        attn_forward_merge_kernel<__nv_bfloat16><<<static_cast<unsigned>(tiles->n_split), merge_threads(h, kHeadDim),
                                                   merge_smem_bytes(h), stream>>>(
            reinterpret_cast<const int4 *>(tiles->split_rows), static_cast<int>(tiles->n_split), part_o, part_ml,
            static_cast<__nv_bfloat16 *>(o), lse, g);
        BPT_LAUNCH_CHECK();
    }
    return BPT_OK;
}

// 0 = every bounded wait of the last bpt_attn_forward_tc5 call on this workspace completed; the call
// clears nothing itself, so the caller zeroes the first 16 bytes of a fresh workspace once.  Waits for the stream.
extern "C" int bpt_attn_forward_tc5_status(const void *workspace, int32_t *status_host, bpt_stream_t stream_) {
    BPT_CHECK_ARG(workspace && status_host, "attn_forward_tc5_status: null argument");
    cudaStream_t stream = as_stream(stream_);
    BPT_CUDA(cudaMemcpyAsync(status_host, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    BPT_CUDA(cudaStreamSynchronize(stream));
    return BPT_OK;
}
