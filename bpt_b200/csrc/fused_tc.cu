// Fused graph attention forward on tensor cores (bf16 storage, fp32 accumulation, head dim 64).
//
// One thread block per (group, head) of the tile plan (tile_plan.cuh): the group's K and V
// rows are gathered ONCE into shared memory, 64 columns per pipeline stage (cp.async,
// kStages deep, 16-byte pieces XOR-swizzled against bank conflicts), together with each
// m-block's 16x64 edge-type tile.  Every warp owns one m-block (<=16 destination rows) and,
// per stage in which it has edges,
//   1. S = Q K^T on tensor cores (ldmatrix B fragments from the K stage),
//   2. adds the relative-position term by looking up QR[row][etype] (QR = Q embed_ak^T, computed
//      on tensor cores once per m-block and head and parked in shared memory) and masks cells
//      without an edge; m-blocks whose rows each have a single edge type skip this: the term is
//      then a per-row constant that cancels in the softmax and is added to lse at the end,
//   3. online softmax in registers, P packed to bf16 A fragments in place,
//   4. O += P V (ldmatrix.trans B fragments from the V stage).
// Scores never leave the SM.  Rows wholly inside one m-block are written as final O / lse; rows
// spread over several m-blocks write (m, l, O) partials that a merge kernel combines in slot
// order, so results are bitwise reproducible.
#include "fused_common.cuh"
#include "plan.cuh"
#include "tile_plan.cuh"

namespace bpt {
namespace {

constexpr int kHeadDim = 64;
constexpr int kStages = 3;
constexpr int kRowBytes = kHeadDim * 2;                  // one head row of K or V: 128 B = 8 pieces of 16 B
constexpr int kKvStageBytes = kTileChunk * kRowBytes;    // 8 KB per matrix per stage

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
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
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// Standard mma A-fragment words of one 64-element row for lane column t: w[2s] = elements
// (16s + 2t, +1), w[2s+1] = (16s + 8 + 2t, +1).
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

// Bytes of one m-block's edge-type tile in a stage: 16 rows of 64 cells + 16 bytes of padding
// per row so that the 8 row groups of a warp hit different banks.
template <typename ET>
__host__ __device__ constexpr int et_row_bytes() { return kTileChunk * static_cast<int>(sizeof(ET)) + 16; }

struct TcParams {
    const int32_t *groups, *mblocks, *cols;
    const void *et;
    const __nv_bfloat16 *q, *k, *v, *ak;
    __nv_bfloat16 *o;
    float *lse, *part_o, *part_ml;
    int n_etypes, H, max_cols_pad, t_max, max_qr_slots;
    float scale;
};

template <typename ET, bool kHasBias>
__global__ void __launch_bounds__(kMaxMBlocks * 32, 2)
attn_forward_group_kernel(const TcParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int n_warps = blockDim.x >> 5;
    constexpr int kEtRow = et_row_bytes<ET>();
    const int et_tile_bytes = kTileRows * kEtRow;
    const int stage_bytes = 2 * kKvStageBytes + n_warps * et_tile_bytes;
    // layout: stages | column ids | QR tables (fp16)
    int32_t *s_cols = reinterpret_cast<int32_t *>(smem + kStages * stage_bytes);
    __half *s_qr_all = reinterpret_cast<__half *>(s_cols + p.max_cols_pad);
    const int qr_stride = p.t_max + 8;
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));

    const int32_t *grp = p.groups + static_cast<int64_t>(blockIdx.x) * kGroupInts;
    const int ncols_pad = grp[kGroupNcolsPad];
    const int n_chunks = ncols_pad / kTileChunk;
    const int n_mb = grp[kGroupMbCount];
    const int h = blockIdx.y, H = p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const bool has_mb = warp < n_mb;
    const int32_t *mb = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + (has_mb ? warp : 0)) * kMbInts;

    {
        const int32_t *gc = p.cols + grp[kGroupColOff];
        for (int i = threadIdx.x; i < ncols_pad; i += blockDim.x) s_cols[i] = gc[i];
    }
    __syncthreads();

    // ---- stage loader: K and V rows of 64 columns, and every m-block's edge-type tile ----
    const ET *et_base = static_cast<const ET *>(p.et);
    auto issue_stage = [&](int chunk) {
        const uint32_t st = smem_base + (chunk % kStages) * stage_bytes;
        for (int id = threadIdx.x; id < kTileChunk * 8; id += blockDim.x) {
            const int r = id >> 3, piece = id & 7;
            const int64_t node = s_cols[chunk * kTileChunk + r];
            const int64_t off = (node * H + h) * kHeadDim + piece * 8;
            const uint32_t dst = r * kRowBytes + ((piece ^ (r & 7)) << 4);
            cp_async16(st + dst, p.k + off);
            cp_async16(st + kKvStageBytes + dst, p.v + off);
        }
        constexpr int kPiecesPerRow = kTileChunk * static_cast<int>(sizeof(ET)) / 16;
        const int pieces = n_mb * kTileRows * kPiecesPerRow;
        for (int id = threadIdx.x; id < pieces; id += blockDim.x) {
            const int m = id / (kTileRows * kPiecesPerRow), rem = id % (kTileRows * kPiecesPerRow);
            const int r = rem / kPiecesPerRow, piece = rem % kPiecesPerRow;
            const int32_t *mrec = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + m) * kMbInts;
            const ET *src = et_base + mrec[kMbEtOff] + (static_cast<int64_t>(chunk) * kTileRows + r) * kTileChunk;
            cp_async16(st + 2 * kKvStageBytes + m * et_tile_bytes + r * kEtRow + piece * 16,
                       reinterpret_cast<const unsigned char *>(src) + piece * 16);
        }
    };

#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (s < n_chunks) issue_stage(s);
        cp_async_commit();
    }

    // ---- per-warp state ----
    const int row_lo = has_mb ? mb[kMbRowOff + g] : -1, row_hi = has_mb ? mb[kMbRowOff + g + 8] : -1;
    const uint32_t chunk_mask = has_mb ? static_cast<uint32_t>(mb[kMbChunkMask]) : 0u;
    const int qr_slot = has_mb ? mb[kMbQrSlot] : -1;
    const bool use_qr = kHasBias && qr_slot >= 0;
    uint32_t q_lo[8], q_hi[8];
    load_a_row(p.q + (static_cast<int64_t>(row_lo < 0 ? 0 : row_lo) * H + h) * kHeadDim, t, q_lo);
    load_a_row(p.q + (static_cast<int64_t>(row_hi < 0 ? 0 : row_hi) * H + h) * kHeadDim, t, q_hi);
    const float sl2 = p.scale * kLog2e;
    __half *s_qr = s_qr_all + static_cast<int64_t>(qr_slot < 0 ? 0 : qr_slot) * kTileRows * qr_stride;
    float bias_lo = 0.f, bias_hi = 0.f;  // per-row constant of m-blocks that skip the table (log2 domain)

    if (kHasBias && has_mb) {
        if (use_qr) {
            // QR[row][type] = <q[row], ak[type]> for the types that occur in this m-block
            const int tq = mb[kMbTq];
            for (int nt = 0; nt < tq; nt += 8) {
                int type = nt + g;
                type = type < p.n_etypes ? type : p.n_etypes - 1;
                uint32_t b[8];
                load_a_row(p.ak + static_cast<int64_t>(type) * kHeadDim, t, b);  // B fragment words have the A layout
                float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    mma_bf16(c, q_lo[2 * s], q_hi[2 * s], q_lo[2 * s + 1], q_hi[2 * s + 1], b[2 * s], b[2 * s + 1]);
                *reinterpret_cast<__half2 *>(s_qr + g * qr_stride + nt + 2 * t) = __floats2half2_rn(c[0], c[1]);
                *reinterpret_cast<__half2 *>(s_qr + (g + 8) * qr_stride + nt + 2 * t) = __floats2half2_rn(c[2], c[3]);
            }
            __syncwarp();
        } else {
            // every row has one edge type: <q[row], ak[type]> shifts all its scores alike
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
                (half ? bias_hi : bias_lo) = sum * sl2;
            }
        }
    }

    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc[i][0] = 0.f; acc[i][1] = 0.f; acc[i][2] = 0.f; acc[i][3] = 0.f; }

    for (int c = 0; c < n_chunks; ++c) {
        cp_async_wait<kStages - 2>();
        __syncthreads();  // stage c has landed for everyone; stage c-1 is free for everyone
        if (c + kStages - 1 < n_chunks) issue_stage(c + kStages - 1);
        cp_async_commit();
        if (!((chunk_mask >> c) & 1u)) continue;

        const uint32_t st = smem_base + (c % kStages) * stage_bytes;
        const unsigned char *st_et = smem + (c % kStages) * stage_bytes + 2 * kKvStageBytes + warp * et_tile_bytes;
        // S = Q K^T for 8 column groups of 8
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            s[nt][0] = 0.f; s[nt][1] = 0.f; s[nt][2] = 0.f; s[nt][3] = 0.f;
            const int r = nt * 8 + (lane & 7);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t b[4];
                const int piece = 4 * j + (lane >> 3);
                ldmatrix_x4(b, st + r * kRowBytes + ((piece ^ (r & 7)) << 4));
                mma_bf16(s[nt], q_lo[4 * j], q_hi[4 * j], q_lo[4 * j + 1], q_hi[4 * j + 1], b[0], b[1]);
                mma_bf16(s[nt], q_lo[4 * j + 2], q_hi[4 * j + 2], q_lo[4 * j + 3], q_hi[4 * j + 3], b[2], b[3]);
            }
        }
        // relative-position term, mask, scale (log2 domain)
        float cmax_lo = -INFINITY, cmax_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            uint32_t e[4];
            if (sizeof(ET) == 1) {
                const uint32_t a = *reinterpret_cast<const uint16_t *>(st_et + g * kEtRow + nt * 8 + 2 * t);
                const uint32_t b = *reinterpret_cast<const uint16_t *>(st_et + (g + 8) * kEtRow + nt * 8 + 2 * t);
                e[0] = a & 0xffu; e[1] = a >> 8; e[2] = b & 0xffu; e[3] = b >> 8;
            } else {
                const uint32_t a = *reinterpret_cast<const uint32_t *>(st_et + g * kEtRow + (nt * 8 + 2 * t) * 2);
                const uint32_t b = *reinterpret_cast<const uint32_t *>(st_et + (g + 8) * kEtRow + (nt * 8 + 2 * t) * 2);
                e[0] = a & 0xffffu; e[1] = a >> 16; e[2] = b & 0xffffu; e[3] = b >> 16;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (e[i] == EtTraits<ET>::kNone) {
                    s[nt][i] = -INFINITY;
                } else {
                    float x = s[nt][i];
                    if (use_qr) x += __half2float(s_qr[(i < 2 ? g : g + 8) * qr_stride + e[i]]);
                    s[nt][i] = x * sl2;
                }
            }
            cmax_lo = fmaxf(cmax_lo, fmaxf(s[nt][0], s[nt][1]));
            cmax_hi = fmaxf(cmax_hi, fmaxf(s[nt][2], s[nt][3]));
        }
        cmax_lo = fmaxf(cmax_lo, __shfl_xor_sync(0xffffffffu, cmax_lo, 1));
        cmax_lo = fmaxf(cmax_lo, __shfl_xor_sync(0xffffffffu, cmax_lo, 2));
        cmax_hi = fmaxf(cmax_hi, __shfl_xor_sync(0xffffffffu, cmax_hi, 1));
        cmax_hi = fmaxf(cmax_hi, __shfl_xor_sync(0xffffffffu, cmax_hi, 2));
        const float mn_lo = fmaxf(m_lo, cmax_lo), mn_hi = fmaxf(m_hi, cmax_hi);
        const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float corr_lo = exp2f(m_lo - ms_lo), corr_hi = exp2f(m_hi - ms_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        l_lo *= corr_lo;
        l_hi *= corr_hi;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc[i][0] *= corr_lo; acc[i][1] *= corr_lo;
            acc[i][2] *= corr_hi; acc[i][3] *= corr_hi;
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            s[nt][0] = exp2f(s[nt][0] - ms_lo);
            s[nt][1] = exp2f(s[nt][1] - ms_lo);
            s[nt][2] = exp2f(s[nt][2] - ms_hi);
            s[nt][3] = exp2f(s[nt][3] - ms_hi);
            l_lo += s[nt][0] + s[nt][1];
            l_hi += s[nt][2] + s[nt][3];
        }
        // O += P V
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint32_t a0 = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
            const uint32_t a1 = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            const uint32_t a2 = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            const uint32_t a3 = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
            const int r = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
            for (int dn = 0; dn < 8; dn += 2) {
                const int piece = dn + (lane >> 4);
                uint32_t b[4];
                ldmatrix_x4_trans(b, st + kKvStageBytes + r * kRowBytes + ((piece ^ (r & 7)) << 4));
                mma_bf16(acc[dn], a0, a1, a2, a3, b[0], b[1]);
                mma_bf16(acc[dn + 1], a0, a1, a2, a3, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    if (!has_mb) return;

    // row sums live per lane: finish them across the quad
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half ? row_hi : row_lo;
        if (row < 0) continue;
        const int slot = mb[kMbSlotOff + g + 8 * half];
        const float m = (half ? m_hi : m_lo) + (half ? bias_hi : bias_lo);
        const float l = half ? l_hi : l_lo;
        if (slot < 0) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16 *dst = p.o + (static_cast<int64_t>(row) * H + h) * kHeadDim + 2 * t;
#pragma unroll
            for (int dn = 0; dn < 8; ++dn)
                *reinterpret_cast<uint32_t *>(dst + dn * 8) = pack_bf16(acc[dn][2 * half] * inv, acc[dn][2 * half + 1] * inv);
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
}

template <typename ET>
size_t tc_smem_bytes(int n_warps, int max_cols_pad, int t_max, int max_qr_slots) {
    return static_cast<size_t>(kStages) * (2 * kKvStageBytes + n_warps * kTileRows * et_row_bytes<ET>()) +
           static_cast<size_t>(max_cols_pad) * 4 + static_cast<size_t>(max_qr_slots) * kTileRows * (t_max + 8) * 2;
}

template <typename ET, bool kHasBias>
int launch_group_kernel(const TcParams &p, int64_t n_groups, int n_warps, size_t smem, cudaStream_t stream) {
    BPT_CUDA(cudaFuncSetAttribute(attn_forward_group_kernel<ET, kHasBias>,
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    const dim3 grid(static_cast<unsigned>(n_groups), static_cast<unsigned>(p.H));
    attn_forward_group_kernel<ET, kHasBias><<<grid, n_warps * 32, smem, stream>>>(p);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

}  // namespace
}  // namespace bpt

using namespace bpt;

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
                                   size_t workspace_bytes, bpt_stream_t stream_) {
    BPT_CHECK_ARG(n_groups >= 0 && n_split >= 0 && n_slots >= 0 && n_row_items >= 0 && h >= 1,
                  "attn_forward_tc: bad sizes");
    if (d != kHeadDim || dtype != BPT_BF16)
        return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc: only bf16 with head dim 64 (got dtype %d, d %d)", dtype, d);
    if (n_groups == 0 && n_row_items == 0) return BPT_OK;
    BPT_CHECK_ARG(q && k && v && o && lse, "attn_forward_tc: null tensor");
    BPT_CHECK_ARG(n_groups == 0 || (groups && mblocks), "attn_forward_tc: null plan arrays");
    BPT_CHECK_ARG(max_cols_pad == 0 || (cols && et), "attn_forward_tc: null plan arrays");
    BPT_CHECK_ARG(et_bytes == 1 || et_bytes == 2, "attn_forward_tc: et_bytes must be 1 or 2");
    BPT_CHECK_ARG(max_cols_pad % kTileChunk == 0 && max_cols_pad <= kMaxChunks * kTileChunk && t_max % 8 == 0 &&
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
                                               h, d, stream))
            return rc;
    }
    if (n_groups > 0) {
        const bool bias = ak != nullptr;
        TcParams p;
        p.groups = groups; p.mblocks = mblocks; p.cols = cols; p.et = et;
        p.q = static_cast<const __nv_bfloat16 *>(q); p.k = static_cast<const __nv_bfloat16 *>(k);
        p.v = static_cast<const __nv_bfloat16 *>(v); p.ak = static_cast<const __nv_bfloat16 *>(ak);
        p.o = static_cast<__nv_bfloat16 *>(o);
        p.lse = lse; p.part_o = part_o; p.part_ml = part_ml;
        p.n_etypes = n_etypes; p.H = h; p.max_cols_pad = max_cols_pad;
        p.t_max = bias ? t_max : 0;
        p.max_qr_slots = bias ? max_qr_slots : 0;
        p.scale = static_cast<float>(scale);
        const int n_warps = max_mblocks < 1 ? 1 : max_mblocks;
        const size_t smem = et_bytes == 1 ? tc_smem_bytes<uint8_t>(n_warps, max_cols_pad, p.t_max, p.max_qr_slots)
                                          : tc_smem_bytes<uint16_t>(n_warps, max_cols_pad, p.t_max, p.max_qr_slots);
        if (smem > 227 * 1024)
            return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc: tile plan needs %zu bytes of shared memory", smem);
        int rc;
        if (et_bytes == 1)
            rc = bias ? launch_group_kernel<uint8_t, true>(p, n_groups, n_warps, smem, stream)
                      : launch_group_kernel<uint8_t, false>(p, n_groups, n_warps, smem, stream);
        else
            rc = bias ? launch_group_kernel<uint16_t, true>(p, n_groups, n_warps, smem, stream)
                      : launch_group_kernel<uint16_t, false>(p, n_groups, n_warps, smem, stream);
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
