// Fused graph attention forward on tensor cores (bf16 storage, fp32 accumulation, head dim 64).
//
// One block per tile of the tile plan (<=16 destination rows x an explicit list of source
// columns), one warp per head.  Per 64-column step a warp
//   1. gathers the K rows of the step's columns straight into mma B fragments (each lane
//      loads two 16-byte pieces of a row; the head dimension is permuted identically for Q, K
//      and embed_ak, which a dot product does not notice),
//   2. S = Q K^T on tensor cores, adds the relative-position term by looking up
//      QR[row][etype] (QR = Q embed_ak^T, also computed on tensor cores once per tile and head
//      and parked in shared memory), masks cells without an edge,
//   3. online softmax in registers, P packed to bf16 A fragments in place,
//   4. O += P V with V staged through swizzled shared memory (cp.async + ldmatrix.trans).
// Scores never leave the SM.  Rows wholly inside one tile are written as final O / lse; rows
// spread over several tiles write (m, l, O) partials that a merge kernel combines in slot
// order, so results are bitwise reproducible.
#include "fused_common.cuh"
#include "plan.cuh"
#include "tile_plan.cuh"

namespace bpt {
namespace {

constexpr int kHeadDim = 64;
constexpr int kWarps = 8;
constexpr int kEtPad = 8;                                  // uint16 padding per etype-tile row (bank spread)
constexpr int kVBytes = kTileChunk * kHeadDim * 2;         // one warp's V stage: 64 rows x 128 B

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
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// A lane's share of one 64-element head row for the QK^T-type products: the two 16-byte pieces
// at elements [8t, 8t+8) and [32+8t, 32+8t+8), t = lane % 4.  Word w[2s], w[2s+1] feed k-step s.
__device__ __forceinline__ void load_row_frag(const __nv_bfloat16 *__restrict__ row, int t, uint32_t (&w)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4 *>(row + 8 * t));
    const uint4 b = __ldg(reinterpret_cast<const uint4 *>(row + 32 + 8 * t));
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}

template <bool kHasBias>
__global__ void __launch_bounds__(kWarps * 32, 2)
attn_forward_tc_kernel(const int32_t *__restrict__ tiles, const int32_t *__restrict__ cols,
                       const uint16_t *__restrict__ et, const __nv_bfloat16 *__restrict__ q,
                       const __nv_bfloat16 *__restrict__ k, const __nv_bfloat16 *__restrict__ v,
                       const __nv_bfloat16 *__restrict__ ak, int n_etypes, float scale,
                       __nv_bfloat16 *__restrict__ o, float *__restrict__ lse, float *__restrict__ part_o,
                       float *__restrict__ part_ml, int H, int max_cols_pad, int t_max) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: V stages (8 x 8 KB, 128-byte aligned) | column ids | etype tile | QR per warp (fp16)
    unsigned char *s_v_all = smem;
    int32_t *s_cols = reinterpret_cast<int32_t *>(smem + kWarps * kVBytes);
    uint16_t *s_et = reinterpret_cast<uint16_t *>(s_cols + max_cols_pad);
    const int et_stride = max_cols_pad + kEtPad;
    __half *s_qr_all = reinterpret_cast<__half *>(s_et + kTileRows * et_stride);
    const int qr_stride = t_max + 8;

    const int32_t *tile = tiles + static_cast<int64_t>(blockIdx.x) * kTileInts;
    const int ncols_pad = tile[kTileNcolsPad];
    const int tq = tile[kTileTq];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    // stage the tile's column list and etype matrix
    {
        const int32_t *gc = cols + tile[kTileColOff];
        for (int i = threadIdx.x; i < ncols_pad; i += blockDim.x) s_cols[i] = gc[i];
        const uint16_t *ge = et + tile[kTileEtOff];
        const int words_per_row = ncols_pad >> 1;
        for (int i = threadIdx.x; i < kTileRows * words_per_row; i += blockDim.x) {
            const int r = i / words_per_row, c2 = i - r * words_per_row;
            reinterpret_cast<uint32_t *>(s_et + r * et_stride)[c2] =
                reinterpret_cast<const uint32_t *>(ge + static_cast<int64_t>(r) * ncols_pad)[c2];
        }
    }
    __syncthreads();

    const int row_lo = tile[kTileRowOff + g], row_hi = tile[kTileRowOff + g + 8];
    const int slot_lo = tile[kTileSlotOff + g], slot_hi = tile[kTileSlotOff + g + 8];
    unsigned char *s_v = s_v_all + warp * kVBytes;
    const uint32_t s_v_addr = static_cast<uint32_t>(__cvta_generic_to_shared(s_v));
    __half *s_qr = s_qr_all + static_cast<int64_t>(warp) * kTileRows * qr_stride;
    const float sl2 = scale * kLog2e;

    for (int h = warp; h < H; h += kWarps) {
        // Q fragments of the two rows this lane serves (unused rows read row 0, never written)
        uint32_t q_lo[8], q_hi[8];
        load_row_frag(q + (static_cast<int64_t>(row_lo < 0 ? 0 : row_lo) * H + h) * kHeadDim, t, q_lo);
        load_row_frag(q + (static_cast<int64_t>(row_hi < 0 ? 0 : row_hi) * H + h) * kHeadDim, t, q_hi);

        if (kHasBias) {
            // QR[row][type] = <q[row], ak[type]> for the types that occur in this tile
            for (int nt = 0; nt < tq; nt += 8) {
                int type = nt + g;
                type = type < n_etypes ? type : n_etypes - 1;
                uint32_t b[8];
                load_row_frag(ak + static_cast<int64_t>(type) * kHeadDim, t, b);
                float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    mma_bf16(c, q_lo[2 * s], q_hi[2 * s], q_lo[2 * s + 1], q_hi[2 * s + 1], b[2 * s], b[2 * s + 1]);
                *reinterpret_cast<__half2 *>(s_qr + g * qr_stride + nt + 2 * t) = __floats2half2_rn(c[0], c[1]);
                *reinterpret_cast<__half2 *>(s_qr + (g + 8) * qr_stride + nt + 2 * t) = __floats2half2_rn(c[2], c[3]);
            }
            __syncwarp();
        }

        float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { acc[i][0] = 0.f; acc[i][1] = 0.f; acc[i][2] = 0.f; acc[i][3] = 0.f; }

        for (int c0 = 0; c0 < ncols_pad; c0 += kTileChunk) {
            // V rows of this step -> shared memory, 16-byte pieces, piece index XOR (row & 7)
#pragma unroll 4
            for (int i = 0; i < 16; ++i) {
                const int id = i * 32 + lane;
                const int r = id >> 3, ch = id & 7;
                const __nv_bfloat16 *src =
                    v + (static_cast<int64_t>(s_cols[c0 + r]) * H + h) * kHeadDim + ch * 8;
                cp_async16(s_v_addr + r * 128 + ((ch ^ (r & 7)) << 4), src);
            }
            // S = Q K^T for 8 column groups of 8
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                uint32_t b[8];
                load_row_frag(k + (static_cast<int64_t>(s_cols[c0 + nt * 8 + g]) * H + h) * kHeadDim, t, b);
                s[nt][0] = 0.f; s[nt][1] = 0.f; s[nt][2] = 0.f; s[nt][3] = 0.f;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_bf16(s[nt], q_lo[2 * ks], q_hi[2 * ks], q_lo[2 * ks + 1], q_hi[2 * ks + 1], b[2 * ks],
                             b[2 * ks + 1]);
            }
            // relative-position term, mask, scale (log2 domain)
            float cmax_lo = -INFINITY, cmax_hi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const uint32_t e_lo = *reinterpret_cast<const uint32_t *>(s_et + g * et_stride + c0 + nt * 8 + 2 * t);
                const uint32_t e_hi = *reinterpret_cast<const uint32_t *>(s_et + (g + 8) * et_stride + c0 + nt * 8 + 2 * t);
                const uint32_t e[4] = {e_lo & 0xffffu, e_lo >> 16, e_hi & 0xffffu, e_hi >> 16};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (e[i] == kNoEdge) {
                        s[nt][i] = -INFINITY;
                    } else {
                        float x = s[nt][i];
                        if (kHasBias) x += __half2float(s_qr[(i < 2 ? g : g + 8) * qr_stride + e[i]]);
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
            cp_async_wait_all();
            __syncwarp();
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint32_t a0 = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
                const uint32_t a1 = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
                const uint32_t a2 = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
                const uint32_t a3 = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
                const int r = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
                for (int dn = 0; dn < 8; dn += 2) {
                    const int ch = dn + (lane >> 4);
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, s_v_addr + r * 128 + ((ch ^ (r & 7)) << 4));
                    mma_bf16(acc[dn], a0, a1, a2, a3, b[0], b[1]);
                    mma_bf16(acc[dn + 1], a0, a1, a2, a3, b[2], b[3]);
                }
            }
            __syncwarp();  // the stage is rewritten by the next step
        }

        // row sums live per lane: finish them across the quad
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
        l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = half ? row_hi : row_lo, slot = half ? slot_hi : slot_lo;
            const float m = half ? m_hi : m_lo, l = half ? l_hi : l_lo;
            if (row < 0) continue;
            if (slot < 0) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                __nv_bfloat16 *dst = o + (static_cast<int64_t>(row) * H + h) * kHeadDim + 2 * t;
#pragma unroll
                for (int dn = 0; dn < 8; ++dn)
                    *reinterpret_cast<uint32_t *>(dst + dn * 8) =
                        pack_bf16(acc[dn][2 * half] * inv, acc[dn][2 * half + 1] * inv);
                if (t == 0) lse[static_cast<int64_t>(row) * H + h] = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;
            } else {
                float *dst = part_o + (static_cast<int64_t>(slot) * H + h) * kHeadDim + 2 * t;
#pragma unroll
                for (int dn = 0; dn < 8; ++dn)
                    *reinterpret_cast<float2 *>(dst + dn * 8) = make_float2(acc[dn][2 * half], acc[dn][2 * half + 1]);
                if (t == 0) {
                    part_ml[(static_cast<int64_t>(slot) * H + h) * 2] = m;
                    part_ml[(static_cast<int64_t>(slot) * H + h) * 2 + 1] = l;
                }
            }
        }
        __syncwarp();
    }
}

size_t tc_smem_bytes(int max_cols_pad, int t_max) {
    return static_cast<size_t>(kWarps) * kVBytes + static_cast<size_t>(max_cols_pad) * 4 +
           static_cast<size_t>(kTileRows) * (max_cols_pad + kEtPad) * 2 +
           static_cast<size_t>(kWarps) * kTileRows * (t_max + 8) * 2;
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" size_t bpt_attn_forward_tc_workspace_bytes(int64_t n_slots, int h) {
    if (n_slots < 0 || h < 1) return 0;
    const size_t s = static_cast<size_t>(n_slots);
    return align_up(s * h * kHeadDim * 4, 256) + align_up(s * h * 2 * 4, 256) + 512;
}

extern "C" int bpt_attn_forward_tc(const int32_t *tiles, int64_t n_tiles, const int32_t *cols, const uint16_t *et,
                                   const int32_t *split_rows, int64_t n_split, int64_t n_slots,
                                   const int32_t *simt_items, int64_t n_simt_items, const void *attn_plan,
                                   const int32_t *counts_host, int64_t n_nodes, int64_t n_edges,
                                   int max_cols_pad, int t_max, int n_etypes, const void *q, const void *k,
                                   const void *v, const void *ak, double scale, void *o, float *lse, int h,
                                   int d, int dtype, void *workspace, size_t workspace_bytes,
                                   bpt_stream_t stream_) {
    BPT_CHECK_ARG(n_tiles >= 0 && n_split >= 0 && n_slots >= 0 && h >= 1, "attn_forward_tc: bad sizes");
    if (d != kHeadDim || dtype != BPT_BF16)
        return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc: only bf16 with head dim 64 (got dtype %d, d %d)", dtype, d);
    if (n_tiles == 0 && n_simt_items == 0) return BPT_OK;
    BPT_CHECK_ARG((n_tiles == 0 || tiles) && q && k && v && o && lse, "attn_forward_tc: null argument");
    BPT_CHECK_ARG(n_simt_items == 0 || (simt_items && attn_plan && counts_host), "attn_forward_tc: null row-item list");
    BPT_CHECK_ARG(n_simt_items >= 0 && n_simt_items < (int64_t(1) << 31), "attn_forward_tc: bad row-item count");
    BPT_CHECK_ARG(max_cols_pad == 0 || (cols && et), "attn_forward_tc: null plan arrays");
    BPT_CHECK_ARG(max_cols_pad % kTileChunk == 0 && t_max % 8 == 0 && n_etypes >= 1, "attn_forward_tc: bad plan sizes");
    BPT_CHECK_ARG(n_tiles < (int64_t(1) << 31), "attn_forward_tc: too many tiles");
    BPT_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                    reinterpret_cast<uintptr_t>(ak) | reinterpret_cast<uintptr_t>(o)) & 15) == 0,
                  "attn_forward_tc: tensors must be 16-byte aligned");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    float *part_o = ws.take<float>(static_cast<size_t>(n_slots) * h * kHeadDim);
    float *part_ml = ws.take<float>(static_cast<size_t>(n_slots) * h * 2);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_forward_tc: workspace of %zu bytes is too small", workspace_bytes);
    const bool bias = ak != nullptr && t_max > 0;
    const size_t smem = tc_smem_bytes(max_cols_pad, bias ? t_max : 0);
    if (smem > 227 * 1024)
        return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc: tile plan needs %zu bytes of shared memory", smem);
    const __nv_bfloat16 *qb = static_cast<const __nv_bfloat16 *>(q), *kb = static_cast<const __nv_bfloat16 *>(k);
    const __nv_bfloat16 *vb = static_cast<const __nv_bfloat16 *>(v), *akb = static_cast<const __nv_bfloat16 *>(ak);
    __nv_bfloat16 *ob = static_cast<__nv_bfloat16 *>(o);
    if (n_simt_items > 0) {
        const PlanView pv = plan_view(const_cast<void *>(attn_plan), n_nodes, counts_host[kCountsNSrc], n_edges, n_etypes);
        if (int rc = launch_forward_items_bf16(reinterpret_cast<const int4 *>(simt_items),
                                               static_cast<int>(n_simt_items), pv.in_src, pv.in_etype, q, k, v, ak,
                                               static_cast<float>(scale), o, lse, h, d, stream))
            return rc;
    }
    if (n_tiles == 0) return BPT_OK;
    if (bias) {
        BPT_CUDA(cudaFuncSetAttribute(attn_forward_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
        attn_forward_tc_kernel<true><<<static_cast<unsigned>(n_tiles), kWarps * 32, smem, stream>>>(
            tiles, cols, et, qb, kb, vb, akb, n_etypes, static_cast<float>(scale), ob, lse, part_o, part_ml, h,
            max_cols_pad, t_max);
    } else {
        BPT_CUDA(cudaFuncSetAttribute(attn_forward_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
        attn_forward_tc_kernel<false><<<static_cast<unsigned>(n_tiles), kWarps * 32, smem, stream>>>(
            tiles, cols, et, qb, kb, vb, akb, n_etypes, static_cast<float>(scale), ob, lse, part_o, part_ml, h,
            max_cols_pad, 0);
    }
    BPT_LAUNCH_CHECK();
    if (n_split > 0) {
        const Geometry g{h, kHeadDim};
        attn_forward_merge_kernel<__nv_bfloat16><<<static_cast<unsigned>(n_split), merge_threads(h, kHeadDim),
                                                   merge_smem_bytes(h), stream>>>(
            reinterpret_cast<const int4 *>(split_rows), static_cast<int>(n_split), part_o, part_ml, ob, lse, g);
        BPT_LAUNCH_CHECK();
    }
    return BPT_OK;
}
