// dK and dV of the fused attention backward on tensor cores (bf16, head dim 64).
//
// Works on the transposed tile plan: an m-block is <=16 SOURCE rows, its columns are the
// destinations that attend to them, and every cell knows its edge's position in the in-CSR.
// The destination-side pass (bpt_attn_backward) has already left P, dP = <dO[dst], v[src]> and
// delta per edge / destination in scratch, so a cell's weights are two gathers away:
//     dV[src] = sum_dst P * dO[dst],   dK[src] = sum_dst scale * P * (dP - delta[dst]) * q[dst].
// One block per m-block, one warp per head; per 32 destinations the warp stages their dO and Q
// rows in swizzled shared memory (cp.async), packs the gathered weights into mma A fragments
// and accumulates both products with ldmatrix.trans B fragments.  A source row wholly inside
// one m-block is written once; rows spread over several m-blocks write fp32 partials that are
// summed in slot order.  No atomics: results are bitwise reproducible.
#include "fused_common.cuh"
#include "tile_plan.cuh"

namespace bpt {
namespace {

constexpr int kHeadDim = 64;
constexpr int kWarps = 8;
constexpr int kHalf = 32;                               // destinations staged per step
constexpr int kRowBytes = kHeadDim * 2;
constexpr int kStageBytes = kHalf * kRowBytes;          // 4 KB per matrix
constexpr int kPosPad = 4;                              // int32 padding per staged position row

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
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

struct DkvParams {
    const int32_t *groups, *mblocks, *cols, *cellpos;
    const float *P, *dP, *delta;
    const __nv_bfloat16 *q, *d_o;
    __nv_bfloat16 *dk, *dv;
    float *part;
    int H, max_cols_pad;
    float scale;
};

__global__ void __launch_bounds__(kWarps * 32, 2)
attn_backward_dkv_tile_kernel(const DkvParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: per warp {dO stage, Q stage} (8 KB) | destination ids | edge positions of the m-block
    int32_t *s_cols = reinterpret_cast<int32_t *>(smem + kWarps * 2 * kStageBytes);
    int32_t *s_pos = s_cols + p.max_cols_pad;
    const int pos_stride = p.max_cols_pad + kPosPad;

    const int32_t *grp = p.groups + static_cast<int64_t>(blockIdx.x) * kGroupInts;
    const int ncols_pad = grp[kGroupNcolsPad];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H;
    const uint32_t s_do = static_cast<uint32_t>(__cvta_generic_to_shared(smem + warp * 2 * kStageBytes));
    const uint32_t s_q = s_do + kStageBytes;
    {
        const int32_t *gc = p.cols + grp[kGroupColOff];
        for (int i = threadIdx.x; i < ncols_pad; i += blockDim.x) s_cols[i] = gc[i];
    }
    for (int mbi = 0; mbi < grp[kGroupMbCount]; ++mbi) {
        const int32_t *mb = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + mbi) * kMbInts;
        const uint32_t chunk_mask = static_cast<uint32_t>(mb[kMbChunkMask]);
        __syncthreads();
        {
            // the cell matrix is [chunk][16][64]; 4 positions (16 bytes) per thread and step
            const int4 *gp = reinterpret_cast<const int4 *>(p.cellpos + mb[kMbEtOff]);
            const int pieces = kTileRows * ncols_pad / 4;
            for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
                const int cell = i * 4;
                const int chunk = cell / (kTileRows * kTileChunk), rem = cell % (kTileRows * kTileChunk);
                const int r = rem / kTileChunk, c = rem % kTileChunk;
                *reinterpret_cast<int4 *>(s_pos + r * pos_stride + chunk * kTileChunk + c) = __ldg(gp + i);
            }
        }
        __syncthreads();
        const int row_lo = mb[kMbRowOff + g], row_hi = mb[kMbRowOff + g + 8];
        for (int h = warp; h < H; h += kWarps) {
            float dk[8][4], dv[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) { dk[i][j] = 0.f; dv[i][j] = 0.f; }
            for (int c0 = 0; c0 < ncols_pad; c0 += kHalf) {
                if (!((chunk_mask >> (c0 / kTileChunk)) & 1u)) continue;
                // dO and Q rows of these 32 destinations -> shared memory
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int id = i * 32 + lane;
                    const int r = id >> 3, piece = id & 7;
                    const int64_t off = (static_cast<int64_t>(s_cols[c0 + r]) * H + h) * kHeadDim + piece * 8;
                    const uint32_t dst = r * kRowBytes + ((piece ^ (r & 7)) << 4);
                    cp_async16(s_do + dst, p.d_o + off);
                    cp_async16(s_q + dst, p.q + off);
                }
                cp_async_commit();
                // weights of this lane's 16 cells: rows g / g+8, destinations c0 + 8nt + 2t, +1
                float wp[4][4], ws[4][4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int c = c0 + nt * 8 + 2 * t;
                    const int2 pos_lo = *reinterpret_cast<const int2 *>(s_pos + g * pos_stride + c);
                    const int2 pos_hi = *reinterpret_cast<const int2 *>(s_pos + (g + 8) * pos_stride + c);
                    const int pos[4] = {pos_lo.x, pos_lo.y, pos_hi.x, pos_hi.y};
                    const float d0 = p.delta[static_cast<int64_t>(s_cols[c]) * H + h];
                    const float d1 = p.delta[static_cast<int64_t>(s_cols[c + 1]) * H + h];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float pr = 0.f, ds = 0.f;
                        if (pos[i] >= 0) {
                            pr = p.P[static_cast<int64_t>(pos[i]) * H + h];
                            ds = p.scale * pr * (p.dP[static_cast<int64_t>(pos[i]) * H + h] - ((i & 1) ? d1 : d0));
                        }
                        wp[nt][i] = pr;
                        ws[nt][i] = ds;
                    }
                }
                cp_async_wait_all();
                __syncwarp();
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    const uint32_t p0 = pack_bf16(wp[2 * ks][0], wp[2 * ks][1]), p1 = pack_bf16(wp[2 * ks][2], wp[2 * ks][3]);
                    const uint32_t p2 = pack_bf16(wp[2 * ks + 1][0], wp[2 * ks + 1][1]);
                    const uint32_t p3 = pack_bf16(wp[2 * ks + 1][2], wp[2 * ks + 1][3]);
                    const uint32_t s0 = pack_bf16(ws[2 * ks][0], ws[2 * ks][1]), s1 = pack_bf16(ws[2 * ks][2], ws[2 * ks][3]);
                    const uint32_t s2 = pack_bf16(ws[2 * ks + 1][0], ws[2 * ks + 1][1]);
                    const uint32_t s3 = pack_bf16(ws[2 * ks + 1][2], ws[2 * ks + 1][3]);
                    const int r = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
#pragma unroll
                    for (int dn = 0; dn < 8; dn += 2) {
                        const int piece = dn + (lane >> 4);
                        const uint32_t off = r * kRowBytes + ((piece ^ (r & 7)) << 4);
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, s_do + off);
                        mma_bf16(dv[dn], p0, p1, p2, p3, b[0], b[1]);
                        mma_bf16(dv[dn + 1], p0, p1, p2, p3, b[2], b[3]);
                        ldmatrix_x4_trans(b, s_q + off);
                        mma_bf16(dk[dn], s0, s1, s2, s3, b[0], b[1]);
                        mma_bf16(dk[dn + 1], s0, s1, s2, s3, b[2], b[3]);
                    }
                }
                __syncwarp();  // the stages are rewritten by the next step
            }
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

// out0[row] | out1[row] = sum over the row's slots, in slot order, of the slot's two halves.
__global__ void dkv_sum_merge_kernel(const int4 *__restrict__ split_rows, int n_split, const float *__restrict__ part,
                                     int width, __nv_bfloat16 *__restrict__ out0, __nv_bfloat16 *__restrict__ out1) {
    const int sr = blockIdx.x;
    if (sr >= n_split) return;
    const int4 rec = split_rows[sr];
    const int row = rec.x, first = rec.y, count = rec.z;
    const int stride = 2 * width;
    for (int c = threadIdx.x; c < stride; c += blockDim.x) {
        const float *src = part + static_cast<int64_t>(first) * stride + c;
        float acc = 0.f;
        int s = 0;
        for (; s + 8 <= count; s += 8) {
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = src[static_cast<int64_t>(s + u) * stride];
#pragma unroll
            for (int u = 0; u < 8; ++u) acc += x[u];
        }
        for (; s < count; ++s) acc += src[static_cast<int64_t>(s) * stride];
        if (c < width) out0[static_cast<int64_t>(row) * width + c] = __float2bfloat16_rn(acc);
        else out1[static_cast<int64_t>(row) * width + (c - width)] = __float2bfloat16_rn(acc);
    }
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" size_t bpt_attn_backward_dkv_tc_workspace_bytes(int64_t n_slots, int h) {
    if (n_slots < 0 || h < 1) return 0;
    return align_up(static_cast<size_t>(n_slots) * 2 * h * kHeadDim * 4, 256) + 256;
}

extern "C" int bpt_attn_backward_dkv_tc(const int32_t *groups, int64_t n_groups, const int32_t *mblocks,
                                        const int32_t *cols, const int32_t *cell_pos, const int32_t *split_rows,
                                        int64_t n_split, int64_t n_slots, int max_cols_pad, const float *P,
                                        const float *dP, const float *delta, const void *q, const void *d_o,
                                        double scale, void *dk, void *dv, int h, int d, int dtype,
                                        void *workspace, size_t workspace_bytes, bpt_stream_t stream_) {
    BPT_CHECK_ARG(n_groups >= 0 && n_split >= 0 && n_slots >= 0 && h >= 1, "attn_backward_dkv_tc: bad sizes");
    if (d != kHeadDim || dtype != BPT_BF16)
        return fail(BPT_ERR_UNSUPPORTED, "attn_backward_dkv_tc: only bf16 with head dim 64 (got dtype %d, d %d)", dtype, d);
    if (n_groups == 0) return BPT_OK;
    BPT_CHECK_ARG(groups && mblocks && P && dP && delta && q && d_o && dk && dv, "attn_backward_dkv_tc: null argument");
    BPT_CHECK_ARG(max_cols_pad == 0 || (cols && cell_pos), "attn_backward_dkv_tc: null plan arrays");
    BPT_CHECK_ARG(max_cols_pad % kTileChunk == 0 && max_cols_pad <= kMaxChunks * kTileChunk,
                  "attn_backward_dkv_tc: bad plan sizes");
    BPT_CHECK_ARG(n_groups < (int64_t(1) << 31), "attn_backward_dkv_tc: too many groups");
    BPT_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(d_o) | reinterpret_cast<uintptr_t>(dk) |
                    reinterpret_cast<uintptr_t>(dv)) & 15) == 0, "attn_backward_dkv_tc: tensors must be 16-byte aligned");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    float *part = ws.take<float>(static_cast<size_t>(n_slots) * 2 * h * kHeadDim);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_backward_dkv_tc: workspace of %zu bytes is too small", workspace_bytes);
    DkvParams p;
    p.groups = groups; p.mblocks = mblocks; p.cols = cols; p.cellpos = cell_pos;
    p.P = P; p.dP = dP; p.delta = delta;
    p.q = static_cast<const __nv_bfloat16 *>(q); p.d_o = static_cast<const __nv_bfloat16 *>(d_o);
    p.dk = static_cast<__nv_bfloat16 *>(dk); p.dv = static_cast<__nv_bfloat16 *>(dv);
    p.part = part; p.H = h; p.max_cols_pad = max_cols_pad; p.scale = static_cast<float>(scale);
    const size_t smem = static_cast<size_t>(kWarps) * 2 * kStageBytes + static_cast<size_t>(max_cols_pad) * 4 +
                        static_cast<size_t>(kTileRows) * (max_cols_pad + kPosPad) * 4;
    if (smem > 227 * 1024)
        return fail(BPT_ERR_UNSUPPORTED, "attn_backward_dkv_tc: tile plan needs %zu bytes of shared memory", smem);
    BPT_CUDA(cudaFuncSetAttribute(attn_backward_dkv_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
    attn_backward_dkv_tile_kernel<<<static_cast<unsigned>(n_groups), kWarps * 32, smem, stream>>>(p);
    BPT_LAUNCH_CHECK();
    if (n_split > 0) {
        dkv_sum_merge_kernel<<<static_cast<unsigned>(n_split), 256, 0, stream>>>(
            reinterpret_cast<const int4 *>(split_rows), static_cast<int>(n_split), part, h * kHeadDim, p.dk, p.dv);
        BPT_LAUNCH_CHECK();
    }
    return BPT_OK;
}
