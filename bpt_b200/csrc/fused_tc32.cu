// Fused graph attention forward for fp32 tensors on tensor cores (head dim 64), within the 1e-5 bar of the
// fp32 path: every product runs as three TF32 products.
//
// A TF32 operand keeps 10 mantissa bits, far short of fp32's 23.  Each fp32 operand x is therefore split
// into hi = x with its low 13 mantissa bits cleared (exactly a TF32 number) and lo = x - hi (exact in fp32,
// at most 13 significant bits, of which the tensor core keeps 10), and a . b is accumulated in fp32 as
// a_lo . b_hi + a_hi . b_lo + a_hi . b_hi; what is dropped (a_lo . b_lo and the tail of lo) is ~2^-21 of
// the product.  The splits are two ALU instructions per operand register, made on the fly.
//
// Same tile plan, same structure and same results layout as the bf16 tile kernel (fused_tc.cu): a warp takes
// one head of a 16-row m-block at a time, S = Q K^T per step of 16 columns, one table lookup per cell for
// the relative-position term and the edge mask (the table is fp32 here), online softmax in registers,
// O += P V, rows spread over several m-blocks write (m, l, O) partials for the merge kernel.  What differs:
//   * mma.sync m16n8k8 (TF32): the A fragment of P . V wants columns (t, t + 4) per lane where the
//     accumulator of S holds (2t, 2t + 1); instead of shuffling, the k index of that product is read as a
//     permutation of the step's columns (k <-> column 2 (k mod 4) + k / 4) and V is fetched accordingly;
//   * K rows (256 bytes) are staged swizzled and read with ldmatrix (an 8 x 16-byte matrix is 8 columns x
//     4 floats: exactly the B fragments of two k-steps); V rows are staged with a 272-byte pitch and read
//     with plain 4-byte loads (bank = 8 t + g: conflict-free);
//   * embed_ak rows are read from global memory (26 KB, L1-resident) when the table is built, so a block
//     needs 65 KB of shared memory and three blocks of four warps share an SM.
#include "fused_common.cuh"
#include "plan.cuh"
#include "tile_plan.cuh"

namespace bpt {
namespace {

constexpr int kHeadDim = 64;
constexpr int kRowBytes = kHeadDim * 4;          // one head row of K or V in fp32: 16 pieces of 16 bytes
constexpr int kStep = 16;                        // source columns per pipeline step
constexpr int kVPitch = kRowBytes + 16;          // staged V rows: 272 bytes apart
constexpr int kKBytes = kStep * kRowBytes;       // 4096
constexpr int kVBytes = kStep * kVPitch;         // 4352
constexpr int kStageBytes = kKBytes + kVBytes;   // per warp
constexpr int kWarps = 4;                        // one tile per block; a warp takes heads w, w + 4, ...
constexpr int kEtPad = 8;
constexpr int kMaxTypes8 = 248;

__device__ __forceinline__ void mma_tf32(float (&c)[4], const float (&a)[4], float b0, float b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])),
          "r"(__float_as_uint(a[3])), "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}
__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
// c += a . b with a and b given in full fp32 precision
__device__ __forceinline__ void mma_3xtf32(float (&c)[4], const float (&a_hi)[4], const float (&a_lo)[4], float b0,
                                           float b1) {
    const float b0h = tf32_hi(b0), b1h = tf32_hi(b1);
    mma_tf32(c, a_lo, b0h, b1h);
    mma_tf32(c, a_hi, b0 - b0h, b1 - b1h);
    mma_tf32(c, a_hi, b0h, b1h);
}
__device__ __forceinline__ void split4(const float (&x)[4], float (&hi)[4], float (&lo)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        hi[i] = tf32_hi(x[i]);
        lo[i] = x[i] - hi[i];
    }
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
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
    return v;
}

template <typename ET> struct EtTraits;
template <> struct EtTraits<uint8_t> { static constexpr uint32_t kNone = kNoEdge8; };
template <> struct EtTraits<uint16_t> { static constexpr uint32_t kNone = kNoEdge; };
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

struct Tc32Params {
    const int32_t *groups, *mblocks, *cols;
    const void *et;
    const float *q, *k, *v, *ak;
    float *o, *lse, *part_o, *part_ml;
    int n_etypes, H, max_cols_pad, t_max, tab_stride;
    int64_t n_groups;
    float scale;
    Dropout drop;
};

// A lane's share of a 64-element fp32 row as A fragments of m16n8k8: for k-step s, elements 8 s + t and
// 8 s + t + 4.  out[s][0], out[s][2] for the row of this call; the caller interleaves the two rows.
__device__ __forceinline__ void load_q_frags(const float *__restrict__ row_lo, const float *__restrict__ row_hi, int t,
                                             float (&qa)[8][4]) {
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        qa[s][0] = __ldg(row_lo + 8 * s + t);
        qa[s][1] = __ldg(row_hi + 8 * s + t);
        qa[s][2] = __ldg(row_lo + 8 * s + t + 4);
        qa[s][3] = __ldg(row_hi + 8 * s + t + 4);
    }
}

// The per-head score table of an m-block, in the log2 domain: with a table (use_qr) entry [row][type] =
// scale * log2(e) * <q[row], ak[type]> for the tq types of the m-block and entry tq = -inf (the cell of a
// missing edge); without one entry 0 = 0, entry 1 = -inf, and when every row has one edge type its
// <q[row], ak[type]> comes back as the row's constant (bias_lo for row g, bias_hi for row g + 8).
// Four groups of eight types per pass share the splits of Q.
template <bool kHasBias>
__device__ __forceinline__ void build_score_table(const float (&qa)[8][4], const float *__restrict__ ak, int n_etypes,
                                                  bool use_qr, int tq, const int32_t *__restrict__ mb, float *s_tab,
                                                  int tab_stride, float sl2, int g, int t, float &bias_lo,
                                                  float &bias_hi) {
    if (use_qr) {
        for (int nt0 = 0; nt0 < tq; nt0 += 32) {
            float c[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) { c[u][0] = 0.f; c[u][1] = 0.f; c[u][2] = 0.f; c[u][3] = 0.f; }
            const float *ak_row[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                int type = nt0 + 8 * u + g;
                type = type < n_etypes ? type : n_etypes - 1;
                ak_row[u] = ak + static_cast<int64_t>(type) * kHeadDim + t;
            }
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                float a_hi[4], a_lo[4];
                split4(qa[s], a_hi, a_lo);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (nt0 + 8 * u < tq)
                        mma_3xtf32(c[u], a_hi, a_lo, __ldg(ak_row[u] + 8 * s), __ldg(ak_row[u] + 8 * s + 4));
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int nt = nt0 + 8 * u;
                if (nt < tq) {
                    s_tab[g * tab_stride + nt + 2 * t] = c[u][0] * sl2;
                    s_tab[g * tab_stride + nt + 2 * t + 1] = c[u][1] * sl2;
                    s_tab[(g + 8) * tab_stride + nt + 2 * t] = c[u][2] * sl2;
                    s_tab[(g + 8) * tab_stride + nt + 2 * t + 1] = c[u][3] * sl2;
                }
            }
        }
        if (t == 0) {
            s_tab[g * tab_stride + tq] = -INFINITY;
            s_tab[(g + 8) * tab_stride + tq] = -INFINITY;
        }
    } else {
        if (t == 0) {
            s_tab[g * tab_stride] = 0.f;
            s_tab[g * tab_stride + 1] = -INFINITY;
            s_tab[(g + 8) * tab_stride] = 0.f;
            s_tab[(g + 8) * tab_stride + 1] = -INFINITY;
        }
        if (kHasBias) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                int type = mb[kMbRowEtOff + g + 8 * half];
                type = type < 0 ? 0 : (type < n_etypes ? type : n_etypes - 1);
                const float *a = ak + static_cast<int64_t>(type) * kHeadDim + t;
                float sum = 0.f;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    sum = fmaf(qa[s][half], __ldg(a + 8 * s), sum);
                    sum = fmaf(qa[s][2 + half], __ldg(a + 8 * s + 4), sum);
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                (half ? bias_hi : bias_lo) = sum * sl2;
            }
        }
    }
}

template <typename ET, bool kHasBias, bool kDrop>
__global__ void __launch_bounds__(kWarps * 32, 3)
attn_forward_tile32_kernel(const Tc32Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: per warp {K buffer 4 KB, V buffer 4.25 KB} | column ids | table indices of the m-block | tables (fp32, per warp)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int idx_stride = p.max_cols_pad + kEtPad;
    int32_t *s_cols = reinterpret_cast<int32_t *>(smem + kWarps * kStageBytes);
    ET *s_idx = reinterpret_cast<ET *>(s_cols + p.max_cols_pad);
    const int tab_stride = p.tab_stride;
    float *s_tab_all = reinterpret_cast<float *>(smem + kWarps * kStageBytes + p.max_cols_pad * 4 +
                                                 (kTileRows * idx_stride * static_cast<int>(sizeof(ET)) + 15) / 16 * 16);
    const int64_t tile = blockIdx.x;
    const int32_t *grp = p.groups + tile * kGroupInts;
    const int n_mblocks = grp[kGroupMbCount];
    if (n_mblocks == 0) return;
    const int ncols_pad = grp[kGroupNcolsPad];
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H;
    const uint32_t s_k_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem + warp * kStageBytes));
    const uint32_t s_v_addr = s_k_addr + kKBytes;
    const int n_steps = ncols_pad / kStep;
    float *s_tab = s_tab_all + static_cast<int64_t>(warp) * kTileRows * tab_stride;
    const uint32_t s_tab_lo = static_cast<uint32_t>(__cvta_generic_to_shared(s_tab + g * tab_stride));
    const uint32_t s_tab_hi = static_cast<uint32_t>(__cvta_generic_to_shared(s_tab + (g + 8) * tab_stride));
    const float sl2 = p.scale * kLog2e;
    const ET *et_base = static_cast<const ET *>(p.et);
    {
        const int32_t *gc = p.cols + grp[kGroupColOff];
        for (int i = threadIdx.x; i < ncols_pad; i += blockDim.x) s_cols[i] = gc[i];
    }
    // Row copies: lane l copies piece (l & 15) of rows (l >> 4) + 2 i.  K pieces are swizzled on their low
    // three bits (ldmatrix reads eight rows at one piece position), V rows are 272 bytes apart.
    const int copy_row = lane >> 4, copy_piece = lane & 15;
    const uint32_t row_pitch = static_cast<uint32_t>(H) * kRowBytes;
    auto issue_k = [&](int h, int j) {
        const char *src = reinterpret_cast<const char *>(p.k) + (h * kRowBytes + copy_piece * 16);
        const int32_t *cj = s_cols + j * kStep + copy_row;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = copy_row + 2 * i;
            cp_async16(s_k_addr + r * kRowBytes + (((copy_piece & 8) | ((copy_piece ^ r) & 7)) << 4),
                       src + static_cast<uint64_t>(static_cast<uint32_t>(cj[2 * i])) * row_pitch);
        }
    };
    auto issue_v = [&](int h, int j) {
        const char *src = reinterpret_cast<const char *>(p.v) + (h * kRowBytes + copy_piece * 16);
        const int32_t *cj = s_cols + j * kStep + copy_row;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = copy_row + 2 * i;
            cp_async16(s_v_addr + r * kVPitch + copy_piece * 16,
                       src + static_cast<uint64_t>(static_cast<uint32_t>(cj[2 * i])) * row_pitch);
        }
    };

    for (int mbi = 0; mbi < n_mblocks; ++mbi) {
        const int32_t *mb = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + mbi) * kMbInts;
        const bool use_qr = kHasBias && mb[kMbQrSlot] >= 0;
        const int tq = use_qr ? mb[kMbTq] : 0;             // table entry tq (or 1) is the -inf entry
        const uint32_t none_idx = use_qr ? tq : 1;
        const uint32_t chunk_mask = static_cast<uint32_t>(mb[kMbChunkMask]);
        // first step after j with an edge in this m-block (one mask bit per 32 columns, two steps); n_steps if none
        static_assert(kMaskCols == 2 * kStep, "two pipeline steps per mask bit");
        auto next_step = [&](int j) {
            ++j;
            while (j < n_steps && !((chunk_mask >> (j >> 1)) & 1u)) ++j;
            return j;
        };
        __syncthreads();  // previous m-block's indices are no longer read; s_cols is visible
        int primed_step = -1;
        if (warp < H) primed_step = next_step(-1);
        if (primed_step >= 0 && primed_step < n_steps) issue_k(warp, primed_step);
        cp_async_commit();
        if (primed_step >= 0 && primed_step < n_steps) issue_v(warp, primed_step);
        cp_async_commit();
        const int row_lo = mb[kMbRowOff + g], row_hi = mb[kMbRowOff + g + 8];
        {
            // stage the m-block's cells as table indices: edge type, or the -inf entry
            constexpr int kCellsPerPiece = 16 / static_cast<int>(sizeof(ET));
            const uint4 *ge = reinterpret_cast<const uint4 *>(et_base + mb[kMbEtOff]);
            const int pieces = kTileRows * ncols_pad / kCellsPerPiece;
            for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
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
        __syncthreads();

        for (int h = warp; h < H; h += kWarps) {
            float qa[8][4];
            load_q_frags(p.q + (static_cast<int64_t>(row_lo < 0 ? 0 : row_lo) * H + h) * kHeadDim,
                         p.q + (static_cast<int64_t>(row_hi < 0 ? 0 : row_hi) * H + h) * kHeadDim, t, qa);
            float bias_lo = 0.f, bias_hi = 0.f;  // per-row constant of m-blocks without a table (log2 domain)
            build_score_table<kHasBias>(qa, p.ak, p.n_etypes, use_qr, tq, mb, s_tab, tab_stride, sl2, g, t, bias_lo, bias_hi);
            __syncwarp();

            float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
            float acc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) { acc[i][0] = 0.f; acc[i][1] = 0.f; acc[i][2] = 0.f; acc[i][3] = 0.f; }

            // K and V each have one buffer: K of the next step is fetched while this step's softmax and PV
            // run, V of the next step while the next step's QK^T runs.  Two cp.async groups per iteration.
            int j = primed_step;
            if (j < 0) {
                j = next_step(-1);
                if (j < n_steps) issue_k(h, j);
                cp_async_commit();
                if (j < n_steps) issue_v(h, j);
                cp_async_commit();
            }
            primed_step = -1;
            while (j < n_steps) {
                const int nj = next_step(j);
                const int c0 = j * kStep;
                cp_async_wait<1>();  // K of this step has landed
                __syncwarp();
                float s[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) { s[nt][0] = 0.f; s[nt][1] = 0.f; s[nt][2] = 0.f; s[nt][3] = 0.f; }
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {  // k-steps 2 sp and 2 sp + 1
                    float a_hi[2][4], a_lo[2][4];
                    split4(qa[2 * sp], a_hi[0], a_lo[0]);
                    split4(qa[2 * sp + 1], a_hi[1], a_lo[1]);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const int r = nt * 8 + (lane & 7), piece = sp * 4 + (lane >> 3);
                        uint32_t b[4];
                        ldmatrix_x4(b, s_k_addr + r * kRowBytes + (((piece & 8) | ((piece ^ r) & 7)) << 4));
                        mma_3xtf32(s[nt], a_hi[0], a_lo[0], __uint_as_float(b[0]), __uint_as_float(b[1]));
                        mma_3xtf32(s[nt], a_hi[1], a_lo[1], __uint_as_float(b[2]), __uint_as_float(b[3]));
                    }
                }
                __syncwarp();  // every lane has read K: its buffer may be refilled
                if (nj < n_steps) issue_k(h, nj);
                cp_async_commit();
                // scale, relative-position term and mask: one table entry per cell
                float cmax_lo = -INFINITY, cmax_hi = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    uint32_t i_lo0, i_lo1, i_hi0, i_hi1;
                    load_idx_pair(s_idx + g * idx_stride + c0 + nt * 8 + 2 * t, i_lo0, i_lo1);
                    load_idx_pair(s_idx + (g + 8) * idx_stride + c0 + nt * 8 + 2 * t, i_hi0, i_hi1);
                    s[nt][0] = fmaf(s[nt][0], sl2, lds_f32(s_tab_lo + 4 * i_lo0));
                    s[nt][1] = fmaf(s[nt][1], sl2, lds_f32(s_tab_lo + 4 * i_lo1));
                    s[nt][2] = fmaf(s[nt][2], sl2, lds_f32(s_tab_hi + 4 * i_hi0));
                    s[nt][3] = fmaf(s[nt][3], sl2, lds_f32(s_tab_hi + 4 * i_hi1));
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
                    const float corr_lo = exp2f(m_lo - ms_lo), corr_hi = exp2f(m_hi - ms_hi);
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
                for (int nt = 0; nt < 2; ++nt) {
                    s[nt][0] = exp2f(s[nt][0] - ms_lo);
                    s[nt][1] = exp2f(s[nt][1] - ms_lo);
                    s[nt][2] = exp2f(s[nt][2] - ms_hi);
                    s[nt][3] = exp2f(s[nt][3] - ms_hi);
                    l_lo += s[nt][0] + s[nt][1];
                    l_hi += s[nt][2] + s[nt][3];
                }
                if (kDrop) {  // the row sums keep every weight; the weights that multiply V are masked and rescaled
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const int src0 = s_cols[c0 + nt * 8 + 2 * t], src1 = s_cols[c0 + nt * 8 + 2 * t + 1];
                        s[nt][0] *= dropout_factor(p.drop, row_lo, src0, h);
                        s[nt][1] *= dropout_factor(p.drop, row_lo, src1, h);
                        s[nt][2] *= dropout_factor(p.drop, row_hi, src0, h);
                        s[nt][3] *= dropout_factor(p.drop, row_hi, src1, h);
                    }
                }
                // O += P V.  k index kk of the product stands for column 8 ks + 2 (kk mod 4) + kk / 4 of the step,
                // so that the accumulators of S are the A fragments as they are.
                cp_async_wait<1>();  // V of this step has landed (the newest group is the next K)
                __syncwarp();
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    const float pa[4] = {s[ks][0], s[ks][2], s[ks][1], s[ks][3]};
                    float p_hi[4], p_lo[4];
                    split4(pa, p_hi, p_lo);
                    const uint32_t v0 = s_v_addr + (8 * ks + 2 * t) * kVPitch + g * 4;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn)
                        mma_3xtf32(acc[dn], p_hi, p_lo, lds_f32(v0 + dn * 32), lds_f32(v0 + kVPitch + dn * 32));
                }
                __syncwarp();  // every lane has read V: its buffer may be refilled
                if (nj < n_steps) issue_v(h, nj);
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
                const int row = half ? row_hi : row_lo;
                if (row < 0) continue;
                const int slot = mb[kMbSlotOff + g + 8 * half];
                const float m = (half ? m_hi : m_lo) + (half ? bias_hi : bias_lo);
                const float l = half ? l_hi : l_lo;
                if (slot < 0) {
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    float *dst = p.o + (static_cast<int64_t>(row) * H + h) * kHeadDim + 2 * t;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn)
                        *reinterpret_cast<float2 *>(dst + dn * 8) =
                            make_float2(acc[dn][2 * half] * inv, acc[dn][2 * half + 1] * inv);
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

int tab_stride32(int t_max) { return t_max + 9; }  // t_max types + the -inf entry, an odd number of words; >= 9
size_t tc32_smem_bytes(int max_cols_pad, int t_max, int et_bytes) {
    return static_cast<size_t>(kWarps) * kStageBytes + static_cast<size_t>(max_cols_pad) * 4 +
           align_up(static_cast<size_t>(kTileRows) * (max_cols_pad + kEtPad) * et_bytes, 16) +
           static_cast<size_t>(kWarps) * kTileRows * tab_stride32(t_max) * 4;
}

template <typename ET, bool kHasBias>
int launch_tile32_kernel(const Tc32Params &p, int64_t n_groups, size_t smem, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>(n_groups);
    if (p.drop.threshold) {
        BPT_CUDA(cudaFuncSetAttribute(attn_forward_tile32_kernel<ET, kHasBias, true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attn_forward_tile32_kernel<ET, kHasBias, true><<<grid, kWarps * 32, smem, stream>>>(p);
    } else {
        BPT_CUDA(cudaFuncSetAttribute(attn_forward_tile32_kernel<ET, kHasBias, false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attn_forward_tile32_kernel<ET, kHasBias, false><<<grid, kWarps * 32, smem, stream>>>(p);
    }
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}


// ------------------------------------------------------------------ backward, destination side
//
// For every (edge, head): p = exp2(s - lse), dp = <dO[dst], v[src]> (times the dropout factor), written to the
// fp32 scratch of the CUDA-core backward (P, dP in [in-CSR position][head] order) with delta = <dO, O> per
// (row, head), so that the source-side and type-bucket passes of that backward run unchanged on it; and the K
// part of dQ, dQ[row] += sum_e dS_e k[src_e] with dS = scale * p * (dp - delta).  The relative-position part
// (sum_e dS_e ak[type_e]) is added afterwards from the scratch.
//
// Same tiles, tables and three-product TF32 scheme as the forward.  Per step of 16 columns a warp holds the K
// rows and the V rows in a swizzled 4 KB tile each, in one of two buffers (the next step's rows travel while
// this step's products run): dP = dO V^T (ldmatrix on V), S = Q K^T (ldmatrix on K), the per-cell work,
// dQ += dS K (K read with plain 4-byte loads: row 8 ks + 2 t (+1), element 8 dn + g of the swizzled tile is
// bank-conflict-free).  Q, dO and the dQ accumulators take 96 registers: two blocks of four warps per SM.
struct Dq32Params {
    const int32_t *groups, *mblocks, *cols, *cellpos;
    const void *et;
    const float *q, *k, *v, *ak, *o, *d_o, *lse;
    float *P, *dP, *delta, *part_dq, *dq;
    int n_etypes, H, max_cols_pad, t_max, tab_stride;
    int64_t n_groups;
    float scale;
    Dropout drop;
};

constexpr int kDqBufBytes = 2 * kKBytes;       // K rows, V rows of one step
constexpr int kDqStageBytes = 2 * kDqBufBytes;  // per warp: two such buffers
#ifndef BPT_DQ32_MIN_BLOCKS
#define BPT_DQ32_MIN_BLOCKS 2
#endif
constexpr int kDqMinBlocks = BPT_DQ32_MIN_BLOCKS;

template <typename ET, bool kHasBias, bool kDrop>
__global__ void __launch_bounds__(kWarps * 32, kDqMinBlocks)
attn_backward_dq_tile32_kernel(const Dq32Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: per warp 2 x {K tile 4 KB, V tile 4 KB} | column ids | table indices of the m-block | tables (fp32, per warp)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int idx_stride = p.max_cols_pad + kEtPad;
    int32_t *s_cols = reinterpret_cast<int32_t *>(smem + kWarps * kDqStageBytes);
    ET *s_idx = reinterpret_cast<ET *>(s_cols + p.max_cols_pad);
    const int tab_stride = p.tab_stride;
    float *s_tab_all = reinterpret_cast<float *>(smem + kWarps * kDqStageBytes + p.max_cols_pad * 4 +
                                                 (kTileRows * idx_stride * static_cast<int>(sizeof(ET)) + 15) / 16 * 16);
    const int64_t tile = blockIdx.x;
    const int32_t *grp = p.groups + tile * kGroupInts;
    const int n_mblocks = grp[kGroupMbCount];
    if (n_mblocks == 0) return;
    const int ncols_pad = grp[kGroupNcolsPad];
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H;
    const uint32_t s_kv_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem + warp * kDqStageBytes));
    const int n_steps = ncols_pad / kStep;
    float *s_tab = s_tab_all + static_cast<int64_t>(warp) * kTileRows * tab_stride;
    const uint32_t s_tab_lo = static_cast<uint32_t>(__cvta_generic_to_shared(s_tab + g * tab_stride));
    const uint32_t s_tab_hi = static_cast<uint32_t>(__cvta_generic_to_shared(s_tab + (g + 8) * tab_stride));
    const float sl2 = p.scale * kLog2e;
    const ET *et_base = static_cast<const ET *>(p.et);
    {
        const int32_t *gc = p.cols + grp[kGroupColOff];
        for (int i = threadIdx.x; i < ncols_pad; i += blockDim.x) s_cols[i] = gc[i];
    }
    // Row copies: lane l copies piece (l & 15) of rows (l >> 4) + 2 i, pieces swizzled on their low three bits.
    const int copy_row = lane >> 4, copy_piece = lane & 15;
    const uint32_t row_pitch = static_cast<uint32_t>(H) * kRowBytes;
    auto issue_kv = [&](int h, int j, int b) {
        const uint64_t head_off = static_cast<uint64_t>(h * kRowBytes + copy_piece * 16);
        const int32_t *cj = s_cols + j * kStep + copy_row;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = copy_row + 2 * i;
            const uint64_t off = static_cast<uint64_t>(static_cast<uint32_t>(cj[2 * i])) * row_pitch + head_off;
            const uint32_t dst = s_kv_addr + b * kDqBufBytes + r * kRowBytes + (((copy_piece & 8) | ((copy_piece ^ r) & 7)) << 4);
            cp_async16(dst, reinterpret_cast<const char *>(p.k) + off);
            cp_async16(dst + kKBytes, reinterpret_cast<const char *>(p.v) + off);
        }
    };
    // dQ += dS K reads element 8 dn + g of rows 8 ks + 2 t and 8 ks + 2 t + 1: piece 2 dn + (g >> 2), whose low
    // three bits are swizzled with the row's
    const uint32_t kb_lo = (2 * t) * kRowBytes + (g & 3) * 4;
    const uint32_t kx_lo = static_cast<uint32_t>((g >> 2) ^ (2 * t)), kx_hi = kx_lo ^ 1u;

    for (int mbi = 0; mbi < n_mblocks; ++mbi) {
        const int32_t *mb = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + mbi) * kMbInts;
        const bool use_qr = kHasBias && mb[kMbQrSlot] >= 0;
        const int tq = use_qr ? mb[kMbTq] : 0;
        const uint32_t none_idx = use_qr ? tq : 1;
        const uint32_t chunk_mask = static_cast<uint32_t>(mb[kMbChunkMask]);
        const int4 *pos_base = reinterpret_cast<const int4 *>(p.cellpos + mb[kMbEtOff]) + lane;
        auto next_step = [&](int j) {
            ++j;
            while (j < n_steps && !((chunk_mask >> (j >> 1)) & 1u)) ++j;
            return j;
        };
        __syncthreads();  // previous m-block's indices are no longer read; s_cols is visible
        int primed_step = -1;
        if (warp < H) primed_step = next_step(-1);
        if (primed_step >= 0 && primed_step < n_steps) issue_kv(warp, primed_step, 0);
        cp_async_commit();
        const int row_lo = mb[kMbRowOff + g], row_hi = mb[kMbRowOff + g + 8];
        {
            constexpr int kCellsPerPiece = 16 / static_cast<int>(sizeof(ET));
            const uint4 *ge = reinterpret_cast<const uint4 *>(et_base + mb[kMbEtOff]);
            const int pieces = kTileRows * ncols_pad / kCellsPerPiece;
            for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
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
        __syncthreads();

        for (int h = warp; h < H; h += kWarps) {
            const int64_t off_lo = (static_cast<int64_t>(row_lo < 0 ? 0 : row_lo) * H + h) * kHeadDim;
            const int64_t off_hi = (static_cast<int64_t>(row_hi < 0 ? 0 : row_hi) * H + h) * kHeadDim;
            float qa[8][4], da[8][4];
            load_q_frags(p.q + off_lo, p.q + off_hi, t, qa);
            load_q_frags(p.d_o + off_lo, p.d_o + off_hi, t, da);
            float delta_lo = 0.f, delta_hi = 0.f;
            {
                const float *o_lo = p.o + off_lo + t, *o_hi = p.o + off_hi + t;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    delta_lo = fmaf(da[s][0], __ldg(o_lo + 8 * s), fmaf(da[s][2], __ldg(o_lo + 8 * s + 4), delta_lo));
                    delta_hi = fmaf(da[s][1], __ldg(o_hi + 8 * s), fmaf(da[s][3], __ldg(o_hi + 8 * s + 4), delta_hi));
                }
                delta_lo += __shfl_xor_sync(0xffffffffu, delta_lo, 1);
                delta_lo += __shfl_xor_sync(0xffffffffu, delta_lo, 2);
                delta_hi += __shfl_xor_sync(0xffffffffu, delta_hi, 1);
                delta_hi += __shfl_xor_sync(0xffffffffu, delta_hi, 2);
            }
            float lse2_lo = row_lo < 0 ? 0.f : p.lse[static_cast<int64_t>(row_lo) * H + h];
            float lse2_hi = row_hi < 0 ? 0.f : p.lse[static_cast<int64_t>(row_hi) * H + h];
            lse2_lo = lse2_lo == -INFINITY ? 0.f : lse2_lo * kLog2e;
            lse2_hi = lse2_hi == -INFINITY ? 0.f : lse2_hi * kLog2e;
            if (t == 0) {
                if (row_lo >= 0) p.delta[static_cast<int64_t>(row_lo) * H + h] = delta_lo;
                if (row_hi >= 0) p.delta[static_cast<int64_t>(row_hi) * H + h] = delta_hi;
            }
            {
                // rows with one edge type: the forward folded scale * <q, ak[type]> into lse; take it out again
                float bias_lo = 0.f, bias_hi = 0.f;
                build_score_table<kHasBias>(qa, p.ak, p.n_etypes, use_qr, tq, mb, s_tab, tab_stride, sl2, g, t, bias_lo, bias_hi);
                lse2_lo -= bias_lo;
                lse2_hi -= bias_hi;
            }
            __syncwarp();

            float acc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) { acc[i][0] = 0.f; acc[i][1] = 0.f; acc[i][2] = 0.f; acc[i][3] = 0.f; }
            float *__restrict__ P_h = p.P + h;
            float *__restrict__ dP_h = p.dP + h;

            int j = primed_step;
            if (j < 0) {
                j = next_step(-1);
                if (j < n_steps) issue_kv(h, j, 0);
                cp_async_commit();
            }
            primed_step = -1;
            int buf = 0;
            while (j < n_steps) {
                const int nj = next_step(j);
                const int c0 = j * kStep;
                if (nj < n_steps) issue_kv(h, nj, buf ^ 1);
                cp_async_commit();
                const uint32_t s_k_addr = s_kv_addr + buf * kDqBufBytes, s_v_addr = s_k_addr + kKBytes;
                // the cells' in-CSR positions, in fragment order (cell_pos_index): column groups 2 j and 2 j + 1
                const int4 pos4[2] = {__ldg(pos_base + (j * 2) * 32), __ldg(pos_base + (j * 2 + 1) * 32)};
                cp_async_wait<1>();  // this step's rows have landed; the newest group is the next step's
                __syncwarp();
                float dp[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) { dp[nt][0] = 0.f; dp[nt][1] = 0.f; dp[nt][2] = 0.f; dp[nt][3] = 0.f; }
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {
                    float a_hi[2][4], a_lo[2][4];
                    split4(da[2 * sp], a_hi[0], a_lo[0]);
                    split4(da[2 * sp + 1], a_hi[1], a_lo[1]);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const int r = nt * 8 + (lane & 7), piece = sp * 4 + (lane >> 3);
                        uint32_t b[4];
                        ldmatrix_x4(b, s_v_addr + r * kRowBytes + (((piece & 8) | ((piece ^ r) & 7)) << 4));
                        mma_3xtf32(dp[nt], a_hi[0], a_lo[0], __uint_as_float(b[0]), __uint_as_float(b[1]));
                        mma_3xtf32(dp[nt], a_hi[1], a_lo[1], __uint_as_float(b[2]), __uint_as_float(b[3]));
                    }
                }
                float s[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) { s[nt][0] = 0.f; s[nt][1] = 0.f; s[nt][2] = 0.f; s[nt][3] = 0.f; }
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {
                    float a_hi[2][4], a_lo[2][4];
                    split4(qa[2 * sp], a_hi[0], a_lo[0]);
                    split4(qa[2 * sp + 1], a_hi[1], a_lo[1]);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const int r = nt * 8 + (lane & 7), piece = sp * 4 + (lane >> 3);
                        uint32_t b[4];
                        ldmatrix_x4(b, s_k_addr + r * kRowBytes + (((piece & 8) | ((piece ^ r) & 7)) << 4));
                        mma_3xtf32(s[nt], a_hi[0], a_lo[0], __uint_as_float(b[0]), __uint_as_float(b[1]));
                        mma_3xtf32(s[nt], a_hi[1], a_lo[1], __uint_as_float(b[2]), __uint_as_float(b[3]));
                    }
                }
                // probabilities, the per-edge scratch, dS (kept in s)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int c = c0 + nt * 8 + 2 * t;
                    uint32_t i_lo0, i_lo1, i_hi0, i_hi1;
                    load_idx_pair(s_idx + g * idx_stride + c, i_lo0, i_lo1);
                    load_idx_pair(s_idx + (g + 8) * idx_stride + c, i_hi0, i_hi1);
                    const float tab[4] = {lds_f32(s_tab_lo + 4 * i_lo0), lds_f32(s_tab_lo + 4 * i_lo1),
                                          lds_f32(s_tab_hi + 4 * i_hi0), lds_f32(s_tab_hi + 4 * i_hi1)};
                    const int pos[4] = {pos4[nt].x, pos4[nt].y, pos4[nt].z, pos4[nt].w};
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
                        const float pr = exp2f(fmaf(s[nt][i], sl2, tab[i]) - (i < 2 ? lse2_lo : lse2_hi));
                        const float dpk = dp[nt][i] * keep[i];
                        if (pos[i] >= 0) {
                            P_h[static_cast<int64_t>(pos[i]) * H] = pr;
                            dP_h[static_cast<int64_t>(pos[i]) * H] = dpk;
                        }
                        s[nt][i] = p.scale * pr * (dpk - (i < 2 ? delta_lo : delta_hi));
                    }
                }
                // dQ += dS K.  k index kk of the product stands for column 8 ks + 2 (kk mod 4) + kk / 4 of the step,
                // so that the accumulators of S are the A fragments as they are.
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    const float pa[4] = {s[ks][0], s[ks][2], s[ks][1], s[ks][3]};
                    float p_hi[4], p_lo[4];
                    split4(pa, p_hi, p_lo);
                    const uint32_t k0 = s_k_addr + kb_lo + ks * 8 * kRowBytes;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn) {
                        const uint32_t piece_off = (dn >> 2) * 128;
                        mma_3xtf32(acc[dn], p_hi, p_lo,
                                   lds_f32(k0 + piece_off + (((2u * (dn & 3)) ^ kx_lo) << 4)),
                                   lds_f32(k0 + kRowBytes + piece_off + (((2u * (dn & 3)) ^ kx_hi) << 4)));
                    }
                }
                __syncwarp();  // these buffers are refilled by the step after next
                j = nj;
                buf ^= 1;
            }
            cp_async_wait<0>();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = half ? row_hi : row_lo;
                if (row < 0) continue;
                const int slot = mb[kMbSlotOff + g + 8 * half];
                float *dst = (slot < 0 ? p.dq + (static_cast<int64_t>(row) * H + h) * kHeadDim
                                       : p.part_dq + (static_cast<int64_t>(slot) * H + h) * kHeadDim) + 2 * t;
#pragma unroll
                for (int dn = 0; dn < 8; ++dn)
                    *reinterpret_cast<float2 *>(dst + dn * 8) = make_float2(acc[dn][2 * half], acc[dn][2 * half + 1]);
            }
            __syncwarp();  // the table is rewritten for the next head
        }
    }
}

size_t dq32_smem_bytes(int max_cols_pad, int t_max, int et_bytes) {
    return static_cast<size_t>(kWarps) * kDqStageBytes + static_cast<size_t>(max_cols_pad) * 4 +
           align_up(static_cast<size_t>(kTileRows) * (max_cols_pad + kEtPad) * et_bytes, 16) +
           static_cast<size_t>(kWarps) * kTileRows * tab_stride32(t_max) * 4;
}

template <typename ET, bool kHasBias>
int launch_dq32_kernel(const Dq32Params &p, int64_t n_groups, size_t smem, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>(n_groups);
    if (p.drop.threshold) {
        BPT_CUDA(cudaFuncSetAttribute(attn_backward_dq_tile32_kernel<ET, kHasBias, true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attn_backward_dq_tile32_kernel<ET, kHasBias, true><<<grid, kWarps * 32, smem, stream>>>(p);
    } else {
        BPT_CUDA(cudaFuncSetAttribute(attn_backward_dq_tile32_kernel<ET, kHasBias, false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attn_backward_dq_tile32_kernel<ET, kHasBias, false><<<grid, kWarps * 32, smem, stream>>>(p);
    }
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}


// ------------------------------------------------------------------ backward, source side
//
// dV[src] = sum_dst p' dO[dst] and dK[src] = sum_dst dS q[dst] on the transposed tile plan (an m-block is <= 16
// source rows, its columns are the destinations that attend to them, every cell knows its edge's in-CSR
// position), from the fp32 scratch the destination side left: p' = p * dropout factor, dS = scale * p *
// (dp - delta[dst]).  One block per tile, a warp takes heads w, w + kDkvWarps, ...; per 16 destinations the
// warp stages their dO and Q rows (272-byte pitch, plain 4-byte loads for the B fragments) while it holds the
// step's 8 + 8 weights per lane, gathered a step ahead; the cell positions come in fragment order, so a lane's
// four cells of a column group are the A fragment of m16n8k8 under the k <-> column permutation of the
// forward.  Rows spread over several m-blocks write fp32 partials that are summed in slot order.
struct Dkv32Params {
    const int32_t *groups, *mblocks, *cols, *cellpos;
    const float *P, *dP, *delta, *q, *d_o;
    float *dk, *dv, *part;
    int H, max_cols_pad;
    float scale;
    Dropout drop;
};
constexpr int kDkvWarps = 4;                         // three blocks per SM at 168 registers
constexpr int kDkvTileBytes = kStep * kVPitch;        // 16 rows, 272 bytes apart
constexpr int kDkvStageBytes = 2 * kDkvTileBytes;     // per warp: dO rows, Q rows of one step

template <bool kDrop>
__global__ void __launch_bounds__(kDkvWarps * 32, 3)
attn_backward_dkv_tile32_kernel(const Dkv32Params p) {
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: per warp {dO tile, Q tile} | destination ids
    int32_t *s_cols = reinterpret_cast<int32_t *>(smem + kDkvWarps * kDkvStageBytes);
    const int32_t *grp = p.groups + static_cast<int64_t>(blockIdx.x) * kGroupInts;
    const int n_mblocks = grp[kGroupMbCount];
    if (n_mblocks == 0) return;
    const int ncols_pad = grp[kGroupNcolsPad];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int H = p.H;
    const uint32_t s_do = static_cast<uint32_t>(__cvta_generic_to_shared(smem + warp * kDkvStageBytes));
    {
        const int32_t *gc = p.cols + grp[kGroupColOff];
        for (int i = threadIdx.x; i < ncols_pad; i += blockDim.x) s_cols[i] = gc[i];
    }
    __syncthreads();
    const int n_steps = ncols_pad / kStep;
    const int copy_row = lane >> 4, copy_piece = lane & 15;
    const uint32_t row_pitch = static_cast<uint32_t>(H) * kRowBytes;
    auto issue_rows = [&](int h, int j) {
        const uint64_t head_off = static_cast<uint64_t>(h * kRowBytes + copy_piece * 16);
        const int32_t *cj = s_cols + j * kStep + copy_row;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint64_t off = static_cast<uint64_t>(static_cast<uint32_t>(cj[2 * i])) * row_pitch + head_off;
            const uint32_t dst = s_do + (copy_row + 2 * i) * kVPitch + copy_piece * 16;
            cp_async16(dst, reinterpret_cast<const char *>(p.d_o) + off);
            cp_async16(dst + kDkvTileBytes, reinterpret_cast<const char *>(p.q) + off);
        }
    };
    for (int mbi = 0; mbi < n_mblocks; ++mbi) {
        const int32_t *mb = p.mblocks + static_cast<int64_t>(grp[kGroupMbFirst] + mbi) * kMbInts;
        const uint32_t chunk_mask = static_cast<uint32_t>(mb[kMbChunkMask]);
        static_assert(kMaskCols == 2 * kStep, "two pipeline steps per mask bit");
        auto next_step = [&](int j) {
            ++j;
            while (j < n_steps && !((chunk_mask >> (j >> 1)) & 1u)) ++j;
            return j;
        };
        const int4 *pos_base = reinterpret_cast<const int4 *>(p.cellpos + mb[kMbEtOff]) + lane;
        const int row_lo = mb[kMbRowOff + g], row_hi = mb[kMbRowOff + g + 8];
        // this lane's 8 cells of step j (rows g / g + 8, destinations 8 nt + 2 t, + 1): p and dp, and delta of its
        // four destinations
        auto gather_weights = [&](int h, int j, float (&wp)[8], float (&wd)[8], float (&dl)[4]) {
            const float *__restrict__ P_h = p.P + h;
            const float *__restrict__ dP_h = p.dP + h;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int4 pos4 = __ldg(pos_base + (j * 2 + nt) * 32);
                const int pos[4] = {pos4.x, pos4.y, pos4.z, pos4.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const bool on = pos[i] >= 0;
                    wp[4 * nt + i] = on ? __ldg(P_h + static_cast<int64_t>(pos[i]) * H) : 0.f;
                    wd[4 * nt + i] = on ? __ldg(dP_h + static_cast<int64_t>(pos[i]) * H) : 0.f;
                }
                const int c = j * kStep + nt * 8 + 2 * t;
                dl[2 * nt] = __ldg(p.delta + static_cast<int64_t>(s_cols[c]) * H + h);
                dl[2 * nt + 1] = __ldg(p.delta + static_cast<int64_t>(s_cols[c + 1]) * H + h);
            }
        };
        for (int h = warp; h < H; h += kDkvWarps) {
            float dk[8][4], dv[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int u = 0; u < 4; ++u) { dk[i][u] = 0.f; dv[i][u] = 0.f; }
            int j = next_step(-1);
            if (j < n_steps) issue_rows(h, j);
            cp_async_commit();
            float wp[8], wd[8], dl[4];
            if (j < n_steps) gather_weights(h, j, wp, wd, dl);
            while (j < n_steps) {
                const int nj = next_step(j);
                // p' (the weight V was summed with) and dS of this step's cells
                float pw[8], ds[8];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    float keep[4] = {1.f, 1.f, 1.f, 1.f};
                    if (kDrop) {
                        const int c = j * kStep + nt * 8 + 2 * t;
                        const int dst0 = s_cols[c], dst1 = s_cols[c + 1];
                        keep[0] = dropout_factor(p.drop, dst0, row_lo, h);
                        keep[1] = dropout_factor(p.drop, dst1, row_lo, h);
                        keep[2] = dropout_factor(p.drop, dst0, row_hi, h);
                        keep[3] = dropout_factor(p.drop, dst1, row_hi, h);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float pr = wp[4 * nt + i];
                        pw[4 * nt + i] = pr * keep[i];
                        ds[4 * nt + i] = p.scale * pr * (wd[4 * nt + i] - dl[2 * nt + (i & 1)]);
                    }
                }
                // the next step's weights travel during this step's products
                if (nj < n_steps) gather_weights(h, nj, wp, wd, dl);
                cp_async_wait<0>();  // this step's rows have landed
                __syncwarp();
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    // cells {(g, c), (g, c + 1), (g + 8, c), (g + 8, c + 1)} -> A fragment {a0, a2, a1, a3}
                    const float ap[4] = {pw[4 * nt], pw[4 * nt + 2], pw[4 * nt + 1], pw[4 * nt + 3]};
                    const float as[4] = {ds[4 * nt], ds[4 * nt + 2], ds[4 * nt + 1], ds[4 * nt + 3]};
                    float p_hi[4], p_lo[4], s_hi[4], s_lo[4];
                    split4(ap, p_hi, p_lo);
                    split4(as, s_hi, s_lo);
                    const uint32_t r0 = s_do + (8 * nt + 2 * t) * kVPitch + g * 4;
#pragma unroll
                    for (int dn = 0; dn < 8; ++dn) {
                        mma_3xtf32(dv[dn], p_hi, p_lo, lds_f32(r0 + dn * 32), lds_f32(r0 + kVPitch + dn * 32));
                        mma_3xtf32(dk[dn], s_hi, s_lo, lds_f32(r0 + kDkvTileBytes + dn * 32),
                                   lds_f32(r0 + kDkvTileBytes + kVPitch + dn * 32));
                    }
                }
                __syncwarp();  // every lane has read the tiles: they may be refilled
                if (nj < n_steps) issue_rows(h, nj);
                cp_async_commit();
                j = nj;
            }
            cp_async_wait<0>();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = half ? row_hi : row_lo;
                if (row < 0) continue;
                const int slot = mb[kMbSlotOff + g + 8 * half];
                float *out_k, *out_v;
                if (slot < 0) {
                    const int64_t off = (static_cast<int64_t>(row) * H + h) * kHeadDim + 2 * t;
                    out_k = p.dk + off;
                    out_v = p.dv + off;
                } else {
                    // partial layout of the sum-merge kernel: [slot][dK (H*64) | dV (H*64)]
                    out_k = p.part + static_cast<int64_t>(slot) * 2 * H * kHeadDim + h * kHeadDim + 2 * t;
                    out_v = out_k + H * kHeadDim;
                }
#pragma unroll
                for (int dn = 0; dn < 8; ++dn) {
                    *reinterpret_cast<float2 *>(out_k + dn * 8) = make_float2(dk[dn][2 * half], dk[dn][2 * half + 1]);
                    *reinterpret_cast<float2 *>(out_v + dn * 8) = make_float2(dv[dn][2 * half], dv[dn][2 * half + 1]);
                }
            }
        }
    }
}

size_t dkv32_smem_bytes(int max_cols_pad) {
    return static_cast<size_t>(kDkvWarps) * kDkvStageBytes + static_cast<size_t>(max_cols_pad) * 4;
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" size_t bpt_attn_forward_tc32_smem_bytes(int max_cols_pad, int t_max, int et_bytes) {
    if (max_cols_pad < 0 || t_max < 0 || (et_bytes != 1 && et_bytes != 2)) return 0;
    return tc32_smem_bytes(max_cols_pad, t_max, et_bytes);
}

extern "C" int bpt_attn_forward_tc32(const bpt_tile_plan_t *tiles, int64_t n_nodes, int n_etypes, const void *q,
                                     const void *k, const void *v, const void *ak, double scale, void *o, float *lse,
                                     int h, int d, void *workspace, size_t workspace_bytes,
                                     const bpt_dropout_t *dropout, bpt_stream_t stream_) {
    BPT_CHECK_ARG(tiles != nullptr, "attn_forward_tc32: null tile plan");
    BPT_CHECK_ARG(dropout == nullptr || (dropout->rate >= 0.0 && dropout->rate < 1.0),
                  "attn_forward_tc32: dropout rate must be in [0, 1)");
    BPT_CHECK_ARG(tiles->n_groups >= 0 && tiles->n_split >= 0 && tiles->n_slots >= 0 && h >= 1 && h <= 65535 &&
                      n_nodes >= 0 && n_etypes >= 1,
                  "attn_forward_tc32: bad sizes");
    if (d != kHeadDim) return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc32: head dim 64 only (got %d)", d);
    if (tiles->n_row_items != 0)
        return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc32: tile plans with CUDA-core row items are not supported");
    if (tiles->n_groups == 0) return BPT_OK;
    BPT_CHECK_ARG(q && k && v && o && lse && tiles->groups && tiles->mblocks, "attn_forward_tc32: null tensor");
    BPT_CHECK_ARG(tiles->max_cols_pad == 0 || (tiles->cols && tiles->et), "attn_forward_tc32: null plan arrays");
    BPT_CHECK_ARG(tiles->et_bytes == 1 || tiles->et_bytes == 2, "attn_forward_tc32: et_bytes must be 1 or 2");
    BPT_CHECK_ARG(tiles->max_cols_pad % kTileChunk == 0 && tiles->t_max % 8 == 0 && tiles->n_groups < (int64_t(1) << 31),
                  "attn_forward_tc32: bad plan sizes");
    BPT_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                    reinterpret_cast<uintptr_t>(ak) | reinterpret_cast<uintptr_t>(o)) & 15) == 0,
                  "attn_forward_tc32: tensors must be 16-byte aligned");
    cudaStream_t stream = as_stream(stream_);
    Workspace ws(workspace, workspace_bytes);
    float *part_o = ws.take<float>(static_cast<size_t>(tiles->n_slots) * h * kHeadDim);
    float *part_ml = ws.take<float>(static_cast<size_t>(tiles->n_slots) * h * 2);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_forward_tc32: workspace of %zu bytes is too small", workspace_bytes);

    const bool bias = ak != nullptr;
    Tc32Params p{};
    p.groups = tiles->groups; p.mblocks = tiles->mblocks; p.cols = tiles->cols; p.et = tiles->et;
    p.q = static_cast<const float *>(q); p.k = static_cast<const float *>(k); p.v = static_cast<const float *>(v);
    p.ak = static_cast<const float *>(ak);
    p.o = static_cast<float *>(o); p.lse = lse; p.part_o = part_o; p.part_ml = part_ml;
    p.n_etypes = n_etypes; p.H = h; p.max_cols_pad = tiles->max_cols_pad;
    p.t_max = bias ? tiles->t_max : 0;
    p.tab_stride = tab_stride32(p.t_max);
    p.scale = static_cast<float>(scale);
    p.n_groups = tiles->n_groups;
    p.drop = make_dropout(dropout);
    if (tiles->et_bytes == 1 && p.t_max > kMaxTypes8)
        return fail(BPT_ERR_INVALID, "attn_forward_tc32: 8-bit cells need t_max <= %d (got %d)", kMaxTypes8, p.t_max);
    const size_t smem = tc32_smem_bytes(tiles->max_cols_pad, p.t_max, tiles->et_bytes);
    if (smem > 227 * 1024)
        return fail(BPT_ERR_UNSUPPORTED, "attn_forward_tc32: tile plan needs %zu bytes of shared memory", smem);
    int rc;
    if (tiles->et_bytes == 1)
        rc = bias ? launch_tile32_kernel<uint8_t, true>(p, tiles->n_groups, smem, stream)
                  : launch_tile32_kernel<uint8_t, false>(p, tiles->n_groups, smem, stream);
    else
        rc = bias ? launch_tile32_kernel<uint16_t, true>(p, tiles->n_groups, smem, stream)
                  : launch_tile32_kernel<uint16_t, false>(p, tiles->n_groups, smem, stream);
    if (rc) return rc;
    if (tiles->n_split > 0) {
        const Geometry g{h, kHeadDim};
        attn_forward_merge_kernel<float><<<static_cast<unsigned>(tiles->n_split), merge_threads(h, kHeadDim),
                                           merge_smem_bytes(h), stream>>>(
            reinterpret_cast<const int4 *>(tiles->split_rows), static_cast<int>(tiles->n_split), part_o, part_ml,
            static_cast<float *>(o), lse, g);
        BPT_LAUNCH_CHECK();
    }
    return BPT_OK;
}

namespace {
size_t dkv_slots(const bpt_tile_plan_t *src_tiles, const int32_t *counts_host) {
    const size_t a = static_cast<size_t>(counts_host[4]);
    const size_t b = src_tiles ? static_cast<size_t>(src_tiles->n_slots) : 0;
    return a > b ? a : b;
}
}  // namespace

extern "C" size_t bpt_attn_backward_tc32_workspace_bytes(const bpt_tile_plan_t *tiles, const bpt_tile_plan_t *src_tiles,
                                                         const int32_t *counts_host, int64_t n_nodes, int64_t n_edges,
                                                         int h) {
    if (!tiles || !counts_host || n_nodes < 0 || n_edges < 0 || h < 1) return 0;
    const size_t e = static_cast<size_t>(n_edges);
    return 2 * align_up(e * h * 4, 256) + align_up(static_cast<size_t>(n_nodes) * h * 4, 256) +
           align_up(static_cast<size_t>(tiles->n_slots) * h * kHeadDim * 4, 256) +
           align_up(dkv_slots(src_tiles, counts_host) * 2 * h * kHeadDim * 4, 256) +
           align_up(static_cast<size_t>(counts_host[7]) * kHeadDim * 4, 256) +
           align_up(type_table_f32_elems(tiles->t_max, n_nodes, h) * 4, 256) + 2048;
}

extern "C" int bpt_attn_backward_tc32(const bpt_tile_plan_t *tiles, const bpt_tile_plan_t *src_tiles,
                                      const void *attn_plan, const int32_t *counts_host, int64_t n_nodes, int64_t n_edges, int n_etypes, const void *q, const void *k,
                                      const void *v, const void *ak, double scale, const void *o, const float *lse,
                                      const void *d_o, void *dq, void *dk, void *dv, float *dak, int h, int d,
                                      void *workspace, size_t workspace_bytes, const bpt_dropout_t *dropout,
                                      bpt_stream_t stream_) {
    BPT_CHECK_ARG(tiles != nullptr && attn_plan != nullptr && counts_host != nullptr, "attn_backward_tc32: null plan");
    BPT_CHECK_ARG(dropout == nullptr || (dropout->rate >= 0.0 && dropout->rate < 1.0),
                  "attn_backward_tc32: dropout rate must be in [0, 1)");
    BPT_CHECK_ARG(tiles->n_groups >= 0 && tiles->n_split >= 0 && tiles->n_slots >= 0 && h >= 1 && h <= 40 &&
                      n_nodes >= 0 && n_edges >= 0 && n_etypes >= 1,
                  "attn_backward_tc32: bad sizes");
    if (d != kHeadDim) return fail(BPT_ERR_UNSUPPORTED, "attn_backward_tc32: head dim 64 only (got %d)", d);
    if (tiles->n_row_items != 0)
        return fail(BPT_ERR_UNSUPPORTED, "attn_backward_tc32: tile plans with CUDA-core row items are not supported");
    if (n_nodes == 0) return BPT_OK;
    BPT_CHECK_ARG(q && k && v && o && lse && d_o && dq, "attn_backward_tc32: null tensor");
    BPT_CHECK_ARG((dk == nullptr) == (dv == nullptr), "attn_backward_tc32: dk and dv must both be given or both be NULL");
    BPT_CHECK_ARG(ak == nullptr || dak != nullptr, "attn_backward_tc32: ak given without dak");
    BPT_CHECK_ARG(tiles->n_groups == 0 || (tiles->groups && tiles->mblocks), "attn_backward_tc32: null plan arrays");
    BPT_CHECK_ARG(tiles->max_cols_pad == 0 || (tiles->cols && tiles->et && tiles->cell_pos),
                  "attn_backward_tc32: the tile plan must carry cell types and cell positions");
    BPT_CHECK_ARG(tiles->et_bytes == 1 || tiles->et_bytes == 2, "attn_backward_tc32: et_bytes must be 1 or 2");
    BPT_CHECK_ARG(tiles->max_cols_pad % kTileChunk == 0 && tiles->t_max % 8 == 0 && tiles->n_groups < (int64_t(1) << 31),
                  "attn_backward_tc32: bad plan sizes");
    BPT_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                    reinterpret_cast<uintptr_t>(ak) | reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(d_o) |
                    reinterpret_cast<uintptr_t>(dq)) & 15) == 0,
                  "attn_backward_tc32: tensors must be 16-byte aligned");
    cudaStream_t stream = as_stream(stream_);
    const PlanView pv = plan_view(const_cast<void *>(attn_plan), n_nodes, counts_host[kCountsNSrc], n_edges, n_etypes);
    Workspace ws(workspace, workspace_bytes);
    const size_t e = static_cast<size_t>(n_edges);
    float *P = ws.take<float>(e * h);
    float *dP = ws.take<float>(e * h);
    float *delta = ws.take<float>(static_cast<size_t>(n_nodes) * h);
    float *part_dq = ws.take<float>(static_cast<size_t>(tiles->n_slots) * h * kHeadDim);
    float *part_dkv = ws.take<float>(dkv_slots(src_tiles, counts_host) * 2 * h * kHeadDim);
    float *part_dak = ws.take<float>(static_cast<size_t>(counts_host[7]) * kHeadDim);
    const size_t table_elems = ak != nullptr ? type_table_f32_elems(tiles->t_max, n_nodes, h) : 0;
    float *G = ws.take<float>(table_elems);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_backward_tc32: workspace of %zu bytes is too small", workspace_bytes);
    const float sc = static_cast<float>(scale);
    const Dropout drop = make_dropout(dropout);
    // Every row is in some m-block of the tile plan (rows without edges form m-blocks without columns), so the
    // tile kernels write every row of dQ, dK and dV; delta is cleared because only the tile kernel's lanes of
    // real rows write it.
    BPT_CUDA(cudaMemsetAsync(delta, 0, static_cast<size_t>(n_nodes) * h * sizeof(float), stream));
    if (tiles->n_groups == 0)  // a plan without a single m-block writes nothing
        BPT_CUDA(cudaMemsetAsync(dq, 0, static_cast<size_t>(n_nodes) * h * kHeadDim * sizeof(float), stream));
    if (tiles->n_groups > 0) {
        const bool bias = ak != nullptr;
        Dq32Params p{};
        p.groups = tiles->groups; p.mblocks = tiles->mblocks; p.cols = tiles->cols; p.cellpos = tiles->cell_pos;
        p.et = tiles->et;
        p.q = static_cast<const float *>(q); p.k = static_cast<const float *>(k); p.v = static_cast<const float *>(v);
        p.ak = static_cast<const float *>(ak); p.o = static_cast<const float *>(o);
        p.d_o = static_cast<const float *>(d_o); p.lse = lse;
        p.P = P; p.dP = dP; p.delta = delta; p.part_dq = part_dq; p.dq = static_cast<float *>(dq);
        p.n_etypes = n_etypes; p.H = h; p.max_cols_pad = tiles->max_cols_pad;
        p.t_max = bias ? tiles->t_max : 0;
        p.tab_stride = tab_stride32(p.t_max);
        p.scale = sc;
        p.n_groups = tiles->n_groups;
        p.drop = drop;
        if (tiles->et_bytes == 1 && p.t_max > kMaxTypes8)
            return fail(BPT_ERR_INVALID, "attn_backward_tc32: 8-bit cells need t_max <= %d (got %d)", kMaxTypes8, p.t_max);
        const size_t smem = dq32_smem_bytes(tiles->max_cols_pad, p.t_max, tiles->et_bytes);
        if (smem > 227 * 1024)
            return fail(BPT_ERR_UNSUPPORTED, "attn_backward_tc32: tile plan needs %zu bytes of shared memory", smem);
        int rc;
        if (tiles->et_bytes == 1)
            rc = bias ? launch_dq32_kernel<uint8_t, true>(p, tiles->n_groups, smem, stream)
                      : launch_dq32_kernel<uint8_t, false>(p, tiles->n_groups, smem, stream);
        else
            rc = bias ? launch_dq32_kernel<uint16_t, true>(p, tiles->n_groups, smem, stream)
                      : launch_dq32_kernel<uint16_t, false>(p, tiles->n_groups, smem, stream);
        if (rc) return rc;
        if (int rc2 = launch_sum_merge_f32(reinterpret_cast<const int4 *>(tiles->split_rows),
                                           static_cast<int>(tiles->n_split), part_dq, h * kHeadDim,
                                           static_cast<float *>(dq), stream))
            return rc2;
    }
    // source side on the transposed tile plan when one is given (else on the CUDA-core kernel below)
    bool dkv_done = false;
    if (src_tiles != nullptr && dk != nullptr && dv != nullptr) {
        BPT_CHECK_ARG(src_tiles->n_groups >= 0 && src_tiles->n_groups < (int64_t(1) << 31) && src_tiles->n_split >= 0 &&
                          src_tiles->n_slots >= 0 && src_tiles->max_cols_pad % kTileChunk == 0,
                      "attn_backward_tc32: bad transposed tile plan sizes");
        BPT_CHECK_ARG(src_tiles->n_groups == 0 || (src_tiles->groups && src_tiles->mblocks),
                      "attn_backward_tc32: null transposed plan arrays");
        BPT_CHECK_ARG(src_tiles->max_cols_pad == 0 || (src_tiles->cols && src_tiles->cell_pos),
                      "attn_backward_tc32: the transposed tile plan must carry cell positions");
        BPT_CHECK_ARG(src_tiles->n_split == 0 || src_tiles->split_rows, "attn_backward_tc32: null split rows");
        BPT_CHECK_ARG(((reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15) == 0,
                      "attn_backward_tc32: tensors must be 16-byte aligned");
        const size_t smem = dkv32_smem_bytes(src_tiles->max_cols_pad);
        if (smem <= 227 * 1024) {
            if (src_tiles->n_groups == 0) {
                const size_t kv_bytes = static_cast<size_t>(counts_host[kCountsNSrc]) * h * kHeadDim * sizeof(float);
                BPT_CUDA(cudaMemsetAsync(dk, 0, kv_bytes, stream));
                BPT_CUDA(cudaMemsetAsync(dv, 0, kv_bytes, stream));
            }
            if (src_tiles->n_groups > 0) {
                Dkv32Params kp{};
                kp.groups = src_tiles->groups; kp.mblocks = src_tiles->mblocks; kp.cols = src_tiles->cols;
                kp.cellpos = src_tiles->cell_pos;
                kp.P = P; kp.dP = dP; kp.delta = delta;
                kp.q = static_cast<const float *>(q); kp.d_o = static_cast<const float *>(d_o);
                kp.dk = static_cast<float *>(dk); kp.dv = static_cast<float *>(dv); kp.part = part_dkv;
                kp.H = h; kp.max_cols_pad = src_tiles->max_cols_pad; kp.scale = sc; kp.drop = drop;
                const unsigned grid = static_cast<unsigned>(src_tiles->n_groups);
                if (drop.threshold) {
                    BPT_CUDA(cudaFuncSetAttribute(attn_backward_dkv_tile32_kernel<true>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
                    attn_backward_dkv_tile32_kernel<true><<<grid, kDkvWarps * 32, smem, stream>>>(kp);
                } else {
                    BPT_CUDA(cudaFuncSetAttribute(attn_backward_dkv_tile32_kernel<false>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
                    attn_backward_dkv_tile32_kernel<false><<<grid, kDkvWarps * 32, smem, stream>>>(kp);
                }
                BPT_LAUNCH_CHECK();
                if (int rc3 = launch_sum_merge_f32(reinterpret_cast<const int4 *>(src_tiles->split_rows),
                                                   static_cast<int>(src_tiles->n_split), part_dkv, h * kHeadDim,
                                                   static_cast<float *>(dk), stream, static_cast<float *>(dv)))
                    return rc3;
            }
            dkv_done = true;
        }
    }
    // relative-position gradients: per-row type table and two fp32 GEMMs where the table applies, else the
    // per-edge CUDA-core kernels below
    bool ak_done = false;
    if (table_elems > 0) {
        if (int rc4 = launch_type_table_terms_f32(pv, tiles->t_max, n_etypes, static_cast<const float *>(q),
                                                  static_cast<const float *>(ak), P, dP, delta, sc,
                                                  static_cast<float *>(dq), dak, G, h, stream))
            return rc4;
        ak_done = true;
    }
    if (ak_done && dkv_done) return BPT_OK;
    if (ak_done) ak = nullptr;
    return launch_backward_rest_f32(pv, counts_host, static_cast<const float *>(q), static_cast<const float *>(ak),
                                    static_cast<const float *>(d_o), P, dP, delta, sc, static_cast<float *>(dq),
                                    dkv_done ? nullptr : static_cast<float *>(dk),
                                    dkv_done ? nullptr : static_cast<float *>(dv), dak, part_dkv, part_dak, h, d,
                                    drop, stream);
}
