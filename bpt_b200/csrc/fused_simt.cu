// Fused graph attention, CUDA-core path: one warp per work item (a destination row or a
// <=128-edge slice of one), any head count, head dim <= 128, fp32 / bf16 / fp16 storage with
// fp32 arithmetic.
//
// Forward = the reference's masked_mm -> node_mul_edge -> scale -> sparse_softmax ->
// vec_spmm chain (modules/attention.py:66-77) in one pass per destination row: scores live
// in shared memory, never in HBM; only O and the row log-sum-exp are written.
// Backward = three segment reductions with one writer per output element:
//   over the in-CSR   : P, dP, delta (scratch) and dQ
//   over the out-CSR  : dK, dV
//   over type buckets : d embed_ak
// Rows longer than a work item are reduced in item order by a merge kernel, so every
// result is bitwise reproducible (the reference's are not: graph_kernel/atomic.cuh).
#include <mutex>

#include "fused_common.cuh"
#include "plan.cuh"

namespace bpt {
namespace {

constexpr int kWarpsPerBlock = 4;

// ---- 16-element slice loads/stores: each lane owns 16 consecutive elements of a head ----

template <typename T, bool kVec>
__device__ __forceinline__ void load16(const T *__restrict__ p, int nvalid, float (&out)[16]);

template <>
__device__ __forceinline__ void load16<float, true>(const float *__restrict__ p, int, float (&out)[16]) {
    const float4 *v = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 x = __ldg(v + i);
        out[4 * i] = x.x; out[4 * i + 1] = x.y; out[4 * i + 2] = x.z; out[4 * i + 3] = x.w;
    }
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16, true>(const __nv_bfloat16 *__restrict__ p, int,
                                                            float (&out)[16]) {
    const uint4 *v = reinterpret_cast<const uint4 *>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint4 x = __ldg(v + i);
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // bf16 -> fp32 is a 16-bit shift
            out[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
            out[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}
template <>
__device__ __forceinline__ void load16<__half, true>(const __half *__restrict__ p, int, float (&out)[16]) {
    const uint4 *v = reinterpret_cast<const uint4 *>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint4 x = __ldg(v + i);
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
            out[8 * i + 2 * j] = f.x;
            out[8 * i + 2 * j + 1] = f.y;
        }
    }
}
template <typename T>
__device__ __forceinline__ void load16_scalar(const T *__restrict__ p, int nvalid, float (&out)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = i < nvalid ? to_acc(p[i]) : 0.f;
}
template <> __device__ __forceinline__ void load16<float, false>(const float *__restrict__ p, int n, float (&o)[16]) { load16_scalar(p, n, o); }
template <> __device__ __forceinline__ void load16<__nv_bfloat16, false>(const __nv_bfloat16 *__restrict__ p, int n, float (&o)[16]) { load16_scalar(p, n, o); }
template <> __device__ __forceinline__ void load16<__half, false>(const __half *__restrict__ p, int n, float (&o)[16]) { load16_scalar(p, n, o); }

template <typename T>
__device__ __forceinline__ void store16(T *__restrict__ p, int nvalid, const float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
        if (i < nvalid) p[i] = from_acc<T>(v[i]);
}

template <int LPH>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int off = LPH / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}


// ------------------------------------------------------------------ forward

template <typename T, int LPH, bool kVec>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attn_forward_kernel(const int4 *__restrict__ items, int n_items, const int32_t *__restrict__ in_src,
                    const int32_t *__restrict__ in_etype, const T *__restrict__ q,
                    const T *__restrict__ k, const T *__restrict__ v, const T *__restrict__ ak,
                    float scale, T *__restrict__ o, float *__restrict__ lse,
                    float *__restrict__ part_o, float *__restrict__ part_ml, Geometry g, Dropout drop) {
    constexpr int HPW = 32 / LPH;
    __shared__ float s_all[kWarpsPerBlock][kSegEdges * HPW];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * kWarpsPerBlock + warp;
    if (item >= n_items) return;
    const int4 it = items[item];
    const int row = it.x, beg = it.y, n = it.z - it.y, slot = it.w;
    const int hl = lane / LPH, gl = lane % LPH;
    const int head = blockIdx.y * HPW + hl;
    const int d0 = gl * 16;
    int nvalid = g.D - d0;
    nvalid = nvalid > 16 ? 16 : nvalid;
    const bool active = head < g.H && nvalid > 0;
    const int H = g.H, D = g.D;
    float *sc = s_all[warp];

    float qf[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) qf[i] = 0.f;
    if (active) load16<T, kVec>(q + (static_cast<int64_t>(row) * H + head) * D + d0, nvalid, qf);
    const float qs = scale * kLog2e;  // scores are kept in the log2 domain
#pragma unroll
    for (int i = 0; i < 16; ++i) qf[i] *= qs;

    for (int j = 0; j < n; ++j) {
        const int src = in_src[beg + j];
        float part = 0.f;
        if (active) {
            float kf[16];
            load16<T, kVec>(k + (static_cast<int64_t>(src) * H + head) * D + d0, nvalid, kf);
            if (ak) {
                float af[16];
                load16<T, kVec>(ak + static_cast<int64_t>(in_etype[beg + j]) * D + d0, nvalid, af);
#pragma unroll
                for (int i = 0; i < 16; ++i) kf[i] += af[i];
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) part = fmaf(qf[i], kf[i], part);
        }
        part = group_sum<LPH>(part);
        if (gl == 0) sc[j * HPW + hl] = part;
    }
    __syncwarp();

    // Row statistics: this lane looks at head (lane % HPW), edges lane / HPW, + LPH, ...
    const int hh = lane % HPW;
    float m = -INFINITY;
    for (int j = lane / HPW; j < n; j += LPH) m = fmaxf(m, sc[j * HPW + hh]);
#pragma unroll
    for (int off = HPW; off < 32; off <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float l = 0.f;
    for (int j = lane / HPW; j < n; j += LPH) {
        const float p = exp2f(sc[j * HPW + hh] - m);
        sc[j * HPW + hh] = p;
        l += p;
    }
#pragma unroll
    for (int off = HPW; off < 32; off <<= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
    __syncwarp();
    const float m_h = __shfl_sync(0xffffffffu, m, hl);  // lane hl holds head hl's statistics
    const float l_h = __shfl_sync(0xffffffffu, l, hl);

    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    if (active) {
        #pragma unroll 4
        for (int j = 0; j < n; ++j) {
            const int src = in_src[beg + j];
            float p = sc[j * HPW + hl];
            if (drop.threshold) p *= dropout_factor(drop, row, src, head);  // the sum l keeps every weight
            float vf[16];
            load16<T, kVec>(v + (static_cast<int64_t>(src) * H + head) * D + d0, nvalid, vf);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = fmaf(p, vf[i], acc[i]);
        }
    }
    if (!active) return;
    if (slot < 0) {
        const float inv = n > 0 ? 1.f / l_h : 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] *= inv;
        store16<T>(o + (static_cast<int64_t>(row) * H + head) * D + d0, nvalid, acc);
        if (gl == 0) lse[static_cast<int64_t>(row) * H + head] = n > 0 ? (m_h + log2f(l_h)) * kLn2 : -INFINITY;
    } else {
        store16<float>(part_o + (static_cast<int64_t>(slot) * H + head) * D + d0, nvalid, acc);
        if (gl == 0) {
            part_ml[(static_cast<int64_t>(slot) * H + head) * 2] = m_h;
            part_ml[(static_cast<int64_t>(slot) * H + head) * 2 + 1] = l_h;
        }
    }
}

// ------------------------------------------------------------------ backward, pass over destinations
//
// With p_e the edge's probability and dp_e = <dO[dst], v[src_e]>, the score gradient is
// dS_e = scale * p_e * (dp_e - delta), delta = sum_e p_e * dp_e.  delta equals <dO, O>, but O
// is stored rounded (bf16), and on rows whose edges all share one type the gradient of
// embed_ak is sum_e dS_e = 0 exactly only if delta is the sum over the same p_e; so delta is
// accumulated here, in fp32, and O is not read at all.  One pass suffices because
//   dQ = scale * (A - delta * B),  A = sum_e p_e dp_e kk_e,  B = sum_e p_e kk_e,
// with kk_e = k[src_e] + ak[etype_e].  P and dP go to scratch in in-CSR order; the later
// passes rebuild dS from them and delta.

template <typename T, int LPH, bool kVec>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attn_backward_dq_kernel(const int4 *__restrict__ items, int n_items, const int32_t *__restrict__ in_src,
                        const int32_t *__restrict__ in_etype, const T *__restrict__ q,
                        const T *__restrict__ k, const T *__restrict__ v, const T *__restrict__ ak,
                        float scale, const float *__restrict__ lse, const T *__restrict__ d_o,
                        float *__restrict__ P, float *__restrict__ dP, float *__restrict__ delta_out,
                        T *__restrict__ dq, float *__restrict__ part_ab, float *__restrict__ part_delta,
                        Geometry g, Dropout drop) {
    constexpr int HPW = 32 / LPH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * kWarpsPerBlock + warp;
    if (item >= n_items) return;
    const int4 it = items[item];
    const int row = it.x, beg = it.y, end = it.z, slot = it.w;
    const int hl = lane / LPH, gl = lane % LPH;
    const int head = blockIdx.y * HPW + hl;
    const int d0 = gl * 16;
    int nvalid = g.D - d0;
    nvalid = nvalid > 16 ? 16 : nvalid;
    const bool active = head < g.H && nvalid > 0;
    const int H = g.H, D = g.D;
    const int64_t row_off = (static_cast<int64_t>(row) * H + head) * D + d0;

    float qf[16], dof[16], fa[16], fb[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) { qf[i] = 0.f; dof[i] = 0.f; fa[i] = 0.f; fb[i] = 0.f; }
    float lse2 = 0.f, delta = 0.f;
    if (active) {
        load16<T, kVec>(q + row_off, nvalid, qf);
        load16<T, kVec>(d_o + row_off, nvalid, dof);
        lse2 = lse[static_cast<int64_t>(row) * H + head] * kLog2e;
    }
    const float qs = scale * kLog2e;
#pragma unroll
    for (int i = 0; i < 16; ++i) qf[i] *= qs;

    for (int j = beg; j < end; ++j) {
        const int src = in_src[j];
        float kf[16];
        float s = 0.f, dp = 0.f;
        if (active) {
            const int64_t src_off = (static_cast<int64_t>(src) * H + head) * D + d0;
            float vf[16];
            load16<T, kVec>(k + src_off, nvalid, kf);
            load16<T, kVec>(v + src_off, nvalid, vf);
            if (ak) {
                float af[16];
                load16<T, kVec>(ak + static_cast<int64_t>(in_etype[j]) * D + d0, nvalid, af);
#pragma unroll
                for (int i = 0; i < 16; ++i) kf[i] += af[i];
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                s = fmaf(qf[i], kf[i], s);
                dp = fmaf(dof[i], vf[i], dp);
            }
        }
        s = group_sum<LPH>(s);
        dp = group_sum<LPH>(dp);
        if (active) {
            // with dropout o = sum p' v, p' = mask * p / (1 - rate): the gradient of p is that of p' times the same factor
            if (drop.threshold) dp *= dropout_factor(drop, row, src, head);
            const float p = exp2f(s - lse2);
            const float pdp = p * dp;
            delta += pdp;
            if (gl == 0) {
                P[static_cast<int64_t>(j) * H + head] = p;
                dP[static_cast<int64_t>(j) * H + head] = dp;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                fa[i] = fmaf(pdp, kf[i], fa[i]);
                fb[i] = fmaf(p, kf[i], fb[i]);
            }
        }
    }
    if (!active) return;
    if (slot < 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) fa[i] = scale * (fa[i] - delta * fb[i]);
        store16<T>(dq + row_off, nvalid, fa);
        if (gl == 0) delta_out[static_cast<int64_t>(row) * H + head] = delta;
    } else {
        const int64_t HD = static_cast<int64_t>(H) * D;
        float *base = part_ab + static_cast<int64_t>(slot) * 2 * HD + static_cast<int64_t>(head) * D + d0;
        store16<float>(base, nvalid, fa);
        store16<float>(base + HD, nvalid, fb);
        if (gl == 0) part_delta[static_cast<int64_t>(slot) * H + head] = delta;
    }
}

// Split rows: delta = sum of the slots' deltas, dQ = scale * (sum A - delta * sum B), slot order.
template <typename T>
__global__ void attn_backward_dq_merge_kernel(const int4 *__restrict__ split_rows, int n_split,
                                              const float *__restrict__ part_ab,
                                              const float *__restrict__ part_delta, float scale,
                                              T *__restrict__ dq, float *__restrict__ delta_out, Geometry g) {
    const int sr = blockIdx.x;
    if (sr >= n_split) return;
    const int4 rec = split_rows[sr];
    const int row = rec.x, first = rec.y, count = rec.z;
    const int HD = g.H * g.D;
    for (int c = threadIdx.x; c < HD; c += blockDim.x) {
        const int head = c / g.D;
        float delta = 0.f, a = 0.f, b = 0.f;
        for (int s = 0; s < count; ++s) {
            delta += part_delta[static_cast<int64_t>(first + s) * g.H + head];
            a += part_ab[static_cast<int64_t>(first + s) * 2 * HD + c];
            b += part_ab[static_cast<int64_t>(first + s) * 2 * HD + HD + c];
        }
        dq[static_cast<int64_t>(row) * HD + c] = from_acc<T>(scale * (a - delta * b));
        if (c % g.D == 0) delta_out[static_cast<int64_t>(row) * g.H + head] = delta;
    }
}

// ------------------------------------------------------------------ backward, pass over sources

template <typename T, int LPH, bool kVec>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attn_backward_dkv_kernel(const int4 *__restrict__ items, int n_items, const int32_t *__restrict__ out_dst,
                         const int32_t *__restrict__ out_inpos, const T *__restrict__ q,
                         const T *__restrict__ d_o, const float *__restrict__ P,
                         const float *__restrict__ dP, const float *__restrict__ delta, float scale,
                         T *__restrict__ dk, T *__restrict__ dv, float *__restrict__ part_dkv, Geometry g,
                         Dropout drop) {
    constexpr int HPW = 32 / LPH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * kWarpsPerBlock + warp;
    if (item >= n_items) return;
    const int4 it = items[item];
    const int row = it.x, beg = it.y, end = it.z, slot = it.w;
    const int hl = lane / LPH, gl = lane % LPH;
    const int head = blockIdx.y * HPW + hl;
    const int d0 = gl * 16;
    int nvalid = g.D - d0;
    nvalid = nvalid > 16 ? 16 : nvalid;
    if (!(head < g.H && nvalid > 0)) return;  // no warp-wide operation below
    const int H = g.H, D = g.D;

    float dkf[16], dvf[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) { dkf[i] = 0.f; dvf[i] = 0.f; }
    #pragma unroll 4
    for (int j = beg; j < end; ++j) {
        const int dst = out_dst[j];
        const int64_t pos = out_inpos[j];
        const float p = P[pos * H + head];
        const float ds = scale * p * (dP[pos * H + head] - delta[static_cast<int64_t>(dst) * H + head]);
        const float pv = drop.threshold ? p * dropout_factor(drop, dst, row, head) : p;  // the weight V was summed with
        const int64_t dst_off = (static_cast<int64_t>(dst) * H + head) * D + d0;
        float qf[16], dof[16];
        load16<T, kVec>(q + dst_off, nvalid, qf);
        load16<T, kVec>(d_o + dst_off, nvalid, dof);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            dkf[i] = fmaf(ds, qf[i], dkf[i]);
            dvf[i] = fmaf(pv, dof[i], dvf[i]);
        }
    }
    const int64_t row_off = (static_cast<int64_t>(row) * H + head) * D + d0;
    if (slot < 0) {
        store16<T>(dk + row_off, nvalid, dkf);
        store16<T>(dv + row_off, nvalid, dvf);
    } else {
        const int64_t HD = static_cast<int64_t>(H) * D;
        float *base = part_dkv + static_cast<int64_t>(slot) * 2 * HD + static_cast<int64_t>(head) * D + d0;
        store16<float>(base, nvalid, dkf);
        store16<float>(base + HD, nvalid, dvf);
    }
}

// ------------------------------------------------------------------ backward, pass over type buckets

// kPacked: the per-edge scratch is one 32-bit word {bf16 p, bf16 dS}, laid out [head][in-CSR position]
// with `ps_edges` positions per head, passed as P.
template <typename T, int LPH, bool kVec, bool kPacked = false>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attn_backward_dak_kernel(const int4 *__restrict__ items, int n_items, const int32_t *__restrict__ et_dst,
                         const int32_t *__restrict__ et_inpos, const T *__restrict__ q,
                         const float *__restrict__ P, const float *__restrict__ dP,
                         const float *__restrict__ delta, float scale, float *__restrict__ dak,
                         float *__restrict__ part_dak, Geometry g, int64_t ps_edges = 0) {
    constexpr int HPW = 32 / LPH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * kWarpsPerBlock + warp;
    if (item >= n_items) return;
    const int4 it = items[item];
    const int row = it.x, beg = it.y, end = it.z, slot = it.w;
    const int hl = lane / LPH, gl = lane % LPH;
    const int d0 = gl * 16;
    int nvalid = g.D - d0;
    nvalid = nvalid > 16 ? 16 : nvalid;
    const int H = g.H, D = g.D;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int h0 = 0; h0 < H; h0 += HPW) {
        const int head = h0 + hl;
        if (head < H && nvalid > 0) {
            #pragma unroll 4
            for (int j = beg; j < end; ++j) {
                const int dst = et_dst[j];
                const int64_t pos = et_inpos[j];
                float ds;
                if (kPacked)
                    ds = __uint_as_float(reinterpret_cast<const uint32_t *>(P)[head * ps_edges + pos] & 0xffff0000u);
                else
                    ds = scale * P[pos * H + head] * (dP[pos * H + head] - delta[static_cast<int64_t>(dst) * H + head]);
                float qf[16];
                load16<T, kVec>(q + (static_cast<int64_t>(dst) * H + head) * D + d0, nvalid, qf);
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] = fmaf(ds, qf[i], acc[i]);
            }
        }
    }
    // Sum over the heads held by lanes with the same gl, in a fixed butterfly order.
#pragma unroll
    for (int off = LPH; off < 32; off <<= 1) {
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
    }
    if (hl == 0 && nvalid > 0) {
        float *out = slot < 0 ? dak + static_cast<int64_t>(row) * D + d0
                              : part_dak + static_cast<int64_t>(slot) * D + d0;
        store16<float>(out, nvalid, acc);
    }
}

// dQ += sum_e dS_e * ak[etype_e]: the relative-position part of dQ, for the tensor-core backward,
// whose destination-side kernel only does the K part and leaves {bf16 p, bf16 dS} per (edge, head).  One warp per
// destination row (whole row, fixed edge order); rows whose edges share one type are skipped:
// their sum of dS is zero.
// kPacked = false: the scratch is fp32 P, dP in [in-CSR position][head] order and delta per (row, head),
// dS = scale * p * (dp - delta).
template <typename T, int LPH, bool kVec, bool kPacked = true>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attn_backward_dq_ak_kernel(const int32_t *__restrict__ in_indptr, const int32_t *__restrict__ in_etype,
                           const int32_t *__restrict__ row_uniform, int n_rows, const T *__restrict__ ak,
                           const uint32_t *__restrict__ PS, int64_t ps_edges, T *__restrict__ dq, Geometry g,
                           const float *__restrict__ P = nullptr, const float *__restrict__ dP = nullptr,
                           const float *__restrict__ delta = nullptr, float scale = 1.f) {
    constexpr int HPW = 32 / LPH;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarpsPerBlock + warp;
    if (row >= n_rows || row_uniform[row]) return;
    const int hl = lane / LPH, gl = lane % LPH;
    const int head = blockIdx.y * HPW + hl;
    const int d0 = gl * 16;
    int nvalid = g.D - d0;
    nvalid = nvalid > 16 ? 16 : nvalid;
    if (!(head < g.H && nvalid > 0)) return;
    const int H = g.H, D = g.D;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    const int beg = in_indptr[row], end = in_indptr[row + 1];
#pragma unroll 4
    const float dl = kPacked ? 0.f : delta[static_cast<int64_t>(row) * H + head];
    for (int j = beg; j < end; ++j) {
        float ds;
        if (kPacked)
            ds = __uint_as_float(PS[head * ps_edges + j] & 0xffff0000u);
        else
            ds = scale * P[static_cast<int64_t>(j) * H + head] * (dP[static_cast<int64_t>(j) * H + head] - dl);
        float af[16];
        load16<T, kVec>(ak + static_cast<int64_t>(in_etype[j]) * D + d0, nvalid, af);
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = fmaf(ds, af[i], acc[i]);
    }
    T *out = dq + (static_cast<int64_t>(row) * H + head) * D + d0;
    float cur[16];
    load16<T, kVec>(out, nvalid, cur);
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] += cur[i];
    store16<T>(out, nvalid, acc);
}

// out[row, c] = sum over the row's slots, in slot order, of part[slot * stride + c], for
// `n_out` output arrays laid side by side in a slot (dK|dV share a slot).
template <typename T>
__global__ void sum_merge_kernel(const int4 *__restrict__ split_rows, int n_split,
                                 const float *__restrict__ part, int width, int n_out,
                                 T *__restrict__ out0, T *__restrict__ out1) {
    const int sr = blockIdx.x;
    if (sr >= n_split) return;
    const int4 rec = split_rows[sr];
    const int row = rec.x, first = rec.y, count = rec.z;
    const int stride = width * n_out;
    for (int c = threadIdx.x; c < stride; c += blockDim.x) {
        float acc = 0.f;
        const float *src = part + static_cast<int64_t>(first) * stride + c;
        for (int s = 0; s < count; s += 16) {  // 16 slots' loads travel together; added in slot order
            float x[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) x[u] = s + u < count ? src[static_cast<int64_t>(s + u) * stride] : 0.f;
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (s + u < count) acc += x[u];
        }
        if (c < width)
            out0[static_cast<int64_t>(row) * width + c] = from_acc<T>(acc);
        else
            out1[static_cast<int64_t>(row) * width + (c - width)] = from_acc<T>(acc);
    }
}

// ------------------------------------------------------------------ built-in scratch
//
// Scratch of bpt_attn_forward_static: lives in the library image, so each GPU that loads the
// library holds these bytes until the process exits.  In host code `g_static_scratch` is only
// a handle for the runtime, not a device address; the address a kernel may use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
constexpr size_t kStaticScratchBytes = BPT_ATTN_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void *g_static_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_static_scratch_mutex;

// Device address of the built-in scratch on the current device (set-up on first use).
int static_scratch_address(void **out) {
    int dev = -1;
    BPT_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(BPT_ERR_INVALID, "attn_forward_static: device %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
        void *ptr = nullptr;
        BPT_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (ptr == nullptr) return fail(BPT_ERR_CUDA, "attn_forward_static: no address for the built-in scratch");
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return BPT_OK;
}

// ------------------------------------------------------------------ host side


size_t forward_ws_bytes(const int32_t *counts, int H, int D) {
    const size_t slots = static_cast<size_t>(counts[1]);
    return align_up(slots * H * D * 4, 256) + align_up(slots * H * 2 * 4, 256) + 512;
}

size_t backward_ws_bytes(int64_t n_nodes, int64_t n_edges, const int32_t *counts, int H, int D) {
    const size_t e = static_cast<size_t>(n_edges);
    return 2 * align_up(e * H * 4, 256) + align_up(static_cast<size_t>(n_nodes) * H * 4, 256) +
           align_up(static_cast<size_t>(counts[1]) * 2 * H * D * 4, 256) +
           align_up(static_cast<size_t>(counts[1]) * H * 4, 256) +
           align_up(static_cast<size_t>(counts[4]) * 2 * H * D * 4, 256) +
           align_up(static_cast<size_t>(counts[7]) * D * 4, 256) + 1024;
}

int pick_lph(int D) { return D <= 32 ? 2 : (D <= 64 ? 4 : 8); }

template <typename T>
bool can_vectorise(int D, int lph, const void *a, const void *b, const void *c, const void *d, const void *e,
                   const void *f) {
    if (D != 16 * lph) return false;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                           reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(d) |
                           reinterpret_cast<uintptr_t>(e) | reinterpret_cast<uintptr_t>(f);
    return (bits & 15) == 0;
}

#define BPT_DISPATCH_LPH_VEC(lph, vec, ...)                                         \
    do {                                                                            \
        if (lph == 2) {                                                             \
            constexpr int LPH = 2;                                                  \
            if (vec) { constexpr bool VEC = true; __VA_ARGS__; } else { constexpr bool VEC = false; __VA_ARGS__; } \
        } else if (lph == 4) {                                                      \
            constexpr int LPH = 4;                                                  \
            if (vec) { constexpr bool VEC = true; __VA_ARGS__; } else { constexpr bool VEC = false; __VA_ARGS__; } \
        } else {                                                                    \
            constexpr int LPH = 8;                                                  \
            if (vec) { constexpr bool VEC = true; __VA_ARGS__; } else { constexpr bool VEC = false; __VA_ARGS__; } \
        }                                                                           \
    } while (0)

template <typename T>
int forward_impl(const PlanView &p, const int32_t *counts, const void *q_, const void *k_, const void *v_,
                 const void *ak_, float scale, void *o_, float *lse, int H, int D, void *ws_ptr,
                 size_t ws_bytes, const Dropout &drop, cudaStream_t stream) {
    const T *q = static_cast<const T *>(q_), *k = static_cast<const T *>(k_), *v = static_cast<const T *>(v_);
    const T *ak = static_cast<const T *>(ak_);
    T *o = static_cast<T *>(o_);
    Workspace ws(ws_ptr, ws_bytes);
    const size_t slots = static_cast<size_t>(counts[1]);
    float *part_o = ws.take<float>(slots * H * D);
    float *part_ml = ws.take<float>(slots * H * 2);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_forward: workspace of %zu bytes is too small", ws_bytes);
    const int n_items = counts[0], n_split = counts[2];
    if (n_items == 0) return BPT_OK;
    const int lph = pick_lph(D);
    const bool vec = can_vectorise<T>(D, lph, q, k, v, ak, o, o);
    const Geometry g{H, D};
    const int hpw = 32 / lph;
    const dim3 grid((n_items + kWarpsPerBlock - 1) / kWarpsPerBlock, (H + hpw - 1) / hpw);
    BPT_DISPATCH_LPH_VEC(lph, vec, (attn_forward_kernel<T, LPH, VEC><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        p.in_work.items, n_items, p.in_src, p.in_etype, q, k, v, ak, scale, o, lse, part_o, part_ml, g, drop)));
    BPT_LAUNCH_CHECK();
    if (n_split > 0) {
        attn_forward_merge_kernel<T><<<n_split, merge_threads(H, D), merge_smem_bytes(H), stream>>>(
            p.in_work.split_rows, n_split, part_o, part_ml, o, lse, g);
        BPT_LAUNCH_CHECK();
    }
    return BPT_OK;
}

template <typename T>
int backward_impl(const PlanView &p, const int32_t *counts, const void *q_, const void *k_, const void *v_,
                  const void *ak_, float scale, const float *lse, const void *do_,
                  void *dq_, void *dk_, void *dv_, float *dak, int H, int D, void *ws_ptr, size_t ws_bytes,
                  const Dropout &drop, cudaStream_t stream) {
    const T *q = static_cast<const T *>(q_), *k = static_cast<const T *>(k_), *v = static_cast<const T *>(v_);
    const T *ak = static_cast<const T *>(ak_), *d_o = static_cast<const T *>(do_);
    T *dq = static_cast<T *>(dq_), *dk = static_cast<T *>(dk_), *dv = static_cast<T *>(dv_);
    Workspace ws(ws_ptr, ws_bytes);
    const size_t e = static_cast<size_t>(p.n_edges);
    float *P = ws.take<float>(e * H);
    float *dP = ws.take<float>(e * H);
    float *delta = ws.take<float>(static_cast<size_t>(p.n_nodes) * H);
    float *part_ab = ws.take<float>(static_cast<size_t>(counts[1]) * 2 * H * D);
    float *part_delta = ws.take<float>(static_cast<size_t>(counts[1]) * H);
    float *part_dkv = ws.take<float>(static_cast<size_t>(counts[4]) * 2 * H * D);
    float *part_dak = ws.take<float>(static_cast<size_t>(counts[7]) * D);
    if (!ws.ok()) return fail(BPT_ERR_WORKSPACE, "attn_backward: workspace of %zu bytes is too small", ws_bytes);
    const int lph = pick_lph(D);
    const bool vec = can_vectorise<T>(D, lph, q, k, v, ak, d_o, d_o) && can_vectorise<T>(D, lph, dq, dk, dv, dq, dq, dq);
    const Geometry g{H, D};
    const int hpw = 32 / lph;
    const unsigned gy = (H + hpw - 1) / hpw;
    if (counts[0] > 0) {
        const dim3 grid((counts[0] + kWarpsPerBlock - 1) / kWarpsPerBlock, gy);
        BPT_DISPATCH_LPH_VEC(lph, vec, (attn_backward_dq_kernel<T, LPH, VEC><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            p.in_work.items, counts[0], p.in_src, p.in_etype, q, k, v, ak, scale, lse, d_o, P, dP, delta, dq,
            part_ab, part_delta, g, drop)));
        BPT_LAUNCH_CHECK();
        if (counts[2] > 0) {
            attn_backward_dq_merge_kernel<T><<<counts[2], 256, 0, stream>>>(
                p.in_work.split_rows, counts[2], part_ab, part_delta, scale, dq, delta, g);
            BPT_LAUNCH_CHECK();
        }
    }
    if (counts[3] > 0 && dk != nullptr && dv != nullptr) {
        const dim3 grid((counts[3] + kWarpsPerBlock - 1) / kWarpsPerBlock, gy);
        BPT_DISPATCH_LPH_VEC(lph, vec, (attn_backward_dkv_kernel<T, LPH, VEC><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            p.out_work.items, counts[3], p.out_dst, p.out_inpos, q, d_o, P, dP, delta, scale, dk, dv, part_dkv, g, drop)));
        BPT_LAUNCH_CHECK();
        if (counts[5] > 0) {
            sum_merge_kernel<T><<<counts[5], 256, 0, stream>>>(p.out_work.split_rows, counts[5], part_dkv, H * D,
                                                              2, dk, dv);
            BPT_LAUNCH_CHECK();
        }
    }
    if (ak != nullptr && dak != nullptr && counts[6] > 0) {
        const dim3 grid((counts[6] + kWarpsPerBlock - 1) / kWarpsPerBlock, 1);
        BPT_DISPATCH_LPH_VEC(lph, vec, (attn_backward_dak_kernel<T, LPH, VEC><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            p.et_work.items, counts[6], p.et_dst, p.et_inpos, q, P, dP, delta, scale, dak, part_dak, g)));
        BPT_LAUNCH_CHECK();
        if (counts[8] > 0) {
            sum_merge_kernel<float><<<counts[8], 128, 0, stream>>>(p.et_work.split_rows, counts[8], part_dak, D, 1,
                                                                  dak, dak);
            BPT_LAUNCH_CHECK();
        }
    }
    return BPT_OK;
}

}  // namespace

int launch_forward_items_bf16(const int4 *items, int n_items, const int32_t *in_src, const int32_t *in_etype,
                              const void *q_, const void *k_, const void *v_, const void *ak_, float scale,
                              void *o_, float *lse, int H, int D, const Dropout &drop, cudaStream_t stream) {
    using T = __nv_bfloat16;
    if (n_items == 0) return BPT_OK;
    const T *q = static_cast<const T *>(q_), *k = static_cast<const T *>(k_), *v = static_cast<const T *>(v_);
    const T *ak = static_cast<const T *>(ak_);
    T *o = static_cast<T *>(o_);
    const int lph = pick_lph(D);
    const bool vec = can_vectorise<T>(D, lph, q, k, v, ak, o, o);
    const Geometry g{H, D};
    const int hpw = 32 / lph;
    const dim3 grid((n_items + kWarpsPerBlock - 1) / kWarpsPerBlock, (H + hpw - 1) / hpw);
    BPT_DISPATCH_LPH_VEC(lph, vec, (attn_forward_kernel<T, LPH, VEC><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
        items, n_items, in_src, in_etype, q, k, v, ak, scale, o, lse, nullptr, nullptr, g, drop)));
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

// The pieces of the CUDA-core backward that the tensor-core backward keeps (bf16): the
// relative-position part of dQ and the gradient of the type table, both from P, dP, delta.
int launch_backward_ak_terms_bf16(const PlanView &p, const int32_t *counts, const void *q_, const void *ak_,
                                  const uint32_t *PS, void *dq_, float *dak, float *part_dak, int H, int D,
                                  cudaStream_t stream) {
    using T = __nv_bfloat16;
    const T *q = static_cast<const T *>(q_), *ak = static_cast<const T *>(ak_);
    T *dq = static_cast<T *>(dq_);
    if (ak == nullptr) return BPT_OK;
    const int lph = pick_lph(D);
    const bool vec = can_vectorise<T>(D, lph, q, ak, dq, dq, dq, dq);
    const Geometry g{H, D};
    const int hpw = 32 / lph;
    if (p.n_nodes > 0) {
        const dim3 grid(static_cast<unsigned>((p.n_nodes + kWarpsPerBlock - 1) / kWarpsPerBlock), (H + hpw - 1) / hpw);
        BPT_DISPATCH_LPH_VEC(lph, vec, (attn_backward_dq_ak_kernel<T, LPH, VEC><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            p.in_indptr, p.in_etype, p.row_uniform, static_cast<int>(p.n_nodes), ak, PS, p.n_edges, dq, g)));
        BPT_LAUNCH_CHECK();
    }
    if (dak != nullptr && counts[6] > 0) {
        const dim3 grid((counts[6] + kWarpsPerBlock - 1) / kWarpsPerBlock, 1);
        BPT_DISPATCH_LPH_VEC(lph, vec, (attn_backward_dak_kernel<T, LPH, VEC, true><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            p.et_work.items, counts[6], p.et_dst, p.et_inpos, q, reinterpret_cast<const float *>(PS), nullptr,
            nullptr, 1.f, dak, part_dak, g, p.n_edges)));
        BPT_LAUNCH_CHECK();
        if (counts[8] > 0) {
            sum_merge_kernel<float><<<counts[8], 128, 0, stream>>>(p.et_work.split_rows, counts[8], part_dak, D, 1,
                                                                  dak, dak);
            BPT_LAUNCH_CHECK();
        }
    }
    return BPT_OK;
}

// The passes of the CUDA-core backward that the fp32 tile backward keeps, all from the fp32 scratch (P, dP in
// [in-CSR position][head] order, delta per (row, head)) that its destination-side kernel leaves: the
// relative-position part of dQ (added to dq), dK and dV over the out-CSR, d embed_ak over the type buckets.
int launch_backward_rest_f32(const PlanView &p, const int32_t *counts, const float *q, const float *ak,
                             const float *d_o, const float *P, const float *dP, const float *delta, float scale,
                             float *dq, float *dk, float *dv, float *dak, float *part_dkv, float *part_dak, int H,
                             int D, const Dropout &drop, cudaStream_t stream) {
    using T = float;
    const int lph = pick_lph(D);
    const bool vec = can_vectorise<T>(D, lph, q, ak, d_o, dq, dk, dv);
    const Geometry g{H, D};
    const int hpw = 32 / lph;
    const unsigned gy = (H + hpw - 1) / hpw;
    if (ak != nullptr && p.n_nodes > 0) {
        const dim3 grid(static_cast<unsigned>((p.n_nodes + kWarpsPerBlock - 1) / kWarpsPerBlock), gy);
        BPT_DISPATCH_LPH_VEC(lph, vec, (attn_backward_dq_ak_kernel<T, LPH, VEC, false><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            p.in_indptr, p.in_etype, p.row_uniform, static_cast<int>(p.n_nodes), ak, nullptr, 0, dq, g, P, dP, delta, scale)));
        BPT_LAUNCH_CHECK();
    }
    if (counts[3] > 0 && dk != nullptr && dv != nullptr) {
        const dim3 grid((counts[3] + kWarpsPerBlock - 1) / kWarpsPerBlock, gy);
        BPT_DISPATCH_LPH_VEC(lph, vec, (attn_backward_dkv_kernel<T, LPH, VEC><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            p.out_work.items, counts[3], p.out_dst, p.out_inpos, q, d_o, P, dP, delta, scale, dk, dv, part_dkv, g, drop)));
        BPT_LAUNCH_CHECK();
        if (counts[5] > 0) {
            sum_merge_kernel<T><<<counts[5], 256, 0, stream>>>(p.out_work.split_rows, counts[5], part_dkv, H * D, 2, dk, dv);
            BPT_LAUNCH_CHECK();
        }
    }
    if (ak != nullptr && dak != nullptr && counts[6] > 0) {
        const dim3 grid((counts[6] + kWarpsPerBlock - 1) / kWarpsPerBlock, 1);
        BPT_DISPATCH_LPH_VEC(lph, vec, (attn_backward_dak_kernel<T, LPH, VEC><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
            p.et_work.items, counts[6], p.et_dst, p.et_inpos, q, P, dP, delta, scale, dak, part_dak, g)));
        BPT_LAUNCH_CHECK();
        if (counts[8] > 0) {
            sum_merge_kernel<float><<<counts[8], 128, 0, stream>>>(p.et_work.split_rows, counts[8], part_dak, D, 1, dak, dak);
            BPT_LAUNCH_CHECK();
        }
    }
    return BPT_OK;
}

// out[row, :] = sum over the row's slots, in slot order, of fp32 partial rows of `width` columns; with out1 a
// slot holds two such rows side by side (out | out1).
int launch_sum_merge_f32(const int4 *split_rows, int n_split, const float *part, int width, float *out,
                         cudaStream_t stream, float *out1) {
    if (n_split <= 0) return BPT_OK;
    sum_merge_kernel<float><<<n_split, 256, 0, stream>>>(split_rows, n_split, part, width, out1 ? 2 : 1, out,
                                                         out1 ? out1 : out);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

namespace {

int check_dropout(const char *name, const bpt_dropout_t *d) {
    BPT_CHECK_ARG(d == nullptr || (d->rate >= 0.0 && d->rate < 1.0), "%s: dropout rate must be in [0, 1)", name);
    return BPT_OK;
}

int check_attn_args(const char *name, const void *plan, const int32_t *counts, int64_t n_nodes,
                    int64_t n_edges, int n_etypes, int H, int D, int dtype) {
    BPT_CHECK_ARG(plan != nullptr && counts != nullptr, "%s: null plan", name);
    BPT_CHECK_ARG(n_nodes >= 0 && n_edges >= 0 && n_etypes >= 1, "%s: bad sizes", name);
    BPT_CHECK_ARG(H >= 1 && D >= 1, "%s: h and d must be positive", name);
    if (D > 128) return fail(BPT_ERR_UNSUPPORTED, "%s: head dim %d > 128 has no kernel", name, D);
    if (H > 40) return fail(BPT_ERR_UNSUPPORTED, "%s: more than 40 heads has no kernel", name);
    if (dtype == BPT_F64) return fail(BPT_ERR_UNSUPPORTED, "%s: fp64 has no fused kernel (use the operators)", name);
    return BPT_OK;
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" size_t bpt_attn_workspace_bytes(int64_t n_nodes, int64_t n_edges, const int32_t *counts, int h, int d,
                                           int backward) {
    if (counts == nullptr || n_nodes < 0 || n_edges < 0 || h < 1 || d < 1) return 0;
    return backward ? backward_ws_bytes(n_nodes, n_edges, counts, h, d) : forward_ws_bytes(counts, h, d);
}

extern "C" int bpt_attn_forward(const void *plan, const int32_t *counts, int64_t n_nodes, int64_t n_edges,
                                int n_etypes, const void *q, const void *k, const void *v, const void *ak,
                                double scale, void *o, float *lse, int h, int d, int dtype, void *workspace,
                                size_t workspace_bytes, const bpt_dropout_t *dropout, bpt_stream_t stream) {
    if (int rc = check_dropout("attn_forward", dropout)) return rc;
    const Dropout drop = make_dropout(dropout);
    if (int rc = check_attn_args("attn_forward", plan, counts, n_nodes, n_edges, n_etypes, h, d, dtype)) return rc;
    BPT_CHECK_ARG(n_nodes == 0 || (q && k && v && o && lse), "attn_forward: null tensor");
    const PlanView p = plan_view(const_cast<void *>(plan), n_nodes, counts[kCountsNSrc], n_edges, n_etypes);
    switch (dtype) {
        case BPT_F32: return forward_impl<float>(p, counts, q, k, v, ak, static_cast<float>(scale), o, lse, h, d, workspace, workspace_bytes, drop, as_stream(stream));
        case BPT_BF16: return forward_impl<__nv_bfloat16>(p, counts, q, k, v, ak, static_cast<float>(scale), o, lse, h, d, workspace, workspace_bytes, drop, as_stream(stream));
        case BPT_F16: return forward_impl<__half>(p, counts, q, k, v, ak, static_cast<float>(scale), o, lse, h, d, workspace, workspace_bytes, drop, as_stream(stream));
        default: return fail(BPT_ERR_UNSUPPORTED, "attn_forward: unknown dtype code %d", dtype);
    }
}

extern "C" int bpt_attn_backward(const void *plan, const int32_t *counts, int64_t n_nodes, int64_t n_edges,
                                 int n_etypes, const void *q, const void *k, const void *v, const void *ak,
                                 double scale, const float *lse, const void *d_o, void *dq,
                                 void *dk, void *dv, float *dak, int h, int d, int dtype, void *workspace,
                                 size_t workspace_bytes, const bpt_dropout_t *dropout, bpt_stream_t stream) {
    if (int rc = check_dropout("attn_backward", dropout)) return rc;
    const Dropout drop = make_dropout(dropout);
    if (int rc = check_attn_args("attn_backward", plan, counts, n_nodes, n_edges, n_etypes, h, d, dtype)) return rc;
    BPT_CHECK_ARG(n_nodes == 0 || (q && k && v && lse && d_o && dq), "attn_backward: null tensor");
    BPT_CHECK_ARG((dk == nullptr) == (dv == nullptr), "attn_backward: dk and dv must both be given or both be NULL");
    BPT_CHECK_ARG(ak == nullptr || dak != nullptr, "attn_backward: ak given without dak");
    const PlanView p = plan_view(const_cast<void *>(plan), n_nodes, counts[kCountsNSrc], n_edges, n_etypes);
    switch (dtype) {
        case BPT_F32: return backward_impl<float>(p, counts, q, k, v, ak, static_cast<float>(scale), lse, d_o, dq, dk, dv, dak, h, d, workspace, workspace_bytes, drop, as_stream(stream));
        case BPT_BF16: return backward_impl<__nv_bfloat16>(p, counts, q, k, v, ak, static_cast<float>(scale), lse, d_o, dq, dk, dv, dak, h, d, workspace, workspace_bytes, drop, as_stream(stream));
        case BPT_F16: return backward_impl<__half>(p, counts, q, k, v, ak, static_cast<float>(scale), lse, d_o, dq, dk, dv, dak, h, d, workspace, workspace_bytes, drop, as_stream(stream));
        default: return fail(BPT_ERR_UNSUPPORTED, "attn_backward: unknown dtype code %d", dtype);
    }
}

// Same computation as bpt_attn_forward, for callers that cannot provide device scratch.
extern "C" int bpt_attn_forward_static(const void *plan, const int32_t *counts, int64_t n_nodes,
                                       int64_t n_edges, int n_etypes, const void *q, const void *k,
                                       const void *v, const void *ak, double scale, void *o, float *lse,
                                       int h, int d, int dtype, bpt_stream_t stream) {
    if (int rc = check_attn_args("attn_forward_static", plan, counts, n_nodes, n_edges, n_etypes, h, d, dtype))
        return rc;
    BPT_CHECK_ARG(n_nodes == 0 || (q && k && v && o && lse), "attn_forward_static: null tensor");
    const size_t need = forward_ws_bytes(counts, h, d);
    if (need > kStaticScratchBytes)
        return fail(BPT_ERR_WORKSPACE,
                    "attn_forward_static: this graph needs %zu bytes of scratch for its split rows but the "
                    "built-in scratch holds %zu; use bpt_attn_forward with a caller-provided workspace",
                    need, kStaticScratchBytes);
    void *scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    return bpt_attn_forward(plan, counts, n_nodes, n_edges, n_etypes, q, k, v, ak, scale, o, lse, h, d, dtype,
                            scratch, kStaticScratchBytes, nullptr, stream);
}

namespace bpt {
namespace {
__global__ void dropout_mask_kernel(const int32_t *__restrict__ src, const int32_t *__restrict__ dst, int64_t n_edges,
                                    int H, Dropout drop, uint8_t *__restrict__ mask) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= n_edges * H) return;
    const int64_t e = i / H;
    const int head = static_cast<int>(i % H);
    mask[i] = !drop.threshold || dropout_factor(drop, dst[e], src[e], head) != 0.f;
}
}  // namespace
}  // namespace bpt

extern "C" int bpt_attn_dropout_mask(const int32_t *src, const int32_t *dst, int64_t n_edges, int h,
                                     const bpt_dropout_t *dropout, uint8_t *mask, bpt_stream_t stream) {
    BPT_CHECK_ARG(n_edges >= 0 && h >= 1, "attn_dropout_mask: bad sizes");
    if (int rc = check_dropout("attn_dropout_mask", dropout)) return rc;
    if (n_edges == 0) return BPT_OK;
    BPT_CHECK_ARG(src && dst && mask, "attn_dropout_mask: null array");
    const int64_t n = n_edges * h;
    dropout_mask_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, as_stream(stream)>>>(src, dst, n_edges, h,
                                                                                            make_dropout(dropout), mask);
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}
