// Pieces shared by the CUDA-core and the tensor-core fused attention kernels.
#pragma once

#include "common.cuh"

namespace bpt {

constexpr float kLog2e = 1.4426950408889634f;

// 2^x in one instruction of the special-function unit (about 2 ulp; denormal results flush to zero;
// ex2(-inf) = 0).  The bf16 tensor-core kernels use it for softmax weights, whose rounding to bf16
// is 2^-9 relative; the fp32 kernels keep exp2f.
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kLn2 = 0.6931471805599453f;

// Dropout on the attention weights (modules/attention.py:73: drop_att between the edge softmax and the
// weighted sum).  An edge's weight for one head is kept when a 32-bit hash of (destination, source, head,
// seed) is at least `threshold` = rate * 2^32, and kept weights are scaled by 1 / (1 - rate).  The mask is a
// pure function of those four numbers: the forward and every backward kernel regenerate it, nothing is
// stored.  Parallel edges between one pair of nodes share their bit.  threshold == 0 switches it off.
struct Dropout {
    uint32_t seed_lo, seed_hi, threshold;
    float keep_scale;
};
inline Dropout make_dropout(const bpt_dropout_t *d) {
    Dropout r{0u, 0u, 0u, 1.f};
    if (d != nullptr && d->rate > 0.0) {
        const double t = d->rate * 4294967296.0;
        r.threshold = t >= 4294967295.0 ? 0xFFFFFFFFu : static_cast<uint32_t>(t);
        r.keep_scale = static_cast<float>(1.0 / (1.0 - d->rate));
        r.seed_lo = static_cast<uint32_t>(d->seed);
        r.seed_hi = static_cast<uint32_t>(d->seed >> 32);
    }
    return r;
}
__host__ __device__ __forceinline__ uint32_t dropout_hash(uint32_t dst, uint32_t src, uint32_t head, uint32_t seed_lo,
                                                          uint32_t seed_hi) {
    uint32_t x = (dst * 0x9E3779B1u) ^ ((src + 0x7F4A7C15u) * 0x85EBCA6Bu) ^ ((head + seed_hi) * 0xC2B2AE35u) ^ seed_lo;
    x ^= x >> 16;
    x *= 0x7FEB352Du;
    x ^= x >> 15;
    x *= 0x846CA68Bu;
    x ^= x >> 16;
    return x;
}
// The factor an attention weight is multiplied by: 1 / (1 - rate) when kept, 0 when dropped.
__device__ __forceinline__ float dropout_factor(const Dropout &d, int dst, int src, int head) {
    return dropout_hash(static_cast<uint32_t>(dst), static_cast<uint32_t>(src), static_cast<uint32_t>(head), d.seed_lo,
                        d.seed_hi) >= d.threshold ? d.keep_scale : 0.f;
}

// Head count and head dim of the feature tensors.
struct Geometry {
    int H, D;
};

// Partial results of a row that is spread over several work items or tiles: per slot and
// head, part_ml = {m, l} (running max of the log2-domain scores, sum of 2^(s-m)) and part_o =
// the unnormalised weighted sum of V rows.
// Combines the partial (m, l, o) triples of a split row, in slot order.  One block per row.
// Slots are taken in batches of kMergeBatch: one thread per head turns the batch's (m, l) into
// weights 2^(m_s - m_run) and the factor that rescales what was accumulated so far, then
// every output column adds its batch of partial values with several loads in flight.
constexpr int kMergeBatch = 128;

template <typename T>
__global__ void attn_forward_merge_kernel(const int4 *__restrict__ split_rows, int n_split,
                                          const float *__restrict__ part_o, const float *__restrict__ part_ml,
                                          T *__restrict__ o, float *__restrict__ lse, Geometry g) {
    extern __shared__ float s_merge[];  // [kMergeBatch][H] m then weights | [kMergeBatch][H] l | [H] rescale | [H] 1/l
    const int sr = blockIdx.x;
    if (sr >= n_split) return;
    const int4 rec = split_rows[sr];
    const int row = rec.x, first = rec.y, count = rec.z;
    const int H = g.H, HD = g.H * g.D;
    float *s_w = s_merge, *s_l = s_merge + kMergeBatch * H, *s_f = s_l + kMergeBatch * H, *s_inv = s_f + H;
    float m_run = -INFINITY, l_run = 0.f;  // meaningful in threads < H
    // Each thread owns columns threadIdx.x, + blockDim.x, ... (at most kMaxCols of them).
    constexpr int kMaxCols = 8;
    float acc[kMaxCols];
#pragma unroll
    for (int u = 0; u < kMaxCols; ++u) acc[u] = 0.f;

    for (int s0 = 0; s0 < count; s0 += kMergeBatch) {
        const int nb = min(kMergeBatch, count - s0);
        __syncthreads();
        for (int i = threadIdx.x; i < nb * H; i += blockDim.x) {
            const float2 ml = *reinterpret_cast<const float2 *>(part_ml + (static_cast<int64_t>(first + s0) * H + i) * 2);
            s_w[i] = ml.x;
            s_l[i] = ml.y;
        }
        __syncthreads();
        if (threadIdx.x < H) {
            const int head = threadIdx.x;
            float m = m_run;
            for (int s = 0; s < nb; ++s) m = fmaxf(m, s_w[s * H + head]);
            const float ms = m == -INFINITY ? 0.f : m;
            const float f = exp2f(m_run - ms);
            float l = l_run * f;
            for (int s = 0; s < nb; ++s) {
                const float w = exp2f(s_w[s * H + head] - ms);
                l = fmaf(s_l[s * H + head], w, l);
                s_w[s * H + head] = w;
            }
            s_f[head] = f;
            m_run = m;
            l_run = l;
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < kMaxCols; ++u) {
            const int c = threadIdx.x + u * blockDim.x;
            if (c >= HD) break;
            const int head = c / g.D;
            const float *src = part_o + static_cast<int64_t>(first + s0) * HD + c;
            float a = acc[u] * s_f[head];
            int s = 0;
            for (; s + 16 <= nb; s += 16) {
                float x[16];
#pragma unroll
                for (int v = 0; v < 16; ++v) x[v] = src[static_cast<int64_t>(s + v) * HD];
#pragma unroll
                for (int v = 0; v < 16; ++v) a = fmaf(x[v], s_w[(s + v) * H + head], a);
            }
            if (s < nb) {  // the last, partial batch: its loads travel together too
                float x[16];
#pragma unroll
                for (int v = 0; v < 16; ++v) x[v] = s + v < nb ? src[static_cast<int64_t>(s + v) * HD] : 0.f;
#pragma unroll
                for (int v = 0; v < 16; ++v)
                    if (s + v < nb) a = fmaf(x[v], s_w[(s + v) * H + head], a);
            }
            acc[u] = a;
        }
    }
    if (threadIdx.x < H) {
        s_inv[threadIdx.x] = l_run > 0.f ? 1.f / l_run : 0.f;
        lse[static_cast<int64_t>(row) * H + threadIdx.x] = l_run > 0.f ? (m_run + log2f(l_run)) * kLn2 : -INFINITY;
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < kMaxCols; ++u) {
        const int c = threadIdx.x + u * blockDim.x;
        if (c >= HD) break;
        o[static_cast<int64_t>(row) * HD + c] = from_acc<T>(acc[u] * s_inv[c / g.D]);
    }
}

// Block size and shared memory of the merge kernel: one output column per thread where that fits
// (a long row's slots are walked once, not once per column).  Needs H <= threads and H*D <= 8*threads.
inline int merge_threads(int H, int D) {
    int t = H * D;
    t = t < H ? H : t;
    t = (t + 31) / 32 * 32;
    return t < 128 ? 128 : (t > 1024 ? 1024 : t);
}
inline size_t merge_smem_bytes(int H) { return (static_cast<size_t>(kMergeBatch) * H * 2 + 2 * H) * sizeof(float); }

// Runs the CUDA-core forward kernel over a caller-given list of whole-row work items
// ({row, begin, end, -1} into the in-CSR arrays); bf16 storage.  Defined in fused_simt.cu.
int launch_forward_items_bf16(const int4 *items, int n_items, const int32_t *in_src, const int32_t *in_etype,
                              const void *q, const void *k, const void *v, const void *ak, float scale,
                              void *o, float *lse, int H, int D, const Dropout &drop, cudaStream_t stream);


struct PlanView;
// Defined in fused_simt.cu: dQ += relative-position part, and d embed_ak (with its split-row merge),
// from the per-edge scratch PS ([head][in-CSR position], one word {bf16 p, bf16 dS} each); bf16
// storage.  part_dak: counts[7] * D floats.
int launch_backward_ak_terms_bf16(const PlanView &p, const int32_t *counts, const void *q, const void *ak,
                                  const uint32_t *PS, void *dq, float *dak, float *part_dak, int H, int D,
                                  cudaStream_t stream);

// Defined in fused_simt.cu: what the fp32 tile backward keeps of the CUDA-core backward, from the fp32 scratch
// (P, dP in [in-CSR position][head] order, delta per (row, head)): dq += relative-position part, dK and dV,
// d embed_ak.  part_dkv: counts[4] * 2 * H * D floats, part_dak: counts[7] * D floats.
int launch_backward_rest_f32(const PlanView &p, const int32_t *counts, const float *q, const float *ak,
                             const float *d_o, const float *P, const float *dP, const float *delta, float scale,
                             float *dq, float *dk, float *dv, float *dak, float *part_dkv, float *part_dak, int H,
                             int D, const Dropout &drop, cudaStream_t stream);
// Defined in fused_tc_bwd.cu: the relative-position gradients of the fp32 backward through a dense per-row type
// table G (fp32, n_nodes * H x tq, made from the fp32 scratch) and two fp32 library GEMMs: dq += G . ak,
// dak = G^T . q.  type_table_f32_elems: floats of G, or 0 when the table does not apply.
size_t type_table_f32_elems(int tq, int64_t n_nodes, int h);
int launch_type_table_terms_f32(const PlanView &pv, int tq, int n_etypes, const float *q, const float *ak,
                                const float *P, const float *dP, const float *delta, float scale, float *dq,
                                float *dak, float *G, int h, cudaStream_t stream);
// out[row, :] = sum over the row's slots ({row, first, count, .} records), in slot order, of fp32 partial rows;
// with out1 a slot holds two rows side by side (out | out1).
int launch_sum_merge_f32(const int4 *split_rows, int n_split, const float *part, int width, float *out,
                         cudaStream_t stream, float *out1 = nullptr);

}  // namespace bpt
