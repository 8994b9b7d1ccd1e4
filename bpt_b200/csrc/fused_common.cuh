// Pieces shared by the CUDA-core and the tensor-core fused attention kernels.
#pragma once

#include "common.cuh"

namespace bpt {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Head count and head dim of the feature tensors.
struct Geometry {
    int H, D;
};

// Partial results of a row that is spread over several work items or tiles: per slot and
// head, part_ml = {m, l} (running max of the log2-domain scores, sum of 2^(s-m)) and part_o =
// the unnormalised weighted sum of V rows.
// Combines the partial (m, l, o) triples of a split row in slot order.
template <typename T>
__global__ void attn_forward_merge_kernel(const int4 *__restrict__ split_rows, int n_split,
                                          const float *__restrict__ part_o, const float *__restrict__ part_ml,
                                          T *__restrict__ o, float *__restrict__ lse, Geometry g) {
    const int sr = blockIdx.x;
    if (sr >= n_split) return;
    const int4 rec = split_rows[sr];
    const int row = rec.x, first = rec.y, count = rec.z;
    const int HD = g.H * g.D;
    for (int c = threadIdx.x; c < HD; c += blockDim.x) {
        const int head = c / g.D;
        float m = -INFINITY;
        for (int s = 0; s < count; ++s) m = fmaxf(m, part_ml[(static_cast<int64_t>(first + s) * g.H + head) * 2]);
        float l = 0.f, acc = 0.f;
        for (int s = 0; s < count; ++s) {
            const int64_t base = static_cast<int64_t>(first + s) * g.H + head;
            const float w = exp2f(part_ml[base * 2] - m);
            l = fmaf(part_ml[base * 2 + 1], w, l);
            acc = fmaf(part_o[static_cast<int64_t>(first + s) * HD + c], w, acc);
        }
        o[static_cast<int64_t>(row) * HD + c] = from_acc<T>(acc / l);
        if (c % g.D == 0) lse[static_cast<int64_t>(row) * g.H + head] = (m + log2f(l)) * kLn2;
    }
}


}  // namespace bpt
