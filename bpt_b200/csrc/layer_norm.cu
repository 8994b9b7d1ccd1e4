// y = LayerNorm(x + r) over the last dimension, one pass over memory.
//
// The block of modules/attention.py ends each of its two halves with `norm(h + sublayer(h))`
// (attention.py:79-81, 141, 168-171).  As two torch operators that is a read of two tensors and a
// write for the sum, then a read and a write for the normalisation; here a warp owns a row, keeps
// the sum in registers (fp32), reduces mean and variance with shuffles and writes the result
// once: 3 passes of N x dim instead of 5.  HBM-bound: (2 reads + 1 write) x N x dim x bytes.
#include "common.cuh"

namespace bpt {
namespace {

constexpr int kLnWarps = 8;

// load8 / store8: 8 elements = one 16-byte piece (bf16, fp16) or two (fp32), widened to fp32.
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __bfloat1622float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}
__device__ __forceinline__ void load8(const __half *p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __half22float2(h[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}
__device__ __forceinline__ void load8(const float *p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16 *p, const float (&f)[8]) {
    uint4 raw;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = raw;
}
__device__ __forceinline__ void store8(__half *p, const float (&f)[8]) {
    uint4 raw;
    __half2 *h = reinterpret_cast<__half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = raw;
}
__device__ __forceinline__ void store8(float *p, const float (&f)[8]) {
    *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4 *>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// kVecs pieces of 8 elements per lane: dim <= 256 * kVecs.  A warp per row.
template <typename T, int kVecs>
__global__ void __launch_bounds__(kLnWarps * 32)
add_layer_norm_kernel(const T *__restrict__ x, const T *__restrict__ r, const T *__restrict__ gamma,
                      const T *__restrict__ beta, float eps, T *__restrict__ y, int64_t n_rows, int dim) {
    const int lane = threadIdx.x & 31;
    const int64_t row = blockIdx.x * static_cast<int64_t>(kLnWarps) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const T *xr = x + row * dim;
    const T *rr = r ? r + row * dim : nullptr;
    float v[kVecs][8];
    float sum = 0.f;
#pragma unroll
    for (int u = 0; u < kVecs; ++u) {
        const int c = (u * 32 + lane) * 8;
        if (c < dim) {
            load8(xr + c, v[u]);
            if (rr) {
                float t[8];
                load8(rr + c, t);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[u][i] += t[i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += v[u][i];
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / static_cast<float>(dim);
    float sq = 0.f;
#pragma unroll
    for (int u = 0; u < kVecs; ++u) {
        const int c = (u * 32 + lane) * 8;
        if (c < dim) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float d = v[u][i] - mean;
                sq = fmaf(d, d, sq);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq / static_cast<float>(dim) + eps);  // biased variance, as torch.nn.LayerNorm
    T *yr = y + row * dim;
#pragma unroll
    for (int u = 0; u < kVecs; ++u) {
        const int c = (u * 32 + lane) * 8;
        if (c < dim) {
            float g[8], b[8], out[8];
            if (gamma) load8(gamma + c, g);
            if (beta) load8(beta + c, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float n = (v[u][i] - mean) * rstd;
                out[i] = fmaf(n, gamma ? g[i] : 1.f, beta ? b[i] : 0.f);
            }
            store8(yr + c, out);
        }
    }
}

template <typename T>
int launch_add_layer_norm(const void *x, const void *r, const void *gamma, const void *beta, float eps, void *y,
                          int64_t n_rows, int dim, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>((n_rows + kLnWarps - 1) / kLnWarps);
    const int vecs = (dim + 255) / 256;
#define BPT_LN_LAUNCH(V)                                                                                      \
    add_layer_norm_kernel<T, V><<<grid, kLnWarps * 32, 0, stream>>>(                                          \
        static_cast<const T *>(x), static_cast<const T *>(r), static_cast<const T *>(gamma),                  \
        static_cast<const T *>(beta), eps, static_cast<T *>(y), n_rows, dim)
    if (vecs <= 1) BPT_LN_LAUNCH(1);
    else if (vecs <= 2) BPT_LN_LAUNCH(2);
    else if (vecs <= 4) BPT_LN_LAUNCH(4);
    else if (vecs <= 8) BPT_LN_LAUNCH(8);
    else BPT_LN_LAUNCH(16);
#undef BPT_LN_LAUNCH
    BPT_LAUNCH_CHECK();
    return BPT_OK;
}

}  // namespace
}  // namespace bpt

using namespace bpt;

extern "C" int bpt_add_layer_norm(const void *x, const void *r, const void *gamma, const void *beta, double eps,
                                  void *y, int64_t n_rows, int dim, int dtype, bpt_stream_t stream_) {
    BPT_CHECK_ARG(n_rows >= 0 && dim >= 8 && dim % 8 == 0 && dim <= 4096,
                  "add_layer_norm: dim must be a multiple of 8 in [8, 4096] (got %d)", dim);
    BPT_CHECK_ARG(n_rows < (int64_t(1) << 31) * kLnWarps, "add_layer_norm: too many rows");
    if (n_rows == 0) return BPT_OK;
    BPT_CHECK_ARG(x && y, "add_layer_norm: null tensor");
    BPT_CHECK_ARG(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(r) | reinterpret_cast<uintptr_t>(gamma) |
                    reinterpret_cast<uintptr_t>(beta) | reinterpret_cast<uintptr_t>(y)) & 15) == 0,
                  "add_layer_norm: tensors must be 16-byte aligned");
    cudaStream_t stream = as_stream(stream_);
    const float e = static_cast<float>(eps);
    switch (dtype) {
        case BPT_F32: return launch_add_layer_norm<float>(x, r, gamma, beta, e, y, n_rows, dim, stream);
        case BPT_BF16: return launch_add_layer_norm<__nv_bfloat16>(x, r, gamma, beta, e, y, n_rows, dim, stream);
        case BPT_F16: return launch_add_layer_norm<__half>(x, r, gamma, beta, e, y, n_rows, dim, stream);
        default: return fail(BPT_ERR_UNSUPPORTED, "add_layer_norm: dtype %d is not supported", dtype);
    }
}
