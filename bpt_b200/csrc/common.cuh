// Shared helpers of the bpt_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/bpt_b200.h"

namespace bpt {

// Thread-local message of the last failing call, returned by bpt_last_error().
char *error_buffer();
int fail(int code, const char *fmt, ...);

#define BPT_CHECK_ARG(cond, ...)                                   \
    do {                                                           \
        if (!(cond)) return ::bpt::fail(BPT_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define BPT_CUDA(call)                                                                      \
    do {                                                                                    \
        cudaError_t err__ = (call);                                                         \
        if (err__ != cudaSuccess)                                                           \
            return ::bpt::fail(BPT_ERR_CUDA, "%s failed: %s (%s:%d)", #call,                \
                               cudaGetErrorString(err__), __FILE__, __LINE__);              \
    } while (0)

#define BPT_LAUNCH_CHECK() BPT_CUDA(cudaGetLastError())

inline cudaStream_t as_stream(bpt_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Carves aligned pieces out of a caller-provided workspace.
struct Workspace {
    char *base;
    size_t size, used;
    Workspace(void *p, size_t n) : base(static_cast<char *>(p)), size(n), used(0) {}
    template <typename T>
    T *take(size_t count) {
        size_t bytes = align_up(count * sizeof(T), 256);
        if (base == nullptr || used + bytes > size) { used = size + 1; return nullptr; }
        T *p = reinterpret_cast<T *>(base + used);
        used += bytes;
        return p;
    }
    bool ok() const { return used <= size; }
};

// Element type traits: storage type -> accumulation type and conversions.
template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v);
template <> __device__ __forceinline__ float to_acc<float>(float v) { return v; }
template <> __device__ __forceinline__ double to_acc<double>(double v) { return v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_acc(typename Acc<T>::type v);
template <> __device__ __forceinline__ float from_acc<float>(float v) { return v; }
template <> __device__ __forceinline__ double from_acc<double>(double v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_acc<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float acc_exp(float x) { return expf(x); }
__device__ __forceinline__ double acc_exp(double x) { return exp(x); }

// Dispatch a BPT_* dtype code to a template instantiation.
#define BPT_DISPATCH_DTYPE(dtype, ...)                                                     \
    switch (dtype) {                                                                       \
        case BPT_F32: { using scalar_t = float; __VA_ARGS__; break; }                      \
        case BPT_F64: { using scalar_t = double; __VA_ARGS__; break; }                     \
        case BPT_BF16: { using scalar_t = __nv_bfloat16; __VA_ARGS__; break; }             \
        case BPT_F16: { using scalar_t = __half; __VA_ARGS__; break; }                     \
        default: return ::bpt::fail(BPT_ERR_UNSUPPORTED, "unknown dtype code %d", dtype);  \
    }

}  // namespace bpt
