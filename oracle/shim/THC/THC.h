/* Stand-in for the <THC/THC.h> that PyTorch no longer ships, put on the include path by
 * oracle/build_ref_graphop.py (test infrastructure) so that the reference's
 * graph_kernel/graphop_kernel.cu compiles unmodified against a current PyTorch.  The reference
 * takes two things from the old header: THCudaCheck (graphop_kernel.cu:264 and after every
 * launch), and -- through AT_DISPATCH_FLOATING_TYPES(x.type(), ...) -- a dispatch on the
 * deprecated type object that Tensor::type() returns, which ATen's dispatch macro no longer
 * accepts.  Both are supplied here; nothing in the reference's sources is touched. */
#pragma once
#include <ATen/ATen.h>
#include <ATen/Dispatch.h>
#include <c10/cuda/CUDAException.h>

#define THCudaCheck(expr) C10_CUDA_CHECK(expr)

namespace detail {
inline at::ScalarType scalar_type(const at::DeprecatedTypeProperties &t) { return t.scalarType(); }
}  // namespace detail
