// Residual adds around the routed-MoE path, with the reference's entry points and arithmetic
// (native/cuda/kernels/residual.cu:18-62 kernels, :1395-1497 entry points): float32 adds whose
// bf16 results are stored by truncation (the reference's f32_to_bf16 keeps the upper 16 bits,
// native/cuda/kernels/common.h:64-66).  A float32 delta is first truncated to bf16.
//
//   residual_add_bf16               out = bf16(residual + delta)
//   residual_add_f32_delta_bf16     out = bf16(residual + bf16(delta_f32))
//   residual_add_shared_f32_delta   out = bf16(residual + bf16(shared + bf16(routed_f32)))
//
// The layer's own forward_residual entry point folds the last form into the combine kernel.
#include "common.cuh"
#include "internal.h"

namespace glmrt {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float trunc_bf16(float x) { return __uint_as_float(__float_as_uint(x) & 0xffff0000u); }
__device__ __forceinline__ uint16_t trunc_bf16_bits(float x) { return static_cast<uint16_t>(__float_as_uint(x) >> 16); }

// kMode 0: bf16 delta; 1: float32 delta; 2: bf16 shared + float32 routed delta
template <int kMode>
__global__ void __launch_bounds__(kThreads)
residual_add_kernel(const uint16_t* __restrict__ residual, const uint16_t* __restrict__ delta_bf16,
                    const float* __restrict__ delta_f32, uint16_t* __restrict__ out, size_t count) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
  for (size_t i = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x; i < count; i += stride) {
    const float res = bf16_bits_to_f32(residual[i]);
    float delta;
    if (kMode == 0) delta = bf16_bits_to_f32(delta_bf16[i]);
    else if (kMode == 1) delta = trunc_bf16(delta_f32[i]);
    else delta = trunc_bf16(__fadd_rn(bf16_bits_to_f32(delta_bf16[i]), trunc_bf16(delta_f32[i])));
    out[i] = trunc_bf16_bits(__fadd_rn(res, delta));
  }
}

template <int kMode>
glmrt_status_t run(const uint16_t* residual, const uint16_t* delta_bf16, const float* delta_f32, uint16_t* out,
                   size_t count, void* cuda_stream, const char* what) {
  if (count == 0) return ok();   // the reference accepts an empty range (residual.cu:1470-1472)
  if (residual == nullptr || out == nullptr || (kMode != 1 && delta_bf16 == nullptr) ||
      (kMode != 0 && delta_f32 == nullptr))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": null pointer argument");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  const size_t blocks = std::min<size_t>((count + kThreads - 1) / kThreads, 148 * 16);
  residual_add_kernel<kMode><<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      residual, delta_bf16, delta_f32, out, count);
  GLMRT_LAUNCH_CHECK(what);
  return ok();
}

glmrt_status_t sync_null(glmrt_status_t st) {
  if (st != GLMRT_STATUS_OK) return st;
  return status_from_cuda(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
}

}  // namespace
}  // namespace glmrt

using namespace glmrt;

extern "C" glmrt_status_t glmrt_cuda_residual_add_bf16_async(const uint16_t* residual, const uint16_t* delta,
                                                             uint16_t* out, size_t count, void* cuda_stream) {
  return run<0>(residual, delta, nullptr, out, count, cuda_stream, "residual_add_bf16");
}
extern "C" glmrt_status_t glmrt_cuda_residual_add_bf16(const uint16_t* residual, const uint16_t* delta, uint16_t* out,
                                                       size_t count) {
  return sync_null(glmrt_cuda_residual_add_bf16_async(residual, delta, out, count, nullptr));
}
extern "C" glmrt_status_t glmrt_cuda_residual_add_f32_delta_bf16_async(const uint16_t* residual, const float* delta_f32,
                                                                       uint16_t* out, size_t count, void* cuda_stream) {
  return run<1>(residual, nullptr, delta_f32, out, count, cuda_stream, "residual_add_f32_delta_bf16");
}
extern "C" glmrt_status_t glmrt_cuda_residual_add_f32_delta_bf16(const uint16_t* residual, const float* delta_f32,
                                                                 uint16_t* out, size_t count) {
  return sync_null(glmrt_cuda_residual_add_f32_delta_bf16_async(residual, delta_f32, out, count, nullptr));
}
extern "C" glmrt_status_t glmrt_cuda_residual_add_shared_f32_delta_bf16_async(
    const uint16_t* residual, const uint16_t* shared_delta, const float* routed_delta_f32, uint16_t* out, size_t count,
    void* cuda_stream) {
  return run<2>(residual, shared_delta, routed_delta_f32, out, count, cuda_stream, "residual_add_shared_f32_delta_bf16");
}
extern "C" glmrt_status_t glmrt_cuda_residual_add_shared_f32_delta_bf16(const uint16_t* residual,
                                                                        const uint16_t* shared_delta,
                                                                        const float* routed_delta_f32, uint16_t* out,
                                                                        size_t count) {
  return sync_null(
      glmrt_cuda_residual_add_shared_f32_delta_bf16_async(residual, shared_delta, routed_delta_f32, out, count, nullptr));
}
