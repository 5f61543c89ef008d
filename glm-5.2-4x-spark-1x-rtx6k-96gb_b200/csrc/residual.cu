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

// bf16 rows -> E4M3 bytes followed by one float32 scale per row (the reference's response dtype
// Fp8E4m3RowScaled, native/cuda/kernels/residual.cu:245-277): scale = max |finite value| / 448 (1 when
// the row is all zero), byte = e4m3(value / scale) with saturation, non-finite values encode 0.
__device__ __forceinline__ float load_value(const uint16_t* p) { return bf16_bits_to_f32(*p); }
__device__ __forceinline__ float load_value(const float* p) { return *p; }

// T = uint16_t (bf16 rows, in place order) or float (float32 rows picked through row_indices:
// the response pack of residual.cu:160-196)
template <typename T>
__global__ void __launch_bounds__(kThreads)
rows_to_fp8_row_scaled_kernel(const T* __restrict__ src, const uint32_t* __restrict__ row_indices,
                              uint8_t* __restrict__ dst, size_t row_width, size_t dst_row_stride_bytes) {
  __shared__ float warp_max[kThreads / 32];
  __shared__ float row_scale;
  const size_t src_row = row_indices != nullptr ? static_cast<size_t>(row_indices[blockIdx.x]) : blockIdx.x;
  const T* source = src + src_row * row_width;
  uint8_t* output = dst + blockIdx.x * dst_row_stride_bytes;
  float m = 0.0f;
  for (size_t col = threadIdx.x; col < row_width; col += kThreads) {
    const float v = load_value(source + col);
    m = fmaxf(m, isfinite(v) ? fabsf(v) : 0.0f);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float all = 0.0f;
    for (int i = 0; i < kThreads / 32; ++i) all = fmaxf(all, warp_max[i]);
    row_scale = all > 0.0f ? __fdiv_rn(all, 448.0f) : 1.0f;
    *reinterpret_cast<float*>(output + row_width) = row_scale;
  }
  __syncthreads();
  const float scale = row_scale;
  for (size_t col = threadIdx.x; col < row_width; col += kThreads) {
    const float v = load_value(source + col);
    output[col] = static_cast<uint8_t>(f32_to_e4m3_satfinite(isfinite(v) ? __fdiv_rn(v, scale) : 0.0f));
  }
}

glmrt_status_t sync_null(glmrt_status_t st) {
  if (st != GLMRT_STATUS_OK) return st;
  return status_from_cuda(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
}

}  // namespace

glmrt_status_t launch_bf16_rows_to_fp8_row_scaled(const uint16_t* src, uint8_t* dst, size_t rows, size_t row_width,
                                                  size_t dst_row_stride_bytes, cudaStream_t stream) {
  rows_to_fp8_row_scaled_kernel<uint16_t><<<static_cast<unsigned>(rows), kThreads, 0, stream>>>(
      src, nullptr, dst, row_width, dst_row_stride_bytes);
  GLMRT_LAUNCH_CHECK("rows_to_fp8_row_scaled_kernel");
  return GLMRT_STATUS_OK;
}

}  // namespace glmrt

using namespace glmrt;

extern "C" glmrt_status_t glmrt_cuda_bf16_rows_to_fp8_e4m3_row_scaled_async(const uint16_t* src, uint8_t* dst, size_t rows,
                                                                            size_t row_width, size_t dst_row_stride_bytes,
                                                                            void* cuda_stream) {
  // validate_bf16_rows_to_fp8_row_scaled_args (residual.cu:724-737)
  if (src == nullptr || dst == nullptr || rows == 0 || row_width == 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "bf16_rows_to_fp8_row_scaled: null pointer or empty shape");
  if (row_width > SIZE_MAX - sizeof(float) || dst_row_stride_bytes < row_width + sizeof(float) ||
      dst_row_stride_bytes % alignof(float) != 0 || row_width % alignof(float) != 0 || rows > SIZE_MAX / row_width ||
      rows > 0x7fffffffull || reinterpret_cast<uintptr_t>(dst) % alignof(float) != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT,
                "bf16_rows_to_fp8_row_scaled: the row stride must hold the row and a float32 scale, 4-byte aligned");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  GLMRT_RETURN_IF_ERROR(launch_bf16_rows_to_fp8_row_scaled(src, dst, rows, row_width, dst_row_stride_bytes,
                                                           static_cast<cudaStream_t>(cuda_stream)));
  return ok();
}

extern "C" glmrt_status_t glmrt_cuda_gather_rows_f32_to_fp8_e4m3_row_scaled_async(
    const float* src, const uint32_t* row_indices, uint8_t* dst, size_t rows, size_t row_width,
    size_t dst_row_stride_bytes, void* cuda_stream) {
  if (src == nullptr || row_indices == nullptr || dst == nullptr || rows == 0 || row_width == 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "gather_rows_f32_to_fp8_row_scaled: null pointer or empty shape");
  if (row_width > SIZE_MAX - sizeof(float) || dst_row_stride_bytes < row_width + sizeof(float) ||
      dst_row_stride_bytes % alignof(float) != 0 || row_width % alignof(float) != 0 || rows > 0x7fffffffull ||
      reinterpret_cast<uintptr_t>(dst) % alignof(float) != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT,
                "gather_rows_f32_to_fp8_row_scaled: the row stride must hold the row and a float32 scale, 4-byte aligned");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  rows_to_fp8_row_scaled_kernel<float><<<static_cast<unsigned>(rows), kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      src, row_indices, dst, row_width, dst_row_stride_bytes);
  GLMRT_LAUNCH_CHECK("rows_to_fp8_row_scaled_kernel");
  return ok();
}
extern "C" glmrt_status_t glmrt_cuda_gather_rows_f32_to_fp8_e4m3_row_scaled(const float* src, const uint32_t* row_indices,
                                                                            uint8_t* dst, size_t rows, size_t row_width,
                                                                            size_t dst_row_stride_bytes) {
  return sync_null(glmrt_cuda_gather_rows_f32_to_fp8_e4m3_row_scaled_async(src, row_indices, dst, rows, row_width,
                                                                           dst_row_stride_bytes, nullptr));
}

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
