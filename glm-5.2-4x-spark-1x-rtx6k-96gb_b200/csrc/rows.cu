// Row gather / scatter-add / shard reduction of the reference ABI around the routed-MoE path
// (native/include/glmrt_native.h:757-836; kernels native/cuda/kernels/residual.cu:133-158,409-589):
// the coordinator-side glue that compacts the rows a host needs, adds the hosts' partial rows back
// into float32 accumulators (from bf16, row-scaled FP8 or NVFP4 wire rows) and sums shard partials.
//
// Scatter-adds of at most 64 compact rows visit the contributions of an output column in wire
// order from one thread (no atomics, fixed summation order), as the reference does for decode and
// verify batches (residual.cu:438-453); larger ones use float32 atomics.
#include "common.cuh"
#include "internal.h"

namespace glmrt {
namespace {

constexpr int kThreads = 256;
constexpr size_t kOrderedMaxRows = 64;

enum Wire { kF32 = 0, kBf16 = 1, kFp8RowScaled = 2, kNvfp4 = 3 };

// value (row r, column c) of a row table in one of the wire formats (residual.cu:544-559)
template <int kWire>
__device__ __forceinline__ float wire_value(const uint8_t* src, size_t stride_bytes, size_t r, size_t c, size_t width) {
  const uint8_t* row = src + r * stride_bytes;
  if (kWire == kF32) return reinterpret_cast<const float*>(row)[c];
  if (kWire == kBf16) return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(row)[c]);
  if (kWire == kFp8RowScaled) return __fmul_rn(e4m3_to_f32(row[c]), *reinterpret_cast<const float*>(row + width));
  const uint32_t byte = row[c / 2];
  return __fmul_rn(e2m1_to_f32(c % 2 == 0 ? (byte & 15u) : (byte >> 4)), e4m3_to_f32(row[width / 2 + c / 16]));
}

template <int kWire>
__global__ void __launch_bounds__(kThreads)
scatter_add_atomic_kernel(const uint8_t* __restrict__ src, size_t stride_bytes, const uint32_t* __restrict__ row_indices,
                          float* __restrict__ dst, size_t rows, size_t width) {
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= rows * width) return;
  const size_t r = gid / width, c = gid % width;
  atomicAdd(&dst[static_cast<size_t>(row_indices[r]) * width + c], wire_value<kWire>(src, stride_bytes, r, c, width));
}

template <int kWire>
__global__ void __launch_bounds__(kThreads)
scatter_add_ordered_kernel(const uint8_t* __restrict__ src, size_t stride_bytes, const uint32_t* __restrict__ row_indices,
                           float* __restrict__ dst, size_t rows, size_t width) {
  const size_t c = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (c >= width) return;
  for (size_t r = 0; r < rows; ++r) {
    float* v = dst + static_cast<size_t>(row_indices[r]) * width + c;
    *v = __fadd_rn(*v, wire_value<kWire>(src, stride_bytes, r, c, width));
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
gather_rows_kernel(const T* __restrict__ src, const uint32_t* __restrict__ row_indices, T* __restrict__ dst, size_t rows,
                   size_t width) {
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= rows * width) return;
  dst[gid] = src[static_cast<size_t>(row_indices[gid / width]) * width + gid % width];
}

// local (float32 or bf16) + up to three peers' wire rows, added in peer order (residual.cu:561-589)
template <int kWire>
__global__ void __launch_bounds__(kThreads)
reduce_shards_kernel(const uint8_t* __restrict__ local, bool local_f32, const uint8_t* __restrict__ p0,
                     const uint8_t* __restrict__ p1, const uint8_t* __restrict__ p2, float* __restrict__ out, size_t rows,
                     size_t width, size_t stride_bytes, uint32_t peers) {
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= rows * width) return;
  const size_t r = gid / width, c = gid % width;
  float sum = local_f32 ? reinterpret_cast<const float*>(local)[gid]
                        : bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(local)[gid]);
  if (peers > 0) sum = __fadd_rn(sum, wire_value<kWire>(p0, stride_bytes, r, c, width));
  if (peers > 1) sum = __fadd_rn(sum, wire_value<kWire>(p1, stride_bytes, r, c, width));
  if (peers > 2) sum = __fadd_rn(sum, wire_value<kWire>(p2, stride_bytes, r, c, width));
  out[gid] = sum;
}

unsigned blocks_for(size_t n) { return static_cast<unsigned>((n + kThreads - 1) / kThreads); }

template <int kWire>
glmrt_status_t scatter_add(const void* src, size_t stride_bytes, const uint32_t* row_indices, float* dst, size_t rows,
                           size_t width, void* cuda_stream, const char* what) {
  if (rows == 0 || width == 0) return ok();   // the reference accepts empty work (residual.cu scatter entry points)
  if (src == nullptr || row_indices == nullptr || dst == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": null pointer argument");
  size_t total = 0;
  if (!checked_mul(rows, width, &total) || total / kThreads + 1 > 0x7fffffffull)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": size overflow");
  const size_t need = kWire == kF32 ? width * 4 : kWire == kBf16 ? width * 2 : kWire == kFp8RowScaled ? width + 4
                                                                                                  : width / 2 + width / 16;
  if (stride_bytes < need || (kWire == kFp8RowScaled && stride_bytes % 4 != 0) || (kWire == kNvfp4 && width % 16 != 0))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": row stride or width does not fit the wire format");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const uint8_t* p = static_cast<const uint8_t*>(src);
  if (rows <= kOrderedMaxRows)
    scatter_add_ordered_kernel<kWire><<<blocks_for(width), kThreads, 0, s>>>(p, stride_bytes, row_indices, dst, rows, width);
  else
    scatter_add_atomic_kernel<kWire><<<blocks_for(total), kThreads, 0, s>>>(p, stride_bytes, row_indices, dst, rows, width);
  GLMRT_LAUNCH_CHECK(what);
  return ok();
}

template <typename T>
glmrt_status_t gather(const T* src, const uint32_t* row_indices, T* dst, size_t rows, size_t width, void* cuda_stream,
                      const char* what) {
  if (src == nullptr || row_indices == nullptr || dst == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": null pointer argument");
  size_t total = 0;
  if (rows == 0 || width == 0 || !checked_mul(rows, width, &total) || total / kThreads + 1 > 0x7fffffffull)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": bad dimensions");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  gather_rows_kernel<T><<<blocks_for(total), kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(src, row_indices, dst,
                                                                                                 rows, width);
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

extern "C" glmrt_status_t glmrt_cuda_gather_rows_f32_async(const float* src, const uint32_t* row_indices, float* dst,
                                                           size_t rows, size_t row_width, void* cuda_stream) {
  return gather<float>(src, row_indices, dst, rows, row_width, cuda_stream, "gather_rows_f32");
}
extern "C" glmrt_status_t glmrt_cuda_gather_rows_f32(const float* src, const uint32_t* row_indices, float* dst, size_t rows,
                                                     size_t row_width) {
  return sync_null(glmrt_cuda_gather_rows_f32_async(src, row_indices, dst, rows, row_width, nullptr));
}
extern "C" glmrt_status_t glmrt_cuda_gather_rows_bf16(const uint16_t* src, const uint32_t* row_indices, uint16_t* dst,
                                                      size_t rows, size_t row_width) {
  return sync_null(glmrt_cuda_gather_rows_bf16_async(src, row_indices, dst, rows, row_width, nullptr));
}

extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_f32_async(const float* src, const uint32_t* row_indices, float* dst,
                                                                size_t rows, size_t row_width, void* cuda_stream) {
  return scatter_add<kF32>(src, row_width * 4, row_indices, dst, rows, row_width, cuda_stream, "scatter_add_rows_f32");
}
extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_f32(const float* src, const uint32_t* row_indices, float* dst,
                                                          size_t rows, size_t row_width) {
  return sync_null(glmrt_cuda_scatter_add_rows_f32_async(src, row_indices, dst, rows, row_width, nullptr));
}
extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_bf16_to_f32_async(const uint16_t* src, const uint32_t* row_indices,
                                                                        float* dst, size_t rows, size_t row_width,
                                                                        void* cuda_stream) {
  return scatter_add<kBf16>(src, row_width * 2, row_indices, dst, rows, row_width, cuda_stream, "scatter_add_rows_bf16_to_f32");
}
extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_bf16_to_f32(const uint16_t* src, const uint32_t* row_indices,
                                                                  float* dst, size_t rows, size_t row_width) {
  return sync_null(glmrt_cuda_scatter_add_rows_bf16_to_f32_async(src, row_indices, dst, rows, row_width, nullptr));
}
extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_fp8_e4m3_row_scaled_to_f32_async(
    const uint8_t* src, size_t src_row_stride_bytes, const uint32_t* row_indices, float* dst, size_t rows, size_t row_width,
    void* cuda_stream) {
  return scatter_add<kFp8RowScaled>(src, src_row_stride_bytes, row_indices, dst, rows, row_width, cuda_stream,
                                    "scatter_add_rows_fp8_e4m3_row_scaled_to_f32");
}
extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_fp8_e4m3_row_scaled_to_f32(const uint8_t* src,
                                                                                 size_t src_row_stride_bytes,
                                                                                 const uint32_t* row_indices, float* dst,
                                                                                 size_t rows, size_t row_width) {
  return sync_null(glmrt_cuda_scatter_add_rows_fp8_e4m3_row_scaled_to_f32_async(src, src_row_stride_bytes, row_indices, dst,
                                                                                rows, row_width, nullptr));
}
extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_nvfp4_e2m1_fp8_e4m3_to_f32_async(
    const uint8_t* src, size_t src_row_stride_bytes, const uint32_t* row_indices, float* dst, size_t rows, size_t row_width,
    void* cuda_stream) {
  return scatter_add<kNvfp4>(src, src_row_stride_bytes, row_indices, dst, rows, row_width, cuda_stream,
                             "scatter_add_rows_nvfp4_e2m1_fp8_e4m3_to_f32");
}
extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_nvfp4_e2m1_fp8_e4m3_to_f32(const uint8_t* src,
                                                                                 size_t src_row_stride_bytes,
                                                                                 const uint32_t* row_indices, float* dst,
                                                                                 size_t rows, size_t row_width) {
  return sync_null(glmrt_cuda_scatter_add_rows_nvfp4_e2m1_fp8_e4m3_to_f32_async(src, src_row_stride_bytes, row_indices, dst,
                                                                                rows, row_width, nullptr));
}

extern "C" glmrt_status_t glmrt_cuda_reduce_route_shards_to_f32_async(const glmrt_route_shard_reduction_buffers_t* buffers,
                                                                      size_t rows, size_t row_width,
                                                                      size_t peer_row_stride_bytes, uint32_t local_dtype,
                                                                      uint32_t peer_dtype, uint32_t peer_count,
                                                                      void* cuda_stream) {
  // validate_route_shard_reduction_args (residual.cu:853-905)
  const char* what = "reduce_route_shards_to_f32";
  if (buffers == nullptr || buffers->local.ptr == nullptr || buffers->output_f32.ptr == nullptr || rows == 0 ||
      row_width == 0 || peer_count == 0 || peer_count > 3)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": null buffer, empty shape or peer count outside 1..3");
  if (local_dtype != GLMRT_ROUTE_SHARD_LOCAL_F32 && local_dtype != GLMRT_ROUTE_SHARD_LOCAL_BF16)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": unknown local dtype");
  size_t values = 0;
  if (!checked_mul(rows, row_width, &values) || values > SIZE_MAX / 4 || values / kThreads + 1 > 0x7fffffffull)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": size overflow");
  const size_t local_bytes = values * (local_dtype == GLMRT_ROUTE_SHARD_LOCAL_F32 ? 4 : 2);
  if (buffers->local.bytes < local_bytes || buffers->output_f32.bytes < values * 4)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": local or output buffer too small");
  size_t min_stride = 0;
  if (peer_dtype == GLMRT_ROUTE_SHARD_WIRE_BF16) min_stride = row_width * 2;
  else if (peer_dtype == GLMRT_ROUTE_SHARD_WIRE_FP8_E4M3_ROW_SCALED && peer_row_stride_bytes % 4 == 0) min_stride = row_width + 4;
  else if (peer_dtype == GLMRT_ROUTE_SHARD_WIRE_NVFP4_E2M1_FP8_E4M3 && row_width % 16 == 0) min_stride = row_width / 2 + row_width / 16;
  else return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": unknown peer dtype or shape unfit for it");
  if (peer_row_stride_bytes < min_stride) return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": peer row stride too small");
  for (uint32_t p = 0; p < peer_count; ++p)
    if (buffers->peers[p].ptr == nullptr || buffers->peers[p].bytes < (rows - 1) * peer_row_stride_bytes + min_stride)
      return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": peer buffer missing or too small");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const uint8_t* l = static_cast<const uint8_t*>(buffers->local.ptr);
  const uint8_t* p0 = static_cast<const uint8_t*>(buffers->peers[0].ptr);
  const uint8_t* p1 = static_cast<const uint8_t*>(buffers->peers[1].ptr);
  const uint8_t* p2 = static_cast<const uint8_t*>(buffers->peers[2].ptr);
  float* out = static_cast<float*>(buffers->output_f32.ptr);
  const bool lf = local_dtype == GLMRT_ROUTE_SHARD_LOCAL_F32;
  const unsigned grid = blocks_for(values);
  if (peer_dtype == GLMRT_ROUTE_SHARD_WIRE_BF16)
    reduce_shards_kernel<kBf16><<<grid, kThreads, 0, s>>>(l, lf, p0, p1, p2, out, rows, row_width, peer_row_stride_bytes, peer_count);
  else if (peer_dtype == GLMRT_ROUTE_SHARD_WIRE_FP8_E4M3_ROW_SCALED)
    reduce_shards_kernel<kFp8RowScaled><<<grid, kThreads, 0, s>>>(l, lf, p0, p1, p2, out, rows, row_width, peer_row_stride_bytes, peer_count);
  else
    reduce_shards_kernel<kNvfp4><<<grid, kThreads, 0, s>>>(l, lf, p0, p1, p2, out, rows, row_width, peer_row_stride_bytes, peer_count);
  GLMRT_LAUNCH_CHECK(what);
  return ok();
}
extern "C" glmrt_status_t glmrt_cuda_reduce_route_shards_to_f32(const glmrt_route_shard_reduction_buffers_t* buffers,
                                                                size_t rows, size_t row_width, size_t peer_row_stride_bytes,
                                                                uint32_t local_dtype, uint32_t peer_dtype,
                                                                uint32_t peer_count) {
  return sync_null(glmrt_cuda_reduce_route_shards_to_f32_async(buffers, rows, row_width, peer_row_stride_bytes, local_dtype,
                                                               peer_dtype, peer_count, nullptr));
}
