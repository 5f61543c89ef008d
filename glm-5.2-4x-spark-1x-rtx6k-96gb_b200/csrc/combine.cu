// Combine: per-route FC2 rows -> one output row per token.
//
//   * combine_routes_kernel restates the accumulation of the Python oracle
//     (python/reference/glmrt_reference/moe_ref.py:30-36): for slot in order,
//     out = bf16(out + bf16(bf16(w) * y)), so the result is independent of how routes were
//     scheduled and bit-reproducible (the reference keeps a fixed-order sum for the same
//     reason: native/cuda/kernels/b12x_direct.cu:203-219, residual.cu:438-453);
//   * sum_topk8, weighted scatter-add and row gather keep the reference entry points
//     (b12x_direct.cu:203-219, residual.cu:666-678, residual.cu:133-158).
#include "common.cuh"
#include "ep_flags.cuh"
#include "internal.h"

GLMRT_CHAIN_TRACE_TU(combine)

namespace glmrt {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t bf16x2_mul_rn(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_add_rn(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// kResidual: the summed routed row is not stored as such but folded into the layer output the way
// the reference's residual kernel does it (native/cuda/kernels/residual.cu:36-62, truncating bf16
// stores): mlp = bf16(shared + routed) when a shared-expert row is given, out = bf16(residual + mlp).
template <bool kResidual>
__global__ void __launch_bounds__(kThreads)
combine_routes_kernel(const uint16_t* __restrict__ route_rows, const float* __restrict__ topk_weights,
                      const int32_t* __restrict__ route_slot, uint16_t* __restrict__ out, int rows, int top_k,
                      int hidden, const uint16_t* __restrict__ residual, const uint16_t* __restrict__ shared,
                      EpWait wait, uint32_t* error_word) {
  GLMRT_CHAIN_SCOPE(kChainCombine);
  pdl_launch_dependents();
  pdl_wait();
  GLMRT_CHAIN_READY();
  if (wait.flags != nullptr) {
    // expert-parallel path: the route rows are stored by the owners of the experts; their flags say when
    __shared__ uint32_t s_wait_err;
    if (threadIdx.x == 0) {
      s_wait_err = ep_wait_all_serial(wait);
      if (s_wait_err != 0u) atomicOr(error_word, s_wait_err);
    }
    __syncthreads();
    if (s_wait_err != 0u) return;
  }
  GLMRT_CHAIN_MARK(0);
  const int vec_per_row = hidden / 8;
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= static_cast<size_t>(rows) * vec_per_row) return;
  const int row = static_cast<int>(gid / vec_per_row);
  const int v = static_cast<int>(gid % vec_per_row);
  // Pairs of bf16 sums.  mul.rn.bf16x2 and add.rn.bf16x2 round the exact product / sum of bf16
  // operands once to bf16, which is what the float32 operation followed by a round-to-nearest-even
  // conversion yields: the product of two 8-bit significands is exact in float32, and a float32 sum
  // of two bf16 values that is not exact differs from the larger operand by less than 2^-15 of it,
  // nowhere near a bf16 rounding boundary.
  uint32_t acc2[4] = {0u, 0u, 0u, 0u};
  // rows are fetched eight routes at a time before any arithmetic, so the loads overlap
  for (int k0 = 0; k0 < top_k; k0 += 8) {
    uint4 y4[8];
    uint32_t w2[8];
    bool use[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int k = k0 + j;
      const int r = row * top_k + k;
      use[j] = k < top_k && (route_slot == nullptr || route_slot[r] >= 0);
      if (use[j]) {
        y4[j] = reinterpret_cast<const uint4*>(route_rows + static_cast<size_t>(r) * hidden)[v];
        const uint32_t wb = f32_to_bf16_rne(topk_weights[r]);
        w2[j] = wb | (wb << 16);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (!use[j]) continue;
      const uint32_t yw[4] = {y4[j].x, y4[j].y, y4[j].z, y4[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) acc2[i] = bf16x2_add_rn(acc2[i], bf16x2_mul_rn(w2[j], yw[i]));
    }
  }
  float acc[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] = __uint_as_float(acc2[i] << 16);
    acc[2 * i + 1] = __uint_as_float(acc2[i] & 0xffff0000u);
  }
  if (kResidual) {
    const size_t off = static_cast<size_t>(row) * hidden;
    const uint4 r4 = reinterpret_cast<const uint4*>(residual + off)[v];
    const uint32_t rw[4] = {r4.x, r4.y, r4.z, r4.w};
    uint32_t sw[4] = {0u, 0u, 0u, 0u};
    if (shared != nullptr) {
      const uint4 s4 = reinterpret_cast<const uint4*>(shared + off)[v];
      sw[0] = s4.x; sw[1] = s4.y; sw[2] = s4.z; sw[3] = s4.w;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float res = __uint_as_float(h == 0 ? rw[i] << 16 : rw[i] & 0xffff0000u);
        float mlp = acc[2 * i + h];
        if (shared != nullptr) {
          const float sh = __uint_as_float(h == 0 ? sw[i] << 16 : sw[i] & 0xffff0000u);
          mlp = __uint_as_float(__float_as_uint(__fadd_rn(sh, mlp)) & 0xffff0000u);
        }
        acc[2 * i + h] = __uint_as_float(__float_as_uint(__fadd_rn(res, mlp)) & 0xffff0000u);
      }
    }
  }
  uint4 o;
  o.x = (__float_as_uint(acc[0]) >> 16) | (__float_as_uint(acc[1]) & 0xffff0000u);
  o.y = (__float_as_uint(acc[2]) >> 16) | (__float_as_uint(acc[3]) & 0xffff0000u);
  o.z = (__float_as_uint(acc[4]) >> 16) | (__float_as_uint(acc[5]) & 0xffff0000u);
  o.w = (__float_as_uint(acc[6]) >> 16) | (__float_as_uint(acc[7]) & 0xffff0000u);
  reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * hidden)[v] = o;
}

// Fixed-order float32 sum of 8 rows of width 6144, truncating bf16 store.
__global__ void __launch_bounds__(kThreads)
sum_topk8_kernel(const uint16_t* __restrict__ routed, uint16_t* __restrict__ out, size_t rows) {
  constexpr int kWidth = 6144, kTop = 8;
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= rows * (kWidth / 2)) return;
  const size_t row = gid / (kWidth / 2);
  const size_t pair = gid % (kWidth / 2);
  float a = 0.0f, b = 0.0f;
#pragma unroll
  for (int k = 0; k < kTop; ++k) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(routed + (row * kTop + k) * kWidth)[pair];
    a = __fadd_rn(a, __uint_as_float(w << 16));
    b = __fadd_rn(b, __uint_as_float(w & 0xffff0000u));
  }
  reinterpret_cast<uint32_t*>(out + row * kWidth)[pair] =
      (__float_as_uint(a) >> 16) | (__float_as_uint(b) & 0xffff0000u);
}

__global__ void __launch_bounds__(kThreads)
scatter_add_weighted_kernel(const uint16_t* __restrict__ src, const uint32_t* __restrict__ row_indices,
                            const float* __restrict__ row_weights, float* __restrict__ dst, size_t rows,
                            size_t width) {
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= rows * width) return;
  const size_t r = gid / width, c = gid % width;
  atomicAdd(&dst[static_cast<size_t>(row_indices[r]) * width + c], row_weights[r] * bf16_bits_to_f32(src[gid]));
}

__global__ void __launch_bounds__(kThreads)
gather_rows_bf16_kernel(const uint16_t* __restrict__ src, const uint32_t* __restrict__ row_indices,
                        uint16_t* __restrict__ dst, size_t rows, size_t width) {
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= rows * width) return;
  const size_t r = gid / width, c = gid % width;
  dst[gid] = src[static_cast<size_t>(row_indices[r]) * width + c];
}

unsigned grid_for(size_t n) { return static_cast<unsigned>((n + kThreads - 1) / kThreads); }

}  // namespace

glmrt_status_t launch_combine_routes(const uint16_t* route_rows, const float* topk_weights,
                                     const int32_t* route_slot, uint16_t* out, int rows, int top_k, int hidden,
                                     cudaStream_t stream, const uint16_t* residual, const uint16_t* shared,
                                     const EpWait* wait, uint32_t* error_word) {
  const unsigned grid = grid_for(static_cast<size_t>(rows) * (hidden / 8));
  EpWait w;
  if (wait != nullptr && error_word != nullptr) w = *wait;
  if (residual != nullptr)
    launch_pdl(combine_routes_kernel<true>, dim3(grid), dim3(kThreads), 0, stream, route_rows, topk_weights, route_slot,
               out, rows, top_k, hidden, residual, shared, w, error_word);
  else
    launch_pdl(combine_routes_kernel<false>, dim3(grid), dim3(kThreads), 0, stream, route_rows, topk_weights, route_slot,
               out, rows, top_k, hidden, static_cast<const uint16_t*>(nullptr), static_cast<const uint16_t*>(nullptr), w,
               error_word);
  GLMRT_LAUNCH_CHECK("combine_routes_kernel");
  return GLMRT_STATUS_OK;
}

}  // namespace glmrt

using namespace glmrt;

extern "C" glmrt_status_t glmrt_cuda_b12x_spark_sum_topk8_bf16_async(glmrt_device_buffer_t routed_bf16,
                                                                     glmrt_device_buffer_t output_bf16,
                                                                     size_t rows, void* cuda_stream) {
  if (routed_bf16.ptr == nullptr || output_bf16.ptr == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "sum_topk8: null buffer");
  if (rows == 0) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "sum_topk8: rows must be > 0");
  size_t out_bytes = 0, in_bytes = 0;
  if (!checked_mul(rows, 6144 * 2, &out_bytes) || !checked_mul(out_bytes, 8, &in_bytes))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "sum_topk8: size overflow");
  if (routed_bf16.bytes < in_bytes || output_bf16.bytes < out_bytes)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "sum_topk8: buffer too small");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  sum_topk8_kernel<<<grid_for(rows * 3072), kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint16_t*>(routed_bf16.ptr), static_cast<uint16_t*>(output_bf16.ptr), rows);
  GLMRT_LAUNCH_CHECK("sum_topk8_kernel");
  return ok();
}

extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_bf16_weighted_to_f32_async(
    const uint16_t* src, const uint32_t* row_indices, const float* row_weights, float* dst, size_t rows,
    size_t row_width, void* cuda_stream) {
  if (src == nullptr || row_indices == nullptr || row_weights == nullptr || dst == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "scatter_add: null pointer argument");
  size_t total = 0;
  if (rows == 0 || row_width == 0 || !checked_mul(rows, row_width, &total))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "scatter_add: bad dimensions");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  scatter_add_weighted_kernel<<<grid_for(total), kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      src, row_indices, row_weights, dst, rows, row_width);
  GLMRT_LAUNCH_CHECK("scatter_add_weighted_kernel");
  return ok();
}
extern "C" glmrt_status_t glmrt_cuda_scatter_add_rows_bf16_weighted_to_f32(const uint16_t* src,
                                                                           const uint32_t* row_indices,
                                                                           const float* row_weights, float* dst,
                                                                           size_t rows, size_t row_width) {
  GLMRT_RETURN_IF_ERROR(glmrt_cuda_scatter_add_rows_bf16_weighted_to_f32_async(src, row_indices, row_weights, dst,
                                                                               rows, row_width, nullptr));
  return status_from_cuda(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
}

extern "C" glmrt_status_t glmrt_cuda_gather_rows_bf16_async(const uint16_t* src, const uint32_t* row_indices,
                                                            uint16_t* dst, size_t rows, size_t row_width,
                                                            void* cuda_stream) {
  if (src == nullptr || row_indices == nullptr || dst == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "gather_rows: null pointer argument");
  size_t total = 0;
  if (rows == 0 || row_width == 0 || !checked_mul(rows, row_width, &total))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "gather_rows: bad dimensions");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  gather_rows_bf16_kernel<<<grid_for(total), kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      src, row_indices, dst, rows, row_width);
  GLMRT_LAUNCH_CHECK("gather_rows_bf16_kernel");
  return ok();
}
