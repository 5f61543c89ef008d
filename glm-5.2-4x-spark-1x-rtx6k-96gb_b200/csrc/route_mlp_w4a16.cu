// Reference-arithmetic route MLP: bf16 activations x NVFP4 weights in float32 (W4A16), the
// computation of the reference's SIMT kernels behind
//   glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_grouped_staged_accumulate_f32[_async]
//   glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_accumulate_f32[_async]
//   glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_single_row_bf16[_async]
// (native/cuda/kernels/mlp.cu:218-518, declared at native/include/glmrt_native.h:572-607):
//   activation[route, m] = silu(x . gate[m]) * (x . up[m])             float32, staged in a workspace
//   accumulator[row, o] += route_weight * (activation[route] . down[o]) float32 atomics
//   single row: out[o] = bf16(sum over the routes of row 0, in route order), truncating, no accumulator
// with every weight dequantised as codebook[code] * e4m3(scale) * scale_2 (common.h:52-58) and no
// quantisation of activations: the arithmetic of the Python reference (moe_ref.py:17-21), unlike
// the layer object's tensor-core path, which is W4A4.  It exists for callers of those symbols and
// as an on-device float32 reference; one warp per output value, lanes stride over the 16-element
// blocks of the reduction (the reference uses one 256-thread CTA per value; the partial sums
// associate differently, results agree to float32 round-off).
#include "common.cuh"
#include "internal.h"

namespace glmrt {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

struct ExpertPtrs {
  const uint8_t* gate_w; const uint8_t* gate_s; const uint8_t* up_w; const uint8_t* up_s;
  const uint8_t* down_w; const uint8_t* down_s;
  size_t intermediate, down_w_stride, down_s_stride;
  float g2, u2, d2;
};

__device__ __forceinline__ ExpertPtrs from_metadata(const glmrt_nvfp4_route_batched_metadata_t& m) {
  ExpertPtrs e;
  e.gate_w = reinterpret_cast<const uint8_t*>(m.gate_weight); e.gate_s = reinterpret_cast<const uint8_t*>(m.gate_scale);
  e.up_w = reinterpret_cast<const uint8_t*>(m.up_weight); e.up_s = reinterpret_cast<const uint8_t*>(m.up_scale);
  e.down_w = reinterpret_cast<const uint8_t*>(m.down_weight); e.down_s = reinterpret_cast<const uint8_t*>(m.down_scale);
  e.intermediate = m.intermediate; e.down_w_stride = m.down_weight_row_stride_bytes;
  e.down_s_stride = m.down_scale_row_stride_bytes;
  e.g2 = m.gate_scale_2; e.u2 = m.up_scale_2; e.d2 = m.down_scale_2;
  return e;
}

// weight value as the reference forms it: (codebook * block scale) * scale_2
__device__ __forceinline__ float wval(uint32_t code, float block_scale, float scale_2) {
  return __fmul_rn(__fmul_rn(e2m1_to_f32(code), block_scale), scale_2);
}

// one warp per (route, intermediate feature)
__global__ void __launch_bounds__(kThreads)
w4a16_activation_kernel(const uint16_t* __restrict__ hidden, const uint32_t* __restrict__ row_indices, ExpertPtrs grouped,
                        const glmrt_nvfp4_route_batched_metadata_t* __restrict__ metadata, float* __restrict__ activations,
                        size_t rows, size_t routes, size_t hidden_dim, size_t hidden_row_stride, size_t max_intermediate) {
  const size_t gw = blockIdx.x * static_cast<size_t>(kWarps) + threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  if (gw >= routes * max_intermediate) return;
  const size_t route = gw / max_intermediate, mid = gw % max_intermediate;
  const ExpertPtrs e = metadata != nullptr ? from_metadata(metadata[route]) : grouped;
  const size_t dest = row_indices[route];
  if (mid >= e.intermediate || dest >= rows) {   // mlp.cu:233-238: out-of-range rows stage a zero
    if (lane == 0) activations[gw] = 0.0f;
    return;
  }
  const uint16_t* x = hidden + dest * hidden_row_stride;
  const size_t kblocks = hidden_dim / 16;
  const uint8_t* gw_row = e.gate_w + mid * (hidden_dim / 2);
  const uint8_t* uw_row = e.up_w + mid * (hidden_dim / 2);
  const uint8_t* gs_row = e.gate_s + mid * kblocks;
  const uint8_t* us_row = e.up_s + mid * kblocks;
  float gate = 0.0f, up = 0.0f;
  for (size_t j = lane; j < kblocks; j += 32) {
    const float gs = e4m3_to_f32(gs_row[j]), us = e4m3_to_f32(us_row[j]);
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const uint32_t gb = gw_row[j * 8 + b], ub = uw_row[j * 8 + b];
      const float x0 = bf16_bits_to_f32(x[j * 16 + 2 * b]), x1 = bf16_bits_to_f32(x[j * 16 + 2 * b + 1]);
      gate = fmaf(x0, wval(gb & 15u, gs, e.g2), gate);
      gate = fmaf(x1, wval(gb >> 4, gs, e.g2), gate);
      up = fmaf(x0, wval(ub & 15u, us, e.u2), up);
      up = fmaf(x1, wval(ub >> 4, us, e.u2), up);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    gate += __shfl_xor_sync(0xffffffffu, gate, off);
    up += __shfl_xor_sync(0xffffffffu, up, off);
  }
  if (lane == 0) activations[gw] = gate * sigmoid_f32(gate) * up;   // mlp.cu:268-271
}

// one warp per (route, output feature)
__global__ void __launch_bounds__(kThreads)
w4a16_down_kernel(const uint32_t* __restrict__ row_indices, const float* __restrict__ route_weights, ExpertPtrs grouped,
                  const glmrt_nvfp4_route_batched_metadata_t* __restrict__ metadata, const float* __restrict__ activations,
                  float* __restrict__ accumulator, size_t rows, size_t routes, size_t max_intermediate, size_t output_dim) {
  const size_t gw = blockIdx.x * static_cast<size_t>(kWarps) + threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  if (gw >= routes * output_dim) return;
  const size_t route = gw / output_dim, out_col = gw % output_dim;
  const size_t dest = row_indices[route];
  if (dest >= rows) return;
  const ExpertPtrs e = metadata != nullptr ? from_metadata(metadata[route]) : grouped;
  const uint8_t* w_row = e.down_w + out_col * e.down_w_stride;
  const uint8_t* s_row = e.down_s + out_col * e.down_s_stride;
  const float* act = activations + route * max_intermediate;
  float acc = 0.0f;
  for (size_t j = lane; j < e.intermediate / 16; j += 32) {
    const float sc = e4m3_to_f32(s_row[j]);
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const uint32_t wb = w_row[j * 8 + b];
      acc = fmaf(act[j * 16 + 2 * b], wval(wb & 15u, sc, e.d2), acc);
      acc = fmaf(act[j * 16 + 2 * b + 1], wval(wb >> 4, sc, e.d2), acc);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) atomicAdd(&accumulator[dest * output_dim + out_col], route_weights[route] * acc);   // mlp.cu:310-312
}

// single row: one warp per output feature walks the routes of row 0 in order (mlp.cu:474-518)
__global__ void __launch_bounds__(kThreads)
w4a16_down_single_row_kernel(const uint32_t* __restrict__ row_indices, const float* __restrict__ route_weights,
                             const glmrt_nvfp4_route_batched_metadata_t* __restrict__ metadata,
                             const float* __restrict__ activations, uint16_t* __restrict__ out, size_t routes,
                             size_t max_intermediate, size_t output_dim) {
  const size_t out_col = blockIdx.x * static_cast<size_t>(kWarps) + threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  if (out_col >= output_dim) return;
  float total = 0.0f;
  for (size_t route = 0; route < routes; ++route) {
    if (row_indices[route] != 0) continue;
    const ExpertPtrs e = from_metadata(metadata[route]);
    const uint8_t* w_row = e.down_w + out_col * e.down_w_stride;
    const uint8_t* s_row = e.down_s + out_col * e.down_s_stride;
    const float* act = activations + route * max_intermediate;
    float acc = 0.0f;
    for (size_t j = lane; j < e.intermediate / 16; j += 32) {
      const float sc = e4m3_to_f32(s_row[j]);
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        const uint32_t wb = w_row[j * 8 + b];
        acc = fmaf(act[j * 16 + 2 * b], wval(wb & 15u, sc, e.d2), acc);
        acc = fmaf(act[j * 16 + 2 * b + 1], wval(wb >> 4, sc, e.d2), acc);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    total = fmaf(route_weights[route], acc, total);
  }
  if (lane == 0) out[out_col] = f32_to_bf16_trunc(total);
}

glmrt_status_t run(const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights, const ExpertPtrs& grouped,
                   const glmrt_nvfp4_route_batched_metadata_t* metadata, float* workspace, float* accumulator, size_t rows,
                   size_t routes, size_t hidden_dim, size_t hidden_row_stride, size_t max_intermediate, size_t output_dim,
                   void* cuda_stream, const char* what, uint16_t* single_row_out = nullptr) {
  if (hidden == nullptr || row_indices == nullptr || route_weights == nullptr || workspace == nullptr ||
      (accumulator == nullptr && single_row_out == nullptr))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": null pointer argument");
  if (rows == 0 || routes == 0 || hidden_dim == 0 || max_intermediate == 0 || output_dim == 0 ||
      hidden_dim % 16 != 0 || max_intermediate % 16 != 0 || hidden_row_stride < hidden_dim)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT,
                std::string(what) + ": dimensions must be positive multiples of 16 and the row stride at least hidden_dim");
  size_t n1 = 0, n2 = 0;
  if (!checked_mul(routes, max_intermediate, &n1) || !checked_mul(routes, output_dim, &n2) ||
      n1 / kWarps + 1 > 0x7fffffffull || n2 / kWarps + 1 > 0x7fffffffull)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": size overflow");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  w4a16_activation_kernel<<<static_cast<unsigned>((n1 + kWarps - 1) / kWarps), kThreads, 0, s>>>(
      hidden, row_indices, grouped, metadata, workspace, rows, routes, hidden_dim, hidden_row_stride, max_intermediate);
  GLMRT_LAUNCH_CHECK("w4a16_activation_kernel");
  if (single_row_out != nullptr) {
    w4a16_down_single_row_kernel<<<static_cast<unsigned>((output_dim + kWarps - 1) / kWarps), kThreads, 0, s>>>(
        row_indices, route_weights, metadata, workspace, single_row_out, routes, max_intermediate, output_dim);
    GLMRT_LAUNCH_CHECK("w4a16_down_single_row_kernel");
    return ok();
  }
  w4a16_down_kernel<<<static_cast<unsigned>((n2 + kWarps - 1) / kWarps), kThreads, 0, s>>>(
      row_indices, route_weights, grouped, metadata, workspace, accumulator, rows, routes, max_intermediate, output_dim);
  GLMRT_LAUNCH_CHECK("w4a16_down_kernel");
  return ok();
}

glmrt_status_t sync_null(glmrt_status_t st) {
  if (st != GLMRT_STATUS_OK) return st;
  return status_from_cuda(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
}

}  // namespace
}  // namespace glmrt

using namespace glmrt;

extern "C" glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_grouped_staged_accumulate_f32_async(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights, const uint8_t* gate_weight,
    const uint8_t* gate_scale, const uint8_t* up_weight, const uint8_t* up_scale, const uint8_t* down_weight,
    const uint8_t* down_scale, float* activation_workspace, float* accumulator, size_t rows, size_t routes,
    size_t hidden_dim, size_t hidden_row_stride, size_t intermediate, size_t output_dim,
    size_t down_weight_row_stride_bytes, size_t down_scale_row_stride_bytes, float gate_scale_2, float up_scale_2,
    float down_scale_2, void* cuda_stream) {
  const char* what = "nvfp4_silu_gated_mlp_route (grouped)";
  if (gate_weight == nullptr || gate_scale == nullptr || up_weight == nullptr || up_scale == nullptr ||
      down_weight == nullptr || down_scale == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": null weight pointer");
  if (down_weight_row_stride_bytes < intermediate / 2 || down_scale_row_stride_bytes < intermediate / 16)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": down row strides smaller than a row");
  ExpertPtrs e{gate_weight, gate_scale, up_weight, up_scale, down_weight, down_scale, intermediate,
               down_weight_row_stride_bytes, down_scale_row_stride_bytes, gate_scale_2, up_scale_2, down_scale_2};
  return run(hidden, row_indices, route_weights, e, nullptr, activation_workspace, accumulator, rows, routes, hidden_dim,
             hidden_row_stride, intermediate, output_dim, cuda_stream, what);
}

extern "C" glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_grouped_staged_accumulate_f32(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights, const uint8_t* gate_weight,
    const uint8_t* gate_scale, const uint8_t* up_weight, const uint8_t* up_scale, const uint8_t* down_weight,
    const uint8_t* down_scale, float* activation_workspace, float* accumulator, size_t rows, size_t routes,
    size_t hidden_dim, size_t hidden_row_stride, size_t intermediate, size_t output_dim,
    size_t down_weight_row_stride_bytes, size_t down_scale_row_stride_bytes, float gate_scale_2, float up_scale_2,
    float down_scale_2) {
  return sync_null(glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_grouped_staged_accumulate_f32_async(
      hidden, row_indices, route_weights, gate_weight, gate_scale, up_weight, up_scale, down_weight, down_scale,
      activation_workspace, accumulator, rows, routes, hidden_dim, hidden_row_stride, intermediate, output_dim,
      down_weight_row_stride_bytes, down_scale_row_stride_bytes, gate_scale_2, up_scale_2, down_scale_2, nullptr));
}

extern "C" glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_accumulate_f32_async(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const glmrt_nvfp4_route_batched_metadata_t* route_metadata, float* activation_workspace, float* accumulator,
    size_t rows, size_t routes, size_t hidden_dim, size_t hidden_row_stride, size_t max_intermediate, size_t output_dim,
    void* cuda_stream) {
  const char* what = "nvfp4_silu_gated_mlp_route (batched)";
  if (route_metadata == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": null route metadata");
  return run(hidden, row_indices, route_weights, ExpertPtrs{}, route_metadata, activation_workspace, accumulator, rows,
             routes, hidden_dim, hidden_row_stride, max_intermediate, output_dim, cuda_stream, what);
}

extern "C" glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_accumulate_f32(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const glmrt_nvfp4_route_batched_metadata_t* route_metadata, float* activation_workspace, float* accumulator,
    size_t rows, size_t routes, size_t hidden_dim, size_t hidden_row_stride, size_t max_intermediate,
    size_t output_dim) {
  return sync_null(glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_accumulate_f32_async(
      hidden, row_indices, route_weights, route_metadata, activation_workspace, accumulator, rows, routes, hidden_dim,
      hidden_row_stride, max_intermediate, output_dim, nullptr));
}

extern "C" glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_single_row_bf16_async(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const glmrt_nvfp4_route_batched_metadata_t* route_metadata, float* activation_workspace, uint16_t* out, size_t rows,
    size_t routes, size_t hidden_dim, size_t hidden_row_stride, size_t max_intermediate, size_t output_dim,
    void* cuda_stream) {
  const char* what = "nvfp4_silu_gated_mlp_route (single row)";
  if (route_metadata == nullptr || out == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": null route metadata or output");
  if (rows != 1) return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": rows must be 1");   // mlp.cu:729-731
  return run(hidden, row_indices, route_weights, ExpertPtrs{}, route_metadata, activation_workspace, nullptr, rows, routes,
             hidden_dim, hidden_row_stride, max_intermediate, output_dim, cuda_stream, what, out);
}

extern "C" glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_single_row_bf16(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const glmrt_nvfp4_route_batched_metadata_t* route_metadata, float* activation_workspace, uint16_t* out, size_t rows,
    size_t routes, size_t hidden_dim, size_t hidden_row_stride, size_t max_intermediate, size_t output_dim) {
  return sync_null(glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_single_row_bf16_async(
      hidden, row_indices, route_weights, route_metadata, activation_workspace, out, rows, routes, hidden_dim,
      hidden_row_stride, max_intermediate, output_dim, nullptr));
}
