// NVFP4 codecs of the routed-MoE path.
//
//   * activation rows -> row payload [cols/2 packed E2M1 | cols/16 E4M3 scales]
//     (replaces native/cuda/kernels/nvfp4_payload.cu:35-73, which runs one 32-thread CTA
//     per 16-element block; here one thread owns one block, a warp reads 1 KiB and
//     writes 256 B contiguously);
//   * weight quantisers (native/cuda/kernels/mlp.cu:98-132 and the benchmark's
//     amax/(6*448) recipe);
//   * payload rows -> bf16 (native/cuda/kernels/b12x_direct.cu:171-201,269-290);
//   * row-major E4M3 scales -> the 128x4 tiled layout read by tcgen05.cp.
#include <cuda_fp4.h>

#include "common.cuh"
#include "internal.h"
#include "quant_block.cuh"

GLMRT_CHAIN_TRACE_TU(quant)

namespace glmrt {
namespace {

constexpr int kThreads = 256;

// ---- activation payload -------------------------------------------------------------
template <bool kNearestLow, bool kVector>
__global__ void __launch_bounds__(kThreads)
quantize_rows_payload_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ payload, size_t rows,
                             int cols) {
  const int blocks_per_row = cols / 16;
  const size_t total = rows * static_cast<size_t>(blocks_per_row);
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= total) return;
  const size_t row = gid / blocks_per_row;
  const int blk = static_cast<int>(gid % blocks_per_row);
  const uint16_t* src = in + row * cols + static_cast<size_t>(blk) * 16;
  float v[16];
  if (kVector) {
    const uint4 a = reinterpret_cast<const uint4*>(src)[0];
    const uint4 b = reinterpret_cast<const uint4*>(src)[1];
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = bf16_bits_to_f32(src[i]);
  }
  uint32_t lo, hi, sbyte;
  quantize_block16<kNearestLow>(v, lo, hi, sbyte);
  uint8_t* prow = payload + row * (static_cast<size_t>(cols) / 2 + blocks_per_row);
  if (kVector) {
    reinterpret_cast<uint2*>(prow)[blk] = make_uint2(lo, hi);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      prow[blk * 8 + i] = static_cast<uint8_t>(lo >> (8 * i));
      prow[blk * 8 + 4 + i] = static_cast<uint8_t>(hi >> (8 * i));
    }
  }
  prow[cols / 2 + blk] = static_cast<uint8_t>(sbyte);
}

// float32 accumulator rows picked through row_indices -> NVFP4 wire rows at a caller row stride
// (the response pack; native/cuda/kernels/nvfp4_payload.cu:75-115 runs a 32-thread CTA per block
// of 16, here a thread owns a block: 64 B read as four 16-byte loads, 8 B + 1 B written).
__global__ void __launch_bounds__(kThreads)
gather_f32_rows_payload_kernel(const float* __restrict__ in, const uint32_t* __restrict__ row_indices,
                               uint8_t* __restrict__ payload, size_t rows, size_t cols, size_t stride_bytes) {
  const size_t blocks_per_row = cols / 16;
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= rows * blocks_per_row) return;
  const size_t row = gid / blocks_per_row, blk = gid % blocks_per_row;
  const float4* src = reinterpret_cast<const float4*>(in + static_cast<size_t>(row_indices[row]) * cols + blk * 16);
  float v[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 q = src[i];
    v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
  }
  uint32_t lo, hi, sbyte;
  quantize_block16<false>(v, lo, hi, sbyte);
  uint8_t* prow = payload + row * stride_bytes;
#pragma unroll
  for (int i = 0; i < 4; ++i) {   // the stride is only byte-granular
    prow[blk * 8 + i] = static_cast<uint8_t>(lo >> (8 * i));
    prow[blk * 8 + 4 + i] = static_cast<uint8_t>(hi >> (8 * i));
  }
  prow[cols / 2 + blk] = static_cast<uint8_t>(sbyte);
}

// ---- weight quantisers -----------------------------------------------------------------
// mlp.cu:98-132: scale = e4m3(amax * g / 6); code = cvt.rn.satfinite.e2m1(v * g / scale).
__global__ void __launch_bounds__(kThreads)
quantize_weight_bf16_mult_kernel(const uint16_t* __restrict__ in, uint8_t* __restrict__ packed,
                                 uint8_t* __restrict__ scales, size_t groups, float g) {
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= groups) return;
  float v[16];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = bf16_bits_to_f32(in[gid * 16 + i]);
    amax = fmaxf(amax, fabsf(v[i]));
  }
  const uint32_t sbyte = f32_to_e4m3_satfinite(__fdiv_rn(__fmul_rn(amax, g), 6.0f));
  const float scale = e4m3_to_f32(sbyte);
  scales[gid] = static_cast<uint8_t>(sbyte);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = scale == 0.0f ? 0.0f : __fdiv_rn(__fmul_rn(v[2 * i], g), scale);
    const float b = scale == 0.0f ? 0.0f : __fdiv_rn(__fmul_rn(v[2 * i + 1], g), scale);
    const uint32_t ca = static_cast<uint32_t>(__nv_cvt_float_to_fp4(a, __NV_E2M1, cudaRoundNearest)) & 0xfu;
    const uint32_t cb = static_cast<uint32_t>(__nv_cvt_float_to_fp4(b, __NV_E2M1, cudaRoundNearest)) & 0xfu;
    packed[gid * 8 + i] = static_cast<uint8_t>(ca | (cb << 4));
  }
}

__global__ void __launch_bounds__(kThreads)
absmax_f32_kernel(const float* __restrict__ in, size_t n, uint32_t* __restrict__ out_bits) {
  float m = 0.0f;
  for (size_t i = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * kThreads)
    m = fmaxf(m, fabsf(in[i]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));  // non-negative floats order as uints
}

// Benchmark recipe: g = amax / (6 * 448); block byte = e4m3(amax_blk / (6 g));
// code = nearest-low(w / (e4m3(byte) * g)).
__global__ void __launch_bounds__(kThreads)
quantize_weight_f32_amax_kernel(const float* __restrict__ in, uint8_t* __restrict__ packed,
                                uint8_t* __restrict__ scales, float* __restrict__ scale_2_out,
                                const uint32_t* __restrict__ amax_bits, size_t groups) {
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  const float g = __fdiv_rn(__uint_as_float(*amax_bits), 2688.0f);
  if (gid == 0) *scale_2_out = g;
  if (gid >= groups) return;
  float v[16];
  const float4* src = reinterpret_cast<const float4*>(in + gid * 16);
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 f = src[i];
    v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float ratio = g == 0.0f ? 0.0f : __fdiv_rn(amax, __fmul_rn(6.0f, g));
  const uint32_t sbyte = f32_to_e4m3_satfinite(ratio);
  const float sg = __fmul_rn(e4m3_to_f32(sbyte), g);
  scales[gid] = static_cast<uint8_t>(sbyte);
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t c = sg == 0.0f ? 0u : fp4_code_nearest_low(__fdiv_rn(v[i], sg));
    if (i < 8) lo |= c << (4 * i); else hi |= c << (4 * (i - 8));
  }
  reinterpret_cast<uint2*>(packed)[gid] = make_uint2(lo, hi);
}

// ---- payload rows -> bf16 (truncating store as the reference's native kernels) ----------
__global__ void __launch_bounds__(kThreads)
gather_payload_rows_bf16_kernel(const uint8_t* __restrict__ payload, size_t source_rows, size_t stride,
                                const uint32_t* __restrict__ row_indices, uint16_t* __restrict__ out,
                                size_t rows, int cols) {
  const size_t total = rows * static_cast<size_t>(cols / 2);
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= total) return;
  const size_t row = gid / (cols / 2);
  const int pair = static_cast<int>(gid % (cols / 2));
  const size_t src_row = row_indices == nullptr ? row : row_indices[row];
  uint32_t packed2 = 0;
  if (src_row < source_rows) {
    const uint8_t* prow = payload + src_row * stride;
    const uint32_t byte = prow[pair];
    const float s = e4m3_to_f32(prow[cols / 2 + pair / 8]);
    const float a = e2m1_to_f32(byte & 0xfu) * s;
    const float b = e2m1_to_f32(byte >> 4) * s;
    packed2 = static_cast<uint32_t>(f32_to_bf16_trunc(a)) | (static_cast<uint32_t>(f32_to_bf16_trunc(b)) << 16);
  }
  reinterpret_cast<uint32_t*>(out)[gid] = packed2;
}

// ---- scale re-tiling ----------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
tile_scales_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, size_t rows, int kblocks,
                   size_t out_row_offset) {
  const size_t total = rows * static_cast<size_t>(kblocks);
  const size_t gid = blockIdx.x * static_cast<size_t>(kThreads) + threadIdx.x;
  if (gid >= total) return;
  const size_t r = gid / kblocks;
  const size_t j = gid % kblocks;
  out[sf_tile_offset(out_row_offset + r, j, kblocks)] = in[gid];
}

unsigned grid_for(size_t n) { return static_cast<unsigned>((n + kThreads - 1) / kThreads); }


// Quantise + dispatch in one pass, one CTA per token row: the row is quantised once into a payload
// image in shared memory, written out as the payload row (the expert-parallel exchange and the
// inspection interface read it) and copied to the slot of each of the row's routes: codes as 16-byte
// vectors, scales as 4-byte words of the tiled layout.  Replaces a launch and the re-read of the
// payload by one warp per route.
constexpr int kFusedThreads = 256;   // measured faster than one thread per 16-element block (384 for hidden 6144)
template <bool kLatency>
__global__ void __launch_bounds__(kFusedThreads)
quantize_dispatch_kernel(const uint16_t* __restrict__ in, DispatchArgs a) {
  GLMRT_CHAIN_SCOPE(kChainQuantDispatch);
  pdl_launch_dependents();
  pdl_wait();
  GLMRT_CHAIN_READY();
  if (static_cast<int>(blockIdx.x) >= a.rows) {
    // an extra CTA: asks the L2 for a quarter of the gate and up weights of one (work item, 128-row
    // tile) pair of FC1's tile order, while the other CTAs quantise and dispatch the rows
    const WeightPrefetch& w = a.prefetch;
    const int id = static_cast<int>(blockIdx.x) - a.rows;
    const int t = id / kPrefetchParts, part = id % kPrefetchParts;
    const int feat_tiles = w.rows_per_expert / 128;
    if (__ldcg(a.counters + kCntError) != 0u || t >= static_cast<int>(__ldcg(a.counters + kCntChunks)) * feat_tiles) return;
    const int expert = __ldcg(&a.chunks[t / feat_tiles].expert);
    const size_t first_row = static_cast<size_t>(expert) * w.rows_per_expert + static_cast<size_t>(t % feat_tiles) * 128;
    prefetch_cta_yield();
    l2_prefetch_weight_tile_part(w.w0, w.sf0, first_row, w.row_bytes, part, kFusedThreads);
    l2_prefetch_weight_tile_part(w.w1, w.sf1, first_row, w.row_bytes, part, kFusedThreads);
    return;
  }
  extern __shared__ uint4 row_img[];
  uint8_t* img = reinterpret_cast<uint8_t*>(row_img);
  const int row = blockIdx.x;
  const int code_bytes = a.hidden / 2;
  const int kblocks = a.hidden / 16;
  const uint16_t* src_row = in + static_cast<size_t>(row) * a.hidden;
  // decode-sized batches: the slots of the row's first eight routes are asked for now and used
  // after the quantisation
  int slots[8];
  if (kLatency) {
#pragma unroll
    for (int j = 0; j < 8; ++j) slots[j] = j < a.top_k ? a.route_slot[row * a.top_k + j] : -1;
  }
  quantize_row_to_image<kLatency>(src_row, img, a.hidden, kFusedThreads);
  __syncthreads();
  GLMRT_CHAIN_MARK(0);
  const int row_vecs = (code_bytes + kblocks) / 16;
  uint4* prow = reinterpret_cast<uint4*>(a.payload_out + static_cast<size_t>(row) * (code_bytes + kblocks));
  for (int i = threadIdx.x; i < row_vecs; i += kFusedThreads) prow[i] = row_img[i];
  const uint32_t* sf_words = reinterpret_cast<const uint32_t*>(img + code_bytes);
  // the slots of up to eight routes are fetched together: one load latency instead of one per route
  for (int k0 = 0; k0 < a.top_k; k0 += 8) {
    if (k0 != 0 || !kLatency) {
#pragma unroll
      for (int j = 0; j < 8; ++j) slots[j] = k0 + j < a.top_k ? a.route_slot[row * a.top_k + k0 + j] : -1;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int slot = slots[j];
      if (slot < 0) continue;   // route of an expert that lives on another shard, or no route
      const int route = row * a.top_k + k0 + j;
      uint4* dst4 = reinterpret_cast<uint4*>(a.act_codes + static_cast<size_t>(slot) * code_bytes);
      for (int i = threadIdx.x; i < code_bytes / 16; i += kFusedThreads) dst4[i] = row_img[i];
      for (int w = threadIdx.x; w < kblocks / 4; w += kFusedThreads)
        *reinterpret_cast<uint32_t*>(a.act_sf + sf_tile_offset(slot, 4 * w, kblocks)) = sf_words[w];
      if (threadIdx.x == 0) {
        if (a.combine_out != nullptr) {
          a.slot_out[slot] = a.combine_out + static_cast<size_t>(row) * a.hidden;
          const uint32_t wb = f32_to_bf16_rne(a.topk_weights[route]);
          a.slot_weight[slot] = wb | (wb << 16);
        } else {
          a.slot_out[slot] = a.route_rows + static_cast<size_t>(route) * a.hidden;
        }
      }
    }
  }
  GLMRT_CHAIN_MARK(1);
}

}  // namespace

bool quantize_dispatch_supported(const uint16_t* in, const DispatchArgs& a) {
  return a.hidden % 128 == 0 && a.hidden <= 16384 && reinterpret_cast<uintptr_t>(in) % 16 == 0 &&
         reinterpret_cast<uintptr_t>(a.payload_out) % 16 == 0;
}

glmrt_status_t launch_quantize_dispatch(const uint16_t* in, const DispatchArgs& a, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(a.hidden) / 2 + a.hidden / 16;
  if (a.rows <= 512)   // a few CTAs per SM at most: the time is the latency of one row
    launch_pdl(quantize_dispatch_kernel<true>, dim3(a.rows + (a.prefetch.w0 != nullptr ? a.prefetch.tiles * kPrefetchParts : 0)),
               dim3(kFusedThreads), smem, stream, in, a);
  else
    launch_pdl(quantize_dispatch_kernel<false>, dim3(a.rows), dim3(kFusedThreads), smem, stream, in, a);
  GLMRT_LAUNCH_CHECK("quantize_dispatch_kernel");
  return GLMRT_STATUS_OK;
}

glmrt_status_t launch_quantize_rows_payload(const uint16_t* in, uint8_t* payload, size_t rows, size_t cols,
                                            uint32_t rule, cudaStream_t stream) {
  const size_t total = rows * (cols / 16);
  const bool vec = (cols % 128 == 0) && (reinterpret_cast<uintptr_t>(in) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(payload) % 8 == 0);
  const int c = static_cast<int>(cols);
  if (rule == GLMRT_B200_FP4_RULE_NEAREST_LOW) {
    if (vec) quantize_rows_payload_kernel<true, true><<<grid_for(total), kThreads, 0, stream>>>(in, payload, rows, c);
    else quantize_rows_payload_kernel<true, false><<<grid_for(total), kThreads, 0, stream>>>(in, payload, rows, c);
  } else {
    if (vec) quantize_rows_payload_kernel<false, true><<<grid_for(total), kThreads, 0, stream>>>(in, payload, rows, c);
    else quantize_rows_payload_kernel<false, false><<<grid_for(total), kThreads, 0, stream>>>(in, payload, rows, c);
  }
  GLMRT_LAUNCH_CHECK("quantize_rows_payload_kernel");
  return GLMRT_STATUS_OK;
}

glmrt_status_t launch_tile_scales(const uint8_t* in, uint8_t* out, size_t rows, size_t kblocks,
                                  size_t out_row_offset, cudaStream_t stream) {
  tile_scales_kernel<<<grid_for(rows * kblocks), kThreads, 0, stream>>>(in, out, rows, static_cast<int>(kblocks),
                                                                        out_row_offset);
  GLMRT_LAUNCH_CHECK("tile_scales_kernel");
  return GLMRT_STATUS_OK;
}

glmrt_status_t launch_quantize_weight_f32(const float* in, uint8_t* packed, uint8_t* scales, float* scale_2_out,
                                          uint32_t* amax_scratch, size_t rows, size_t cols, cudaStream_t stream) {
  const size_t n = rows * cols;
  cudaError_t err = cudaMemsetAsync(amax_scratch, 0, sizeof(uint32_t), stream);
  if (err != cudaSuccess) return status_from_cuda(err, "cudaMemsetAsync");
  const unsigned g1 = static_cast<unsigned>(std::min<size_t>((n + kThreads - 1) / kThreads, 148 * 8));
  absmax_f32_kernel<<<g1, kThreads, 0, stream>>>(in, n, amax_scratch);
  GLMRT_LAUNCH_CHECK("absmax_f32_kernel");
  quantize_weight_f32_amax_kernel<<<grid_for(n / 16), kThreads, 0, stream>>>(in, packed, scales, scale_2_out,
                                                                              amax_scratch, n / 16);
  GLMRT_LAUNCH_CHECK("quantize_weight_f32_amax_kernel");
  return GLMRT_STATUS_OK;
}

}  // namespace glmrt

using namespace glmrt;

namespace {
glmrt_status_t payload_entry(glmrt_device_buffer_t input, glmrt_device_buffer_t payload, size_t rows,
                             size_t hidden_dim, uint32_t rule, void* cuda_stream) {
  if (input.ptr == nullptr || payload.ptr == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "payload quantiser: null buffer");
  if (rows == 0 || hidden_dim == 0 || hidden_dim % 16 != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "payload quantiser: rows > 0 and hidden_dim a positive multiple of 16 required");
  if (rule > GLMRT_B200_FP4_RULE_NEAREST_LOW)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "payload quantiser: unknown code rule");
  size_t values = 0, in_bytes = 0, out_bytes = 0;
  if (!checked_mul(rows, hidden_dim, &values) || !checked_mul(values, 2, &in_bytes) ||
      !checked_mul(rows, hidden_dim / 2 + hidden_dim / 16, &out_bytes))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "payload quantiser: size overflow");
  if (input.bytes < in_bytes || payload.bytes < out_bytes)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "payload quantiser: buffer too small");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  GLMRT_RETURN_IF_ERROR(launch_quantize_rows_payload(static_cast<const uint16_t*>(input.ptr),
                                                     static_cast<uint8_t*>(payload.ptr), rows, hidden_dim, rule,
                                                     static_cast<cudaStream_t>(cuda_stream)));
  return ok();
}
}  // namespace

extern "C" glmrt_status_t glmrt_cuda_b12x_quantize_bf16_nvfp4_row_payload_async(
    glmrt_device_buffer_t input, glmrt_device_buffer_t payload, size_t rows, size_t hidden_dim, void* cuda_stream) {
  return payload_entry(input, payload, rows, hidden_dim, GLMRT_B200_FP4_RULE_RNE_PAYLOAD, cuda_stream);
}

extern "C" glmrt_status_t glmrt_b200_quantize_bf16_nvfp4_row_payload_async(
    glmrt_device_buffer_t input, glmrt_device_buffer_t payload, size_t rows, size_t hidden_dim, uint32_t rule,
    void* cuda_stream) {
  return payload_entry(input, payload, rows, hidden_dim, rule, cuda_stream);
}

extern "C" glmrt_status_t glmrt_cuda_quantize_bf16_weight_nvfp4_async(
    glmrt_device_buffer_t input, glmrt_device_buffer_t packed, glmrt_device_buffer_t scales, size_t rows,
    size_t cols, float global_scale, void* cuda_stream) {
  if (input.ptr == nullptr || packed.ptr == nullptr || scales.ptr == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "weight quantiser: null buffer");
  if (rows == 0 || cols == 0 || cols % 16 != 0 || !(global_scale > 0.0f) || !isfinite(global_scale))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "weight quantiser: rows > 0, cols a positive multiple of 16 and a finite positive global scale required");
  size_t values = 0;
  if (!checked_mul(rows, cols, &values)) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "weight quantiser: size overflow");
  if (input.bytes < values * 2 || packed.bytes < values / 2 || scales.bytes < values / 16)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "weight quantiser: buffer too small");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  quantize_weight_bf16_mult_kernel<<<grid_for(values / 16), kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint16_t*>(input.ptr), static_cast<uint8_t*>(packed.ptr), static_cast<uint8_t*>(scales.ptr),
      values / 16, global_scale);
  GLMRT_LAUNCH_CHECK("quantize_weight_bf16_mult_kernel");
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_quantize_f32_weight_nvfp4_async(
    glmrt_device_buffer_t input, glmrt_device_buffer_t packed, glmrt_device_buffer_t scales,
    glmrt_device_buffer_t scale_2_out, glmrt_device_buffer_t scratch, size_t rows, size_t cols, void* cuda_stream) {
  if (input.ptr == nullptr || packed.ptr == nullptr || scales.ptr == nullptr || scale_2_out.ptr == nullptr ||
      scratch.ptr == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "weight quantiser: null buffer");
  if (rows == 0 || cols == 0 || cols % 16 != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "weight quantiser: rows > 0 and cols a positive multiple of 16 required");
  size_t values = 0;
  if (!checked_mul(rows, cols, &values)) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "weight quantiser: size overflow");
  if (input.bytes < values * 4 || packed.bytes < values / 2 || scales.bytes < values / 16 ||
      scale_2_out.bytes < 4 || scratch.bytes < 4)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "weight quantiser: buffer too small");
  if (reinterpret_cast<uintptr_t>(input.ptr) % 16 != 0 || reinterpret_cast<uintptr_t>(packed.ptr) % 8 != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "weight quantiser: input must be 16-byte and packed 8-byte aligned");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  GLMRT_RETURN_IF_ERROR(launch_quantize_weight_f32(
      static_cast<const float*>(input.ptr), static_cast<uint8_t*>(packed.ptr), static_cast<uint8_t*>(scales.ptr),
      static_cast<float*>(scale_2_out.ptr), static_cast<uint32_t*>(scratch.ptr), rows, cols,
      static_cast<cudaStream_t>(cuda_stream)));
  return ok();
}

extern "C" glmrt_status_t glmrt_cuda_b12x_gather_nvfp4_rows_bf16_async(
    glmrt_device_buffer_t payload, size_t source_rows, size_t source_row_stride_bytes,
    glmrt_device_buffer_t row_indices, glmrt_device_buffer_t output, size_t rows, size_t hidden_dim,
    void* cuda_stream) {
  if (payload.ptr == nullptr || output.ptr == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "payload gather: null buffer");
  if (rows == 0 || source_rows == 0 || hidden_dim == 0 || hidden_dim % 16 != 0 ||
      source_row_stride_bytes < hidden_dim / 2 + hidden_dim / 16)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "payload gather: bad dimensions or row stride");
  size_t src_bytes = 0, out_values = 0;
  if (!checked_mul(source_rows, source_row_stride_bytes, &src_bytes) || !checked_mul(rows, hidden_dim, &out_values))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "payload gather: size overflow");
  // the last row only needs its payload bytes, not a full stride
  if (payload.bytes < src_bytes - source_row_stride_bytes + hidden_dim / 2 + hidden_dim / 16 ||
      output.bytes < out_values * 2 || (row_indices.ptr != nullptr && row_indices.bytes < rows * 4))
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "payload gather: buffer too small");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  gather_payload_rows_bf16_kernel<<<grid_for(out_values / 2), kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint8_t*>(payload.ptr), source_rows, source_row_stride_bytes,
      static_cast<const uint32_t*>(row_indices.ptr), static_cast<uint16_t*>(output.ptr), rows,
      static_cast<int>(hidden_dim));
  GLMRT_LAUNCH_CHECK("gather_payload_rows_bf16_kernel");
  return ok();
}

extern "C" glmrt_status_t glmrt_cuda_gather_rows_f32_to_nvfp4_e2m1_fp8_e4m3_async(
    const float* src, const uint32_t* row_indices, uint8_t* dst, size_t rows, size_t row_width,
    size_t dst_row_stride_bytes, void* cuda_stream) {
  if (src == nullptr || row_indices == nullptr || dst == nullptr || rows == 0 || row_width == 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "gather_rows_f32_to_nvfp4: null pointer or empty shape");
  if (row_width % 16 != 0 || dst_row_stride_bytes < row_width / 2 + row_width / 16)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT,
                "gather_rows_f32_to_nvfp4: the width must be a multiple of 16 and the row stride must hold codes and scales");
  if (reinterpret_cast<uintptr_t>(src) % 16 != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "gather_rows_f32_to_nvfp4: the source must be 16-byte aligned");
  size_t blocks = 0;
  if (!checked_mul(rows, row_width / 16, &blocks) || blocks / kThreads + 1 > 0x7fffffffull)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "gather_rows_f32_to_nvfp4: size overflow");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  gather_f32_rows_payload_kernel<<<grid_for(blocks), kThreads, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      src, row_indices, dst, rows, row_width, dst_row_stride_bytes);
  GLMRT_LAUNCH_CHECK("gather_f32_rows_payload_kernel");
  return ok();
}

extern "C" glmrt_status_t glmrt_cuda_gather_rows_f32_to_nvfp4_e2m1_fp8_e4m3(
    const float* src, const uint32_t* row_indices, uint8_t* dst, size_t rows, size_t row_width,
    size_t dst_row_stride_bytes) {
  const glmrt_status_t st = glmrt_cuda_gather_rows_f32_to_nvfp4_e2m1_fp8_e4m3_async(src, row_indices, dst, rows, row_width,
                                                                                   dst_row_stride_bytes, nullptr);
  if (st != GLMRT_STATUS_OK) return st;
  return status_from_cuda(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
}
