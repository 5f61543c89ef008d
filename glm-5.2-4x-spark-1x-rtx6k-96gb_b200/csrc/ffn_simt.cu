// SIMT verification engine for the NVFP4 expert FFN.
//
// Computes exactly the arithmetic the tensor-core engine is specified to compute --
// FP4 x FP4 products, per-16 block scales, SwiGLU, NVFP4 requantisation of the
// intermediate, down projection -- with one thread per output element and a float64
// accumulator, so it serves as an on-device cross-check at sizes the CPU oracle cannot
// reach.  It reads the same buffers (tiled scales, slot layout, chunk list) as the
// tensor-core kernels.  It corresponds to the reference's SIMT route MLP
// (native/cuda/kernels/mlp.cu:218-314) but is W4A4 like the rest of this library.
// Selected with GLMRT_B200_LAYER_ENGINE_SIMT; never used unless asked for.
#include "common.cuh"
#include "epilogue.cuh"
#include "internal.h"

namespace glmrt {
namespace {

// sum_i a_i * w_i over one 16-element block given 8 packed bytes each (exact in float32).
__device__ __forceinline__ float block_dot(uint2 a, uint2 w) {
  float s = 0.0f;
  const uint32_t aw[2] = {a.x, a.y}, ww[2] = {w.x, w.y};
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int i = 0; i < 8; ++i)
      s += e2m1_to_f32((aw[h] >> (4 * i)) & 0xfu) * e2m1_to_f32((ww[h] >> (4 * i)) & 0xfu);
  return s;
}

__global__ void __launch_bounds__(128) simt_fc1_kernel(FfnArgs a) {
  const int chunk_id = blockIdx.x;
  if (chunk_id >= static_cast<int>(a.counters[kCntChunks])) return;
  const Chunk ch = a.chunks[chunk_id];
  const int f = blockIdx.y * 128 + threadIdx.x;
  const int kb_count = a.hidden / 16;
  const size_t wrow = static_cast<size_t>(ch.expert) * a.inter + f;
  const uint2* gw = reinterpret_cast<const uint2*>(a.gate_codes + wrow * (a.hidden / 2));
  const uint2* uw = reinterpret_cast<const uint2*>(a.up_codes + wrow * (a.hidden / 2));
  const float sg2 = a.scale2[ch.expert * 3 + 0], su2 = a.scale2[ch.expert * 3 + 1];
  for (int n = 0; n < ch.tokens; ++n) {
    const size_t slot = static_cast<size_t>(ch.slot_base) + n;
    const uint2* xa = reinterpret_cast<const uint2*>(a.act1_codes + slot * (a.hidden / 2));
    double accg = 0.0, accu = 0.0;
    for (int kb = 0; kb < kb_count; ++kb) {
      const float sa = e4m3_to_f32(a.act1_sf[sf_tile_offset(slot, kb, kb_count)]);
      const float sgw = e4m3_to_f32(a.gate_sf[sf_tile_offset(wrow, kb, kb_count)]);
      const float suw = e4m3_to_f32(a.up_sf[sf_tile_offset(wrow, kb, kb_count)]);
      const uint2 x = xa[kb];
      accg += static_cast<double>(sa * sgw * block_dot(x, gw[kb]));
      accu += static_cast<double>(sa * suw * block_dot(x, uw[kb]));
    }
    const float g = __fmul_rn(static_cast<float>(accg), sg2);
    const float u = __fmul_rn(static_cast<float>(accu), su2);
    swiglu_requant_store<false>(g, u, f, slot, a.inter, a.act2_codes, a.act2_sf);
  }
}

__global__ void __launch_bounds__(128) simt_fc2_kernel(FfnArgs a) {
  const int chunk_id = blockIdx.x;
  if (chunk_id >= static_cast<int>(a.counters[kCntChunks])) return;
  const Chunk ch = a.chunks[chunk_id];
  const int h = blockIdx.y * 128 + threadIdx.x;
  const int kb_count = a.inter / 16;
  const size_t wrow = static_cast<size_t>(ch.expert) * a.hidden + h;
  const uint2* dw = reinterpret_cast<const uint2*>(a.down_codes + wrow * (a.inter / 2));
  const float sd2 = a.scale2[ch.expert * 3 + 2];
  for (int n = 0; n < ch.tokens; ++n) {
    const size_t slot = static_cast<size_t>(ch.slot_base) + n;
    const uint2* xa = reinterpret_cast<const uint2*>(a.act2_codes + slot * (a.inter / 2));
    double acc = 0.0;
    for (int kb = 0; kb < kb_count; ++kb) {
      const float sa = e4m3_to_f32(a.act2_sf[sf_tile_offset(slot, kb, kb_count)]);
      const float sw = e4m3_to_f32(a.down_sf[sf_tile_offset(wrow, kb, kb_count)]);
      acc += static_cast<double>(sa * sw * block_dot(xa[kb], dw[kb]));
    }
    const float y = __fmul_rn(static_cast<float>(acc), sd2);
    a.slot_out[slot][h] = f32_to_bf16_rne(y);
  }
}

}  // namespace

glmrt_status_t launch_fc1_simt(const FfnArgs& a, cudaStream_t stream) {
  simt_fc1_kernel<<<dim3(a.max_chunks, a.inter / 128), 128, 0, stream>>>(a);
  GLMRT_LAUNCH_CHECK("simt_fc1_kernel");
  return GLMRT_STATUS_OK;
}

glmrt_status_t launch_fc2_simt(const FfnArgs& a, cudaStream_t stream) {
  simt_fc2_kernel<<<dim3(a.max_chunks, a.hidden / 128), 128, 0, stream>>>(a);
  GLMRT_LAUNCH_CHECK("simt_fc2_kernel");
  return GLMRT_STATUS_OK;
}

}  // namespace glmrt
