// Epilogue arithmetic shared by the tensor-core engine and the SIMT verification engine.
#pragma once

#include "common.cuh"

namespace glmrt {

// SwiGLU + NVFP4 requantisation of one (feature, token) value per lane.
//
// Called by a full warp whose lanes hold 32 consecutive intermediate features
// (feature = f0 + lane, f0 a multiple of 32) of one token slot.  a = silu(g) * u as
// python/reference/glmrt_reference/moe_ref.py:18-20; the 16-feature block scale is
// e4m3(amax / 6) and codes follow quant_ref.py:41-46 (x / scale, ties to the lower
// magnitude) so the result matches a quantise->dequantise of the float32 intermediate.
// Writes 16 code bytes and 2 scale bytes per warp.
__device__ __forceinline__ void swiglu_requant_store(float g, float u, int feature, size_t slot, int inter,
                                                     uint8_t* __restrict__ act2_codes,
                                                     uint8_t* __restrict__ act2_sf) {
  const int lane = threadIdx.x & 31;
  const float a = __fmul_rn(__fmul_rn(g, sigmoid_f32(g)), u);
  float amax = fabsf(a);
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const uint32_t sbyte = f32_to_e4m3_satfinite(__fdiv_rn(amax, 6.0f));
  const float scale = e4m3_to_f32(sbyte);
  const uint32_t code = scale == 0.0f ? 0u : fp4_code_nearest_low(__fdiv_rn(a, scale));
  uint32_t v = code << (4 * (lane & 7));
  v |= __shfl_xor_sync(0xffffffffu, v, 1);
  v |= __shfl_xor_sync(0xffffffffu, v, 2);
  v |= __shfl_xor_sync(0xffffffffu, v, 4);
  if ((lane & 7) == 0)
    *reinterpret_cast<uint32_t*>(act2_codes + slot * static_cast<size_t>(inter / 2) + feature / 2) = v;
  if ((lane & 15) == 0) act2_sf[sf_tile_offset(slot, feature / 16, inter / 16)] = static_cast<uint8_t>(sbyte);
}

}  // namespace glmrt
