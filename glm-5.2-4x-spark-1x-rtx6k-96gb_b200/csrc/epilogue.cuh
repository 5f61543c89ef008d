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
//
// kFast selects the arithmetic: false = IEEE exp and divisions exactly as the oracle states them
// (the SIMT verification engine); true = the tensor-core engines' form, hardware exp2/reciprocal for
// the sigmoid (relative error about 1e-6) and code selection by comparing |a| with threshold*scale
// (exact products) instead of dividing by the scale.  The two agree except on values within
// rounding distance of a code boundary.
template <bool kFast>
__device__ __forceinline__ float swiglu_value(float g, float u) {
  if (kFast) {
    const float sig = __fdividef(1.0f, 1.0f + __expf(-g));
    return __fmul_rn(__fmul_rn(g, sig), u);
  }
  return __fmul_rn(__fmul_rn(g, sigmoid_f32(g)), u);
}
template <bool kFast>
__device__ __forceinline__ uint32_t fp4_code_of(float a, float scale) {
  if (scale == 0.0f) return 0u;
  if (kFast) {
    const float m = fabsf(a);
    const uint32_t mag = (m > 0.25f * scale) + (m > 0.75f * scale) + (m > 1.25f * scale) + (m > 1.75f * scale) +
                         (m > 2.5f * scale) + (m > 3.5f * scale) + (m > 5.0f * scale);
    return mag | ((a < 0.0f && mag != 0u) ? 8u : 0u);
  }
  return fp4_code_nearest_low(__fdiv_rn(a, scale));
}

template <bool kFast>
__device__ __forceinline__ void swiglu_requant_store(float g, float u, int feature, size_t slot, int inter,
                                                     uint8_t* __restrict__ act2_codes,
                                                     uint8_t* __restrict__ act2_sf) {
  const int lane = threadIdx.x & 31;
  const float a = swiglu_value<kFast>(g, u);
  float amax = fabsf(a);
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const uint32_t sbyte = f32_to_e4m3_satfinite(__fdiv_rn(amax, 6.0f));
  const float scale = e4m3_to_f32(sbyte);
  const uint32_t code = fp4_code_of<kFast>(a, scale);
  uint32_t v = code << (4 * (lane & 7));
  v |= __shfl_xor_sync(0xffffffffu, v, 1);
  v |= __shfl_xor_sync(0xffffffffu, v, 2);
  v |= __shfl_xor_sync(0xffffffffu, v, 4);
  if ((lane & 7) == 0)
    *reinterpret_cast<uint32_t*>(act2_codes + slot * static_cast<size_t>(inter / 2) + feature / 2) = v;
  if ((lane & 15) == 0) act2_sf[sf_tile_offset(slot, feature / 16, inter / 16)] = static_cast<uint8_t>(sbyte);
}

// One thread, one token slot, 16 consecutive features: raw gate/up accumulators -> packed codes
// (lo = features 0..7, hi = 8..15, low nibble first) and the block's E4M3 scale byte.
__device__ __forceinline__ void swiglu_requant_block16(const uint32_t (&g)[16], const uint32_t (&u)[16], float s2g,
                                                       float s2u, uint32_t& lo, uint32_t& hi, uint32_t& sbyte) {
  float v[16];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = swiglu_value<true>(__fmul_rn(__uint_as_float(g[i]), s2g), __fmul_rn(__uint_as_float(u[i]), s2u));
    amax = fmaxf(amax, fabsf(v[i]));
  }
  sbyte = f32_to_e4m3_satfinite(__fdiv_rn(amax, 6.0f));
  const float scale = e4m3_to_f32(sbyte);
  lo = 0;
  hi = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t c = fp4_code_of<true>(v[i], scale);
    if (i < 8) lo |= c << (4 * i); else hi |= c << (4 * (i - 8));
  }
}

}  // namespace glmrt
