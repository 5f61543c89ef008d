// Quantiser of one 16-element block of activations, shared by the stand-alone payload quantiser,
// the fused quantise + dispatch kernel and the expert-parallel push kernel.
#pragma once

#include "common.cuh"

namespace glmrt {

// One 16-element block: E4M3 scale of amax/6, then E2M1 codes, low nibble first.
//
// kNearestLow is the rule of the Python reference (quant_ref.py:41-46): the code nearest to the
// IEEE quotient x / scale, ties towards the smaller magnitude.  The quotient is never formed:
// for a bf16 x (8 significant bits), an E4M3 scale (4 bits) and a code midpoint m (0.25 .. 5),
// x / scale is either exactly m or differs from it by more than 2^-9 relative, far more than the
// rounding of the division, so fl(x / scale) > m holds exactly when |x| > m * scale, and m * scale
// is exact in float32.  Seven comparisons against exact products replace sixteen divisions.
template <bool kNearestLow>
__device__ __forceinline__ void quantize_block16(const float (&v)[16], uint32_t& lo, uint32_t& hi, uint32_t& sbyte) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  sbyte = f32_to_e4m3_satfinite(__fdiv_rn(amax, 6.0f));
  const float scale = e4m3_to_f32(sbyte);
  lo = 0; hi = 0;
  if (kNearestLow) {
    if (scale != 0.0f) {
      const float t0 = 0.25f * scale, t1 = 0.75f * scale, t2 = 1.25f * scale, t3 = 1.75f * scale, t4 = 2.5f * scale,
                  t5 = 3.5f * scale, t6 = 5.0f * scale;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float m = fabsf(v[i]);
        const uint32_t mag = (m > t0) + (m > t1) + (m > t2) + (m > t3) + (m > t4) + (m > t5) + (m > t6);
        const uint32_t c = mag | ((v[i] < 0.0f && mag != 0u) ? 8u : 0u);
        if (i < 8) lo |= c << (4 * i); else hi |= c << (4 * (i - 8));
      }
    }
  } else {
    const float inv = scale == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float q = fminf(fmaxf(__fmul_rn(v[i], inv), -6.0f), 6.0f);
      const uint32_t c = fp4_code_rne_payload(q);
      if (i < 8) lo |= c << (4 * i); else hi |= c << (4 * (i - 8));
    }
  }
}

// bf16 row [hidden] -> payload image [hidden/2 codes | hidden/16 scale bytes] in shared memory, by
// all `threads` threads of the CTA (nearest-low rule).  The caller synchronises afterwards.
// kLatency: two blocks per thread and pass with their four loads in flight together; one memory
// round trip less for a row of 6144 on 256 threads, which is what a decode-sized batch (a CTA or
// two per SM) waits for.  It costs 24 registers, so prefill-sized batches, bound by how many rows an SM
// holds at once, use the plain form.
template <bool kLatency>
__device__ __forceinline__ void quantize_row_to_image(const uint16_t* __restrict__ src_row, uint8_t* img, int hidden,
                                                      int threads) {
  const int code_bytes = hidden / 2, kblocks = hidden / 16;
  auto one_block = [&](const uint4& x0, const uint4& x1, int blk) {
    const uint32_t w[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
    uint32_t lo, hi, sbyte;
    quantize_block16<true>(v, lo, hi, sbyte);
    reinterpret_cast<uint2*>(img)[blk] = make_uint2(lo, hi);
    img[code_bytes + blk] = static_cast<uint8_t>(sbyte);
  };
  if (kLatency) {
    for (int blk0 = threadIdx.x; blk0 < kblocks; blk0 += 2 * threads) {
      const int blk1 = blk0 + threads;
      const bool two = blk1 < kblocks;
      const uint4 a0 = reinterpret_cast<const uint4*>(src_row + blk0 * 16)[0];
      const uint4 a1 = reinterpret_cast<const uint4*>(src_row + blk0 * 16)[1];
      const uint4 b0 = two ? reinterpret_cast<const uint4*>(src_row + blk1 * 16)[0] : make_uint4(0u, 0u, 0u, 0u);
      const uint4 b1 = two ? reinterpret_cast<const uint4*>(src_row + blk1 * 16)[1] : make_uint4(0u, 0u, 0u, 0u);
      one_block(a0, a1, blk0);
      if (two) one_block(b0, b1, blk1);
    }
  } else {
    for (int blk = threadIdx.x; blk < kblocks; blk += threads)
      one_block(reinterpret_cast<const uint4*>(src_row + blk * 16)[0], reinterpret_cast<const uint4*>(src_row + blk * 16)[1], blk);
  }
}

}  // namespace glmrt
