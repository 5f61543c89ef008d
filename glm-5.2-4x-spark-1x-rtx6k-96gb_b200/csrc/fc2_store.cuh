// FC2 epilogue of the token-major tensor-core kernels: accumulator columns -> bf16 result rows.
//
// A thread of the epilogue owns one token row (its tensor-memory lane), but a row's 256 bytes
// should leave as whole lines: 32 lanes each storing a piece of a different row would touch 32
// lines per instruction, and one asynchronous bulk copy per lane serialises in the copy engine
// (measured: about 2000 cycles per warp for 32 copies of 128 bytes, which made the down projection
// epilogue-bound).  So the warp parks its 32 x 128 tile in shared memory (row pitch = row bytes +
// 16: the 16-byte accesses of a quarter warp fall on distinct banks both ways) and writes it out
// several rows per instruction, each row's bytes contiguous over neighbouring lanes, to local
// memory or a peer's alike.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace glmrt {
namespace tc {

// kPass = columns parked per pass: 128 (one pass, 272-byte pitch, two rows per store instruction)
// or 64 (two passes through half the staging space, 144-byte pitch, four rows per instruction).
template <int kPass>
struct Fc2Stage {
  static_assert(kPass == 64 || kPass == 128, "columns per pass");
  static constexpr int kPitch = kPass * 2 + 16;
  static constexpr int kBytesPerWarp = 32 * kPitch;
  static constexpr int kLanesPerRow = kPass * 2 / 16;
  static constexpr int kRowsPerStore = 32 / kLanesPerRow;
};

// Sixteen bytes of bf16 pairs added to global memory, each 16-bit lane rounded to nearest even
// (one instruction instead of a load, eight additions and a store; performed by the L2).
__device__ __forceinline__ void red_add_bf16x8(void* dst, const uint4& v) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// t_acc: tensor-memory address (lane quadrant and first column) of the warp's 128 columns;
// dst: this lane's destination (row pointer plus the tile's first feature) or nullptr for a slot
// without a token; stage: the warp's Fc2Stage<kPass>::kBytesPerWarp bytes; release(): called by
// lane 0 once all 128 columns are in registers, hands the accumulator back to the MMA issuer.
// kFused: the destination is the token's row of the layer output and `weight2` holds the route
// weight as a bf16 pair: bf16(weight * bf16(y)) is ADDED to the destination (the weighted
// scatter-add combine of moe_ref.py:35-36 inside the down projection; the products are rounded as
// the oracle rounds them, the sums in the order the routes happen to finish).
template <int kPass, bool kFused = false, typename Release>
__device__ __forceinline__ void fc2_emit_128_columns(uint32_t t_acc, float s2, uint16_t* dst, uint8_t* stage, int lane,
                                                     Release&& release, uint32_t weight2 = 0u) {
  using S = Fc2Stage<kPass>;
  uint8_t* mine = stage + lane * S::kPitch;
  const int sub = lane / S::kLanesPerRow, piece = lane % S::kLanesPerRow;
  const unsigned long long my_dst = reinterpret_cast<unsigned long long>(dst);
  uint32_t w[2][4][8];   // the row's 128 columns as bf16 pairs
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t y[4][16];
#pragma unroll
    for (int q = 0; q < 4; ++q) tc_load16(t_acc + half * 64 + q * 16, y[q]);
    tc_wait_ld();
    if (half == 1) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) release();
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(__fmul_rn(__uint_as_float(y[q][2 * i]), s2),
                                                       __fmul_rn(__uint_as_float(y[q][2 * i + 1]), s2));
        w[half][q][i] = *reinterpret_cast<const uint32_t*>(&p);
        if (kFused) asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(w[half][q][i]) : "r"(weight2), "r"(w[half][q][i]));
      }
    }
  }
#pragma unroll
  for (int pass = 0; pass < 128 / kPass; ++pass) {
    __syncwarp();   // the rows parked before have been read out
#pragma unroll
    for (int h = 0; h < kPass / 64; ++h) {
      const int half = kPass == 128 ? h : pass;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4* s4 = reinterpret_cast<uint4*>(mine + h * 128 + q * 32);
        s4[0] = make_uint4(w[half][q][0], w[half][q][1], w[half][q][2], w[half][q][3]);
        s4[1] = make_uint4(w[half][q][4], w[half][q][5], w[half][q][6], w[half][q][7]);
      }
    }
    __syncwarp();
#pragma unroll 4
    for (int r = 0; r < 32 / S::kRowsPerStore; ++r) {
      const int row = S::kRowsPerStore * r + sub;
      const unsigned long long p = __shfl_sync(0xffffffffu, my_dst, row);
      const uint4 v = *reinterpret_cast<const uint4*>(stage + row * S::kPitch + piece * 16);
      if (p != 0ull) {
        uint8_t* where = reinterpret_cast<uint8_t*>(p) + pass * kPass * 2 + piece * 16;
        if (kFused) red_add_bf16x8(where, v); else *reinterpret_cast<uint4*>(where) = v;
      }
    }
  }
}

}  // namespace tc
}  // namespace glmrt
