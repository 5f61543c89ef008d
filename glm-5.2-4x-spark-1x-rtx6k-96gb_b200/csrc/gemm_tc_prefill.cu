// Tensor-core engine for prefill-sized batches: grouped NVFP4 x NVFP4 expert GEMMs on tcgen05 with
// "tokens as A".
//
// Same role as gemm_tc.cu (the reference's fused-MoE kernels, native/cuda/kernels/
// b12x_direct.cu:479-647, and SIMT route MLP, mlp.cu:218-314), for token chunks of up to 128 rows:
// the 128 rows of the UMMA tile are the token slots of one expert, the 128 columns are weight rows.
//
//   FC1  B = 64 gate rows stacked on the 64 up rows of the same features (two TMA boxes into one
//        shared-memory tile, scales pre-tiled in the same stacking), so one thread of the epilogue
//        owns one token and finds gate and up of 16 consecutive features in its own registers:
//        SwiGLU, block amax, E4M3 scale, FP4 codes and packing need no cross-lane traffic, and the
//        result leaves as one 8-byte store per block plus one 4-byte store of scales per tile.
//   FC2  B = 128 down rows; the epilogue thread scales, rounds to bf16 and writes 256 contiguous
//        bytes of its token's result row.
//
// Accumulators (128 columns) are double-buffered in tensor memory, so the epilogue of one tile runs
// under the MMAs of the next.  Producer, issuer and epilogue roles, bounded waits and the work-item
// cache are as in gemm_tc.cu.  TMA loads read local memory only and use no cluster multicast.
#include <cuda.h>

#include "common.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace glmrt {
namespace {

using namespace tc;

constexpr int kPfStages = 6;
constexpr int kPfABytes = 128 * kStageBytesK;   // 128 token rows
constexpr int kPfBBytes = 128 * kStageBytesK;   // 128 weight rows
constexpr int kPfStageBytes = kPfABytes + kPfBBytes + 2 * kSfStageBytes;   // 36 KiB
constexpr int kPfChunkCache = 256;
constexpr size_t kPfSmemBytes = static_cast<size_t>(kPfStages) * kPfStageBytes + 1024 + 256 + kPfChunkCache * sizeof(Chunk);
constexpr int kPfAccCols = 128;
constexpr int kPfSfCol = 2 * kPfAccCols;        // scales after the two accumulator buffers
constexpr int kPfTmemCols = 512;

__device__ __forceinline__ void tc_load16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

template <bool kFC1>
__global__ void __launch_bounds__(kThreadsTC, 1)
expert_gemm_tokens_kernel(FfnArgs a, const __grid_constant__ CUtensorMap map_act,
                          const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kPfStages) * kPfStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kPfStages;
  uint64_t* acc_full = bars + 2 * kPfStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  Chunk* chunk_cache = reinterpret_cast<Chunk*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int k_bytes = (kFC1 ? a.hidden : a.inter) / 2;
  const int k_stages = k_bytes / kStageBytesK;
  const int k_tiles64 = k_bytes / 32;
  const int feat_per_tile = kFC1 ? 64 : 128;
  const int out_rows = kFC1 ? a.inter : a.hidden;
  const int feat_tiles = out_rows / feat_per_tile;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPfStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) tmem_alloc(tmem_slot, kPfTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_chunks = static_cast<int>(a.counters[kCntChunks]);
  const int num_tiles = num_chunks * feat_tiles;
  for (int i = threadIdx.x; i < kPfChunkCache; i += kThreadsTC) {
    const long long tile = static_cast<long long>(blockIdx.x) + static_cast<long long>(i) * gridDim.x;
    if (tile < num_tiles) chunk_cache[i] = a.chunks[tile / feat_tiles];
  }
  __syncthreads();
  auto chunk_of = [&](int it, int tile) -> Chunk {
    return it < kPfChunkCache ? chunk_cache[it] : a.chunks[tile / feat_tiles];
  };

  if (warp == 0) {
    // ================= TMA producer =================
    const uint64_t pol_w = policy_evict_last();   // a weight tile is used by every chunk of its expert
    const uint64_t pol_x = policy_evict_last();   // a chunk's rows are used by every feature tile
    const uint8_t* sfa = kFC1 ? a.act1_sf : a.act2_sf;
    const uint8_t* sfb = kFC1 ? a.gu_sf64 : a.down_sf;
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x, ++it) {
      const Chunk ch = chunk_of(it, tile);
      const int ft = tile % feat_tiles;
      const int w_row = ch.expert * out_rows + ft * feat_per_tile;
      const size_t sfa_tile0 = static_cast<size_t>(ch.slot_base / 128) * k_tiles64;
      const size_t sfb_tile0 =
          (kFC1 ? static_cast<size_t>(ch.expert) * feat_tiles + ft : static_cast<size_t>(w_row / 128)) * k_tiles64;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_warp(&empty_bar[stage], phase ^ 1u, abort_flag)) { alive = false; break; }
        if (elect_one()) {
          const uint32_t s_a = smem_u32(smem + static_cast<size_t>(stage) * kPfStageBytes);
          const uint32_t s_b = s_a + kPfABytes;
          const uint32_t s_sfa = s_b + kPfBBytes;
          const uint32_t s_sfb = s_sfa + kSfStageBytes;
          mbar_expect_tx(&full_bar[stage], kPfStageBytes);
          tma_load_2d(s_a, &map_act, &full_bar[stage], ks * kStageBytesK, ch.slot_base, pol_x);
          if (kFC1) {
            tma_load_2d(s_b, &map_w0, &full_bar[stage], ks * kStageBytesK, w_row, pol_w);                // 64 gate rows
            tma_load_2d(s_b + 64 * kStageBytesK, &map_w1, &full_bar[stage], ks * kStageBytesK, w_row, pol_w);  // 64 up rows
          } else {
            tma_load_2d(s_b, &map_w0, &full_bar[stage], ks * kStageBytesK, w_row, pol_w);                // 128 down rows
          }
          bulk_load(s_sfa, sfa + (sfa_tile0 + static_cast<size_t>(ks) * 4) * 512, kSfStageBytes, &full_bar[stage], pol_x);
          bulk_load(s_sfb, sfb + (sfb_tile0 + static_cast<size_t>(ks) * 4) * 512, kSfStageBytes, &full_bar[stage], pol_w);
        }
        __syncwarp();
        if (++stage == kPfStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    int stage = 0;
    uint32_t phase = 0;
    int abuf = 0;
    uint32_t aphase = 0;
    bool alive = true;
    const uint32_t t_sfa = tmem_base + kPfSfCol;
    const uint32_t t_sfb = t_sfa + 16;
    const uint32_t idesc = idesc_nvf4(128);
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      if (!mbar_wait_warp(&acc_empty[abuf], aphase ^ 1u, abort_flag)) { alive = false; break; }
      tc_fence_after();
      const uint32_t d0 = tmem_base + abuf * kPfAccCols;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag)) { alive = false; break; }
        tc_fence_after();
        if (elect_one()) {
          const uint32_t s_a = smem_u32(smem + static_cast<size_t>(stage) * kPfStageBytes);
          const uint32_t s_b = s_a + kPfABytes;
          const uint32_t s_sfa = s_b + kPfBBytes;
          const uint32_t s_sfb = s_sfa + kSfStageBytes;
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            tc_copy_sf(t_sfa + kb * 4, desc_sf(s_sfa + kb * 512));
            tc_copy_sf(t_sfb + kb * 4, desc_sf(s_sfb + kb * 512));
          }
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            tc_mma_nvf4(d0, desc_sw128(s_a + kb * 32), desc_sw128(s_b + kb * 32), idesc, t_sfa + kb * 4,
                        t_sfb + kb * 4, (ks | kb) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == kPfStages) { stage = 0; phase ^= 1u; }
      }
      if (!alive) break;
      if (elect_one()) tc_commit(&acc_full[abuf]);
      __syncwarp();
      abuf ^= 1;
      if (abuf == 0) aphase ^= 1u;
    }
  } else {
    // ================= epilogue (warps 2..5): one thread per token slot =================
    const int quad = warp & 3;
    const int row = quad * 32 + lane;                 // token slot inside the chunk = tensor-memory lane
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    int abuf = 0;
    uint32_t aphase = 0;
    bool alive = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x, ++it) {
      const Chunk ch = chunk_of(it, tile);
      const int ft = tile % feat_tiles;
      const bool valid = row < ch.tokens;
      const size_t slot = static_cast<size_t>(ch.slot_base) + row;
      const float s2a = a.scale2[ch.expert * 3 + (kFC1 ? 0 : 2)];
      const float s2b = kFC1 ? a.scale2[ch.expert * 3 + 1] : 0.0f;
      uint16_t* dst = (!kFC1 && valid) ? a.slot_out[slot] : nullptr;
      if (!mbar_wait_warp(&acc_full[abuf], aphase, abort_flag)) { alive = false; break; }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base + abuf * kPfAccCols;
      if (kFC1) {
        uint32_t sbytes = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {              // four 16-feature blocks of this 64-feature tile
          uint32_t g[16], u[16];
          tc_load16(t_acc + b * 16, g);
          tc_load16(t_acc + 64 + b * 16, u);
          tc_wait_ld();
          float v[16];
          float amax = 0.0f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float gg = __fmul_rn(__uint_as_float(g[i]), s2a);
            const float uu = __fmul_rn(__uint_as_float(u[i]), s2b);
            v[i] = __fmul_rn(__fmul_rn(gg, sigmoid_f32(gg)), uu);   // moe_ref.py:18-20
            amax = fmaxf(amax, fabsf(v[i]));
          }
          const uint32_t sbyte = f32_to_e4m3_satfinite(__fdiv_rn(amax, 6.0f));
          const float scale = e4m3_to_f32(sbyte);
          uint32_t lo = 0, hi = 0;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint32_t c = scale == 0.0f ? 0u : fp4_code_nearest_low(__fdiv_rn(v[i], scale));
            if (i < 8) lo |= c << (4 * i); else hi |= c << (4 * (i - 8));
          }
          sbytes |= sbyte << (8 * b);
          if (valid)
            *reinterpret_cast<uint2*>(a.act2_codes + slot * static_cast<size_t>(a.inter / 2) + (ft * 64 + b * 16) / 2) =
                make_uint2(lo, hi);
        }
        // the four scale bytes of this tile are consecutive in the tiled layout (blocks ft*4 .. ft*4+3)
        if (valid) *reinterpret_cast<uint32_t*>(a.act2_sf + sf_tile_offset(slot, ft * 4, a.inter / 16)) = sbytes;
      } else {
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 16) {
          uint32_t y[16];
          tc_load16(t_acc + c0, y);
          tc_wait_ld();
          if (valid) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              w[i] = static_cast<uint32_t>(f32_to_bf16_rne(__fmul_rn(__uint_as_float(y[2 * i]), s2a))) |
                     (static_cast<uint32_t>(f32_to_bf16_rne(__fmul_rn(__uint_as_float(y[2 * i + 1]), s2a))) << 16);
            uint4* d4 = reinterpret_cast<uint4*>(dst + ft * 128 + c0);
            d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
            d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[abuf]);
      abuf ^= 1;
      if (abuf == 0) aphase ^= 1u;
    }
  }

  // ---- teardown ----
  __syncwarp();
  if (*abort_flag != 0u) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);   // let copies in flight land
    if (threadIdx.x == 0) atomicOr(a.error_word, static_cast<uint32_t>(kErrWaitTimeout));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kPfTmemCols);
}

template <bool kFC1>
glmrt_status_t launch_tokens(const FfnArgs& a, const CUtensorMap& act, const CUtensorMap& w0, const CUtensorMap& w1,
                             int sm_count, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(expert_gemm_tokens_kernel<kFC1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(kPfSmemBytes));
    if (err != cudaSuccess)
      return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaFuncSetAttribute(expert_gemm_tokens_kernel)", err);
    configured = true;
  }
  expert_gemm_tokens_kernel<kFC1><<<sm_count, kThreadsTC, kPfSmemBytes, stream>>>(a, act, w0, w1);
  GLMRT_LAUNCH_CHECK("expert_gemm_tokens_kernel");
  return GLMRT_STATUS_OK;
}

}  // namespace

glmrt_status_t launch_fc1_tc_prefill(const FfnArgs& a, const TensorMaps& m, int sm_count, cudaStream_t stream) {
  return launch_tokens<true>(a, m.act1, m.gate64, m.up64, sm_count, stream);
}
glmrt_status_t launch_fc2_tc_prefill(const FfnArgs& a, const TensorMaps& m, int sm_count, cudaStream_t stream) {
  return launch_tokens<false>(a, m.act2, m.down, m.down, sm_count, stream);
}

}  // namespace glmrt
