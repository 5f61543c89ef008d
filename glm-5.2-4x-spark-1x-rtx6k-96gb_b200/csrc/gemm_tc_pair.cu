// Expert GEMMs of large prefill batches on CTA pairs (tcgen05 cta_group::2).
//
// FC2 instance: the pair's B tile is 256 down rows (128 per CTA), each CTA's accumulator is 128
// slots x 256 features and leaves as whole row pieces like the one-CTA FC2 kernel's (fc2_store.cuh).
//
// FC1: same computation as the FC1 instance of gemm_tc_prefill.cu (the reference's fused-MoE FC1 stage,
// native/cuda/kernels/b12x_direct.cu:479-508, and SIMT gate/up MLP, mlp.cu:218-273), for experts
// that received well over 128 tokens.  One work item is (expert, 256 token slots, 128 features):
// the two CTAs of a cluster each hold 128 of the token slots as their A rows and one half of the
// 256 B rows - the leader the 128 gate rows, its peer the 128 up rows of the same features - and a
// single M = 256 MMA per K block, issued by the leader, fills a 128 x 256 accumulator in each CTA's
// tensor memory.  Per unit of math a CTA brings 38 KB instead of 54 KB into shared memory, which
// buys a fifth pipeline stage.  Measured on the GLM-5.2 layer it is exactly as fast as the one-CTA
// kernel (T = 8192: 1.19 vs 1.14 ms, T = 16384: 1.88 vs 1.89 ms) and bit-identical: what each SM no
// longer loads from L2 it now reads from its peer's shared memory, and the 256-slot items are
// emptier on average; FC2 on pairs measures 0.93 vs 0.86 ms and 1.60 vs 1.62 ms.  The layer
// therefore uses these kernels only when asked (GLMRT_B200_LAYER_PAIR_FC1 / _FC2).
//
// Protocol (every wait bounded, as in gemm_tc.cu):
//   * both producers wait on their own `empty` barrier and load into their own shared memory; all
//     bytes of a stage, from both CTAs, are counted on the leader's `full` barrier (the TMA loads
//     carry cta_group::2 so that the barrier may live in the other CTA of the pair; the scale tiles
//     therefore also travel as 2-D TMA boxes of 16 rows x 128 bytes);
//   * the leader's issuing warp copies the scales (each CTA's own tile into its own tensor
//     memory), issues the MMAs and commits to the `empty` barrier of both CTAs, and after the last
//     stage to both `acc_full` barriers;
//   * the epilogue warps of both CTAs read their own accumulator and arrive on the leader's
//     `acc_empty` barrier.
// Every TMA load reads this GPU's own memory into the shared memory of the CTA that issued it.
#include <cuda.h>

#include "common.cuh"
#include "epilogue.cuh"
#include "fc2_store.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace glmrt {
namespace {

using namespace tc;

template <bool kFC1>
struct PairCfg {
  static constexpr int kABytes = 128 * kStageBytesK;      // this CTA's 128 token slots
  static constexpr int kBBytes = 128 * kStageBytesK;      // this CTA's half of the 256 weight rows
  static constexpr int kSfaBytes = kSfStageBytes;         // scales of this CTA's slots
  static constexpr int kSfbBytes = 2 * kSfStageBytes;     // scales of all 256 weight rows (both CTAs need them)
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // 38912
  static constexpr int kStages = kFC1 ? 5 : 4;            // FC2 leaves room for the staging rows of its epilogue
  static constexpr int kAccCols = 256;
  static constexpr int kSfSetCols = 16 + 32;
  static constexpr int kSfCol = kAccCols;
  static constexpr int kTmemCols = 512;
  static constexpr int kFeatPerTile = kFC1 ? 128 : 256;
  static constexpr int kEpiWarps = kFC1 ? 16 : 8;
  static constexpr int kThreads = 32 * (2 + kEpiWarps);
  static constexpr int kChunkCache = 256;
  static constexpr int kOutBytes = kFC1 ? 0 : kEpiWarps * Fc2Stage<128>::kBytesPerWarp;   // FC2: a 32 x 128 staging tile per warp
  static constexpr size_t kSmemBytes =
      static_cast<size_t>(kStages) * kStageBytes + 1024 + 256 + kChunkCache * sizeof(Chunk) + kOutBytes;
};

// act / act_sf: this GEMM's activation codes and scales; w0 / w0_sf: the weight rows the leader
// loads (FC1 gate, FC2 down) and their scales; w1 / w1_sf: the peer's (FC1 up, FC2 down again).
struct PairMaps {
  CUtensorMap act, w0, w1, act_sf, w0_sf, w1_sf;
};

template <bool kFC1>
__global__ void __launch_bounds__(PairCfg<kFC1>::kThreads, 1)
expert_pair_kernel(FfnArgs a, const __grid_constant__ PairMaps maps) {
  using C = PairCfg<kFC1>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(C::kStages) * C::kStageBytes);
  uint64_t* full_bar = bars;                     // used in the leader only
  uint64_t* empty_bar = bars + C::kStages;       // one set per CTA
  uint64_t* acc_full = bars + 2 * C::kStages;    // one per CTA
  uint64_t* acc_empty = acc_full + 1;            // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  Chunk* chunk_cache = reinterpret_cast<Chunk*>(reinterpret_cast<uint8_t*>(bars) + 256);
  uint8_t* out_stage = reinterpret_cast<uint8_t*>(chunk_cache + C::kChunkCache);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();       // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int k_bytes = (kFC1 ? a.hidden : a.inter) / 2;
  const int k_stages = k_bytes / kStageBytesK;
  const int k_tiles64 = k_bytes / 32;
  const int out_rows = kFC1 ? a.inter : a.hidden;
  const int feat_tiles = out_rows / C::kFeatPerTile;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 2 * C::kEpiWarps);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) tmem_alloc_pair(tmem_slot, C::kTmemCols);
  tc_fence_before();
  cluster_sync_all();          // barriers of both CTAs initialised, tensor memory of both allocated
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_chunks = static_cast<int>(a.counters[kCntChunks]);
  const int num_tiles = num_chunks * feat_tiles;
  for (int i = threadIdx.x; i < C::kChunkCache; i += C::kThreads) {
    const long long tile = static_cast<long long>(pair) + static_cast<long long>(i) * num_pairs;
    if (tile < num_tiles) chunk_cache[i] = a.chunks[tile / feat_tiles];
  }
  __syncthreads();
  auto chunk_of = [&](int it, int tile) -> Chunk {
    return it < C::kChunkCache ? chunk_cache[it] : a.chunks[tile / feat_tiles];
  };

  if (warp == 0) {
    // ================= TMA producer (both CTAs) =================
    const uint64_t pol = policy_evict_last();
    const CUtensorMap* map_w = rank == 0 ? &maps.w0 : &maps.w1;
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    int it = 0;
    for (int tile = pair; tile < num_tiles && alive; tile += num_pairs, ++it) {
      const Chunk ch = chunk_of(it, tile);
      const int ft = tile % feat_tiles;
      const int w_row = ch.expert * out_rows + ft * C::kFeatPerTile;
      // FC1: both CTAs take rows w_row.. of their own projection; FC2: the peer takes the second 128 rows
      const int my_w_row = w_row + (kFC1 ? 0 : 128 * static_cast<int>(rank));
      const int slot0 = ch.slot_base + 128 * static_cast<int>(rank);
      // rows of the scale maps are 128 bytes: one 512-byte scale tile = 4 rows
      const int sfa_row0 = (slot0 / 128) * k_tiles64 * 4;
      const int sfb_row0 = (w_row / 128) * k_tiles64 * 4;
      const int sfb_row1 = kFC1 ? sfb_row0 : (w_row / 128 + 1) * k_tiles64 * 4;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_warp(&empty_bar[stage], phase ^ 1u, abort_flag)) { alive = false; break; }
        if (elect_one()) {
          const uint32_t s_a = smem_u32(smem + static_cast<size_t>(stage) * C::kStageBytes);
          const uint32_t s_b = s_a + C::kABytes;
          const uint32_t s_sfa = s_b + C::kBBytes;
          const uint32_t s_sfb = s_sfa + C::kSfaBytes;
          const uint32_t full = cluster_addr(smem_u32(&full_bar[stage]), 0);
          const int kx = ks * kStageBytesK;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * C::kStageBytes);
          tma_load_2d_pair(s_a, &maps.act, full, kx, slot0, pol);
          tma_load_2d_pair(s_b, map_w, full, kx, my_w_row, pol);
          tma_load_2d_pair(s_sfa, &maps.act_sf, full, 0, sfa_row0 + ks * 16, pol);
          tma_load_2d_pair(s_sfb, &maps.w0_sf, full, 0, sfb_row0 + ks * 16, pol);
          tma_load_2d_pair(s_sfb + kSfStageBytes, &maps.w1_sf, full, 0, sfb_row1 + ks * 16, pol);
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer (leader only) =================
    if (rank == 0) {
      int stage = 0;
      uint32_t phase = 0, aphase = 0, sf_flip = 0;
      bool alive = true;
      const uint32_t idesc = idesc_nvf4_pair(256);
      const uint32_t peer_acc_full = cluster_addr(smem_u32(acc_full), 1);
      for (int tile = pair; tile < num_tiles && alive; tile += num_pairs) {
        if (!mbar_wait_warp(acc_empty, aphase ^ 1u, abort_flag)) { alive = false; break; }
        tc_fence_after();
        for (int ks = 0; ks < k_stages; ++ks) {
          if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag)) { alive = false; break; }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + C::kSfCol + sf_flip * C::kSfSetCols;
          const uint32_t t_sfb = t_sfa + 16;
          sf_flip ^= 1u;
          if (elect_one()) {
            const uint32_t s_a = smem_u32(smem + static_cast<size_t>(stage) * C::kStageBytes);
            const uint32_t s_b = s_a + C::kABytes;
            const uint32_t s_sfa = s_b + C::kBBytes;
            const uint32_t s_sfb = s_sfa + C::kSfaBytes;
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
              tc_copy_sf_pair(t_sfa + kb * 4, desc_sf(s_sfa + kb * 512));
              tc_copy_sf_pair(t_sfb + kb * 8, desc_sf(s_sfb + kb * 512));                       // B rows 0..127
              tc_copy_sf_pair(t_sfb + kb * 8 + 4, desc_sf(s_sfb + kSfStageBytes + kb * 512));   // B rows 128..255
            }
#pragma unroll
            for (int kb = 0; kb < 4; ++kb)
              tc_mma_nvf4_pair(tmem_base, desc_sw128(s_a + kb * 32), desc_sw128(s_b + kb * 32), idesc, t_sfa + kb * 4,
                               t_sfb + kb * 8, (ks | kb) != 0 ? 1u : 0u);
            tc_commit_pair(smem_u32(&empty_bar[stage]));
            tc_commit_pair(cluster_addr(smem_u32(&empty_bar[stage]), 1));
          }
          __syncwarp();
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        if (elect_one()) {
          tc_commit_pair(smem_u32(acc_full));
          tc_commit_pair(peer_acc_full);
        }
        __syncwarp();
        aphase ^= 1u;
      }
    }
  } else {
    // ================= epilogue (both CTAs): one thread per (token slot, share of the features) =================
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;                 // FC1 0..3: 32 of the tile's 128 features; FC2 0..1: 128 of its 256
    const int row = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t lead_acc_empty = cluster_addr(smem_u32(acc_empty), 0);
    uint32_t aphase = 0;
    bool alive = true;
    int it = 0;
    for (int tile = pair; tile < num_tiles && alive; tile += num_pairs, ++it) {
      const Chunk ch = chunk_of(it, tile);
      const int ft = tile % feat_tiles;
      const int here = min(128, max(0, ch.tokens - 128 * static_cast<int>(rank)));
      const bool valid = row < here;
      const size_t slot = static_cast<size_t>(ch.slot_base) + 128 * rank + row;
      const float s2g = a.scale2[ch.expert * 3 + (kFC1 ? 0 : 2)];
      const float s2u = kFC1 ? a.scale2[ch.expert * 3 + 1] : 0.0f;
      uint16_t* dst = (!kFC1 && valid) ? a.slot_out[slot] : nullptr;
      if (!mbar_wait_warp(acc_full, aphase, abort_flag)) { alive = false; break; }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base;
      if (kFC1) {
        // Both 16-feature blocks of this warp are read out first and the accumulator is handed back
        // before any arithmetic, so the next item's MMAs run under this item's SwiGLU and stores.
        uint32_t g[2][16], u[2][16];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tc_load16(t_acc + (part * 2 + j) * 16, g[j]);
          tc_load16(t_acc + 128 + (part * 2 + j) * 16, u[j]);
        }
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_acc_empty);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int b = part * 2 + j;                   // 16-feature block of the tile
          uint32_t lo, hi, sbyte;
          swiglu_requant_block16(g[j], u[j], s2g, s2u, lo, hi, sbyte);
          if (valid) {
            const int feature = ft * C::kFeatPerTile + b * 16;
            *reinterpret_cast<uint2*>(a.act2_codes + slot * static_cast<size_t>(a.inter / 2) + feature / 2) =
                make_uint2(lo, hi);
            a.act2_sf[sf_tile_offset(slot, feature / 16, a.inter / 16)] = static_cast<uint8_t>(sbyte);
          }
        }
      } else {
        // this warp's 128 of the CTA's 256 columns leave as whole rows through its staging tile
        fc2_emit_128_columns<128>(t_acc + part * 128, s2g, valid ? dst + ft * C::kFeatPerTile + part * 128 : nullptr,
                             out_stage + static_cast<size_t>(warp - 2) * Fc2Stage<128>::kBytesPerWarp, lane,
                             [&] { mbar_arrive_cluster(lead_acc_empty); });
      }
      aphase ^= 1u;
    }
  }

  // ---- teardown ----
  if (*abort_flag != 0u) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);   // let copies in flight land
    if (threadIdx.x == 0) atomicOr(a.error_word, static_cast<uint32_t>(kErrWaitTimeout));
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // neither CTA frees tensor memory the other may still be written through
  if (warp == 1) tmem_dealloc_pair(tmem_base, C::kTmemCols);
}

}  // namespace

bool pair_tiles_supported(const FfnArgs& a, int sm_count) {
  return a.chunk_tokens == 256 && a.inter % 256 == 0 && a.hidden % 256 == 0 && sm_count % 2 == 0;
}

namespace {
template <bool kFC1>
glmrt_status_t launch_pair(const FfnArgs& a, const PairMaps& maps, int sm_count, cudaStream_t stream) {
  using C = PairCfg<kFC1>;
  static std::atomic<uint64_t> configured{0};
  GLMRT_RETURN_IF_ERROR(ensure_smem_limit(configured, expert_pair_kernel<kFC1>, C::kSmemBytes,
                                          "cudaFuncSetAttribute(expert_pair_kernel)"));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(sm_count & ~1));
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  cudaError_t err = cudaLaunchKernelEx(&cfg, expert_pair_kernel<kFC1>, a, maps);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "launch expert_pair_kernel", err);
  count_launch();
  return GLMRT_STATUS_OK;
}
}  // namespace

glmrt_status_t launch_fc1_tc_pair(const FfnArgs& a, const TensorMaps& m, int sm_count, cudaStream_t stream) {
  PairMaps maps;
  maps.act = m.act1; maps.w0 = m.gate; maps.w1 = m.up;
  maps.act_sf = m.act1_sf; maps.w0_sf = m.gate_sf; maps.w1_sf = m.up_sf;
  return launch_pair<true>(a, maps, sm_count, stream);
}

glmrt_status_t launch_fc2_tc_pair(const FfnArgs& a, const TensorMaps& m, int sm_count, cudaStream_t stream) {
  PairMaps maps;
  maps.act = m.act2; maps.w0 = m.down; maps.w1 = m.down;
  maps.act_sf = m.act2_sf; maps.w0_sf = m.down_sf; maps.w1_sf = m.down_sf;
  return launch_pair<false>(a, maps, sm_count, stream);
}

}  // namespace glmrt
