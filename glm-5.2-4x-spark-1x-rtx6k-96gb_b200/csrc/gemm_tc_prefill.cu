// Tensor-core engine for prefill-sized batches: grouped NVFP4 x NVFP4 expert GEMMs on tcgen05 with
// "tokens as A".
//
// Same role as gemm_tc.cu (the reference's fused-MoE kernels, native/cuda/kernels/
// b12x_direct.cu:479-647, and SIMT route MLP, mlp.cu:218-314), for token chunks of up to 128 rows:
// the 128 rows of the UMMA tile are the token slots of one expert, the 128 columns are weight rows.
//
//   FC1  B = 128 gate rows followed by the 128 up rows of the same features (two TMA boxes into one
//        256-row shared-memory tile, one scale tile each), so one thread of the epilogue owns one
//        token and finds gate and up of 16 consecutive features in its own registers: SwiGLU, block
//        amax, E4M3 scale, FP4 codes and packing need no cross-lane traffic, and the result leaves
//        as one 8-byte store of codes and one scale byte per block.
//   FC2  B = 128 down rows, accumulators double-buffered in tensor memory: its K loop is only eight
//        stages long, so an epilogue that held the single buffer of a 256-column tile drained the
//        pipeline at every tile (measured at T = 8192: 1.08 ms with N = 256, 0.86 ms with N = 128).
//        The epilogue warp scales, rounds to bf16, parks its 32 rows x 128 columns in shared memory
//        and writes them out as whole 256-byte row pieces (fc2_store.cuh).
//
// FC1 uses N = 256: half the scale copies and fewer bytes brought into shared memory per unit of
// math than N = 128 (measured: FC1 1.63 -> 1.33 ms at T = 8192); its 48-stage K loop hides the one
// non-overlapped epilogue per tile, which sixteen epilogue warps keep short.  Producer, issuer and
// epilogue roles, bounded waits and the work-item cache are as in gemm_tc.cu.  Every TMA load reads
// this GPU's own memory into one CTA.
#include <cuda.h>

#include "common.cuh"
#include "ep_flags.cuh"
#include "epilogue.cuh"
#include "fc2_store.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace glmrt {

// Optional timeline of one CTA (build.py --trace defines GLMRT_B200_TRACE and builds a separate
// library): clock64 stamps of the producer (slot free seen, loads issued), the issuer (stage full
// seen, MMAs issued; accumulator wait begin / end per tile) and the first epilogue warp
// (accumulator full wait begin / end, accumulator released, tile done).  [kernel: 0 FC1, 1 FC2].
#ifdef GLMRT_B200_TRACE
constexpr int kTraceCta = 5, kTraceStages = 2048, kTraceTiles = 256;
__device__ long long g_prefill_stage_trace[2][4][kTraceStages];
__device__ long long g_prefill_tile_trace[2][6][kTraceTiles];
#define GLMRT_TRACE_STAGE(kind, ev, n)                                                        \
  do {                                                                                        \
    if (blockIdx.x == kTraceCta && (n) < kTraceStages) g_prefill_stage_trace[kind][ev][n] = clock64(); \
  } while (0)
#define GLMRT_TRACE_TILE(kind, ev, n)                                                         \
  do {                                                                                        \
    if (blockIdx.x == kTraceCta && (n) < kTraceTiles) g_prefill_tile_trace[kind][ev][n] = clock64(); \
  } while (0)
#else
#define GLMRT_TRACE_STAGE(kind, ev, n) ((void)0)
#define GLMRT_TRACE_TILE(kind, ev, n) ((void)0)
#endif

namespace {

using namespace tc;

// Tile geometry.  kWN = weight rows (UMMA N) per tile: 128 with the accumulators double-buffered
// (FC2), or 256 = 128 gate + 128 up with a single accumulator buffer (FC1).
template <bool kFC1, int kWN>
struct PfCfg {
  static constexpr int kBTiles = kWN / 128;                          // 128-row boxes / scale tiles of B
  static constexpr int kABytes = 128 * kStageBytesK;                 // 128 token rows
  static constexpr int kBBytes = kWN * kStageBytesK;
  static constexpr int kStageBytes = kABytes + kBBytes + (1 + kBTiles) * kSfStageBytes;
  // FC2 gives one pipeline stage up for the staging rows of its epilogue
  // FC2 parks its result rows in shared memory before they leave: a whole 128-column pass per warp
  // with N = 128 (one pipeline stage given up for it), two 64-column passes with N = 256.
  static constexpr int kPass = kWN == 128 ? 128 : 64;
  static constexpr int kStages = kFC1 ? 221184 / kStageBytes : (kWN == 128 ? 221184 / kStageBytes - 1 : 3);   // 4 (FC1) / 5 (FC2, N=128) / 3 (FC2, N=256)
  static constexpr int kAccBufs = kWN == 128 ? 2 : 1;
  static constexpr int kSfSetCols = 16 + 16 * kBTiles;               // scale columns of one stage
  static constexpr int kSfCol = kAccBufs * kWN;                      // two alternating sets follow the accumulators
  static constexpr int kTmemCols = 512;
  static constexpr int kFeatPerTile = kFC1 ? kWN / 2 : kWN;
  // The FC1 epilogue is arithmetic-heavy (SwiGLU, quantisation): with one warp per scheduler it
  // could not hide its own latencies and bounded the kernel, so it gets sixteen warps, four per
  // tensor-memory quadrant.  FC2's scale-and-round needs one warp per 128 columns and quadrant.
  static constexpr int kEpiWarps = kFC1 ? 16 : 4 * kBTiles;
  static constexpr int kParts = kEpiWarps / 4;
  static constexpr int kThreads = 32 * (2 + kEpiWarps);
  static constexpr int kChunkCache = 256;
  // FC2 epilogue: every warp parks its 32 rows x 128 columns before they leave as whole rows
  static constexpr int kOutBytes = kFC1 ? 0 : kEpiWarps * Fc2Stage<kPass>::kBytesPerWarp;
  static constexpr size_t kSmemBytes =
      static_cast<size_t>(kStages) * kStageBytes + 1024 + 256 + kChunkCache * sizeof(Chunk) + kOutBytes;
};

// kFusedCombine (FC2 only): results are not stored as one row per route but added, weighted, into
// the token's row of the layer output (a.slot_out holds those rows, a.slot_weight the weights).
template <bool kFC1, int kWN, bool kFusedCombine = false>
__global__ void __launch_bounds__(PfCfg<kFC1, kWN>::kThreads, 1)
expert_gemm_tokens_kernel(FfnArgs a, const __grid_constant__ CUtensorMap map_act,
                          const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1) {
  using C = PfCfg<kFC1, kWN>;
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(C::kStages) * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* acc_full = bars + 2 * C::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  Chunk* chunk_cache = reinterpret_cast<Chunk*>(reinterpret_cast<uint8_t*>(bars) + 256);
  uint8_t* out_stage = reinterpret_cast<uint8_t*>(chunk_cache + C::kChunkCache);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int k_bytes = (kFC1 ? a.hidden : a.inter) / 2;
  const int k_stages = k_bytes / kStageBytesK;
  const int k_tiles64 = k_bytes / 32;
  const int out_rows = kFC1 ? a.inter : a.hidden;
  const int feat_tiles = out_rows / C::kFeatPerTile;

  if (threadIdx.x == 32) {   // the maps are kernel parameters: fetched while the previous kernel still runs
    prefetch_tensormap(&map_act);
    prefetch_tensormap(&map_w0);
    if (kFC1) prefetch_tensormap(&map_w1);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], C::kEpiWarps);
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();   // set-up above overlapped the previous kernel's tail; its results are read from here on
  // A plan made of 256-slot chunks (for the CTA-pair FC1 kernel) is taken as two halves of 128
  // slots; a half without tokens is skipped by every role alike.
  const int halves = a.chunk_tokens > 128 ? a.chunk_tokens / 128 : 1;
  // a step that has already reported an error runs no expert work (and tells no peer it did)
  const bool step_failed = *reinterpret_cast<const volatile uint32_t*>(a.error_word) != 0u;
  const int num_chunks = step_failed ? 0 : static_cast<int>(a.counters[kCntChunks]);
  const int num_tiles = num_chunks * halves * feat_tiles;
  auto load_chunk = [&](int tile) -> Chunk {
    Chunk c = a.chunks[tile / (feat_tiles * halves)];
    const int half = (tile / feat_tiles) % halves;
    c.slot_base += 128 * half;
    c.tokens = min(128, max(0, c.tokens - 128 * half));
    return c;
  };
  for (int i = threadIdx.x; i < C::kChunkCache; i += C::kThreads) {
    const long long tile = static_cast<long long>(blockIdx.x) + static_cast<long long>(i) * gridDim.x;
    if (tile < num_tiles) chunk_cache[i] = load_chunk(static_cast<int>(tile));
  }
  __syncthreads();
  auto chunk_of = [&](int it, int tile) -> Chunk { return it < C::kChunkCache ? chunk_cache[it] : load_chunk(tile); };

  if (warp == 0) {
    // ================= TMA producer =================
    const uint64_t pol = policy_evict_last();   // weight tiles serve every chunk of their expert, rows every feature tile
    const uint8_t* sfa = kFC1 ? a.act1_sf : a.act2_sf;
    [[maybe_unused]] int traced = 0;
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    int it = 0;
    if (kFC1 && a.wait.flags != nullptr && (blockIdx.x == 0 || static_cast<int>(blockIdx.x) < num_tiles)) {
      // expert-parallel path: the rows this kernel reads are pushed by the peers (CTA 0 waits even
      // without work, so that no rank ever runs a step ahead of a peer that is still pushing)
      uint32_t werr = lane == 0 ? ep_wait_all_serial(a.wait) : 0u;
      werr = __shfl_sync(0xffffffffu, werr, 0);
      if (werr != 0) {
        if (lane == 0) *abort_flag = werr == kErrWaitTimeout ? 1u : 2u;
        alive = false;
      }
      asm volatile("fence.proxy.async;" ::: "memory");
      __syncwarp();
    }
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x, ++it) {
      const Chunk ch = chunk_of(it, tile);
      if (ch.tokens == 0) continue;
      const int ft = tile % feat_tiles;
      const int w_row = ch.expert * out_rows + ft * C::kFeatPerTile;   // first weight row (per projection)
      const size_t sfa_tile0 = static_cast<size_t>(ch.slot_base / 128) * k_tiles64;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_warp(&empty_bar[stage], phase ^ 1u, abort_flag)) { alive = false; break; }
        if (lane == 0) GLMRT_TRACE_STAGE(kFC1 ? 0 : 1, 0, traced);
        if (elect_one()) {
          const uint32_t s_a = smem_u32(smem + static_cast<size_t>(stage) * C::kStageBytes);
          const uint32_t s_b = s_a + C::kABytes;
          const uint32_t s_sfa = s_b + C::kBBytes;
          const uint32_t s_sfb = s_sfa + kSfStageBytes;
          const int kx = ks * kStageBytesK;
          const size_t ksf = static_cast<size_t>(ks) * 4;
          mbar_expect_tx(&full_bar[stage], C::kStageBytes);
          // weight tiles first: they come from HBM, the rows from L2 (measured: 1 % of the step)
          if (kFC1) {
            // 128 gate rows, then 128 up rows, each with its own scale tile
            tma_load_2d(s_b, &map_w0, &full_bar[stage], kx, w_row, pol);
            tma_load_2d(s_b + 128 * kStageBytesK, &map_w1, &full_bar[stage], kx, w_row, pol);
            const size_t t0 = static_cast<size_t>(w_row / 128) * k_tiles64 + ksf;
            bulk_load(s_sfb, a.gate_sf + t0 * 512, kSfStageBytes, &full_bar[stage], pol);
            bulk_load(s_sfb + kSfStageBytes, a.up_sf + t0 * 512, kSfStageBytes, &full_bar[stage], pol);
          } else {
#pragma unroll
            for (int t = 0; t < C::kBTiles; ++t) {
              tma_load_2d(s_b + t * 128 * kStageBytesK, &map_w0, &full_bar[stage], kx, w_row + t * 128, pol);
              bulk_load(s_sfb + t * kSfStageBytes,
                        a.down_sf + ((static_cast<size_t>(w_row / 128) + t) * k_tiles64 + ksf) * 512, kSfStageBytes,
                        &full_bar[stage], pol);
            }
          }
          tma_load_2d(s_a, &map_act, &full_bar[stage], kx, ch.slot_base, pol);
          bulk_load(s_sfa, sfa + (sfa_tile0 + ksf) * 512, kSfStageBytes, &full_bar[stage], pol);
        }
        __syncwarp();
        if (lane == 0) GLMRT_TRACE_STAGE(kFC1 ? 0 : 1, 1, traced);
        ++traced;
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    [[maybe_unused]] int traced = 0;
    int stage = 0;
    uint32_t phase = 0;
    int abuf = 0;
    uint32_t aphase = 0;
    bool alive = true;
    const uint32_t idesc = idesc_nvf4(kWN);
    uint32_t sf_flip = 0;   // scale columns alternate between two sets: copies of one stage run under the MMAs of the previous
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x, ++it) {
      if (halves > 1 && chunk_of(it, tile).tokens == 0) continue;
      if (lane == 0) GLMRT_TRACE_TILE(kFC1 ? 0 : 1, 0, it);
      if (!mbar_wait_warp(&acc_empty[abuf], aphase ^ 1u, abort_flag)) { alive = false; break; }
      tc_fence_after();
      if (lane == 0) GLMRT_TRACE_TILE(kFC1 ? 0 : 1, 1, it);
      const uint32_t d0 = tmem_base + abuf * kWN;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag)) { alive = false; break; }
        tc_fence_after();
        if (lane == 0) GLMRT_TRACE_STAGE(kFC1 ? 0 : 1, 2, traced);
        const uint32_t t_sfa = tmem_base + C::kSfCol + sf_flip * C::kSfSetCols;
        const uint32_t t_sfb = t_sfa + 16;
        sf_flip ^= 1u;
        if (elect_one()) {
          const uint32_t s_a = smem_u32(smem + static_cast<size_t>(stage) * C::kStageBytes);
          const uint32_t s_b = s_a + C::kABytes;
          const uint32_t s_sfa = s_b + C::kBBytes;
          const uint32_t s_sfb = s_sfa + kSfStageBytes;
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            tc_copy_sf(t_sfa + kb * 4, desc_sf(s_sfa + kb * 512));
#pragma unroll
            for (int t = 0; t < C::kBTiles; ++t)   // rows 128t.. of B live in columns 4t.. of the k-block's group
              tc_copy_sf(t_sfb + kb * 4 * C::kBTiles + t * 4, desc_sf(s_sfb + t * kSfStageBytes + kb * 512));
          }
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            tc_mma_nvf4(d0, desc_sw128(s_a + kb * 32), desc_sw128(s_b + kb * 32), idesc, t_sfa + kb * 4,
                        t_sfb + kb * 4 * C::kBTiles, (ks | kb) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (lane == 0) GLMRT_TRACE_STAGE(kFC1 ? 0 : 1, 3, traced);
        ++traced;
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
      if (!alive) break;
      if (elect_one()) tc_commit(&acc_full[abuf]);
      __syncwarp();
      if (C::kAccBufs == 2) { abuf ^= 1; if (abuf == 0) aphase ^= 1u; } else { aphase ^= 1u; }
    }
  } else {
    // ================= epilogue: one thread per (token slot, share of the columns) =================
    const int quad = warp & 3;                        // tensor-memory lanes 32*quad .. 32*quad+31
    const int part = (warp - 2) >> 2;                 // which share of the tile's columns
    const int row = quad * 32 + lane;                 // token slot inside the chunk
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    int abuf = 0;
    uint32_t aphase = 0;
    bool alive = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x, ++it) {
      const Chunk ch = chunk_of(it, tile);
      if (ch.tokens == 0) continue;
      const int ft = tile % feat_tiles;
      const bool valid = row < ch.tokens;
      const size_t slot = static_cast<size_t>(ch.slot_base) + row;
      const float s2a = a.scale2[ch.expert * 3 + (kFC1 ? 0 : 2)];
      const float s2b = kFC1 ? a.scale2[ch.expert * 3 + 1] : 0.0f;
      uint16_t* dst = (!kFC1 && valid) ? a.slot_out[slot] : nullptr;
      const uint32_t weight2 = (kFusedCombine && valid) ? a.slot_weight[slot] : 0u;
      if (warp == 2 && lane == 0) GLMRT_TRACE_TILE(kFC1 ? 0 : 1, 2, it);
      if (!mbar_wait_warp(&acc_full[abuf], aphase, abort_flag)) { alive = false; break; }
      tc_fence_after();
      if (warp == 2 && lane == 0) GLMRT_TRACE_TILE(kFC1 ? 0 : 1, 3, it);
      const uint32_t t_acc = tmem_base + lane_base + abuf * kWN;
      if (kFC1) {
        // gate occupies columns [0, kWN/2), up [kWN/2, kWN); 16 warps share the 16-feature blocks
        // All blocks of this warp are read out first and the accumulator is handed back before
        // any arithmetic: the next tile's MMAs run under this tile's SwiGLU and stores.
        constexpr int kBlocksPerWarp = (kWN / 32) / C::kParts;   // 1 (N=128) or 2 (N=256)
        uint32_t g[kBlocksPerWarp][16], u[kBlocksPerWarp][16];
#pragma unroll
        for (int j = 0; j < kBlocksPerWarp; ++j) {
          tc_load16(t_acc + (part * kBlocksPerWarp + j) * 16, g[j]);
          tc_load16(t_acc + kWN / 2 + (part * kBlocksPerWarp + j) * 16, u[j]);
        }
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[abuf]);
        if (warp == 2 && lane == 0) GLMRT_TRACE_TILE(0, 4, it);
#pragma unroll
        for (int j = 0; j < kBlocksPerWarp; ++j) {
          const int b = part * kBlocksPerWarp + j;
          uint32_t lo, hi, sbyte;
          swiglu_requant_block16(g[j], u[j], s2a, s2b, lo, hi, sbyte);
          if (valid) {
            const int feature = ft * C::kFeatPerTile + b * 16;
            *reinterpret_cast<uint2*>(a.act2_codes + slot * static_cast<size_t>(a.inter / 2) + feature / 2) =
                make_uint2(lo, hi);
            a.act2_sf[sf_tile_offset(slot, feature / 16, a.inter / 16)] = static_cast<uint8_t>(sbyte);
          }
        }
      } else {
        uint16_t* where = valid ? dst + ft * C::kFeatPerTile + part * 128 : nullptr;
        uint8_t* park = out_stage + static_cast<size_t>(warp - 2) * Fc2Stage<C::kPass>::kBytesPerWarp;
        fc2_emit_128_columns<C::kPass, kFusedCombine>(t_acc + part * 128, s2a, where, park, lane,
                                                 [&] { mbar_arrive(&acc_empty[abuf]); }, weight2);
      }
      if (warp == 2 && lane == 0) GLMRT_TRACE_TILE(kFC1 ? 0 : 1, 5, it);
      if (C::kAccBufs == 2) { abuf ^= 1; if (abuf == 0) aphase ^= 1u; } else { aphase ^= 1u; }
    }
  }

  // ---- teardown ----
  const uint32_t aborted = *abort_flag;
  if (aborted != 0u) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);   // let copies in flight land
    if (threadIdx.x == 0) atomicOr(a.error_word, static_cast<uint32_t>(aborted == 2u ? kErrPeerFailed : kErrWaitTimeout));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
  if (!kFC1 && a.signal.ticket != nullptr && aborted == 0u && !step_failed) ep_signal_last_cta(a.signal);
}

template <bool kFC1, int kWN, bool kFusedCombine = false>
glmrt_status_t launch_tokens(const FfnArgs& a, const CUtensorMap& act, const CUtensorMap& w0, const CUtensorMap& w1,
                             int sm_count, cudaStream_t stream) {
  using C = PfCfg<kFC1, kWN>;
  static std::atomic<uint64_t> configured{0};
  GLMRT_RETURN_IF_ERROR(ensure_smem_limit(configured, expert_gemm_tokens_kernel<kFC1, kWN, kFusedCombine>, C::kSmemBytes, "cudaFuncSetAttribute(expert_gemm_tokens_kernel)"));
  launch_pdl(expert_gemm_tokens_kernel<kFC1, kWN, kFusedCombine>, dim3(sm_count), dim3(C::kThreads), C::kSmemBytes, stream, a, act, w0, w1);
  GLMRT_LAUNCH_CHECK("expert_gemm_tokens_kernel");
  return GLMRT_STATUS_OK;
}

}  // namespace

glmrt_status_t launch_fc1_tc_prefill(const FfnArgs& a, const TensorMaps& m, int sm_count, cudaStream_t stream) {
  return launch_tokens<true, 256>(a, m.act1, m.gate, m.up, sm_count, stream);
}
glmrt_status_t launch_fc2_tc_prefill(const FfnArgs& a, const TensorMaps& m, int sm_count, cudaStream_t stream) {
  // 128-feature tiles with two accumulator buffers.  A 256-feature tile (a quarter fewer bytes into
  // shared memory per unit of math, but one accumulator buffer and only three 54 KB stages beside
  // the staging rows) measured the same or slower: FC2 0.89 vs 0.87 ms at T = 8192, 0.41 vs 0.37 ms
  // at T = 2048, 1.58 vs 1.60 ms at T = 16384.
  if (a.slot_weight != nullptr) return launch_tokens<false, 128, true>(a, m.act2, m.down, m.down, sm_count, stream);
  return launch_tokens<false, 128>(a, m.act2, m.down, m.down, sm_count, stream);
}

}  // namespace glmrt

#ifdef GLMRT_B200_TRACE
// Copies the last launches' stamps to the host: stages [2][4][2048], tiles [2][6][256] (int64).
extern "C" int glmrt_b200_debug_prefill_trace(long long* stages, long long* tiles) {
  cudaError_t e = cudaMemcpyFromSymbol(stages, glmrt::g_prefill_stage_trace, sizeof(glmrt::g_prefill_stage_trace));
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(tiles, glmrt::g_prefill_tile_trace, sizeof(glmrt::g_prefill_tile_trace));
  return static_cast<int>(e);
}
#endif
