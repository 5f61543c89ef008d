// Tensor-core engine: grouped NVFP4 x NVFP4 expert GEMMs on tcgen05 (sm_100a).
//
// Replaces the reference's CuTe-DSL W4A16 fused-MoE kernels (launch glue
// native/cuda/kernels/b12x_direct.cu:479-647,989-1541; kernel source not in the reference
// tree) and its SIMT route MLP (native/cuda/kernels/mlp.cu:218-314) with two persistent,
// warp-specialised kernels built on the same template:
//
//   FC1: for every (expert, token chunk, 128-feature tile): gate and up projections as two
//        block-scaled UMMA accumulators in tensor memory, then SwiGLU and NVFP4
//        requantisation straight from the float32 accumulators (moe_ref.py:18-20 followed by
//        the activation quantiser) into the slot-ordered operand of FC2.
//   FC2: down projection, scaled by the tensor's global scale, rounded to bf16 and stored to
//        the destination row of each route (moe_ref.py:21); the weighted sum over a token's
//        routes happens in the combine kernel in the oracle's order.
//
// Operand orientation is "weights as A": the 128 rows of the MMA tile are weight rows, the N
// columns are the tokens of one expert (16..BN), so at decode sizes every weight byte is
// streamed exactly once through a TMA pipeline while the tensor core merely keeps up, and at
// prefill sizes N grows to BN.  Scales travel as pre-tiled 512-byte blocks (128 rows x 4
// sixteen-element groups) that tcgen05.cp places in tensor memory.
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and tensor-memory
// owner, warps 2..5 = epilogue (one per 32-lane quadrant of tensor memory).
// Every wait is bounded: on expiry the kernel records kErrWaitTimeout, lets outstanding
// copies land, releases tensor memory and returns.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "ep_flags.cuh"
#include "epilogue.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

GLMRT_CHAIN_TRACE_TU(gemm)

namespace glmrt {
namespace {

using namespace tc;

template <bool kFC1, int kBN>
struct Cfg {
  static constexpr int kNumA = kFC1 ? 2 : 1;
  static constexpr int kABytes = kTileRows * kStageBytesK;                 // 16 KiB per weight tile
  static constexpr int kBBytes = kBN * kStageBytesK;
  static constexpr int kSfbTiles = (kBN + 127) / 128;                      // scale tiles per k-block for B
  static constexpr int kStageBytes = kNumA * kABytes + kBBytes + kNumA * kSfStageBytes + kSfbTiles * kSfStageBytes;
  static constexpr int kStages = (221184 / kStageBytes) > 10 ? 10 : (221184 / kStageBytes);
  // One issuing warp, kept converged, hands the instructions of a stage to one elected lane
  // (elect.sync); issuing from a divergent `lane == 0` branch had limited the tensor pipe.
  static constexpr int kAccCols = kNumA * kBN;                             // accumulator columns per buffer
  static constexpr int kAccBufs = (2 * kAccCols + 16 * kNumA + 16 * kSfbTiles <= 512) ? 2 : 1;
  static constexpr int kSfCol = kAccBufs * kAccCols;                       // first scale column
  static constexpr int kColsUsed = kSfCol + 16 * kNumA + 16 * kSfbTiles;
  static constexpr int kTmemCols = kColsUsed <= 32 ? 32 : kColsUsed <= 64 ? 64 : kColsUsed <= 128 ? 128
                                   : kColsUsed <= 256 ? 256 : 512;
  static constexpr uint32_t kTxBytes = kStageBytes;
  static constexpr int kChunkCache = 256;  // work items of this CTA's first tiles, staged in shared memory
  static constexpr int kBarrierBytes = 768; // mbarriers, the tensor-memory slot, the abort word and the tile ring
  static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024 /*align*/ + kBarrierBytes +
                                       kChunkCache * sizeof(Chunk);
};

// One entry of the tile ring of the overlapped FC2 kernel: a scheduling warp draws tiles from a
// global counter and hands each one, with its work item and once its operand rows are there, to the
// producer, the issuing warp and the epilogue warps.
struct TileSlot {
  Chunk ch;
  int32_t tile;      // -1: no more tiles
  int32_t pad[3];
};
constexpr int kTileRing = 8;
constexpr int kThreadsOverlapFc2 = kThreadsTC + 32;   // the six warps of every instance + the scheduling warp

// Destination-row pointers are written by an earlier kernel (or by a peer rank); the overlapped
// FC2 may share an SM's L1 with that earlier kernel's traffic, so it reads them from the L2.
__device__ __forceinline__ uint16_t* load_row_pointer(uint16_t* const* p) {
  return reinterpret_cast<uint16_t*>(__ldcg(reinterpret_cast<const unsigned long long*>(p)));
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// kOverlap: FC1 and FC2 of a decode-sized step run as one pipeline over two launches.  FC1 lets its
// successor start once FC1 itself may run (griddepcontrol.launch_dependents after its own
// griddepcontrol.wait, so everything older than FC1 is complete when FC2 begins) and counts, per work
// item, the epilogue warps that have stored intermediate rows.  FC2 does not wait for FC1 to
// complete: its CTAs take the SMs FC1's CTAs have left, draw tiles from a global counter (the CTAs
// that start early take more) and wait, per tile, until the work item's intermediate rows are all
// there.  On an expert-parallel shard with 28 experts FC1 is 448 tiles on 148 SMs: during its
// fourth wave 144 SMs would otherwise idle.
template <bool kFC1, int kBN, bool kOverlap>
__global__ void __launch_bounds__(kOverlap && !kFC1 ? kThreadsOverlapFc2 : kThreadsTC, 1)
expert_gemm_kernel(FfnArgs a, const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                   const __grid_constant__ CUtensorMap map_b) {
  using C = Cfg<kFC1, kBN>;
  constexpr bool kDynamic = kOverlap && !kFC1;   // tiles drawn from a counter instead of a fixed stride
  GLMRT_CHAIN_SCOPE(kFC1 ? kChainFc1 : kChainFc2);
  if (!(kOverlap && kFC1)) pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  // stage buffers need 1024-byte alignment for the 128-byte swizzle
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(C::kStages) * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* acc_full = bars + 2 * C::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* ring_full = acc_empty + 2;
  uint64_t* ring_empty = ring_full + kTileRing;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ring_empty + kTileRing);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  TileSlot* ring = reinterpret_cast<TileSlot*>(reinterpret_cast<uint8_t*>(bars) + 384);   // 8 x 32 bytes
  Chunk* chunk_cache = reinterpret_cast<Chunk*>(reinterpret_cast<uint8_t*>(bars) + C::kBarrierBytes);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  // K (reduction) and output-feature geometry of this GEMM
  const int k_bytes = (kFC1 ? a.hidden : a.inter) / 2;       // packed bytes per operand row
  const int k_stages = k_bytes / kStageBytesK;
  const int out_rows = kFC1 ? a.inter : a.hidden;            // weight rows per expert
  const int feat_tiles = out_rows / kTileRows;
  const int k_tiles64 = k_bytes / 32;                        // scale tiles (64 elements) along K

  if (threadIdx.x == 32) {   // the maps are kernel parameters: fetched while the previous kernel still runs
    prefetch_tensormap(&map_a0);
    if (kFC1) prefetch_tensormap(&map_a1);
    prefetch_tensormap(&map_b);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    for (int r = 0; r < kTileRing; ++r) {
      mbar_init(&ring_full[r], 1);
      mbar_init(&ring_empty[r], 6);   // the producer, the issuing warp and four epilogue warps have read the entry
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

  // Everything above (barriers, tensor memory) ran while the previous kernel was finishing; from
  // here on this kernel reads what earlier kernels wrote.  The overlapped FC2 does not wait for
  // FC1's completion (FC1 raised launch_dependents only after everything older than itself was
  // complete); it reads what it needs of FC1 tile by tile, below.
  // cache policies of the loads (register-only; created before the wait, off the critical path)
  const uint64_t pol_w = policy_evict_first();   // weights are read once
  const uint64_t pol_x = policy_evict_last();    // activations are re-read by every feature tile
  if (!kDynamic) pdl_wait();
  GLMRT_CHAIN_READY();
  if (kOverlap && kFC1) pdl_launch_dependents();
  // a step that has already reported an error runs no expert work (and tells no peer it did)
  const uint32_t planned_chunks = __ldcg(a.counters + kCntChunks);   // both loads in flight together
  const bool step_failed = *reinterpret_cast<const volatile uint32_t*>(a.error_word) != 0u;
  const int num_chunks = step_failed ? 0 : static_cast<int>(planned_chunks);
  const int num_tiles = num_chunks * feat_tiles;
  if (!kDynamic) {
    // The work items of this CTA's tiles are fetched once, up front: a global load at the head of
    // every tile would stall each role for a memory round trip and drain the TMA pipeline.
    // The loads do not depend on the chunk count (entries past it are never used), so both memory
    // round trips of this prologue overlap.
    for (int i = threadIdx.x; i < C::kChunkCache; i += blockDim.x) {
      const long long ci = (static_cast<long long>(blockIdx.x) + static_cast<long long>(i) * gridDim.x) / feat_tiles;
      if (ci < a.max_chunks) chunk_cache[i] = a.chunks[ci];
    }
    __syncthreads();
  }
  GLMRT_CHAIN_MARK(0);
  // Tile sequence of a consumer role (every lane of the warp calls it; the warp stays converged).
  auto next_tile = [&](int it, TileSlot& ts) -> bool {
    if (!kDynamic) {
      const long long tile = static_cast<long long>(blockIdx.x) + static_cast<long long>(it) * gridDim.x;
      if (tile >= num_tiles) return false;
      ts.tile = static_cast<int32_t>(tile);
      ts.ch = it < C::kChunkCache ? chunk_cache[it] : a.chunks[tile / feat_tiles];
      return true;
    }
    const int r = it % kTileRing;
    if (!mbar_wait_warp(&ring_full[r], static_cast<uint32_t>(it / kTileRing) & 1u, abort_flag)) return false;
    ts = ring[r];
    __syncwarp();
    if (lane == 0) mbar_arrive(&ring_empty[r]);
    return ts.tile >= 0;
  };

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      const uint8_t* sfa0 = kFC1 ? a.gate_sf : a.down_sf;
      const uint8_t* sfa1 = a.up_sf;
      const uint8_t* sfb = kFC1 ? a.act1_sf : a.act2_sf;
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      if (kFC1 && a.wait.flags != nullptr && (blockIdx.x == 0 || static_cast<int>(blockIdx.x) < num_tiles)) {
        // expert-parallel path: the rows this kernel reads are pushed by the peers (CTA 0 waits even
        // without work, so that no rank ever runs a step ahead of a peer that is still pushing)
        const uint32_t werr = ep_wait_all_serial(a.wait);
        if (werr != 0) {
          *abort_flag = werr == kErrWaitTimeout ? 1u : 2u;
          alive = false;
        }
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      for (int it = 0; alive; ++it) {
        TileSlot ts;
        if (kDynamic) {
          // the scheduling warp hands over tiles whose operand rows are complete
          const int r = it % kTileRing;
          if (!mbar_wait(&ring_full[r], static_cast<uint32_t>(it / kTileRing) & 1u, abort_flag)) { alive = false; break; }
          ts = ring[r];
          mbar_arrive(&ring_empty[r]);
          if (ts.tile < 0) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");   // FC1 wrote the rows with ordinary stores; TMA reads them
        } else if (!next_tile(it, ts)) {
          break;
        }
        const Chunk ch = ts.ch;
        const int tile = ts.tile;
        const int ft = tile % feat_tiles;
        const int w_row = ch.expert * out_rows + ft * kTileRows;
        const size_t sfa_tile0 = static_cast<size_t>(w_row / 128) * k_tiles64;
        const size_t sfb_tile0 = static_cast<size_t>(ch.slot_base / 128) * k_tiles64;
        for (int ks = 0; ks < k_stages; ++ks) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { alive = false; break; }
          uint8_t* st = smem + static_cast<size_t>(stage) * C::kStageBytes;
          const uint32_t s_a0 = smem_u32(st);
          const uint32_t s_b = s_a0 + C::kNumA * C::kABytes;
          const uint32_t s_sfa0 = s_b + C::kBBytes;
          const uint32_t s_sfb = s_sfa0 + C::kNumA * kSfStageBytes;
          mbar_expect_tx(&full_bar[stage], C::kTxBytes);
          if (it == 0 && ks == 0) GLMRT_CHAIN_MARK_HERE(1);
          tma_load_2d(s_a0, &map_a0, &full_bar[stage], ks * kStageBytesK, w_row, pol_w);
          if (kFC1) tma_load_2d(s_a0 + C::kABytes, &map_a1, &full_bar[stage], ks * kStageBytesK, w_row, pol_w);
          tma_load_2d(s_b, &map_b, &full_bar[stage], ks * kStageBytesK, ch.slot_base, pol_x);
          bulk_load(s_sfa0, sfa0 + (sfa_tile0 + static_cast<size_t>(ks) * 4) * 512, kSfStageBytes, &full_bar[stage], pol_w);
          if (kFC1)
            bulk_load(s_sfa0 + kSfStageBytes, sfa1 + (sfa_tile0 + static_cast<size_t>(ks) * 4) * 512, kSfStageBytes,
                      &full_bar[stage], pol_w);
#pragma unroll
          for (int t = 0; t < C::kSfbTiles; ++t)
            bulk_load(s_sfb + t * kSfStageBytes,
                      sfb + (sfb_tile0 + static_cast<size_t>(t) * k_tiles64 + static_cast<size_t>(ks) * 4) * 512,
                      kSfStageBytes, &full_bar[stage], pol_x);
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
      GLMRT_CHAIN_MARK_HERE(2);
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    {   // the whole warp runs the loop; one elected lane issues
      int stage = 0;
      uint32_t phase = 0;
      int abuf = 0;
      uint32_t aphase = 0;
      bool alive = true;
      const uint32_t t_sfa0 = tmem_base + C::kSfCol;
      const uint32_t t_sfb = t_sfa0 + 16 * C::kNumA;
      TileSlot ts;
      for (int it = 0; alive && next_tile(it, ts); ++it) {
        const Chunk ch = ts.ch;
        const uint32_t n_mma = static_cast<uint32_t>(max(16, (ch.tokens + 15) & ~15));
        const uint32_t idesc = idesc_nvf4(n_mma);
        const uint32_t sfb_q = static_cast<uint32_t>((ch.slot_base & 127) >> 5);  // 32-row quadrant inside the scale tile
        if (!mbar_wait_warp(&acc_empty[abuf], aphase ^ 1u, abort_flag)) { alive = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + abuf * C::kAccCols;
        for (int ks = 0; ks < k_stages; ++ks) {
          if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag)) { alive = false; break; }
          tc_fence_after();
          if (it == 0 && ks == 0 && lane == 0) GLMRT_CHAIN_MARK_HERE(3);
          uint8_t* st = smem + static_cast<size_t>(stage) * C::kStageBytes;
          const uint32_t s_a0 = smem_u32(st);
          const uint32_t s_b = s_a0 + C::kNumA * C::kABytes;
          const uint32_t s_sfa0 = s_b + C::kBBytes;
          const uint32_t s_sfb = s_sfa0 + C::kNumA * kSfStageBytes;
          if (elect_one()) {
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            tc_copy_sf(t_sfa0 + kb * 4, desc_sf(s_sfa0 + kb * 512));
            if (kFC1) tc_copy_sf(t_sfa0 + 16 + kb * 4, desc_sf(s_sfa0 + kSfStageBytes + kb * 512));
#pragma unroll
            for (int t = 0; t < C::kSfbTiles; ++t)
              tc_copy_sf(t_sfb + kb * 4 * C::kSfbTiles + t * 4, desc_sf(s_sfb + t * kSfStageBytes + kb * 512));
          }
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            const uint32_t acc = (ks | kb) != 0 ? 1u : 0u;
            const uint32_t dset = d0;
            const uint64_t bdesc = desc_sw128(s_b + kb * 32);
            const uint32_t sfb_addr = t_sfb + kb * 4 * C::kSfbTiles + sfb_q;
            tc_mma_nvf4(dset, desc_sw128(s_a0 + kb * 32), bdesc, idesc, t_sfa0 + kb * 4, sfb_addr, acc);
            if (kFC1)
              tc_mma_nvf4(dset + kBN, desc_sw128(s_a0 + C::kABytes + kb * 32), bdesc, idesc, t_sfa0 + 16 + kb * 4,
                          sfb_addr, acc);
          }
          tc_commit(&empty_bar[stage]);  // frees the stage once the MMAs above have read it
          }
          __syncwarp();
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        if (elect_one()) tc_commit(&acc_full[abuf]);      // accumulators complete
        __syncwarp();
        if (C::kAccBufs == 2) { abuf ^= 1; if (abuf == 0) aphase ^= 1u; } else { aphase ^= 1u; }
      }
      if (lane == 0) GLMRT_CHAIN_MARK_HERE(4);
    }
  } else if (warp >= 6) {
    // ================= tile scheduler (overlapped FC2 only) =================
    // Draws tiles from the global counter (the CTAs that start early, on SMs FC1 has already left,
    // take more), waits until every FC1 epilogue warp has stored its share of the tile's work item
    // (bounded; a step that has reported an error ends the wait), and hands the tile to the ring.
    if (kDynamic && lane == 0) {
      const uint32_t need = 4u * static_cast<uint32_t>(a.inter / kTileRows);
      int ready_chunk = -1;
      Chunk ch = Chunk{0, 0, 0, 0};
      bool alive = true;
      for (int it = 0; alive; ++it) {
        TileSlot ts;
        ts.pad[0] = ts.pad[1] = ts.pad[2] = 0;
        const int t = static_cast<int>(atomicAdd(a.fc_sync, 1u));
        if (t >= num_tiles) {
          ts.tile = -1;
          ts.ch = Chunk{0, 0, 0, 0};
        } else {
          const int ci = t / feat_tiles;
          if (ci != ready_chunk) {
            const int4 c4 = __ldcg(reinterpret_cast<const int4*>(a.chunks + ci));   // from L2: written by an earlier kernel
            ch = Chunk{c4.x, c4.y, c4.z, c4.w};
            const uint32_t* done = a.fc_sync + kFcSyncHeader + ci;
            if (ld_acquire_gpu(done) < need) {
              const uint64_t t0 = global_timer_ns();
              while (ld_acquire_gpu(done) < need) {
                if (*reinterpret_cast<const volatile uint32_t*>(a.error_word) != 0u || *abort_flag != 0u ||
                    global_timer_ns() - t0 > kWaitLimitNs) {
                  *abort_flag = 1u;
                  alive = false;
                  break;
                }
                __nanosleep(64);
              }
              if (!alive) break;
            }
            ready_chunk = ci;
          }
          ts.tile = t;
          ts.ch = ch;
        }
        const int r = it % kTileRing;
        if (!mbar_wait(&ring_empty[r], (static_cast<uint32_t>(it / kTileRing) & 1u) ^ 1u, abort_flag)) break;
        ring[r] = ts;
        mbar_arrive(&ring_full[r]);     // release: the entry is visible to the roles that wait on it
        if (ts.tile < 0) break;
      }
    }
  } else {
    // ================= epilogue (warps 2..5) =================
    const int quad = warp & 3;                       // tensor-memory lanes 32*quad .. 32*quad+31
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    int abuf = 0;
    uint32_t aphase = 0;
    bool alive = true;
    TileSlot ts;
    for (int it = 0; alive && next_tile(it, ts); ++it) {
      const Chunk ch = ts.ch;
      const int tile = ts.tile;
      const int ft = tile % feat_tiles;
      const int feature = ft * kTileRows + quad * 32 + lane;   // output row of this lane inside the expert
      // everything the epilogue needs from global memory is fetched before the accumulators are
      // awaited, so these latencies overlap the tile's main loop
      const float s2a = a.scale2[ch.expert * 3 + (kFC1 ? 0 : 2)];
      const float s2b = kFC1 ? a.scale2[ch.expert * 3 + 1] : 0.0f;
      uint16_t* dst_lane = nullptr;   // FC2: lane j holds the destination row of token column j (of the current 32)
      if (!kFC1 && lane < ch.tokens) dst_lane = load_row_pointer(a.slot_out + ch.slot_base + lane);
      // lane 0 waits (bounded) and the warp takes one common decision, so that the full-mask
      // shuffles of the epilogue can never run with part of the warp gone
      uint32_t ready = lane == 0 ? (mbar_wait(&acc_full[abuf], aphase, abort_flag) ? 1u : 0u) : 0u;
      ready = __shfl_sync(0xffffffffu, ready, 0);
      if (ready == 0u) { alive = false; break; }
      (void)mbar_try_wait(&acc_full[abuf], aphase);  // phase already complete: every lane observes it
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base + abuf * C::kAccCols;
      if (kFC1) {
        for (int c0 = 0; c0 < ch.tokens; c0 += 8) {
          uint32_t g[8], u[8];
          tc_load8(t_acc + c0, g);
          tc_load8(t_acc + kBN + c0, u);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (c0 + j < ch.tokens)  // uniform across the warp
              swiglu_requant_store<true>(__fmul_rn(__uint_as_float(g[j]), s2a), __fmul_rn(__uint_as_float(u[j]), s2b),
                                   feature, static_cast<size_t>(ch.slot_base) + c0 + j, a.inter, a.act2_codes,
                                   a.act2_sf);
          }
        }
        if (kOverlap) {
          // this warp's share of the work item's intermediate rows is stored: count it for FC2
          asm volatile("fence.proxy.async.global;" ::: "memory");
          __threadfence();
          __syncwarp();
          if (lane == 0) atomicAdd(a.fc_sync + kFcSyncHeader + tile / feat_tiles, 1u);
        }
      } else {
        for (int c0 = 0; c0 < ch.tokens; c0 += 8) {
          if (c0 != 0 && (c0 & 31) == 0)
            dst_lane = (c0 + lane < ch.tokens) ? load_row_pointer(a.slot_out + ch.slot_base + c0 + lane) : nullptr;
          uint32_t y[8];
          tc_load8(t_acc + c0, y);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const unsigned long long p =
                __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(dst_lane), (c0 + j) & 31);
            if (c0 + j < ch.tokens && p != 0ull)   // a slot nobody gave a destination is skipped
              reinterpret_cast<uint16_t*>(p)[feature] = f32_to_bf16_rne(__fmul_rn(__uint_as_float(y[j]), s2a));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[abuf]);
      if (C::kAccBufs == 2) { abuf ^= 1; if (abuf == 0) aphase ^= 1u; } else { aphase ^= 1u; }
    }
  }

  if (warp == 2 && lane == 0) GLMRT_CHAIN_MARK_HERE(5);
  // ---- teardown ----
  __syncwarp();
  const uint32_t aborted = *abort_flag;
  if (aborted != 0u) {
    // let copies already in flight land before shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (threadIdx.x == 0) atomicOr(a.error_word, static_cast<uint32_t>(aborted == 2u ? kErrPeerFailed : kErrWaitTimeout));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
  if (!kFC1 && a.signal.ticket != nullptr && aborted == 0u && !step_failed) ep_signal_last_cta(a.signal);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

template <bool kFC1, int kBN, bool kOverlap>
glmrt_status_t launch_one(const FfnArgs& a, const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b,
                          int sm_count, cudaStream_t stream) {
  using C = Cfg<kFC1, kBN>;
  static std::atomic<uint64_t> configured{0};
  GLMRT_RETURN_IF_ERROR(ensure_smem_limit(configured, expert_gemm_kernel<kFC1, kBN, kOverlap>, C::kSmemBytes, "cudaFuncSetAttribute(expert_gemm_kernel)"));
  launch_pdl(expert_gemm_kernel<kFC1, kBN, kOverlap>, dim3(sm_count), dim3(kOverlap && !kFC1 ? kThreadsOverlapFc2 : kThreadsTC),
             C::kSmemBytes, stream, a, a0, a1, b);
  GLMRT_LAUNCH_CHECK("expert_gemm_kernel");
  return GLMRT_STATUS_OK;
}

// FC2 may start under FC1's tail only when the two are launched with the programmatic launch
// attribute (otherwise FC2 starts after FC1 has completed anyway and the plain pair is used).
bool fc_overlap(const FfnArgs& a) {
  static const bool off = []() {
    const char* v = std::getenv("GLMRT_B200_NO_FC_OVERLAP");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return a.fc_sync != nullptr && !off && pdl_enabled();
}

}  // namespace

glmrt_status_t make_codes_tensor_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes,
                                     uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(GLMRT_STATUS_CUDA_UNAVAILABLE, "cuTensorMapEncodeTiled is not available");
  if (row_bytes % 128 != 0 || reinterpret_cast<uintptr_t>(base) % 16 != 0 || box_rows == 0 || box_rows > 256)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "tensor map: rows must be multiples of 128 bytes on a 16-byte aligned base");
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GLMRT_STATUS_INTERNAL_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
  return GLMRT_STATUS_OK;
}

glmrt_status_t make_scale_tensor_map(CUtensorMap* out, const void* base, uint64_t bytes) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(GLMRT_STATUS_CUDA_UNAVAILABLE, "cuTensorMapEncodeTiled is not available");
  if (bytes == 0 || bytes % 2048 != 0 || reinterpret_cast<uintptr_t>(base) % 128 != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "scale tensor map: needs whole 2 KB groups on a 128-byte aligned base");
  const cuuint64_t dims[2] = {128, bytes / 128};
  const cuuint64_t strides[1] = {128};
  const cuuint32_t box[2] = {128, 16};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GLMRT_STATUS_INTERNAL_ERROR, "cuTensorMapEncodeTiled (scales) failed with code " + std::to_string(static_cast<int>(r)));
  return GLMRT_STATUS_OK;
}

glmrt_status_t launch_fc1_tc(const FfnArgs& a, const TensorMaps& m, int sm_count, cudaStream_t stream) {
  if (a.chunk_tokens == 32)
    return fc_overlap(a) ? launch_one<true, 32, true>(a, m.gate, m.up, m.act1, sm_count, stream)
                         : launch_one<true, 32, false>(a, m.gate, m.up, m.act1, sm_count, stream);
  return fail(GLMRT_STATUS_INTERNAL_ERROR, "tensor-core engine: unsupported chunk size");
}

glmrt_status_t launch_fc2_tc(const FfnArgs& a, const TensorMaps& m, int sm_count, cudaStream_t stream) {
  if (a.chunk_tokens == 32)
    return fc_overlap(a) ? launch_one<false, 32, true>(a, m.down, m.down, m.act2, sm_count, stream)
                         : launch_one<false, 32, false>(a, m.down, m.down, m.act2, sm_count, stream);
  return fail(GLMRT_STATUS_INTERNAL_ERROR, "tensor-core engine: unsupported chunk size");
}

}  // namespace glmrt
