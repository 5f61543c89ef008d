// Route plan of one batch by ONE CTA: counting sort of the rows * top_k routes by expert (the
// device-side form of plan_packed_w4a16_topk8_prefill_flat,
// rust/crates/glmrt-daemon/src/commands/real_full/sparse_mlp/route.rs:3727-3828).  A device function
// so that it can run as a kernel of its own or as the tail of the router's selection kernel (one
// launch less on the decode path).  Called by every thread of the CTA; nthreads = its size
// (a multiple of 32).  Uses 8 KB of static shared memory.
#pragma once

#include "common.cuh"
#include "internal.h"

namespace glmrt {

constexpr int kMaxLocalExperts = 1024;

// chunk_tokens is 32, 128 or 256: the slot arithmetic of expert_slot_span / slot_of_position with
// shifts (this runs on the critical path of every decode step).
__device__ __forceinline__ int plan_slot_span(int count, int chunk_tokens, int shift) {
  return chunk_tokens < 128 ? ((count + chunk_tokens - 1) >> shift) * 128 : (count + 127) & ~127;
}
__device__ __forceinline__ int plan_slot_of_position(int pos, int chunk_tokens, int shift) {
  return chunk_tokens < 128 ? (pos >> shift) * 128 + (pos & (chunk_tokens - 1)) : pos;
}

// The plan of at most 32 routes (up to four rows of top-8: the single-row decode step) by one warp,
// without the shared-memory histogram and its barriers: a lane per route, `match.any` finds the
// routes of the same expert (position = lower lanes among them, count = all of them), an expert's
// rank among the touched experts (in expert order, as the counting sort places them) is counted over
// the 32 lanes, and every touched expert gets one work item in a 128-slot group of its own.  Same
// outputs as the general body below for the same routes, except that a route's position inside its
// expert follows the route order (there: the order of the atomic counter).  Decode layout only
// (32-token work items), all experts local.
__device__ __forceinline__ void route_plan_tiny(const PlanArgs& a, int nthreads) {
  const int n = a.rows * a.top_k;
  for (int i = threadIdx.x; i < a.experts; i += nthreads) a.expert_counts[i] = 0;
  __syncthreads();   // the counts of the touched experts are stored after the zeros
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  const uint32_t e = lane < n ? a.topk_indices[lane] : kNoRoute;
  const bool valid = e != kNoRoute && e < static_cast<uint32_t>(a.experts);
  const unsigned bad = __ballot_sync(0xffffffffu, lane < n && e != kNoRoute && e >= static_cast<uint32_t>(a.experts));
  const unsigned peers = __match_any_sync(0xffffffffu, valid ? e : (0x80000000u | static_cast<uint32_t>(lane)));
  const int pos = __popc(peers & ((1u << lane) - 1u));
  const int count = __popc(peers);
  const bool leader = valid && pos == 0;
  int rank = 0;
#pragma unroll 8
  for (int k = 0; k < 32; ++k) {
    const uint32_t ek = __shfl_sync(0xffffffffu, e, k);
    const int lk = __shfl_sync(0xffffffffu, leader ? 1 : 0, k);
    rank += (lk != 0 && ek < e) ? 1 : 0;
  }
  const int distinct = __popc(__ballot_sync(0xffffffffu, leader));
  const int routes = __popc(__ballot_sync(0xffffffffu, valid));
  const int total_slots = 128 * distinct;
  int err = bad != 0u ? static_cast<int>(kErrBadExpert) : 0;
  if (total_slots > a.max_slots) err |= static_cast<int>(kErrSlotOverflow);
  if (distinct > a.max_chunks) err |= static_cast<int>(kErrChunkOverflow);
  if (leader) {
    a.expert_counts[e] = count;
    if (err == 0) {
      Chunk ch;
      ch.expert = static_cast<int32_t>(e);
      ch.slot_base = rank * 128;
      ch.tokens = count;
      ch.reserved = 0;
      a.chunks[rank] = ch;
    }
  }
  if (lane < n) {
    const int slot = (valid && err == 0) ? rank * 128 + pos : -1;
    a.route_slot[lane] = slot;
    if (slot >= 0) a.slot_route[slot] = lane;
  }
  if (a.fc_sync != nullptr && err == 0)
    for (int i = lane; i < kFcSyncHeader + distinct; i += 32) a.fc_sync[i] = 0u;
  if (lane == 0) {
    a.counters[kCntChunks] = err != 0 ? 0u : static_cast<uint32_t>(distinct);   // never launch expert work on an inconsistent plan
    a.counters[kCntSlots] = static_cast<uint32_t>(total_slots);
    a.counters[kCntError] = static_cast<uint32_t>(err);   // also clears the word for the kernels that follow
    a.counters[kCntDistinct] = static_cast<uint32_t>(distinct);
    a.counters[kCntLocalRoutes] = static_cast<uint32_t>(routes);
  }
}

constexpr int kPlanKeep = 4;   // routes a thread keeps in registers between the counting and the placing pass

__device__ __forceinline__ void route_plan_body(const PlanArgs& a, int nthreads) {
  __shared__ int cnt[kMaxLocalExperts];
  __shared__ int base[kMaxLocalExperts];
  __shared__ int s_error;
  __shared__ int s_total_chunks;
  if (a.rows * a.top_k <= 32 && a.ep_world == 1 && a.chunk_tokens == 32) {
    route_plan_tiny(a, nthreads);
    return;
  }
  const int local_experts = (a.experts - a.ep_rank + a.ep_world - 1) / a.ep_world;
  const int shift = 31 - __clz(a.chunk_tokens);
  for (int i = threadIdx.x; i < local_experts; i += nthreads) cnt[i] = 0;
  if (threadIdx.x == 0) s_error = 0;
  __syncthreads();
  const int n = a.rows * a.top_k;
  // Up to kPlanKeep * nthreads routes (64 rows of top-8 on 128 threads) stay in registers from the
  // counting pass to the placing pass: their expert ids are loaded once, all loads of a thread in
  // flight together, and route_slot is written once.
  const bool keep = n <= kPlanKeep * nthreads;
  int kept_le[kPlanKeep], kept_pos[kPlanKeep];
  for (int r0 = 0; r0 < n; r0 += kPlanKeep * nthreads) {
    uint32_t e[kPlanKeep];
#pragma unroll
    for (int j = 0; j < kPlanKeep; ++j) {
      const int r = r0 + j * nthreads + threadIdx.x;
      e[j] = r < n ? a.topk_indices[r] : kNoRoute;
    }
#pragma unroll
    for (int j = 0; j < kPlanKeep; ++j) {
      const int r = r0 + j * nthreads + threadIdx.x;
      int pos = -1, le = 0;
      if (e[j] == kNoRoute) {
        // nothing to do for this entry
      } else if (e[j] >= static_cast<uint32_t>(a.experts)) {
        atomicOr(&s_error, static_cast<int>(kErrBadExpert));
      } else if (a.ep_world == 1) {
        le = static_cast<int>(e[j]);
        pos = atomicAdd(&cnt[le], 1);
      } else if (static_cast<int>(e[j] % a.ep_world) == a.ep_rank) {
        le = static_cast<int>(e[j] / a.ep_world);
        pos = atomicAdd(&cnt[le], 1);
      }
      kept_le[j] = le;
      kept_pos[j] = pos;
      if (!keep && r < n) a.route_slot[r] = pos;
    }
  }
  __syncthreads();
  GLMRT_CHAIN_MARK(3);
  if (threadIdx.x < 32) {
    // warp 0: each lane owns a contiguous run of experts; exclusive scan of slots and chunks
    const int lane = threadIdx.x;
    const int per_lane = (local_experts + 31) / 32;
    const int le0 = lane * per_lane, le1 = min(local_experts, le0 + per_lane);
    int slots = 0, chunks = 0, distinct = 0, routes = 0;
    for (int le = le0; le < le1; ++le) {
      const int c = cnt[le];
      slots += plan_slot_span(c, a.chunk_tokens, shift);
      chunks += (c + a.chunk_tokens - 1) >> shift;
      distinct += c != 0;
      routes += c;
    }
    int slot_off = slots, chunk_off = chunks;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int s = __shfl_up_sync(0xffffffffu, slot_off, d);
      const int c = __shfl_up_sync(0xffffffffu, chunk_off, d);
      if (lane >= d) { slot_off += s; chunk_off += c; }
    }
    const int total_slots = __shfl_sync(0xffffffffu, slot_off, 31);
    const int total_chunks = __shfl_sync(0xffffffffu, chunk_off, 31);
    slot_off -= slots;    // inclusive -> exclusive
    chunk_off -= chunks;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      distinct += __shfl_xor_sync(0xffffffffu, distinct, d);
      routes += __shfl_xor_sync(0xffffffffu, routes, d);
    }
    int err = s_error;
    if (total_slots > a.max_slots) err |= static_cast<int>(kErrSlotOverflow);
    if (total_chunks > a.max_chunks) err |= static_cast<int>(kErrChunkOverflow);
    for (int le = le0; le < le1; ++le) {
      const int c = cnt[le];
      base[le] = slot_off;
      a.expert_counts[le] = c;
      if (err == 0) {
        for (int off = 0; off < c; off += a.chunk_tokens) {
          Chunk ch;
          ch.expert = le;
          ch.slot_base = slot_off + plan_slot_of_position(off, a.chunk_tokens, shift);
          ch.tokens = min(a.chunk_tokens, c - off);
          ch.reserved = 0;
          a.chunks[chunk_off++] = ch;
        }
      }
      slot_off += plan_slot_span(c, a.chunk_tokens, shift);
    }
    if (lane == 0) {
      s_total_chunks = err != 0 ? 0 : total_chunks;
      s_error = err;
      // never launch expert work on an inconsistent plan
      a.counters[kCntChunks] = err != 0 ? 0u : static_cast<uint32_t>(total_chunks);
      a.counters[kCntSlots] = static_cast<uint32_t>(total_slots);
      a.counters[kCntError] = static_cast<uint32_t>(err);   // also clears the word for the kernels that follow
      a.counters[kCntDistinct] = static_cast<uint32_t>(distinct);
      a.counters[kCntLocalRoutes] = static_cast<uint32_t>(routes);
    }
  }
  __syncthreads();
  GLMRT_CHAIN_MARK(4);
  if (a.fc_sync != nullptr) {
    // the decode GEMMs' hand-over words: FC2's tile counter and one "rows stored" count per work item
    for (int i = threadIdx.x; i < kFcSyncHeader + s_total_chunks; i += nthreads) a.fc_sync[i] = 0u;
  }
  const bool bad = s_error != 0;
  GLMRT_CHAIN_MARK(5);
  if (keep) {
#pragma unroll
    for (int j = 0; j < kPlanKeep; ++j) {
      const int r = j * nthreads + threadIdx.x;
      if (r >= n) continue;
      int slot = -1;
      if (kept_pos[j] >= 0 && !bad) {
        slot = base[kept_le[j]] + plan_slot_of_position(kept_pos[j], a.chunk_tokens, shift);
        if (slot >= a.max_slots) slot = -1;
      }
      a.route_slot[r] = slot;
      if (slot >= 0) a.slot_route[slot] = r;
    }
    return;
  }
  for (int r = threadIdx.x; r < n; r += nthreads) {
    const int pos = a.route_slot[r];
    if (pos < 0) continue;
    const uint32_t e = a.topk_indices[r];
    const int slot = base[e / a.ep_world] + plan_slot_of_position(pos, a.chunk_tokens, shift);
    if (bad || slot >= a.max_slots) {
      a.route_slot[r] = -1;
    } else {
      a.route_slot[r] = slot;
      a.slot_route[slot] = r;
    }
  }
}

}  // namespace glmrt
