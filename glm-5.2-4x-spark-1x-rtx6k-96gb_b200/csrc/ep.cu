// Expert-parallel exchange over NVLink peer memory.
//
// The reference moves routed rows between the coordinator and its expert hosts as
// ExpertProtocolV2 frames over TCP or RDMA (rust/crates/glmrt-transport/src/protocol_v2.rs:236-310,
// protocol_v2_tcp.rs:333-420) and, between shards, with an NCCL row all-to-all
// (native/src/glmrt_native.cc:1593-1659).  On one NVSwitch box both directions become stores into
// the peer's own memory issued from inside kernels:
//
//   counts    every rank publishes its routes-per-expert histogram to every peer; from the N
//             histograms each rank derives the SAME slot layout for every owner, so no reply is
//             needed before rows can be pushed;
//   dispatch  the home rank of a token stores the route's NVFP4 row (codes, tiled scales) and the
//             address of its result row straight into the owning rank's slot buffers;
//   combine   the owner's FC2 epilogue stores each route's bf16 result row through that address
//             into the home rank's staging rows; the home rank then runs the ordinary combine.
//
// Flags are epoch counters that only grow (no reset races across layers or steps).  Every wait is
// bounded and reports kErrWaitTimeout instead of spinning forever.  All loads that feed TMA or the
// tensor core read local memory only; peers are only ever written to.
#include "common.cuh"
#include "internal.h"

namespace glmrt {
namespace {

constexpr int kEpThreads = 1024;
constexpr uint64_t kFlagWaitLimitNs = 2000000000ull;

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *flag >= epoch.  Returns false on expiry.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = timer_ns();
  while (true) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (timer_ns() - t0 > kFlagWaitLimitNs) return false;
    __nanosleep(200);
  }
}

// ---- counts: histogram of this rank's routes, published to every rank ----------------------
__global__ void __launch_bounds__(kEpThreads) ep_count_kernel(EpArgs a, const uint32_t* topk_indices, int routes) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < a.experts; e += kEpThreads) hist[e] = 0;
  __shared__ int s_err;
  if (threadIdx.x == 0) s_err = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < routes; r += kEpThreads) {
    const uint32_t e = topk_indices[r];
    if (e >= static_cast<uint32_t>(a.experts)) atomicOr(&s_err, static_cast<int>(kErrBadExpert));
    else atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.experts; e += kEpThreads) {
    const int c = hist[e];
    for (int p = 0; p < a.world; ++p) a.peer_ctrl[p]->counts_all[a.rank * kEpMaxExperts + e] = c;
    a.ctrl->cursor[e] = 0;
  }
  if (threadIdx.x == 0) a.counters[kCntError] = static_cast<uint32_t>(s_err);  // also clears the word
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world) st_release_sys(&a.peer_ctrl[threadIdx.x]->flag_counts[a.rank], a.epoch);
}

// ---- plan: wait for all histograms, derive every owner's slot layout, build own chunk list ----
__global__ void __launch_bounds__(kEpThreads) ep_plan_kernel(EpArgs a, PlanArgs p) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world && !wait_flag(&a.ctrl->flag_counts[threadIdx.x], a.epoch)) s_ok = 0;
  __syncthreads();
  const bool ok = s_ok != 0;
  EpControl* c = a.ctrl;
  // totals per expert and this rank's offset inside each expert's slot range
  for (int e = threadIdx.x; e < a.experts; e += kEpThreads) {
    int tot = 0, mine = 0;
    for (int s = 0; s < a.world; ++s) {
      const int v = ok ? c->counts_all[s * kEpMaxExperts + e] : 0;
      if (s < a.rank) mine += v;
      tot += v;
    }
    c->total[e] = tot;
    c->my_offset[e] = mine;
  }
  __syncthreads();
  // one thread per owner walks that owner's experts in local order
  if (threadIdx.x < a.world) {
    const int owner = threadIdx.x;
    int running = 0, chunks = 0, distinct = 0, routes = 0;
    bool overflow = false;
    for (int e = owner; e < a.experts; e += a.world) {
      const int tot = c->total[e];
      c->base_slot[e] = running;
      if (owner == a.rank) {
        p.expert_counts[e / a.world] = tot;
        distinct += tot != 0;
        routes += tot;
        for (int off = 0; off < tot; off += p.chunk_tokens) {
          if (chunks < p.max_chunks) {
            Chunk ch;
            ch.expert = e / a.world;
            ch.slot_base = running + slot_of_position(off, p.chunk_tokens);
            ch.tokens = min(p.chunk_tokens, tot - off);
            ch.reserved = 0;
            p.chunks[chunks] = ch;
          }
          ++chunks;
        }
      }
      running += expert_slot_span(tot, p.chunk_tokens);
    }
    if (running > p.max_slots) overflow = true;
    if (overflow) atomicOr(&c->plan_error, 1);
    if (owner == a.rank) {
      uint32_t err = 0;
      if (!ok) err |= kErrWaitTimeout;
      if (chunks > p.max_chunks) err |= kErrChunkOverflow;
      p.counters[kCntSlots] = static_cast<uint32_t>(running);
      p.counters[kCntDistinct] = static_cast<uint32_t>(distinct);
      p.counters[kCntLocalRoutes] = static_cast<uint32_t>(routes);
      p.counters[kCntChunks] = static_cast<uint32_t>(chunks);  // finalised below
      if (err != 0) atomicOr(&p.counters[kCntError], err);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // any owner over capacity (every rank computes the same answer) or a failed wait: no expert work
    if (c->plan_error != 0) atomicOr(&p.counters[kCntError], static_cast<uint32_t>(kErrSlotOverflow));
    if (p.counters[kCntError] != 0) p.counters[kCntChunks] = 0;
    c->plan_error = 0;
  }
}

// ---- dispatch: push each local route's row into its owner's slot buffers --------------------
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(EpArgs a, const uint8_t* payload, const uint32_t* topk_indices, int32_t* route_slot, int rows,
                   int top_k, int hidden, const uint32_t* counters) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  const int n = rows * top_k;
  const bool bad_plan = counters[kCntError] != 0;
  if (warp < n && !bad_plan) {
    const uint32_t e = topk_indices[warp];
    if (e < static_cast<uint32_t>(a.experts)) {
      int pos = 0;
      if (lane == 0) pos = atomicAdd(&a.ctrl->cursor[e], 1);
      pos = __shfl_sync(0xffffffffu, pos, 0);
      const int owner = static_cast<int>(e % a.world);
      const int slot = a.ctrl->base_slot[e] + slot_of_position(a.ctrl->my_offset[e] + pos, a.chunk_tokens);
      const int row = warp / top_k;
      const int code_bytes = hidden / 2, kblocks = hidden / 16;
      const uint8_t* src = payload + static_cast<size_t>(row) * (code_bytes + kblocks);
      const uint4* src4 = reinterpret_cast<const uint4*>(src);
      uint4* dst4 = reinterpret_cast<uint4*>(a.peer_act_codes[owner] + static_cast<size_t>(slot) * code_bytes);
      for (int i = lane; i < code_bytes / 16; i += 32) dst4[i] = src4[i];
      // scales leave as 4-byte words: four consecutive blocks of a slot are contiguous in the tiled layout
      uint8_t* sf = a.peer_act_sf[owner];
      const uint32_t* sf_words = reinterpret_cast<const uint32_t*>(src + code_bytes);
      for (int j = lane; j < kblocks / 4; j += 32)
        *reinterpret_cast<uint32_t*>(sf + sf_tile_offset(slot, 4 * j, kblocks)) = sf_words[j];
      if (lane == 0) {
        a.peer_slot_out[owner][slot] = a.my_rows_in_peer[owner] + static_cast<size_t>(warp) * hidden;
        route_slot[warp] = slot;
      }
    } else if (lane == 0) {
      route_slot[warp] = -1;
    }
  } else if (warp < n && lane == 0) {
    route_slot[warp] = -1;
  }
  // last CTA to finish tells every owner that this rank's rows have landed
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(&a.ctrl->done, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x == 0) a.ctrl->done = 0;
    if (threadIdx.x < a.world) st_release_sys(&a.peer_ctrl[threadIdx.x]->flag_dispatch[a.rank], a.epoch);
  }
}

__global__ void ep_wait_kernel(const uint32_t* flags, int world, uint32_t epoch, uint32_t* error_word,
                               uint32_t* chunk_count) {
  if (threadIdx.x < world && !wait_flag(&flags[threadIdx.x], epoch)) {
    atomicOr(error_word, static_cast<uint32_t>(kErrWaitTimeout));
    if (chunk_count != nullptr) *chunk_count = 0;   // never start expert work on rows that did not arrive
  }
}

__global__ void ep_signal_kernel(EpArgs a, int which) {
  __threadfence_system();
  if (threadIdx.x < a.world) {
    EpControl* pc = a.peer_ctrl[threadIdx.x];
    st_release_sys(which == 0 ? &pc->flag_dispatch[a.rank] : &pc->flag_combine[a.rank], a.epoch);
  }
}

}  // namespace

glmrt_status_t launch_ep_count(const EpArgs& a, const uint32_t* topk_indices, int routes, cudaStream_t stream) {
  ep_count_kernel<<<1, kEpThreads, a.experts * sizeof(int), stream>>>(a, topk_indices, routes);
  GLMRT_LAUNCH_CHECK("ep_count_kernel");
  return GLMRT_STATUS_OK;
}
glmrt_status_t launch_ep_plan(const EpArgs& a, const PlanArgs& p, cudaStream_t stream) {
  ep_plan_kernel<<<1, kEpThreads, 0, stream>>>(a, p);
  GLMRT_LAUNCH_CHECK("ep_plan_kernel");
  return GLMRT_STATUS_OK;
}
glmrt_status_t launch_ep_dispatch(const EpArgs& a, const uint8_t* payload, const uint32_t* topk_indices,
                                  int32_t* route_slot, int rows, int top_k, int hidden, const uint32_t* counters,
                                  cudaStream_t stream) {
  const int n = rows * top_k;
  ep_dispatch_kernel<<<(n + 7) / 8, 256, 0, stream>>>(a, payload, topk_indices, route_slot, rows, top_k, hidden,
                                                      counters);
  GLMRT_LAUNCH_CHECK("ep_dispatch_kernel");
  return GLMRT_STATUS_OK;
}
glmrt_status_t launch_ep_wait(const uint32_t* flags, int world, uint32_t epoch, uint32_t* error_word,
                              uint32_t* chunk_count, cudaStream_t stream) {
  ep_wait_kernel<<<1, 32, 0, stream>>>(flags, world, epoch, error_word, chunk_count);
  GLMRT_LAUNCH_CHECK("ep_wait_kernel");
  return GLMRT_STATUS_OK;
}
glmrt_status_t launch_ep_signal(const EpArgs& a, int which, cudaStream_t stream) {
  ep_signal_kernel<<<1, 32, 0, stream>>>(a, which);
  GLMRT_LAUNCH_CHECK("ep_signal_kernel");
  return GLMRT_STATUS_OK;
}

}  // namespace glmrt
