// Expert-parallel exchange over NVLink peer memory.
//
// The reference moves routed rows between the coordinator and its expert hosts as
// ExpertProtocolV2 frames over TCP or RDMA (rust/crates/glmrt-transport/src/protocol_v2.rs:236-310,
// protocol_v2_tcp.rs:333-420) and, between shards, with an NCCL row all-to-all
// (native/src/glmrt_native.cc:1593-1659).  On one NVSwitch box both directions become stores into
// the peer's own memory issued from inside kernels:
//
//   counts    every rank publishes its routes-per-expert histogram to every peer (from the tail of
//             the router's selection kernel); from the N histograms each rank derives the SAME
//             slot layout for every owner, so no reply is needed before rows can be pushed;
//   dispatch  one kernel per rank waits for the histograms, derives the layout, quantises each of
//             its token rows once in shared memory and stores the row (codes, tiled scales) and
//             the address of the route's result row straight into the owning rank's slot buffers;
//   combine   the owner's FC1 kernel waits for the pushed rows, its FC2 epilogue stores each
//             route's bf16 result row through that address into the home rank's staging rows and
//             the last CTA raises the "combine" flag; the home rank's combine kernel waits for it.
//
// Flags are epoch counters that only grow (no reset races across layers or steps).  Every wait is
// bounded and reports kErrWaitTimeout instead of spinning forever.  A rank without a valid plan
// (a histogram never arrived, the layout does not fit) pushes nothing and says so (poison word),
// so that no owner computes on slots nobody filled.  All loads that feed TMA or the tensor core
// read local memory only; peers are only ever written to.
#include "common.cuh"
#include "ep_flags.cuh"
#include "internal.h"
#include "quant_block.cuh"

GLMRT_CHAIN_TRACE_TU(ep)

namespace glmrt {
namespace {

constexpr int kEpThreads = 1024;
constexpr int kPushThreads = 256;

// ---- counts: histogram of a rank without rows (ranks with rows publish from the router's tail) ----
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
  }
  if (threadIdx.x == 0) a.counters[kCntError] = static_cast<uint32_t>(s_err);  // also clears the word
  __syncthreads();   // the release below is cumulative over what the barrier ordered before it
  if (threadIdx.x < a.world) st_release_sys(&a.peer_ctrl[threadIdx.x]->flag_counts[a.rank], a.epoch);
}

// ---- plan + quantise + dispatch ---------------------------------------------------------------
// Every CTA derives the layout itself (the tables are small and sit in L2): totals per expert,
// this rank's offset inside each expert's range, and per owner the first slot of each of its
// experts.  CTA 0 also writes this rank's own work-item list and counters.  Then the CTAs walk the
// token rows (row = CTA index, + grid size, ...): quantise once, push to the owner of each route.
__global__ void __launch_bounds__(kPushThreads)
ep_plan_dispatch_kernel(EpArgs a, PlanArgs p, const uint16_t* __restrict__ hidden, uint8_t* __restrict__ payload,
                        int rows, int top_k, int hidden_dim) {
  extern __shared__ uint4 ep_smem[];
  // layout tables first (3 ints per expert), then the payload image of the row
  int* s_tot = reinterpret_cast<int*>(ep_smem);
  int* s_mine = s_tot + a.experts;
  int* s_base = s_mine + a.experts;
  uint8_t* img = reinterpret_cast<uint8_t*>(ep_smem) + ((static_cast<size_t>(a.experts) * 12 + 15) & ~size_t(15));
  __shared__ int s_err;
  __shared__ int s_owner_slots[kEpMaxWorld];
  __shared__ int s_pos[64];
  __shared__ int s_expert[64];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

  GLMRT_CHAIN_SCOPE(kChainEpPlanDispatch);
  pdl_launch_dependents();
  if (threadIdx.x == 0) s_err = 0;
  __syncthreads();
  pdl_wait();   // the routes and their positions come from the router's kernels
  GLMRT_CHAIN_READY();
  if (threadIdx.x < a.world && !wait_flag(&a.ctrl->flag_counts[threadIdx.x], a.epoch))
    atomicOr(&s_err, static_cast<int>(kErrWaitTimeout));
  __syncthreads();
  GLMRT_CHAIN_MARK(0);
  const bool have_counts = s_err == 0;
  for (int e = threadIdx.x; e < a.experts; e += kPushThreads) {
    int tot = 0, mine = 0;
    for (int s = 0; s < a.world; ++s) {
      const int v = have_counts ? a.ctrl->counts_all[s * kEpMaxExperts + e] : 0;
      if (s < a.rank) mine += v;
      tot += v;
    }
    s_tot[e] = tot;
    s_mine[e] = mine;
  }
  __syncthreads();
  // warp o scans owner o's experts (e = o, o + world, ...) in local order: first slot of each
  if (warp < a.world) {
    const int owner = warp;
    const int n_local = (a.experts - owner + a.world - 1) / a.world;
    int running = 0;
    for (int i0 = 0; i0 < n_local; i0 += 32) {
      const int i = i0 + lane;
      const int e = owner + i * a.world;
      const int span = i < n_local ? expert_slot_span(s_tot[e], a.chunk_tokens) : 0;
      int incl = span;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
      }
      if (i < n_local) s_base[e] = running + incl - span;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      s_owner_slots[owner] = running;
      if (running > p.max_slots) atomicOr(&s_err, static_cast<int>(kErrSlotOverflow));
    }
  }
  __syncthreads();
  GLMRT_CHAIN_MARK(1);

  if (blockIdx.x == 0) {
    // this rank's own work items: chunk offsets by a scan over its experts (warp 0), then every
    // thread writes the chunks of the experts it owns
    __shared__ int s_chunk_total;
    const int n_local = (a.experts - a.rank + a.world - 1) / a.world;
    __shared__ int s_coff[kEpMaxExperts];
    if (warp == 0) {
      int running = 0, distinct = 0, routes = 0;
      for (int i0 = 0; i0 < n_local; i0 += 32) {
        const int i = i0 + lane;
        const int tot = i < n_local ? s_tot[a.rank + i * a.world] : 0;
        const int n = (tot + p.chunk_tokens - 1) / p.chunk_tokens;
        int incl = n;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += v;
        }
        if (i < n_local) s_coff[i] = running + incl - n;
        running += __shfl_sync(0xffffffffu, incl, 31);
        distinct += tot != 0;
        routes += tot;
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        distinct += __shfl_xor_sync(0xffffffffu, distinct, d);
        routes += __shfl_xor_sync(0xffffffffu, routes, d);
      }
      if (lane == 0) {
        s_chunk_total = running;
        if (running > p.max_chunks) atomicOr(&s_err, static_cast<int>(kErrChunkOverflow));
        p.counters[kCntSlots] = static_cast<uint32_t>(s_owner_slots[a.rank]);
        p.counters[kCntDistinct] = static_cast<uint32_t>(distinct);
        p.counters[kCntLocalRoutes] = static_cast<uint32_t>(routes);
      }
    }
    __syncthreads();
    const bool plan_ok = s_err == 0;
    for (int i = threadIdx.x; i < n_local; i += kPushThreads) {
      const int e = a.rank + i * a.world;
      const int tot = s_tot[e];
      p.expert_counts[i] = tot;
      if (plan_ok) {
        int c = s_coff[i];
        for (int off = 0; off < tot; off += p.chunk_tokens, ++c) {
          Chunk ch;
          ch.expert = i;
          ch.slot_base = s_base[e] + slot_of_position(off, p.chunk_tokens);
          ch.tokens = min(p.chunk_tokens, tot - off);
          ch.reserved = 0;
          p.chunks[c] = ch;
        }
      }
    }
    if (p.fc_sync != nullptr && plan_ok)   // hand-over words of the decode GEMMs (FfnArgs::fc_sync)
      for (int i = threadIdx.x; i < kFcSyncHeader + s_chunk_total; i += kPushThreads) p.fc_sync[i] = 0u;
    if (threadIdx.x == 0) {
      // never start expert work on an inconsistent plan
      p.counters[kCntChunks] = plan_ok ? static_cast<uint32_t>(s_chunk_total) : 0u;
      if (!plan_ok) atomicOr(&p.counters[kCntError], static_cast<uint32_t>(s_err));
    }
  }
  __syncthreads();
  const bool plan_ok = s_err == 0;
  if (!plan_ok && threadIdx.x == 0) {
    atomicOr(&p.counters[kCntError], static_cast<uint32_t>(s_err));
    atomicOr(&a.ctrl->plan_failed, 1);   // read by the last CTA: one failing CTA poisons the whole push
  }

  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const int code_bytes = hidden_dim / 2, kblocks = hidden_dim / 16;
    __syncthreads();   // the previous row's image and positions have been read
    const size_t row_bytes = static_cast<size_t>(code_bytes + kblocks);
    if (plan_ok) {
      // positions of the row's routes among this rank's routes of each expert: asked for first, the
      // round trip of the loads runs under the quantisation of the row
      if (threadIdx.x < top_k) {
        const uint32_t e = p.topk_indices[row * top_k + threadIdx.x];
        s_expert[threadIdx.x] = static_cast<int>(e);
        // its position among this rank's routes of that expert was counted by the router's tail
        s_pos[threadIdx.x] = e < static_cast<uint32_t>(a.experts) ? p.route_slot[row * top_k + threadIdx.x] : -1;
      }
      if (hidden != nullptr) {
        if (a.chunk_tokens < 128)   // decode-sized step
          quantize_row_to_image<true>(hidden + static_cast<size_t>(row) * hidden_dim, img, hidden_dim, kPushThreads);
        else
          quantize_row_to_image<false>(hidden + static_cast<size_t>(row) * hidden_dim, img, hidden_dim, kPushThreads);
      } else {
        const uint4* src = reinterpret_cast<const uint4*>(payload + row * row_bytes);
        for (int i = threadIdx.x; i < static_cast<int>(row_bytes / 16); i += kPushThreads)
          reinterpret_cast<uint4*>(img)[i] = src[i];
      }
      __syncthreads();
      GLMRT_CHAIN_MARK(3);
      if (hidden != nullptr) {
        uint4* prow = reinterpret_cast<uint4*>(payload + row * row_bytes);
        for (int i = threadIdx.x; i < static_cast<int>(row_bytes / 16); i += kPushThreads)
          prow[i] = reinterpret_cast<const uint4*>(img)[i];
      }
      const uint32_t* sf_words = reinterpret_cast<const uint32_t*>(img + code_bytes);
      GLMRT_CHAIN_MARK(4);
      for (int k = 0; k < top_k; ++k) {
        const int route = row * top_k + k;
        const int pos = s_pos[k];
        if (pos < 0) {
          if (threadIdx.x == 0) p.route_slot[route] = -1;
          continue;
        }
        const int e = s_expert[k];
        const int owner = e % a.world;
        const int slot = s_base[e] + slot_of_position(s_mine[e] + pos, a.chunk_tokens);
        uint4* dst4 = reinterpret_cast<uint4*>(a.peer_act_codes[owner] + static_cast<size_t>(slot) * code_bytes);
        for (int i = threadIdx.x; i < code_bytes / 16; i += kPushThreads) dst4[i] = reinterpret_cast<const uint4*>(img)[i];
        if (a.chunk_tokens >= 128) {
          // prefill-sized step: the slot's scale bytes leave as one contiguous row, the owner re-tiles
          uint4* srow = reinterpret_cast<uint4*>(a.peer_act_sf_rows[owner] + static_cast<size_t>(slot) * kblocks);
          const uint4* s4 = reinterpret_cast<const uint4*>(img + code_bytes);
          for (int j = threadIdx.x; j < kblocks / 16; j += kPushThreads) srow[j] = s4[j];
        } else {
          // decode-sized step: 4-byte words straight into the tiled layout (four consecutive blocks of
          // a slot are contiguous there)
          uint8_t* sf = a.peer_act_sf[owner];
          for (int j = threadIdx.x; j < kblocks / 4; j += kPushThreads)
            *reinterpret_cast<uint32_t*>(sf + sf_tile_offset(slot, 4 * j, kblocks)) = sf_words[j];
        }
        if (threadIdx.x == 0) {
          a.peer_slot_out[owner][slot] = a.my_rows_in_peer[owner] + static_cast<size_t>(route) * hidden_dim;
          p.route_slot[route] = slot;
        }
      }
    } else {
      for (int k = threadIdx.x; k < top_k; k += kPushThreads) p.route_slot[row * top_k + k] = -1;
    }
  }

  // last CTA to finish tells every owner that this rank's rows have landed -- or that none will
  // (one thread fences for the CTA: the barrier orders every thread's stores before its fence)
  __syncthreads();
  GLMRT_CHAIN_MARK(2);
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = atomicAdd(&a.ctrl->ticket_dispatch, 1) == static_cast<int>(gridDim.x) - 1;
    if (s_last) __threadfence_system();
  }
  __syncthreads();
  if (s_last) {
    const bool failed = *reinterpret_cast<volatile int32_t*>(&a.ctrl->plan_failed) != 0;
    __syncthreads();
    if (threadIdx.x == 0) {
      a.ctrl->ticket_dispatch = 0;
      a.ctrl->plan_failed = 0;
    }
    if (threadIdx.x < a.world) {
      EpControl* pc = a.peer_ctrl[threadIdx.x];
      if (failed) {
        pc->poison_dispatch[a.rank] = a.epoch;
        __threadfence_system();
      }
      st_release_sys(&pc->flag_dispatch[a.rank], a.epoch);
    }
  }
}

// Owner side of a prefill-sized push: wait for every rank's rows, then move the scale rows of the
// occupied slots into the tiled layout.  One thread per (slot, group of four blocks).
__global__ void __launch_bounds__(256)
ep_retile_scales_kernel(EpWait w, const uint8_t* __restrict__ sf_rows, uint8_t* __restrict__ sf_tiled, int kblocks,
                        const uint32_t* counters, uint32_t* error_word, uint32_t* chunk_count) {
  GLMRT_CHAIN_SCOPE(kChainEpRetile);
  pdl_launch_dependents();
  pdl_wait();
  GLMRT_CHAIN_READY();
  __shared__ uint32_t s_err;
  if (threadIdx.x == 0) {
    s_err = ep_wait_all_serial(w);
    if (s_err != 0u) {
      atomicOr(error_word, s_err);
      if (blockIdx.x == 0) *chunk_count = 0;   // never start expert work on rows that did not arrive
    }
  }
  __syncthreads();
  if (s_err != 0u) return;
  const int slots = static_cast<int>(counters[kCntSlots]);
  const int words = kblocks / 4;
  const long long total = static_cast<long long>(slots) * words;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
    const int slot = static_cast<int>(i / words), j = static_cast<int>(i % words);
    const uint32_t v = reinterpret_cast<const uint32_t*>(sf_rows + static_cast<size_t>(slot) * kblocks)[j];
    *reinterpret_cast<uint32_t*>(sf_tiled + sf_tile_offset(slot, 4 * j, kblocks)) = v;
  }
}

// Stand-alone wait / signal for engines whose kernels do not carry them (the SIMT verification engine).
__global__ void ep_wait_kernel(EpWait w, uint32_t* error_word, uint32_t* chunk_count) {
  if (threadIdx.x != 0) return;
  const uint32_t err = ep_wait_all_serial(w);
  if (err != 0) {
    atomicOr(error_word, err);
    if (chunk_count != nullptr) *chunk_count = 0;   // never start expert work on rows that did not arrive
  }
}
__global__ void ep_signal_kernel(EpSignal s, const uint32_t* error_word) {
  if (*error_word != 0u) return;   // a failed step tells no home rank that results have arrived
  __threadfence_system();
  if (threadIdx.x < s.world) st_release_sys(s.peer_flags[threadIdx.x], s.epoch);
}

}  // namespace

glmrt_status_t launch_ep_retile_scales(const EpArgs& a, const uint8_t* sf_rows, uint8_t* sf_tiled, int kblocks,
                                       const uint32_t* counters, uint32_t* error_word, uint32_t* chunk_count,
                                       cudaStream_t stream) {
  launch_pdl(ep_retile_scales_kernel, dim3(592), dim3(256), 0, stream, ep_wait_dispatch(a), sf_rows, sf_tiled, kblocks,
             counters, error_word, chunk_count);
  GLMRT_LAUNCH_CHECK("ep_retile_scales_kernel");
  return GLMRT_STATUS_OK;
}
glmrt_status_t launch_ep_wait(const EpWait& w, uint32_t* error_word, uint32_t* chunk_count, cudaStream_t stream) {
  ep_wait_kernel<<<1, 32, 0, stream>>>(w, error_word, chunk_count);
  GLMRT_LAUNCH_CHECK("ep_wait_kernel");
  return GLMRT_STATUS_OK;
}
glmrt_status_t launch_ep_signal(const EpSignal& s, const uint32_t* error_word, cudaStream_t stream) {
  ep_signal_kernel<<<1, 32, 0, stream>>>(s, error_word);
  GLMRT_LAUNCH_CHECK("ep_signal_kernel");
  return GLMRT_STATUS_OK;
}

glmrt_status_t launch_ep_count(const EpArgs& a, const uint32_t* topk_indices, int routes, cudaStream_t stream) {
  ep_count_kernel<<<1, kEpThreads, a.experts * sizeof(int), stream>>>(a, topk_indices, routes);
  GLMRT_LAUNCH_CHECK("ep_count_kernel");
  return GLMRT_STATUS_OK;
}

RouterCountTail ep_count_tail(const EpArgs& a) {
  RouterCountTail t{};
  t.world = a.world;
  t.epoch = a.epoch;
  for (int p = 0; p < a.world; ++p) {
    t.peer_counts[p] = a.peer_ctrl[p]->counts_all + a.rank * kEpMaxExperts;   // address arithmetic only
    t.peer_flags[p] = a.peer_ctrl[p]->flag_counts + a.rank;
  }
  t.error_word = a.counters + kCntError;
  t.ticket = &a.ctrl->ticket_select;
  return t;
}

glmrt_status_t launch_ep_plan_dispatch(const EpArgs& a, const PlanArgs& p, const uint16_t* hidden, uint8_t* payload,
                                       int rows, int top_k, int hidden_dim, cudaStream_t stream) {
  if (top_k > 64 || hidden_dim % 256 != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "expert-parallel dispatch: top_k must be <= 64 and hidden a multiple of 256");
  const size_t smem = ((static_cast<size_t>(a.experts) * 12 + 15) & ~size_t(15)) + hidden_dim / 2 + hidden_dim / 16;
  if (smem > 40 * 1024) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "expert-parallel dispatch: hidden too large");
  // every CTA derives the layout once, so large batches walk their rows with a bounded grid
  const int grid = rows > 0 ? (rows < 1184 ? rows : 1184) : 1;
  launch_pdl(ep_plan_dispatch_kernel, dim3(grid), dim3(kPushThreads), smem, stream, a, p, hidden, payload,
             rows, top_k, hidden_dim);
  GLMRT_LAUNCH_CHECK("ep_plan_dispatch_kernel");
  return GLMRT_STATUS_OK;
}

EpWait ep_wait_dispatch(const EpArgs& a) {
  EpWait w;
  w.flags = a.ctrl->flag_dispatch;
  w.poison = a.ctrl->poison_dispatch;
  w.world = a.world;
  w.epoch = a.epoch;
  return w;
}
EpWait ep_wait_combine(const EpArgs& a) {
  EpWait w;
  w.flags = a.ctrl->flag_combine;
  w.poison = nullptr;
  w.world = a.world;
  w.epoch = a.epoch;
  return w;
}
EpSignal ep_signal_combine(const EpArgs& a) {
  EpSignal s{};
  for (int p = 0; p < a.world; ++p) s.peer_flags[p] = a.peer_ctrl[p]->flag_combine + a.rank;
  s.ticket = &a.ctrl->ticket_fc2;
  s.world = a.world;
  s.epoch = a.epoch;
  return s;
}

}  // namespace glmrt
