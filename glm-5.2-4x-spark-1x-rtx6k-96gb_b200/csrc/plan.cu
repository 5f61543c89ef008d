// Route plan and dispatch.
//
// route plan: counting sort of the rows * top_k routes by expert on the device, replacing the
// host-side plan_packed_w4a16_topk8_prefill_flat of the reference
// (rust/crates/glmrt-daemon/src/commands/real_full/sparse_mlp/route.rs:3727-3828).  Each local
// expert receives a contiguous slot range that starts on a multiple of 128 slots (the row
// granularity of the tiled scale layout) and is cut into chunks of `chunk_tokens` slots, the
// work items of the expert GEMM kernels.  The order of routes inside an expert is arbitrary;
// every route's result is independent of its slot, so outputs stay bit-reproducible.
//
// dispatch: copies each route's NVFP4 activation payload row into its slot (codes row-major,
// scales into the tiled layout) -- the single-GPU form of the all-to-all send.
#include "common.cuh"
#include "internal.h"
#include "plan_body.cuh"

GLMRT_CHAIN_TRACE_TU(plan)

namespace glmrt {
namespace {

constexpr int kPlanThreads = 1024;

__global__ void __launch_bounds__(kPlanThreads) route_plan_kernel(PlanArgs a) {
  GLMRT_CHAIN_SCOPE(kChainPlan);
  pdl_launch_dependents();
  pdl_wait();   // the routes come from the router's kernels
  GLMRT_CHAIN_READY();
  route_plan_body(a, kPlanThreads);
}

// ---- large batches: the same plan in three grid-wide steps ---------------------------------
// Slots follow the order of the routes block by block (256 routes = 32 rows of a top-8 batch), so
// the rows an expert's chunk reads and the result rows it writes stay close together in memory;
// a purely atomic assignment scatters them over the whole batch and costs DRAM locality.
constexpr int kPlanBlock = 256;

// count: per-block histogram; each route keeps its arrival position inside (block, expert)
__global__ void __launch_bounds__(kPlanBlock) plan_count_kernel(PlanArgs a, int local_experts) {
  extern __shared__ int hist[];
  for (int i = threadIdx.x; i < local_experts; i += kPlanBlock) hist[i] = 0;
  __syncthreads();
  const int r = blockIdx.x * kPlanBlock + threadIdx.x;
  if (r < a.rows * a.top_k) {
    const uint32_t e = a.topk_indices[r];
    int pos = -1;
    if (e == kNoRoute) {
      // nothing to do for this entry
    } else if (e >= static_cast<uint32_t>(a.experts)) {
      atomicOr(&a.counters[kCntError], static_cast<uint32_t>(kErrBadExpert));
    } else if (static_cast<int>(e % a.ep_world) == a.ep_rank) {
      pos = atomicAdd(&hist[e / a.ep_world], 1);
    }
    a.route_slot[r] = pos;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < local_experts; i += kPlanBlock)
    a.block_hist[static_cast<size_t>(blockIdx.x) * local_experts + i] = hist[i];
}
// scan: per expert, exclusive prefix over the blocks; then one warp turns the totals into slot
// bases and the chunk list.  The blocks of an expert are cut into segments, one thread each
// (neighbouring threads hold neighbouring experts, so every access is a full line); values are
// fetched eight at a time before anything is stored, so the loads do not queue behind the stores.
__global__ void __launch_bounds__(1024) plan_scan_kernel(PlanArgs a, int local_experts, int blocks) {
  __shared__ int seg_sum[1024];
  const int segs = local_experts <= 1024 ? min(32, 1024 / local_experts) : 1;
  const int per_seg = (blocks + segs - 1) / segs;
  for (int le0 = 0; le0 < local_experts; le0 += 1024) {   // one pass unless there are more than 1024 experts
    const int seg = segs > 1 ? threadIdx.x / local_experts : 0;
    const int le = segs > 1 ? threadIdx.x % local_experts : le0 + threadIdx.x;
    const bool active = seg < segs && le < local_experts;
    const int b0 = min(blocks, seg * per_seg), b1 = min(blocks, b0 + per_seg);
    int sum = 0;
    if (active) {
      for (int b = b0; b < b1; b += 8) {
        int c[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) c[j] = b + j < b1 ? a.block_hist[static_cast<size_t>(b + j) * local_experts + le] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += c[j];
      }
    }
    __syncthreads();   // the previous pass has read seg_sum
    seg_sum[threadIdx.x] = sum;
    __syncthreads();
    if (active) {
      int running = 0;
      for (int s2 = 0; s2 < seg; ++s2) running += seg_sum[s2 * local_experts + le];
      if (seg == segs - 1) a.expert_counts[le] = running + sum;
      for (int b = b0; b < b1; b += 8) {
        int c[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) c[j] = b + j < b1 ? a.block_hist[static_cast<size_t>(b + j) * local_experts + le] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (b + j < b1) a.block_hist[static_cast<size_t>(b + j) * local_experts + le] = running;
          running += c[j];
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  const int per_lane = (local_experts + 31) / 32;
  const int le0 = lane * per_lane, le1 = min(local_experts, le0 + per_lane);
  int slots = 0, chunks = 0, distinct = 0, routes = 0;
  for (int le = le0; le < le1; ++le) {
    const int c = a.expert_counts[le];
    slots += expert_slot_span(c, a.chunk_tokens);
    chunks += (c + a.chunk_tokens - 1) / a.chunk_tokens;
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
  slot_off -= slots;
  chunk_off -= chunks;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    distinct += __shfl_xor_sync(0xffffffffu, distinct, d);
    routes += __shfl_xor_sync(0xffffffffu, routes, d);
  }
  uint32_t err = a.counters[kCntError];
  if (total_slots > a.max_slots) err |= kErrSlotOverflow;
  if (total_chunks > a.max_chunks) err |= kErrChunkOverflow;
  for (int le = le0; le < le1; ++le) {
    const int c = a.expert_counts[le];
    a.expert_base[le] = slot_off;
    if (err == 0) {
      for (int off = 0; off < c; off += a.chunk_tokens) {
        Chunk ch;
        ch.expert = le;
        ch.slot_base = slot_off + slot_of_position(off, a.chunk_tokens);
        ch.tokens = min(a.chunk_tokens, c - off);
        ch.reserved = 0;
        a.chunks[chunk_off++] = ch;
      }
    }
    slot_off += expert_slot_span(c, a.chunk_tokens);
  }
  if (lane == 0) {
    a.counters[kCntChunks] = err != 0 ? 0u : static_cast<uint32_t>(total_chunks);
    a.counters[kCntSlots] = static_cast<uint32_t>(total_slots);
    a.counters[kCntError] = err;
    a.counters[kCntDistinct] = static_cast<uint32_t>(distinct);
    a.counters[kCntLocalRoutes] = static_cast<uint32_t>(routes);
  }
}
// place: position inside the expert -> slot
__global__ void __launch_bounds__(kPlanBlock) plan_place_kernel(PlanArgs a, int local_experts) {
  const int r = blockIdx.x * kPlanBlock + threadIdx.x;
  if (r >= a.rows * a.top_k) return;
  const int pos = a.route_slot[r];
  if (pos < 0) return;
  const bool bad = a.counters[kCntError] != 0;
  const int le = static_cast<int>(a.topk_indices[r] / a.ep_world);
  const int slot = a.expert_base[le] +
                   slot_of_position(a.block_hist[static_cast<size_t>(blockIdx.x) * local_experts + le] + pos, a.chunk_tokens);
  if (bad || slot >= a.max_slots) {
    a.route_slot[r] = -1;
  } else {
    a.route_slot[r] = slot;
    a.slot_route[slot] = r;
  }
}

// One warp per route.
__global__ void __launch_bounds__(256) dispatch_kernel(DispatchArgs a) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  const int n = a.rows * a.top_k;
  if (warp >= n) return;
  const int slot = a.route_slot[warp];
  if (slot < 0) return;
  const int row = warp / a.top_k;
  const int code_bytes = a.hidden / 2;
  const int kblocks = a.hidden / 16;
  const uint8_t* src = a.payload + static_cast<size_t>(row) * (code_bytes + kblocks);
  const uint4* src4 = reinterpret_cast<const uint4*>(src);
  uint4* dst4 = reinterpret_cast<uint4*>(a.act_codes + static_cast<size_t>(slot) * code_bytes);
  for (int i = lane; i < code_bytes / 16; i += 32) dst4[i] = src4[i];
  const uint8_t* ssrc = src + code_bytes;
  for (int j = lane; j < kblocks; j += 32) a.act_sf[sf_tile_offset(slot, j, kblocks)] = ssrc[j];
  if (lane == 0) a.slot_out[slot] = a.route_rows + static_cast<size_t>(warp) * a.hidden;
}

}  // namespace

glmrt_status_t launch_route_plan(const PlanArgs& a, cudaStream_t stream) {
  const int n = a.rows * a.top_k;
  if (n <= 8192) {   // one CTA, one launch
    launch_pdl(route_plan_kernel, dim3(1), dim3(kPlanThreads), 0, stream, a);
    GLMRT_LAUNCH_CHECK("route_plan_kernel");
    return GLMRT_STATUS_OK;
  }
  const int local_experts = (a.experts - a.ep_rank + a.ep_world - 1) / a.ep_world;
  const int blocks = (n + kPlanBlock - 1) / kPlanBlock;
  cudaError_t err = cudaMemsetAsync(a.counters + kCntError, 0, sizeof(uint32_t), stream);
  if (err != cudaSuccess) return status_from_cuda(err, "cudaMemsetAsync(route plan)");
  plan_count_kernel<<<blocks, kPlanBlock, local_experts * sizeof(int), stream>>>(a, local_experts);
  GLMRT_LAUNCH_CHECK("plan_count_kernel");
  plan_scan_kernel<<<1, 1024, 0, stream>>>(a, local_experts, blocks);
  GLMRT_LAUNCH_CHECK("plan_scan_kernel");
  plan_place_kernel<<<blocks, kPlanBlock, 0, stream>>>(a, local_experts);
  GLMRT_LAUNCH_CHECK("plan_place_kernel");
  return GLMRT_STATUS_OK;
}

glmrt_status_t launch_dispatch(const DispatchArgs& a, cudaStream_t stream) {
  const int n = a.rows * a.top_k;
  dispatch_kernel<<<(n + 7) / 8, 256, 0, stream>>>(a);
  GLMRT_LAUNCH_CHECK("dispatch_kernel");
  return GLMRT_STATUS_OK;
}

}  // namespace glmrt
