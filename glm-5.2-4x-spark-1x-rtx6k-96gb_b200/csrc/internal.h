// Internal launch interfaces shared by the translation units of libglmrt_b200.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace glmrt {

// Error bits a kernel may set in the layer's device error word.
enum DeviceError : uint32_t {
  kErrWaitTimeout = 1u,       // a bounded mbarrier / flag wait gave up
  kErrSlotOverflow = 2u,      // route plan needs more slots than the layer holds
  kErrChunkOverflow = 4u,     // more (expert, token-chunk) work items than the layer holds
  kErrBadExpert = 8u,         // a route names an expert id >= experts
  kErrPeerFailed = 16u,       // a peer rank declared that it had no valid plan this step and pushed nothing
};

// Counters written by the route-plan kernel (device memory, uint32 each).
enum Counter : int {
  kCntChunks = 0,
  kCntSlots = 1,
  kCntError = 2,
  kCntDistinct = 3,
  kCntLocalRoutes = 4,
  kCntRouterError = 5,   // error word of the tensor-core router kernel (cleared by that kernel)
  kCntTicket = 6,        // last-CTA ticket of the router's selection kernel (zero between launches)
  kCntWords = 8,
};

struct Chunk {      // one (expert, block of <= BN tokens) work item
  int32_t expert;      // local expert index
  int32_t slot_base;   // first slot (multiple of 32)
  int32_t tokens;      // valid slots in this chunk
  int32_t reserved;
};

// ---- router.cu ----
struct RouterCountTail;
glmrt_status_t launch_router(const void* hidden, bool hidden_bf16, const void* weight, bool weight_bf16,
                             const float* bias, float* logits, uint32_t* idx, float* scores, float* weights,
                             size_t rows, size_t hidden_dim, size_t experts, size_t top_k, float scaling,
                             cudaStream_t stream, const RouterCountTail* tail = nullptr);

// splits in 2..8: `logits` holds that many partial tables [splits][rows][experts], added in order
constexpr int kEpMaxWorld = 8;
struct RouterCountTail;
glmrt_status_t launch_router_select(const float* logits, const float* bias, uint32_t* idx, float* scores,
                                    float* weights, size_t rows, size_t experts, size_t top_k, float scaling,
                                    cudaStream_t stream, int splits = 1, const RouterCountTail* tail = nullptr);
// ---- router_tc.cu (prefill-sized batches) ----
glmrt_status_t launch_split_router_weight(const float* w, uint16_t* w3, size_t experts, size_t hidden,
                                          cudaStream_t stream);
bool router_tc_supported(size_t rows, size_t hidden, size_t experts, const void* x);
int router_tc_splits(size_t rows, size_t hidden, size_t experts, int sm_count);
// splits > 1 writes partial tables [splits][rows][experts] for launch_router_select to add up
glmrt_status_t launch_router_logits_tc(const uint16_t* x, const CUtensorMap& map_w3, float* logits, size_t rows,
                                       size_t hidden, size_t experts, uint32_t* error_word, int sm_count,
                                       cudaStream_t stream, int splits = 1);

// ---- quant.cu ----
glmrt_status_t launch_quantize_rows_payload(const uint16_t* in, uint8_t* payload, size_t rows, size_t cols,
                                            uint32_t rule, cudaStream_t stream);
glmrt_status_t launch_tile_scales(const uint8_t* in, uint8_t* out, size_t rows, size_t kblocks,
                                  size_t out_row_offset, cudaStream_t stream);
glmrt_status_t launch_quantize_weight_f32(const float* in, uint8_t* packed, uint8_t* scales, float* scale_2_out,
                                          uint32_t* amax_scratch, size_t rows, size_t cols, cudaStream_t stream);

// ---- plan.cu ----
// Slot layout of one expert.  Work items of 128 or 256 slots tile the expert's range densely (the
// range is rounded up to the 128-row granularity of the tiled scales).  Work items of 32 slots
// (decode kernels) each get a 128-slot group of their own, so that the scales of a work item always
// start at column 0 of a scale tile in tensor memory: the block-scaled MMA was only ever run, and
// is only known to work, with its B-scale address on such a boundary.
#if defined(__CUDACC__)
#define GLMRT_HD __host__ __device__
#else
#define GLMRT_HD
#endif
GLMRT_HD inline int expert_slot_span(int count, int chunk_tokens) {
  return chunk_tokens < 128 ? ((count + chunk_tokens - 1) / chunk_tokens) * 128 : (count + 127) & ~127;
}
// slot (relative to the expert's first slot) of the expert's route number `pos`
GLMRT_HD inline int slot_of_position(int pos, int chunk_tokens) {
  return chunk_tokens < 128 ? (pos / chunk_tokens) * 128 + pos % chunk_tokens : pos;
}

// A route entry with this expert id is "no route": it gets no slot and is not an error (the
// expert worker's view of a request may name fewer than top_k experts for a row).
constexpr uint32_t kNoRoute = 0xffffffffu;
// Weights of the first FC1 work of a decode step, asked into the L2 while the rows are quantised and
// dispatched: between the route plan and the first weight byte FC1 itself asks for, the memory
// system is otherwise idle for several microseconds.  One SM turns out about one 128-byte request
// per clock (256 GB/s), so the requests are spread over extra CTAs of the dispatch kernel: four per
// (work item, 128-row tile) pair of FC1's tile order.  (One GPU only: on the expert-parallel push
// kernel the same CTAs changed nothing.)
struct WeightPrefetch {
  const uint8_t* w0 = nullptr;    // gate codes [local experts * rows_per_expert, row_bytes]; nullptr: no prefetch
  const uint8_t* w1 = nullptr;    // up codes, same shape
  const uint8_t* sf0 = nullptr;   // their tiled scales
  const uint8_t* sf1 = nullptr;
  int rows_per_expert = 0, row_bytes = 0;
  int tiles = 0;                  // pairs asked for (kPrefetchParts extra CTAs each)
};
struct PlanArgs {
  const uint32_t* topk_indices;  // [rows * top_k] global expert ids
  int rows, top_k, experts;      // experts = global count
  int ep_world, ep_rank;
  int chunk_tokens;              // BN: tokens per chunk (32, 128 or 256)
  int max_slots, max_chunks;
  int32_t* route_slot;           // [rows * top_k] -> slot or -1
  int32_t* slot_route;           // [max_slots] -> route or -1
  int32_t* expert_counts;        // [local experts]
  int32_t* expert_base;          // [local experts] first slot of each expert (large-batch plan)
  int32_t* block_hist;           // [ceil(routes / 256)][local experts] per-block counts, then prefixes
  Chunk* chunks;                 // [max_chunks]
  uint32_t* counters;            // [kCntWords]
  uint32_t* fc_sync = nullptr;   // [kFcSyncHeader + max_chunks] cleared by the plan: see FfnArgs::fc_sync
};
// Optional tails of the router's selection kernel, run by the last CTA of its grid to finish.
//   expert-parallel path (world > 0): count this rank's routes per expert, store the histogram into
//     every rank's count table, number each route among this rank's routes of its expert, clear the layer's error word, and
//     raise the per-peer "counts" epoch flag;
//   one GPU, decode-sized batches (do_plan): build the route plan right there (one launch less).
struct RouterCountTail {
  int world = 0;                         // 0: no histogram publish
  uint32_t epoch = 0;
  int32_t* peer_counts[kEpMaxWorld];     // this rank's row of each rank's count table
  uint32_t* peer_flags[kEpMaxWorld];     // this rank's "counts" flag at each rank
  int32_t* route_pos = nullptr;          // [routes], local: a route's number among this rank's routes of its expert (-1: no valid expert)
  uint32_t* error_word;                  // local
  int32_t* ticket = nullptr;             // local, zero between launches
  int do_plan = 0;
  PlanArgs plan;
};
glmrt_status_t launch_route_plan(const PlanArgs& a, cudaStream_t stream);

struct DispatchArgs {
  const uint8_t* payload;        // [rows, H/2 + H/16]
  const int32_t* route_slot;     // [rows * top_k]
  int rows, top_k, hidden;
  uint8_t* act_codes;            // [max_slots, H/2]
  uint8_t* act_sf;               // tiled scales, H/16 blocks per slot
  uint16_t* route_rows;          // bf16 [rows * top_k, H]: destination rows of FC2
  uint16_t** slot_out;           // [max_slots] destination row pointer per slot
  uint8_t* payload_out;          // fused quantise + dispatch only: where the payload rows are written
  // Fused combine (the down GEMM adds weight * row straight into the layer output): a slot's
  // destination is then its token's output row and its route weight travels beside it.
  uint16_t* combine_out = nullptr;       // [rows, hidden] bf16 layer output, or nullptr: per-route rows
  const float* topk_weights = nullptr;   // [rows * top_k]
  uint32_t* slot_weight = nullptr;       // [max_slots] the route weight as a bf16 pair
  // fused quantise + dispatch of a decode-sized step: CTAs past `rows` prefetch FC1 weights
  WeightPrefetch prefetch;
  const Chunk* chunks = nullptr;
  const uint32_t* counters = nullptr;
};
glmrt_status_t launch_dispatch(const DispatchArgs& a, cudaStream_t stream);
// quant.cu: quantises bf16 rows [rows, hidden] and dispatches them in one kernel (payload rows
// go to payload_out; `payload` is not read).  Needs hidden % 128 == 0 and 16-byte aligned rows.
bool quantize_dispatch_supported(const uint16_t* in, const DispatchArgs& a);
glmrt_status_t launch_quantize_dispatch(const uint16_t* in, const DispatchArgs& a, cudaStream_t stream);

// ---- ep.cu (expert-parallel exchange over peer memory) ----
constexpr int kEpMaxExperts = 1024;
struct EpControl {
  // written by peers
  int32_t counts_all[kEpMaxWorld * kEpMaxExperts];  // [source rank][global expert] routes
  uint32_t flag_counts[kEpMaxWorld];                 // epoch of the last histogram received from each rank
  uint32_t flag_dispatch[kEpMaxWorld];               // epoch of the last completed row push from each rank
  uint32_t poison_dispatch[kEpMaxWorld];             // epoch in which that rank had no valid plan and pushed nothing
  uint32_t flag_combine[kEpMaxWorld];                // epoch of the last completed result push from each owner
  // local only
  int32_t ticket_select;              // last-CTA tickets of the kernels that end with a publish step
  int32_t ticket_dispatch;
  int32_t ticket_fc2;
  int32_t plan_failed;                // set by any CTA of the push kernel whose plan is invalid
};
struct EpArgs {
  int world, rank, experts;
  int chunk_tokens;              // work-item size of this step (decides the slot layout, see expert_slot_span)
  uint32_t epoch;
  EpControl* ctrl;
  uint32_t* counters;
  EpControl* peer_ctrl[kEpMaxWorld];
  uint8_t* peer_act_codes[kEpMaxWorld];
  uint8_t* peer_act_sf[kEpMaxWorld];
  uint8_t* peer_act_sf_rows[kEpMaxWorld];   // row-major scale staging of prefill-sized pushes
  uint16_t** peer_slot_out[kEpMaxWorld];
  uint16_t* my_rows_in_peer[kEpMaxWorld];   // this rank's route_rows as addressed from each peer
};
// Histogram publish of a rank without rows (the ranks with rows publish from the router's tail).
glmrt_status_t launch_ep_count(const EpArgs& a, const uint32_t* topk_indices, int routes, cudaStream_t stream);
RouterCountTail ep_count_tail(const EpArgs& a);
// Waits for every rank's histogram, derives the slot layout, quantises this rank's rows (or takes
// their payload rows when `hidden` is null) and stores each route's row into its owner's slot
// buffers; CTA 0 also writes this rank's own work-item list; the last CTA raises the "dispatch" flag.
glmrt_status_t launch_ep_plan_dispatch(const EpArgs& a, const PlanArgs& p, const uint16_t* hidden, uint8_t* payload,
                                       int rows, int top_k, int hidden_dim, cudaStream_t stream);
// Flags another kernel waits on before it touches what peers have written / raises when it is done.
struct EpWait {
  const uint32_t* flags = nullptr;    // [world], nullptr: nothing to wait for
  const uint32_t* poison = nullptr;   // [world] or nullptr
  int world = 0;
  uint32_t epoch = 0;
};
struct EpSignal {
  uint32_t* peer_flags[kEpMaxWorld];  // this rank's flag at each rank
  int32_t* ticket = nullptr;          // nullptr: nothing to signal
  int world = 0;
  uint32_t epoch = 0;
};
glmrt_status_t launch_ep_wait(const EpWait& w, uint32_t* error_word, uint32_t* chunk_count, cudaStream_t stream);
glmrt_status_t launch_ep_signal(const EpSignal& s, const uint32_t* error_word, cudaStream_t stream);
// Prefill-sized steps: the home ranks push each slot's scale bytes as one contiguous row (a few
// full lines over NVLink instead of a hundred 4-byte words); the owner waits for the pushes and
// moves the rows of its occupied slots into the tiled layout the GEMM reads.
glmrt_status_t launch_ep_retile_scales(const EpArgs& a, const uint8_t* sf_rows, uint8_t* sf_tiled, int kblocks,
                                       const uint32_t* counters, uint32_t* error_word, uint32_t* chunk_count,
                                       cudaStream_t stream);
EpWait ep_wait_dispatch(const EpArgs& a);
EpWait ep_wait_combine(const EpArgs& a);
EpSignal ep_signal_combine(const EpArgs& a);

// ---- combine.cu ----
// residual / shared (optional, [rows, hidden] bf16): fold the routed sum into the layer output,
// out = bf16(residual + bf16(shared + routed)), instead of storing it.
struct EpWait;
glmrt_status_t launch_combine_routes(const uint16_t* route_rows, const float* topk_weights,
                                     const int32_t* route_slot, uint16_t* out, int rows, int top_k, int hidden,
                                     cudaStream_t stream, const uint16_t* residual = nullptr,
                                     const uint16_t* shared = nullptr, const EpWait* wait = nullptr,
                                     uint32_t* error_word = nullptr);

// ---- residual.cu ----
glmrt_status_t launch_bf16_rows_to_fp8_row_scaled(const uint16_t* src, uint8_t* dst, size_t rows, size_t row_width,
                                                  size_t dst_row_stride_bytes, cudaStream_t stream);

// ---- layer.cu: entry used by the ExpertProtocolV2 executor (protocol_v2.cu) ----
struct LayerDims { uint32_t hidden, experts, top_k, max_tokens, ep_world, ep_rank; };
glmrt_status_t layer_dims(void* layer, LayerDims* out);
// Forgets a streamed request that is still pending on this layer handle (called when the handle dies).
void drop_stream_session(void* layer);
// Runs `rows` host rows (bf16, or NVFP4 payload rows when hidden_is_payload) with host route tables
// [rows, top_k] (expert kNoRoute = none) through the layer and writes bf16 rows, or NVFP4 payload
// rows in the native rounding rule (out_kind 1) or row-scaled FP8 rows (out_kind 2), to host memory.
// Synchronises the stream and reports the device error word.
enum { kOutBf16 = 0, kOutNvfp4Payload = 1, kOutFp8RowScaled = 2 };
glmrt_status_t layer_execute_host_rows(void* layer, const void* hidden_host, bool hidden_is_payload, size_t hidden_stride,
                                       size_t rows, const uint32_t* idx_host, const float* w_host, int out_kind,
                                       void* out_host, size_t out_stride, cudaStream_t stream);

// ---- ffn_simt.cu (verification engine) ----
struct FfnArgs {
  // weights of local experts, stacked
  const uint8_t* gate_codes; const uint8_t* up_codes; const uint8_t* down_codes;   // [E_l*I, H/2] x2, [E_l*H, I/2]
  const uint8_t* gate_sf; const uint8_t* up_sf; const uint8_t* down_sf;            // tiled scales
  const float* scale2;                                                                // [E_l][3]
  const uint8_t* act1_codes; const uint8_t* act1_sf;                                   // dispatch output
  uint8_t* act2_codes; uint8_t* act2_sf;                                               // FC1 output
  uint16_t* const* slot_out;                                                           // FC2 destination rows
  const uint32_t* slot_weight = nullptr;   // non-null: FC2 adds weight * row into the destination (fused combine)
  const Chunk* chunks; const uint32_t* counters;
  int hidden, inter, max_chunks, chunk_tokens;
  uint32_t* error_word;
  // expert-parallel path: FC1 waits for the rows its peers push, FC2 tells the home ranks when its
  // result rows have been stored
  EpWait wait;
  EpSignal signal;
  // Decode kernels: FC2 starts on the SMs FC1 has left while FC1's last tiles still run.  Word 0 is
  // FC2's next-tile counter, words kFcSyncHeader + c count the FC1 epilogue warps that have stored
  // work item c's intermediate rows (4 per feature tile); both are cleared by the route plan.
  // nullptr: FC2 starts when FC1 has completed, as every other kernel pair does.
  uint32_t* fc_sync = nullptr;
};
constexpr int kFcSyncHeader = 8;
glmrt_status_t launch_fc1_simt(const FfnArgs& a, cudaStream_t stream);
glmrt_status_t launch_fc2_simt(const FfnArgs& a, cudaStream_t stream);

// ---- gemm_tc.cu (tcgen05 engine) ----
struct TensorMaps {
  CUtensorMap gate, up, down;   // weight codes, 128-row boxes
  CUtensorMap act1, act2;       // activation codes (box rows = chunk_tokens)
  CUtensorMap act1_sf, gate_sf, up_sf, act2_sf, down_sf;   // tiled scales seen as rows of 128 bytes, 2 KB boxes (CTA-pair kernels)
};
// Encodes a 2D uint8 tensor map [rows, row_bytes] with a {128 B, box_rows} box and 128-byte swizzle.
glmrt_status_t make_codes_tensor_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes,
                                     uint32_t box_rows);
// Encodes a byte range as [bytes / 128, 128] with a {128 B, 16 rows} box and no swizzle: one box = 2 KB of scale tiles.
glmrt_status_t make_scale_tensor_map(CUtensorMap* out, const void* base, uint64_t bytes);
glmrt_status_t launch_fc1_tc(const FfnArgs& a, const TensorMaps& maps, int sm_count, cudaStream_t stream);
glmrt_status_t launch_fc2_tc(const FfnArgs& a, const TensorMaps& maps, int sm_count, cudaStream_t stream);
// gemm_tc_prefill.cu: 128-token chunks, tokens on the MMA rows
glmrt_status_t launch_fc1_tc_prefill(const FfnArgs& a, const TensorMaps& maps, int sm_count, cudaStream_t stream);
glmrt_status_t launch_fc2_tc_prefill(const FfnArgs& a, const TensorMaps& maps, int sm_count, cudaStream_t stream);
// gemm_tc_pair.cu: 256-token chunks on CTA pairs (the one-CTA kernels above take such a chunk as
// two halves of 128, so either GEMM of a 256-slot plan may run on either kind of kernel)
bool pair_tiles_supported(const FfnArgs& a, int sm_count);
glmrt_status_t launch_fc1_tc_pair(const FfnArgs& a, const TensorMaps& maps, int sm_count, cudaStream_t stream);
glmrt_status_t launch_fc2_tc_pair(const FfnArgs& a, const TensorMaps& maps, int sm_count, cudaStream_t stream);

}  // namespace glmrt
