// Layer object: owns the NVFP4 expert weights of one sparse layer in tensor-core layout and all
// work buffers, and sequences the kernels of one forward pass.
//
// It stands where the reference has RealNvfp4ProtocolV2Executor (resident expert preload:
// rust/crates/glmrt-daemon/src/commands/expertd.rs:246-259, route.rs:2793-3054; per-request
// execution: expert_probe/protocol_v2_executor.rs:1882-2493) plus the coordinator's router and
// activation quantiser.
//
// A layer handle joins two blocks of device memory with separate lifetimes: the WEIGHTS of its
// local experts (with the router) and a WORKSPACE (route tables, slot-ordered operands, result rows,
// exchange buffers and flags).  glmrt_b200_moe_layer_create makes both.  A lane
// (glmrt_b200_moe_layer_create_lane) shares the weights of an existing layer and owns a fresh
// workspace, so several host threads / streams can run the same experts at once, as the
// reference's executor does with one route-tensor cache per execution lane
// (expert_probe/protocol_v2_executor.rs:123-126,674-690; at most 8 lanes,
// rust/crates/glmrt-transport/src/host_batch_set.rs:52).  A stacked layer
// (glmrt_b200_moe_layer_create_stacked) owns its weights and shares the workspace of another
// layer of the same shape: the 75 sparse layers of a model run one after another on one stream
// and need one workspace between them.  One handle is driven by one host thread at a time;
// handles that share a workspace must be used on one stream, in order.
#include <cstdlib>
#include <cstring>
#include <memory>
#include <new>
#include <vector>

#include "common.cuh"
#include "internal.h"

namespace glmrt {
namespace {

// Device allocations (and peer mappings) that live and die together.
struct Block {
  std::vector<void*> allocations;
  std::vector<void*> ipc_mappings;
  ~Block() {
    for (void* p : ipc_mappings) cudaIpcCloseMemHandle(p);
    for (void* p : allocations) cudaFree(p);
  }
};

// Expert-parallel exchange state of one workspace (shared by every handle on that workspace: the
// epoch must grow across all of them).
struct EpState {
  EpArgs args{};
  bool attached = false;
  uint32_t epoch = 0;
  uint32_t global_rows = 0;   // rows of the whole batch over all ranks when the caller has said so, else 0
};

struct Layer {
  glmrt_b200_moe_config_t cfg{};
  int device = 0;
  int sm_count = 0;
  int local_experts = 0;
  int max_slots = 0;
  int max_chunks = 0;
  bool have_sf_maps = false;   // the scale arrays are whole 2 KB groups: the CTA-pair FC1 kernel may run
  std::shared_ptr<Block> weights_block, work_block;
  std::shared_ptr<EpState> eps;
  // weights (local experts stacked)
  uint8_t *gate_codes = nullptr, *up_codes = nullptr, *down_codes = nullptr;
  uint8_t *gate_sf = nullptr, *up_sf = nullptr, *down_sf = nullptr;
  float* scale2 = nullptr;
  float *router_w = nullptr, *router_b = nullptr;
  uint16_t* router_w3 = nullptr;   // [experts, 3 * hidden] bf16 split of router_w for the tensor-core router
  CUtensorMap map_w3{};
  bool have_w3 = false;
  float* logits_partial = nullptr;  // [splits][rows][experts] partial logits (tensor-core router, rows below one wave of tiles)
  size_t logits_partial_floats = 0;
  // work buffers
  float *logits = nullptr, *topk_w = nullptr, *topk_scores = nullptr;
  uint32_t* topk_idx = nullptr;
  uint8_t* payload = nullptr;
  int32_t *route_slot = nullptr, *slot_route = nullptr, *expert_counts = nullptr, *expert_base = nullptr,
          *block_hist = nullptr;
  Chunk* chunks = nullptr;
  uint32_t* counters = nullptr;
  uint8_t *act1_codes = nullptr, *act1_sf = nullptr, *act2_codes = nullptr, *act2_sf = nullptr;
  uint16_t* route_rows = nullptr;
  uint16_t** slot_out = nullptr;
  uint32_t* slot_weight = nullptr;   // route weight per slot (fused combine of large batches)
  uint32_t* fc_sync = nullptr;       // hand-over words between the decode FC1 and FC2 kernels
  uint16_t *hidden_stage = nullptr, *out_stage = nullptr;
  // scratch for weight loading
  float* wtmp = nullptr;
  uint8_t* sftmp = nullptr;
  uint32_t* amax_tmp = nullptr;
  TensorMaps maps32{}, maps128{};
  bool have_maps = false;
  uint32_t launches_last = 0;
  uint32_t last_rows = 0;
  // optional per-stage timing of the last forward (events recorded on the caller's stream)
  bool profiling = false;
  cudaEvent_t stage_events[GLMRT_B200_STAGE_COUNT + 1] = {};
  bool stage_valid = false;
  // expert-parallel exchange (control block and scale staging in the workspace)
  EpControl* ep_ctrl = nullptr;
  uint8_t* act1_sf_rows = nullptr;
};

void mark(Layer* l, int stage_begin, cudaStream_t s) {
  if (l->profiling) cudaEventRecord(l->stage_events[stage_begin], s);
}

size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }

template <typename T>
glmrt_status_t dev_alloc(Block* b, T** out, size_t count, bool zero = false) {
  void* p = nullptr;
  const size_t bytes = round_up(count * sizeof(T), 256);
  cudaError_t err = cudaMalloc(&p, bytes);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return fail_cuda(GLMRT_STATUS_ALLOCATION_FAILED, "cudaMalloc (layer buffer)", err);
  }
  b->allocations.push_back(p);
  if (zero) cudaMemset(p, 0, bytes);
  *out = static_cast<T*>(p);
  return GLMRT_STATUS_OK;
}

void destroy(Layer* l) {
  for (cudaEvent_t e : l->stage_events)
    if (e != nullptr) cudaEventDestroy(e);
  delete l;   // the blocks free their memory when the last handle that shares them goes
}

bool local_expert(const Layer* l, uint32_t e) { return e % l->cfg.ep_world == l->cfg.ep_rank; }

glmrt_status_t check_buf(const glmrt_device_buffer_t& b, size_t need, const char* what) {
  if (b.ptr == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, std::string(what) + ": null buffer");
  if (b.bytes < need) return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, std::string(what) + ": buffer too small");
  return GLMRT_STATUS_OK;
}

// Seeded synthetic weights: N(0, std) from a counter-based generator (one Box-Muller pair per
// two elements), so any expert can be regenerated independently of the others.
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}
__global__ void synth_normal_kernel(float* out, size_t n, uint64_t stream_key, float std) {
  const size_t i = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 2;
  if (i >= n) return;
  const uint64_t r = mix64(stream_key ^ mix64(i));
  const float u1 = (static_cast<float>(static_cast<uint32_t>(r >> 40)) + 1.0f) * (1.0f / 16777216.0f);
  const float u2 = static_cast<float>(static_cast<uint32_t>(r) >> 8) * (1.0f / 16777216.0f);
  const float rad = sqrtf(-2.0f * logf(u1)) * std;
  float s, c;
  sincospif(2.0f * u2, &s, &c);
  out[i] = rad * c;
  if (i + 1 < n) out[i + 1] = rad * s;
}

glmrt_status_t build_maps(Layer* l) {
  const auto& c = l->cfg;
  const uint64_t wrows_fc1 = static_cast<uint64_t>(l->local_experts) * c.intermediate_dim;
  const uint64_t wrows_fc2 = static_cast<uint64_t>(l->local_experts) * c.hidden_dim;
  for (TensorMaps* m : {&l->maps32, &l->maps128}) {
    const uint32_t box = (m == &l->maps32) ? 32 : 128;
    GLMRT_RETURN_IF_ERROR(make_codes_tensor_map(&m->gate, l->gate_codes, wrows_fc1, c.hidden_dim / 2, 128));
    GLMRT_RETURN_IF_ERROR(make_codes_tensor_map(&m->up, l->up_codes, wrows_fc1, c.hidden_dim / 2, 128));
    GLMRT_RETURN_IF_ERROR(make_codes_tensor_map(&m->down, l->down_codes, wrows_fc2, c.intermediate_dim / 2, 128));
    GLMRT_RETURN_IF_ERROR(make_codes_tensor_map(&m->act1, l->act1_codes, l->max_slots, c.hidden_dim / 2, box));
    GLMRT_RETURN_IF_ERROR(make_codes_tensor_map(&m->act2, l->act2_codes, l->max_slots, c.intermediate_dim / 2, box));
    const uint64_t sf_fc1 = wrows_fc1 * (c.hidden_dim / 16);
    const uint64_t sf_fc2 = wrows_fc2 * (c.intermediate_dim / 16);
    const uint64_t sf_act1 = static_cast<uint64_t>(l->max_slots) * (c.hidden_dim / 16);
    const uint64_t sf_act2 = static_cast<uint64_t>(l->max_slots) * (c.intermediate_dim / 16);
    if (sf_fc1 % 2048 == 0 && sf_act1 % 2048 == 0 && sf_fc2 % 2048 == 0 && sf_act2 % 2048 == 0) {
      GLMRT_RETURN_IF_ERROR(make_scale_tensor_map(&m->gate_sf, l->gate_sf, sf_fc1));
      GLMRT_RETURN_IF_ERROR(make_scale_tensor_map(&m->up_sf, l->up_sf, sf_fc1));
      GLMRT_RETURN_IF_ERROR(make_scale_tensor_map(&m->act1_sf, l->act1_sf, sf_act1));
      GLMRT_RETURN_IF_ERROR(make_scale_tensor_map(&m->down_sf, l->down_sf, sf_fc2));
      GLMRT_RETURN_IF_ERROR(make_scale_tensor_map(&m->act2_sf, l->act2_sf, sf_act2));
      l->have_sf_maps = true;
    }
  }
  l->have_maps = true;
  return GLMRT_STATUS_OK;
}

// batch_rows: rows of the whole batch (over all ranks where known).  The FC1 -> FC2 overlap of the
// decode kernels pays from about eight rows on (64 routes); below that FC2's tile scheduling costs
// more than the overlap saves (measured at one row: +1.3 us on 67), so tiny batches run the plain pair.
// How many (work item, 128-row tile) pairs of FC1's weights a decode-sized step asks into the L2
// while its rows are quantised and dispatched: GLMRT_B200_PREFETCH_FC1, default 48 (38 MB of the
// GLM-5.2 shape; measured at 1 / 64 rows: 32 pairs -2.7 / -2 us, 64 pairs -1.6 / -8 us, 128 pairs
// +5 / -10 us of 62 / 751 us); 0 turns it off.
int prefetch_tiles_fc1() {
  static const int n = [] {
    const char* v = std::getenv("GLMRT_B200_PREFETCH_FC1");
    if (v == nullptr || *v == '\0') return 48;
    const long x = std::strtol(v, nullptr, 10);
    return static_cast<int>(x < 0 ? 0 : x > 1024 ? 1024 : x);
  }();
  return n;
}
WeightPrefetch fc1_prefetch(const Layer* l, int chunk_tokens) {
  const auto& c = l->cfg;
  WeightPrefetch w;
  if (chunk_tokens == 32 && !(c.flags & GLMRT_B200_LAYER_ENGINE_SIMT) && c.intermediate_dim % 128 == 0 &&
      c.hidden_dim % 256 == 0 && prefetch_tiles_fc1() > 0) {
    w.w0 = l->gate_codes; w.w1 = l->up_codes; w.sf0 = l->gate_sf; w.sf1 = l->up_sf;
    w.rows_per_expert = static_cast<int>(c.intermediate_dim);
    w.row_bytes = static_cast<int>(c.hidden_dim / 2);
    w.tiles = prefetch_tiles_fc1();
  }
  return w;
}

FfnArgs ffn_args(const Layer* l, int chunk_tokens, size_t batch_rows) {
  FfnArgs a{};
  a.gate_codes = l->gate_codes; a.up_codes = l->up_codes; a.down_codes = l->down_codes;
  a.gate_sf = l->gate_sf; a.up_sf = l->up_sf; a.down_sf = l->down_sf;
  a.scale2 = l->scale2;
  a.act1_codes = l->act1_codes; a.act1_sf = l->act1_sf;
  a.act2_codes = l->act2_codes; a.act2_sf = l->act2_sf;
  a.slot_out = l->slot_out;
  a.chunks = l->chunks; a.counters = l->counters;
  a.hidden = static_cast<int>(l->cfg.hidden_dim); a.inter = static_cast<int>(l->cfg.intermediate_dim);
  a.max_chunks = l->max_chunks; a.chunk_tokens = chunk_tokens;
  a.error_word = l->counters + kCntError;
  a.fc_sync = chunk_tokens == 32 && batch_rows * l->cfg.top_k >= 64 && !(l->cfg.flags & GLMRT_B200_LAYER_ENGINE_SIMT)
                  ? l->fc_sync : nullptr;
  return a;
}

// Router: tensor-core logits for prefill-sized batches, SIMT kernels otherwise.
glmrt_status_t run_router(Layer* l, const void* hidden, size_t rows, cudaStream_t s,
                          const RouterCountTail* tail = nullptr) {
  const auto& c = l->cfg;
  if (l->have_w3 && router_tc_supported(rows, c.hidden_dim, c.experts, hidden)) {
    int splits = router_tc_splits(rows, c.hidden_dim, c.experts, l->sm_count);
    if (static_cast<size_t>(splits) * rows * c.experts > l->logits_partial_floats) splits = 1;
    float* table = splits > 1 ? l->logits_partial : l->logits;
    GLMRT_RETURN_IF_ERROR(launch_router_logits_tc(static_cast<const uint16_t*>(hidden), l->map_w3, table, rows,
                                                  c.hidden_dim, c.experts, l->counters + kCntRouterError,
                                                  l->sm_count, s, splits));
    return launch_router_select(table, l->router_b, l->topk_idx, l->topk_scores, l->topk_w, rows, c.experts,
                                c.top_k, c.routed_scaling, s, splits, tail);
  }
  return launch_router(hidden, true, l->router_w, false, l->router_b, l->logits, l->topk_idx, l->topk_scores,
                       l->topk_w, rows, c.hidden_dim, c.experts, c.top_k, c.routed_scaling, s, tail);
}

PlanArgs plan_args(const Layer* l, size_t rows, int chunk_tokens) {
  const auto& c = l->cfg;
  PlanArgs p{};
  p.topk_indices = l->topk_idx;
  p.rows = static_cast<int>(rows); p.top_k = static_cast<int>(c.top_k); p.experts = static_cast<int>(c.experts);
  p.ep_world = static_cast<int>(c.ep_world); p.ep_rank = static_cast<int>(c.ep_rank);
  p.chunk_tokens = chunk_tokens; p.max_slots = l->max_slots; p.max_chunks = l->max_chunks;
  p.route_slot = l->route_slot; p.slot_route = l->slot_route; p.expert_counts = l->expert_counts;
  p.expert_base = l->expert_base; p.block_hist = l->block_hist;
  p.chunks = l->chunks; p.counters = l->counters;
  p.fc_sync = chunk_tokens == 32 ? l->fc_sync : nullptr;
  return p;
}

// Decode-sized batches on one GPU: the route plan runs as the tail of the router's selection kernel.
bool plan_in_router_tail(const Layer* l, size_t rows) { return rows <= 256 && l->cfg.ep_world == 1; }

// Router followed by the routed path, for the entry points that route themselves.
glmrt_status_t run_routed(Layer* l, const uint16_t* hidden, size_t rows, uint16_t* out, cudaStream_t stream,
                          const uint16_t* residual = nullptr, const uint16_t* shared = nullptr, bool plan_done = false);
glmrt_status_t run_router_and_routed(Layer* l, const uint16_t* hidden, size_t rows, uint16_t* out, cudaStream_t s,
                                     const uint16_t* residual = nullptr, const uint16_t* shared = nullptr) {
  mark(l, GLMRT_B200_STAGE_ROUTER, s);
  const bool tail_plan = plan_in_router_tail(l, rows);
  if (tail_plan) {
    RouterCountTail tail{};
    tail.do_plan = 1;
    tail.plan = plan_args(l, rows, 32);
    tail.ticket = reinterpret_cast<int32_t*>(l->counters + kCntTicket);
    GLMRT_RETURN_IF_ERROR(run_router(l, hidden, rows, s, &tail));
  } else {
    GLMRT_RETURN_IF_ERROR(run_router(l, hidden, rows, s));
  }
  return run_routed(l, hidden, rows, out, s, residual, shared, tail_plan);
}

// Everything after the router: quantise, plan, dispatch, expert FFN, combine.
// `hidden` == nullptr: the payload rows are already in l->payload (a request that carried NVFP4 rows).
// plan_done: the route plan has already been made (by the router's tail).
glmrt_status_t run_routed(Layer* l, const uint16_t* hidden, size_t rows, uint16_t* out, cudaStream_t stream,
                          const uint16_t* residual, const uint16_t* shared, bool plan_done) {
  const auto& c = l->cfg;
  // Work-item size: 32 slots for decode batches (weights on the MMA rows), 128 for prefill (tokens
  // on the MMA rows); on request 256 (GEMMs on CTA pairs) once the average expert receives more than
  // 192 routes, i.e. when most 256-slot items are better than half full.
  int chunk_tokens = rows <= 256 ? 32 : 128;
  if (chunk_tokens == 128 && (c.flags & GLMRT_B200_LAYER_PAIR_TILES) && !(c.flags & GLMRT_B200_LAYER_ENGINE_SIMT) &&
      l->sm_count % 2 == 0 && c.hidden_dim % 256 == 0 && c.intermediate_dim % 256 == 0 &&
      rows * c.top_k > static_cast<size_t>(192) * c.experts) {
    if (!l->have_maps) GLMRT_RETURN_IF_ERROR(build_maps(l));
    if (l->have_sf_maps) chunk_tokens = 256;
  }
  DispatchArgs d{};
  d.payload = l->payload; d.payload_out = l->payload; d.route_slot = l->route_slot;
  d.rows = static_cast<int>(rows); d.top_k = static_cast<int>(c.top_k); d.hidden = static_cast<int>(c.hidden_dim);
  d.act_codes = l->act1_codes; d.act_sf = l->act1_sf; d.route_rows = l->route_rows; d.slot_out = l->slot_out;
  d.prefetch = fc1_prefetch(l, chunk_tokens); d.chunks = l->chunks; d.counters = l->counters;
  // The plan needs only the routes, so it runs first and the rows are quantised and dispatched by
  // one kernel (its time is reported as the dispatch stage, the quantise stage then reads 0).
  const bool fused = hidden != nullptr && quantize_dispatch_supported(hidden, d);
  // Large batches with all experts local: the down projection adds weight * row straight into the
  // output rows (no per-route rows, no combine pass).  Batches of at most 256 rows keep the
  // ordered combine: there a row must not depend on its batch, bit for bit.
  const bool fused_combine = fused && chunk_tokens == 128 && c.ep_world == 1 && residual == nullptr && shared == nullptr &&
                             l->slot_weight != nullptr &&
                             !(c.flags & (GLMRT_B200_LAYER_ENGINE_SIMT | GLMRT_B200_LAYER_ORDERED_COMBINE));
  if (fused_combine) {
    d.combine_out = out;
    d.topk_weights = l->topk_w;
    d.slot_weight = l->slot_weight;
    cudaError_t zerr = cudaMemsetAsync(out, 0, rows * static_cast<size_t>(c.hidden_dim) * 2, stream);
    if (zerr != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "clear the output rows", zerr);
  }
  mark(l, GLMRT_B200_STAGE_QUANTIZE, stream);
  if (!fused && hidden != nullptr)
    GLMRT_RETURN_IF_ERROR(launch_quantize_rows_payload(hidden, l->payload, rows, c.hidden_dim,
                                                       GLMRT_B200_FP4_RULE_NEAREST_LOW, stream));
  mark(l, GLMRT_B200_STAGE_PLAN, stream);
  if (!plan_done) GLMRT_RETURN_IF_ERROR(launch_route_plan(plan_args(l, rows, chunk_tokens), stream));
  mark(l, GLMRT_B200_STAGE_DISPATCH, stream);
  GLMRT_RETURN_IF_ERROR(fused ? launch_quantize_dispatch(hidden, d, stream) : launch_dispatch(d, stream));
  FfnArgs f = ffn_args(l, chunk_tokens, rows);
  if (fused_combine) f.slot_weight = l->slot_weight;
  mark(l, GLMRT_B200_STAGE_FC1, stream);
  if (c.flags & GLMRT_B200_LAYER_ENGINE_SIMT) {
    GLMRT_RETURN_IF_ERROR(launch_fc1_simt(f, stream));
    mark(l, GLMRT_B200_STAGE_FC2, stream);
    GLMRT_RETURN_IF_ERROR(launch_fc2_simt(f, stream));
  } else {
    if (!l->have_maps) GLMRT_RETURN_IF_ERROR(build_maps(l));
    const TensorMaps& maps = chunk_tokens == 32 ? l->maps32 : l->maps128;
    const bool pair1 = chunk_tokens == 256 && (c.flags & GLMRT_B200_LAYER_PAIR_FC1);
    const bool pair2 = chunk_tokens == 256 && (c.flags & GLMRT_B200_LAYER_PAIR_FC2);
    GLMRT_RETURN_IF_ERROR(chunk_tokens == 32 ? launch_fc1_tc(f, maps, l->sm_count, stream)
                          : pair1            ? launch_fc1_tc_pair(f, maps, l->sm_count, stream)
                                             : launch_fc1_tc_prefill(f, maps, l->sm_count, stream));
    mark(l, GLMRT_B200_STAGE_FC2, stream);
    GLMRT_RETURN_IF_ERROR(chunk_tokens == 32 ? launch_fc2_tc(f, maps, l->sm_count, stream)
                          : pair2            ? launch_fc2_tc_pair(f, maps, l->sm_count, stream)
                                             : launch_fc2_tc_prefill(f, maps, l->sm_count, stream));
  }
  mark(l, GLMRT_B200_STAGE_COMBINE, stream);
  // routes without a slot (another shard's expert, a "no route" entry, a refused plan) are skipped
  const int32_t* mask = l->route_slot;
  if (!fused_combine)
    GLMRT_RETURN_IF_ERROR(launch_combine_routes(l->route_rows, l->topk_w, mask, out, static_cast<int>(rows),
                                                static_cast<int>(c.top_k), static_cast<int>(c.hidden_dim), stream,
                                                residual, shared));
  mark(l, GLMRT_B200_STAGE_COUNT, stream);
  l->stage_valid = l->profiling;
  l->last_rows = static_cast<uint32_t>(rows);
  return GLMRT_STATUS_OK;
}

glmrt_status_t validate_forward(Layer* l, size_t rows) {
  if (l == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer is null");
  if (rows == 0 || rows > l->cfg.max_tokens)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward: rows must be in 1..max_tokens");
  return GLMRT_STATUS_OK;
}

}  // namespace
}  // namespace glmrt

using namespace glmrt;

namespace glmrt {
namespace {

glmrt_status_t validate_config(const glmrt_b200_moe_config_t& c) {
  if (c.hidden_dim == 0 || c.hidden_dim % 256 != 0 || c.intermediate_dim == 0 || c.intermediate_dim % 256 != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer create: hidden_dim and intermediate_dim must be positive multiples of 256");
  if (c.experts == 0 || c.experts > 1024 || c.top_k == 0 || c.top_k > 16 || c.top_k > c.experts)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer create: experts must be 1..1024 and top_k 1..min(16, experts)");
  if (c.max_tokens == 0 || c.max_tokens > (1u << 20))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer create: max_tokens must be 1..1048576");
  if (c.ep_world == 0 || c.ep_rank >= c.ep_world || c.ep_world > c.experts || c.ep_world > kEpMaxWorld)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer create: need 0 <= ep_rank < ep_world <= min(experts, 8)");
  if (!(c.routed_scaling > 0.0f)) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer create: routed_scaling must be positive");
  return GLMRT_STATUS_OK;
}

// Geometry every handle derives from its configuration alone.
void set_geometry(Layer* l) {
  const auto& c = l->cfg;
  cudaGetDevice(&l->device);
  cudaDeviceGetAttribute(&l->sm_count, cudaDevAttrMultiProcessorCount, l->device);
  l->local_experts = static_cast<int>((c.experts - c.ep_rank + c.ep_world - 1) / c.ep_world);
  const size_t E = l->local_experts, T = c.max_tokens, K = c.top_k;
  // Routes this shard's experts may receive in one step.  With all experts local that is T * K.  An
  // expert-parallel shard receives T * K when the routing is balanced and up to world times that
  // when every route of every rank goes to its experts; it is sized for twice the balanced load
  // (popularity ~ rank^-1.2 with the hot experts spread over the ranks gives 1.6), beyond which a
  // step is refused with kErrSlotOverflow.
  const size_t routes = c.ep_world > 1 ? T * K * std::min<size_t>(2, c.ep_world) : T * K;
  // Dense work items (128 / 256 slots): every expert's range is rounded up to 128 slots.  Batches of
  // at most 256 rows use 32-slot work items, each in a 128-slot group of its own (expert_slot_span).
  // (a decode-sized batch is small enough to provide for all of it landing on one shard)
  const size_t decode_routes = std::min<size_t>(T * c.ep_world, 256) * K;
  const size_t decode_slots = 128 * (std::min(E, decode_routes) + decode_routes / 32 + 1);
  l->max_slots = static_cast<int>(std::max(round_up(routes + E * 127, 128), decode_slots));
  l->max_chunks = static_cast<int>(E + (routes + 31) / 32);
}

glmrt_status_t alloc_weights(Layer* l) {
  const auto& c = l->cfg;
  l->weights_block = std::make_shared<Block>();
  Block* b = l->weights_block.get();
  const size_t H = c.hidden_dim, I = c.intermediate_dim, E = l->local_experts;
  glmrt_status_t st = GLMRT_STATUS_OK;
  auto A = [&](glmrt_status_t s) { if (st == GLMRT_STATUS_OK) st = s; };
  A(dev_alloc(b, &l->gate_codes, E * I * H / 2));
  A(dev_alloc(b, &l->up_codes, E * I * H / 2));
  A(dev_alloc(b, &l->down_codes, E * H * I / 2));
  A(dev_alloc(b, &l->gate_sf, E * I * H / 16));
  A(dev_alloc(b, &l->up_sf, E * I * H / 16));
  A(dev_alloc(b, &l->down_sf, E * H * I / 16));
  A(dev_alloc(b, &l->scale2, E * 3, true));
  A(dev_alloc(b, &l->router_w, static_cast<size_t>(c.experts) * H, true));
  A(dev_alloc(b, &l->router_b, c.experts, true));
  A(dev_alloc(b, &l->router_w3, static_cast<size_t>(c.experts) * 3 * H, true));
  l->have_w3 = false;
  // the tensor-core router reads the split weight through a tensor map (lanes made later inherit it)
  if (st == GLMRT_STATUS_OK && c.experts % 128 == 0 && c.hidden_dim % 64 == 0) {
    st = make_codes_tensor_map(&l->map_w3, l->router_w3, c.experts, static_cast<uint64_t>(c.hidden_dim) * 3 * 2, 128);
    l->have_w3 = st == GLMRT_STATUS_OK;
  }
  return st;
}

glmrt_status_t alloc_workspace(Layer* l) {
  const auto& c = l->cfg;
  l->work_block = std::make_shared<Block>();
  l->eps = std::make_shared<EpState>();
  Block* b = l->work_block.get();
  const size_t H = c.hidden_dim, I = c.intermediate_dim, E = l->local_experts, T = c.max_tokens, K = c.top_k;
  const size_t routes = T * K;
  glmrt_status_t st = GLMRT_STATUS_OK;
  auto A = [&](glmrt_status_t s) { if (st == GLMRT_STATUS_OK) st = s; };
  A(dev_alloc(b, &l->logits, T * c.experts));
  A(dev_alloc(b, &l->topk_w, routes));
  A(dev_alloc(b, &l->topk_scores, routes));
  A(dev_alloc(b, &l->topk_idx, routes));
  A(dev_alloc(b, &l->payload, T * (H / 2 + H / 16)));
  A(dev_alloc(b, &l->route_slot, routes));
  A(dev_alloc(b, &l->slot_route, static_cast<size_t>(l->max_slots)));
  A(dev_alloc(b, &l->expert_counts, E));
  A(dev_alloc(b, &l->expert_base, E));
  A(dev_alloc(b, &l->block_hist, ((routes + 255) / 256 + 1) * E));
  A(dev_alloc(b, &l->chunks, static_cast<size_t>(l->max_chunks)));
  A(dev_alloc(b, &l->counters, kCntWords, true));
  A(dev_alloc(b, &l->fc_sync, static_cast<size_t>(kFcSyncHeader) + l->max_chunks, true));
  // slot-ordered operands; zero-filled once so that padding slots hold finite values
  A(dev_alloc(b, &l->act1_codes, static_cast<size_t>(l->max_slots) * H / 2, true));
  A(dev_alloc(b, &l->act1_sf, static_cast<size_t>(l->max_slots) * H / 16, true));
  A(dev_alloc(b, &l->act2_codes, static_cast<size_t>(l->max_slots) * I / 2, true));
  A(dev_alloc(b, &l->act2_sf, static_cast<size_t>(l->max_slots) * I / 16, true));
  A(dev_alloc(b, &l->route_rows, routes * H));
  // destinations start out null: a slot nobody dispatched to is skipped by the FC2 epilogues
  A(dev_alloc(b, &l->slot_out, static_cast<size_t>(l->max_slots), true));
  if (c.max_tokens > 256 && c.ep_world == 1) A(dev_alloc(b, &l->slot_weight, static_cast<size_t>(l->max_slots), true));
  A(dev_alloc(b, &l->hidden_stage, T * H));
  A(dev_alloc(b, &l->out_stage, T * H));
  A(dev_alloc(b, &l->wtmp, std::max(I * H, static_cast<size_t>(1))));
  A(dev_alloc(b, &l->sftmp, I * H / 16));
  A(dev_alloc(b, &l->amax_tmp, 1, true));
  if (c.ep_world > 1) {
    A(dev_alloc(b, &l->ep_ctrl, 1, true));
    A(dev_alloc(b, &l->act1_sf_rows, static_cast<size_t>(l->max_slots) * H / 16, true));
  }
  // partial logits of the tensor-core router: largest splits * rows over the batch sizes this
  // workspace can see (splits * tiles <= SM count)
  l->logits_partial = nullptr;
  l->logits_partial_floats = 0;
  if (c.max_tokens > 128 && c.experts % 128 == 0 && c.hidden_dim % 64 == 0) {
    size_t need = 0;
    for (size_t rows = 129; rows <= c.max_tokens; rows += 128) {
      const size_t r = std::min<size_t>(rows + 127, c.max_tokens);
      const int sp = router_tc_splits(r, c.hidden_dim, c.experts, l->sm_count);
      if (sp > 1) need = std::max(need, static_cast<size_t>(sp) * r * c.experts);
    }
    if (need != 0) {
      A(dev_alloc(b, &l->logits_partial, need));
      if (st == GLMRT_STATUS_OK) l->logits_partial_floats = need;
    }
  }
  return st;
}

// Per-handle state that must not be inherited when a handle is cloned.
void reset_instance_state(Layer* l) {
  l->have_maps = false;
  l->have_sf_maps = false;
  l->launches_last = 0;
  l->last_rows = 0;
  l->profiling = false;
  l->stage_valid = false;
  for (cudaEvent_t& e : l->stage_events) e = nullptr;
}

bool same_shape(const glmrt_b200_moe_config_t& a, const glmrt_b200_moe_config_t& b) {
  return a.hidden_dim == b.hidden_dim && a.intermediate_dim == b.intermediate_dim && a.experts == b.experts &&
         a.top_k == b.top_k && a.max_tokens == b.max_tokens && a.ep_world == b.ep_world && a.ep_rank == b.ep_rank;
}

}  // namespace
}  // namespace glmrt

extern "C" glmrt_status_t glmrt_b200_moe_layer_create(const glmrt_b200_moe_config_t* config, void** out_layer) {
  if (config == nullptr || out_layer == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer create: null argument");
  *out_layer = nullptr;
  GLMRT_RETURN_IF_ERROR(validate_config(*config));
  GLMRT_RETURN_IF_ERROR(require_cuda());
  Layer* l = new (std::nothrow) Layer();
  if (l == nullptr) return fail(GLMRT_STATUS_ALLOCATION_FAILED, "layer create: out of host memory");
  l->cfg = *config;
  set_geometry(l);
  glmrt_status_t st = alloc_weights(l);
  if (st == GLMRT_STATUS_OK) st = alloc_workspace(l);
  if (st != GLMRT_STATUS_OK) {
    destroy(l);
    return st;
  }
  *out_layer = l;
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_create_lane(void* layer, uint32_t max_tokens, void** out_lane) {
  Layer* parent = static_cast<Layer*>(layer);
  if (parent == nullptr || out_lane == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "create_lane: null argument");
  *out_lane = nullptr;
  if (max_tokens > (1u << 20)) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "create_lane: max_tokens must be at most 1048576");
  int dev = -1;
  cudaGetDevice(&dev);
  if (dev != parent->device) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "create_lane: the layer's device must be current");
  Layer* l = new (std::nothrow) Layer(*parent);   // weight pointers and their block are shared
  if (l == nullptr) return fail(GLMRT_STATUS_ALLOCATION_FAILED, "create_lane: out of host memory");
  reset_instance_state(l);
  if (max_tokens != 0) l->cfg.max_tokens = max_tokens;
  set_geometry(l);
  glmrt_status_t st = alloc_workspace(l);          // replaces every work pointer and the exchange state
  if (st != GLMRT_STATUS_OK) {
    destroy(l);
    return st;
  }
  *out_lane = l;
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_create_stacked(const glmrt_b200_moe_config_t* config,
                                                              void* workspace_layer, void** out_layer) {
  Layer* donor = static_cast<Layer*>(workspace_layer);
  if (config == nullptr || donor == nullptr || out_layer == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "create_stacked: null argument");
  *out_layer = nullptr;
  GLMRT_RETURN_IF_ERROR(validate_config(*config));
  if (!same_shape(*config, donor->cfg))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "create_stacked: the layer must have the shape, max_tokens and shard of the layer whose workspace it shares");
  int dev = -1;
  cudaGetDevice(&dev);
  if (dev != donor->device) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "create_stacked: the donor layer's device must be current");
  Layer* l = new (std::nothrow) Layer(*donor);     // work pointers, their block and the exchange state are shared
  if (l == nullptr) return fail(GLMRT_STATUS_ALLOCATION_FAILED, "create_stacked: out of host memory");
  reset_instance_state(l);
  l->cfg = *config;
  glmrt_status_t st = alloc_weights(l);            // replaces every weight pointer
  if (st != GLMRT_STATUS_OK) {
    destroy(l);
    return st;
  }
  *out_layer = l;
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_destroy(void* layer) {
  if (layer == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer is null");
  cudaDeviceSynchronize();
  drop_stream_session(layer);
  destroy(static_cast<Layer*>(layer));
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_set_router(void* layer, glmrt_device_buffer_t weight_f32,
                                                          glmrt_device_buffer_t bias_f32, void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  if (l == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer is null");
  const size_t wbytes = static_cast<size_t>(l->cfg.experts) * l->cfg.hidden_dim * 4, bbytes = l->cfg.experts * 4;
  GLMRT_RETURN_IF_ERROR(check_buf(weight_f32, wbytes, "set_router weight"));
  GLMRT_RETURN_IF_ERROR(check_buf(bias_f32, bbytes, "set_router bias"));
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t err = cudaMemcpyAsync(l->router_w, weight_f32.ptr, wbytes, cudaMemcpyDeviceToDevice, s);
  if (err == cudaSuccess) err = cudaMemcpyAsync(l->router_b, bias_f32.ptr, bbytes, cudaMemcpyDeviceToDevice, s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "set_router copy", err);
  GLMRT_RETURN_IF_ERROR(launch_split_router_weight(l->router_w, l->router_w3, l->cfg.experts, l->cfg.hidden_dim, s));
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_set_expert(
    void* layer, uint32_t expert_id, glmrt_device_buffer_t gate_codes, glmrt_device_buffer_t gate_scales,
    glmrt_device_buffer_t up_codes, glmrt_device_buffer_t up_scales, glmrt_device_buffer_t down_codes,
    glmrt_device_buffer_t down_scales, float gate_scale_2, float up_scale_2, float down_scale_2, void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  if (l == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer is null");
  if (expert_id >= l->cfg.experts || !local_expert(l, expert_id))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "set_expert: expert is not local to this shard");
  if (!isfinite(gate_scale_2) || !isfinite(up_scale_2) || !isfinite(down_scale_2))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "set_expert: second-level scales must be finite");
  const size_t H = l->cfg.hidden_dim, I = l->cfg.intermediate_dim;
  GLMRT_RETURN_IF_ERROR(check_buf(gate_codes, I * H / 2, "set_expert gate codes"));
  GLMRT_RETURN_IF_ERROR(check_buf(up_codes, I * H / 2, "set_expert up codes"));
  GLMRT_RETURN_IF_ERROR(check_buf(down_codes, H * I / 2, "set_expert down codes"));
  GLMRT_RETURN_IF_ERROR(check_buf(gate_scales, I * H / 16, "set_expert gate scales"));
  GLMRT_RETURN_IF_ERROR(check_buf(up_scales, I * H / 16, "set_expert up scales"));
  GLMRT_RETURN_IF_ERROR(check_buf(down_scales, H * I / 16, "set_expert down scales"));
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const size_t le = expert_id / l->cfg.ep_world;
  cudaError_t err = cudaMemcpyAsync(l->gate_codes + le * I * H / 2, gate_codes.ptr, I * H / 2, cudaMemcpyDeviceToDevice, s);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(l->up_codes + le * I * H / 2, up_codes.ptr, I * H / 2, cudaMemcpyDeviceToDevice, s);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(l->down_codes + le * H * I / 2, down_codes.ptr, H * I / 2, cudaMemcpyDeviceToDevice, s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "set_expert copy", err);
  GLMRT_RETURN_IF_ERROR(launch_tile_scales(static_cast<const uint8_t*>(gate_scales.ptr), l->gate_sf, I, H / 16, le * I, s));
  GLMRT_RETURN_IF_ERROR(launch_tile_scales(static_cast<const uint8_t*>(up_scales.ptr), l->up_sf, I, H / 16, le * I, s));
  GLMRT_RETURN_IF_ERROR(launch_tile_scales(static_cast<const uint8_t*>(down_scales.ptr), l->down_sf, H, I / 16, le * H, s));
  const float s2[3] = {gate_scale_2, up_scale_2, down_scale_2};
  err = cudaMemcpyAsync(l->scale2 + le * 3, s2, sizeof(s2), cudaMemcpyHostToDevice, s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "set_expert scale copy", err);
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_fill_synthetic(void* layer, uint64_t seed, float weight_std,
                                                              void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  if (l == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer is null");
  if (!(weight_std > 0.0f)) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "fill_synthetic: weight_std must be positive");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const size_t H = l->cfg.hidden_dim, I = l->cfg.intermediate_dim, n = I * H;
  const unsigned blocks = static_cast<unsigned>((n / 2 + 255) / 256);
  for (int le = 0; le < l->local_experts; ++le) {
    const uint64_t e = static_cast<uint64_t>(le) * l->cfg.ep_world + l->cfg.ep_rank;  // global expert id
    for (int t = 0; t < 3; ++t) {
      const uint64_t key = seed * 0x100000001b3ull + e * 3 + t + 1;
      synth_normal_kernel<<<blocks, 256, 0, s>>>(l->wtmp, n, key, weight_std);
      GLMRT_LAUNCH_CHECK("synth_normal_kernel");
      uint8_t* codes = t == 0 ? l->gate_codes : t == 1 ? l->up_codes : l->down_codes;
      uint8_t* sf = t == 0 ? l->gate_sf : t == 1 ? l->up_sf : l->down_sf;
      const size_t rows = t == 2 ? H : I, cols = t == 2 ? I : H;
      GLMRT_RETURN_IF_ERROR(launch_quantize_weight_f32(l->wtmp, codes + static_cast<size_t>(le) * n / 2, l->sftmp,
                                                       l->scale2 + le * 3 + t, l->amax_tmp, rows, cols, s));
      GLMRT_RETURN_IF_ERROR(launch_tile_scales(l->sftmp, sf, rows, cols / 16, static_cast<size_t>(le) * rows, s));
    }
  }
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_forward_async(void* layer, glmrt_device_buffer_t hidden_bf16,
                                                             size_t rows, glmrt_device_buffer_t output_bf16,
                                                             glmrt_device_buffer_t topk_indices,
                                                             glmrt_device_buffer_t topk_weights, void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(validate_forward(l, rows));
  if (l->cfg.ep_world != 1)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward: this entry point needs ep_world == 1");
  const size_t row_bytes = static_cast<size_t>(l->cfg.hidden_dim) * 2, routes = rows * l->cfg.top_k;
  GLMRT_RETURN_IF_ERROR(check_buf(hidden_bf16, rows * row_bytes, "forward hidden"));
  GLMRT_RETURN_IF_ERROR(check_buf(output_bf16, rows * row_bytes, "forward output"));
  if (topk_indices.ptr != nullptr && topk_indices.bytes < routes * 4)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "forward topk_indices: buffer too small");
  if (topk_weights.ptr != nullptr && topk_weights.bytes < routes * 4)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "forward topk_weights: buffer too small");
  if (reinterpret_cast<uintptr_t>(hidden_bf16.ptr) % 16 != 0 || reinterpret_cast<uintptr_t>(output_bf16.ptr) % 16 != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward: hidden and output must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const uint64_t before = launches_total();
  GLMRT_RETURN_IF_ERROR(run_router_and_routed(l, static_cast<const uint16_t*>(hidden_bf16.ptr), rows,
                                              static_cast<uint16_t*>(output_bf16.ptr), s));
  l->launches_last = static_cast<uint32_t>(launches_total() - before);
  cudaError_t err = cudaSuccess;
  if (topk_indices.ptr != nullptr)
    err = cudaMemcpyAsync(topk_indices.ptr, l->topk_idx, routes * 4, cudaMemcpyDeviceToDevice, s);
  if (err == cudaSuccess && topk_weights.ptr != nullptr)
    err = cudaMemcpyAsync(topk_weights.ptr, l->topk_w, routes * 4, cudaMemcpyDeviceToDevice, s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "forward route copy", err);
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_forward_residual_async(
    void* layer, glmrt_device_buffer_t hidden_bf16, size_t rows, glmrt_device_buffer_t residual_bf16,
    glmrt_device_buffer_t shared_delta_bf16, glmrt_device_buffer_t output_bf16, void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(validate_forward(l, rows));
  if (l->cfg.ep_world != 1)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_residual: this entry point needs ep_world == 1");
  const size_t row_bytes = static_cast<size_t>(l->cfg.hidden_dim) * 2;
  GLMRT_RETURN_IF_ERROR(check_buf(hidden_bf16, rows * row_bytes, "forward_residual hidden"));
  GLMRT_RETURN_IF_ERROR(check_buf(residual_bf16, rows * row_bytes, "forward_residual residual"));
  GLMRT_RETURN_IF_ERROR(check_buf(output_bf16, rows * row_bytes, "forward_residual output"));
  if (shared_delta_bf16.ptr != nullptr && shared_delta_bf16.bytes < rows * row_bytes)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "forward_residual shared_delta: buffer too small");
  for (const void* p : {hidden_bf16.ptr, residual_bf16.ptr, shared_delta_bf16.ptr, output_bf16.ptr})
    if (reinterpret_cast<uintptr_t>(p) % 16 != 0)
      return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_residual: buffers must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const uint64_t before = launches_total();
  GLMRT_RETURN_IF_ERROR(run_router_and_routed(l, static_cast<const uint16_t*>(hidden_bf16.ptr), rows,
                                              static_cast<uint16_t*>(output_bf16.ptr), s,
                                              static_cast<const uint16_t*>(residual_bf16.ptr),
                                              static_cast<const uint16_t*>(shared_delta_bf16.ptr)));
  l->launches_last = static_cast<uint32_t>(launches_total() - before);
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_forward_routed_async(
    void* layer, glmrt_device_buffer_t hidden_bf16, size_t rows, glmrt_device_buffer_t topk_indices,
    glmrt_device_buffer_t topk_weights, glmrt_device_buffer_t output_bf16, void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(validate_forward(l, rows));
  const size_t row_bytes = static_cast<size_t>(l->cfg.hidden_dim) * 2, routes = rows * l->cfg.top_k;
  GLMRT_RETURN_IF_ERROR(check_buf(hidden_bf16, rows * row_bytes, "forward_routed hidden"));
  GLMRT_RETURN_IF_ERROR(check_buf(output_bf16, rows * row_bytes, "forward_routed output"));
  GLMRT_RETURN_IF_ERROR(check_buf(topk_indices, routes * 4, "forward_routed topk_indices"));
  GLMRT_RETURN_IF_ERROR(check_buf(topk_weights, routes * 4, "forward_routed topk_weights"));
  if (reinterpret_cast<uintptr_t>(hidden_bf16.ptr) % 16 != 0 || reinterpret_cast<uintptr_t>(output_bf16.ptr) % 16 != 0)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_routed: hidden and output must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const uint64_t before = launches_total();
  mark(l, GLMRT_B200_STAGE_ROUTER, s);
  cudaError_t err = cudaMemcpyAsync(l->topk_idx, topk_indices.ptr, routes * 4, cudaMemcpyDeviceToDevice, s);
  if (err == cudaSuccess) err = cudaMemcpyAsync(l->topk_w, topk_weights.ptr, routes * 4, cudaMemcpyDeviceToDevice, s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "forward_routed route copy", err);
  GLMRT_RETURN_IF_ERROR(run_routed(l, static_cast<const uint16_t*>(hidden_bf16.ptr), rows,
                                   static_cast<uint16_t*>(output_bf16.ptr), s));
  l->launches_last = static_cast<uint32_t>(launches_total() - before);
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_forward_host(void* layer, const void* hidden_host, size_t rows,
                                                            void* output_host, void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(validate_forward(l, rows));
  if (hidden_host == nullptr || output_host == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_host: null host pointer");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const size_t bytes = rows * static_cast<size_t>(l->cfg.hidden_dim) * 2;
  cudaError_t err = cudaMemcpyAsync(l->hidden_stage, hidden_host, bytes, cudaMemcpyHostToDevice, s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "forward_host input copy", err);
  glmrt_device_buffer_t in{l->hidden_stage, bytes, l->device, 0}, out{l->out_stage, bytes, l->device, 0};
  glmrt_device_buffer_t none{nullptr, 0, l->device, 0};
  GLMRT_RETURN_IF_ERROR(glmrt_b200_moe_layer_forward_async(layer, in, rows, out, none, none, cuda_stream));
  err = cudaMemcpyAsync(output_host, l->out_stage, bytes, cudaMemcpyDeviceToHost, s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "forward_host output copy", err);
  err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "forward_host synchronize", err);
  return ok();
}

namespace glmrt {

glmrt_status_t layer_dims(void* layer, LayerDims* out) {
  Layer* l = static_cast<Layer*>(layer);
  if (l == nullptr || out == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer is null");
  const auto& c = l->cfg;
  *out = LayerDims{c.hidden_dim, c.experts, c.top_k, c.max_tokens, c.ep_world, c.ep_rank};
  return GLMRT_STATUS_OK;
}

glmrt_status_t layer_execute_host_rows(void* layer, const void* hidden_host, bool hidden_is_payload, size_t hidden_stride,
                                       size_t rows, const uint32_t* idx_host, const float* w_host, int out_kind,
                                       void* out_host, size_t out_stride, cudaStream_t s) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(validate_forward(l, rows));
  const auto& c = l->cfg;
  const size_t H = c.hidden_dim, routes = rows * c.top_k;
  const size_t payload_row = H / 2 + H / 16, bf16_row = H * 2;
  cudaError_t err = cudaMemcpyAsync(l->topk_idx, idx_host, routes * 4, cudaMemcpyHostToDevice, s);
  if (err == cudaSuccess) err = cudaMemcpyAsync(l->topk_w, w_host, routes * 4, cudaMemcpyHostToDevice, s);
  if (err == cudaSuccess)
    err = hidden_is_payload ? cudaMemcpy2DAsync(l->payload, payload_row, hidden_host, hidden_stride, payload_row, rows,
                                                cudaMemcpyHostToDevice, s)
                            : cudaMemcpy2DAsync(l->hidden_stage, bf16_row, hidden_host, hidden_stride, bf16_row, rows,
                                                cudaMemcpyHostToDevice, s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "executor input copy", err);
  const uint64_t before = launches_total();
  mark(l, GLMRT_B200_STAGE_ROUTER, s);
  GLMRT_RETURN_IF_ERROR(run_routed(l, hidden_is_payload ? nullptr : l->hidden_stage, rows, l->out_stage, s));
  if (out_kind == kOutNvfp4Payload) {
    // response rows in the wire format, with the native kernel's rounding rule (nvfp4_payload.cu:11-33)
    GLMRT_RETURN_IF_ERROR(launch_quantize_rows_payload(l->out_stage, l->payload, rows, H, GLMRT_B200_FP4_RULE_RNE_PAYLOAD, s));
    err = cudaMemcpy2DAsync(out_host, out_stride, l->payload, payload_row, payload_row, rows, cudaMemcpyDeviceToHost, s);
  } else if (out_kind == kOutFp8RowScaled) {
    // H + 4 bytes per row; the input stage is free again and large enough (2H per row)
    uint8_t* fp8 = reinterpret_cast<uint8_t*>(l->hidden_stage);
    GLMRT_RETURN_IF_ERROR(launch_bf16_rows_to_fp8_row_scaled(l->out_stage, fp8, rows, H, H + 4, s));
    err = cudaMemcpy2DAsync(out_host, out_stride, fp8, H + 4, H + 4, rows, cudaMemcpyDeviceToHost, s);
  } else {
    err = cudaMemcpy2DAsync(out_host, out_stride, l->out_stage, bf16_row, bf16_row, rows, cudaMemcpyDeviceToHost, s);
  }
  l->launches_last = static_cast<uint32_t>(launches_total() - before);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "executor output copy", err);
  return glmrt_b200_moe_layer_check(layer, s);
}

}  // namespace glmrt

extern "C" glmrt_status_t glmrt_b200_moe_layer_check(void* layer, void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  if (l == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer is null");
  uint32_t host[kCntWords] = {0};
  cudaError_t err = cudaStreamSynchronize(static_cast<cudaStream_t>(cuda_stream));
  if (err == cudaSuccess) err = cudaMemcpy(host, l->counters, sizeof(host), cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "layer check", err);
  const uint32_t e = host[kCntError] | host[kCntRouterError];
  if (e == 0) return ok();
  std::string msg = "device reported:";
  if (e & kErrWaitTimeout) msg += " a bounded wait expired;";
  if (e & kErrSlotOverflow) msg += " route plan exceeds slot capacity;";
  if (e & kErrChunkOverflow) msg += " route plan exceeds chunk capacity;";
  if (e & kErrBadExpert) msg += " a route names an expert id outside the layer;";
  if (e & kErrPeerFailed) msg += " a peer rank had no valid plan this step and sent no rows;";
  return fail(GLMRT_STATUS_INTERNAL_ERROR, msg);
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_debug_buffer(void* layer, uint32_t which, glmrt_device_buffer_t* out) {
  Layer* l = static_cast<Layer*>(layer);
  if (l == nullptr || out == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "debug_buffer: null argument");
  const auto& c = l->cfg;
  const size_t H = c.hidden_dim, I = c.intermediate_dim, T = c.max_tokens, K = c.top_k, S = l->max_slots,
               E = l->local_experts;
  void* p = nullptr;
  size_t bytes = 0;
  switch (which) {
    case GLMRT_B200_DEBUG_PAYLOAD: p = l->payload; bytes = T * (H / 2 + H / 16); break;
    case GLMRT_B200_DEBUG_ROUTE_SLOT: p = l->route_slot; bytes = T * K * 4; break;
    case GLMRT_B200_DEBUG_ACT1_CODES: p = l->act1_codes; bytes = S * H / 2; break;
    case GLMRT_B200_DEBUG_ACT1_SF: p = l->act1_sf; bytes = S * H / 16; break;
    case GLMRT_B200_DEBUG_ACT2_CODES: p = l->act2_codes; bytes = S * I / 2; break;
    case GLMRT_B200_DEBUG_ACT2_SF: p = l->act2_sf; bytes = S * I / 16; break;
    case GLMRT_B200_DEBUG_ROUTE_ROWS: p = l->route_rows; bytes = T * K * H * 2; break;
    case GLMRT_B200_DEBUG_COUNTERS: p = l->counters; bytes = kCntWords * 4; break;
    case GLMRT_B200_DEBUG_CHUNKS: p = l->chunks; bytes = static_cast<size_t>(l->max_chunks) * sizeof(Chunk); break;
    case GLMRT_B200_DEBUG_EXPERT_COUNTS: p = l->expert_counts; bytes = E * 4; break;
    case GLMRT_B200_DEBUG_GATE_CODES: p = l->gate_codes; bytes = E * I * H / 2; break;
    case GLMRT_B200_DEBUG_UP_CODES: p = l->up_codes; bytes = E * I * H / 2; break;
    case GLMRT_B200_DEBUG_DOWN_CODES: p = l->down_codes; bytes = E * H * I / 2; break;
    case GLMRT_B200_DEBUG_GATE_SF: p = l->gate_sf; bytes = E * I * H / 16; break;
    case GLMRT_B200_DEBUG_UP_SF: p = l->up_sf; bytes = E * I * H / 16; break;
    case GLMRT_B200_DEBUG_DOWN_SF: p = l->down_sf; bytes = E * H * I / 16; break;
    case GLMRT_B200_DEBUG_SCALE2: p = l->scale2; bytes = E * 3 * 4; break;
    case GLMRT_B200_DEBUG_TOPK_IDX: p = l->topk_idx; bytes = T * K * 4; break;
    case GLMRT_B200_DEBUG_TOPK_W: p = l->topk_w; bytes = T * K * 4; break;
    default: return fail(GLMRT_STATUS_INVALID_ARGUMENT, "debug_buffer: unknown buffer id");
  }
  out->ptr = p;
  out->bytes = bytes;
  out->device_id = l->device;
  out->flags = 0;
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_stats(void* layer, glmrt_b200_layer_stats_t* out) {
  Layer* l = static_cast<Layer*>(layer);
  if (l == nullptr || out == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer stats: null argument");
  uint32_t host[kCntWords] = {0};
  cudaError_t err = cudaMemcpy(host, l->counters, sizeof(host), cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "layer stats", err);
  std::memset(out, 0, sizeof(*out));
  out->launches_total = launches_total();
  out->launches_last_forward = l->launches_last;
  out->chunks = host[kCntChunks];
  out->slots = host[kCntSlots];
  out->distinct_experts = host[kCntDistinct];
  out->device_error = host[kCntError] | host[kCntRouterError];
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_set_profiling(void* layer, int enable) {
  Layer* l = static_cast<Layer*>(layer);
  if (l == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer is null");
  if (enable != 0 && l->stage_events[0] == nullptr) {
    for (cudaEvent_t& e : l->stage_events) {
      cudaError_t err = cudaEventCreate(&e);
      if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaEventCreate", err);
    }
  }
  l->profiling = enable != 0;
  l->stage_valid = false;
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_stage_times(void* layer, float* out_ms, size_t count) {
  Layer* l = static_cast<Layer*>(layer);
  if (l == nullptr || out_ms == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "stage_times: null argument");
  if (count < GLMRT_B200_STAGE_COUNT) return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "stage_times: need GLMRT_B200_STAGE_COUNT floats");
  if (!l->stage_valid) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "stage_times: no profiled forward has run");
  cudaError_t err = cudaEventSynchronize(l->stage_events[GLMRT_B200_STAGE_COUNT]);
  for (int i = 0; i < GLMRT_B200_STAGE_COUNT && err == cudaSuccess; ++i)
    err = cudaEventElapsedTime(&out_ms[i], l->stage_events[i], l->stage_events[i + 1]);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "stage_times", err);
  return ok();
}

// ---------------------------------------------------------------------------------------------
// Expert-parallel forward
// ---------------------------------------------------------------------------------------------
namespace {

glmrt_status_t require_ep(Layer* l, bool attached) {
  if (l == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "layer is null");
  if (l->cfg.ep_world < 2 || l->ep_ctrl == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "expert-parallel entry point on a layer created with ep_world == 1");
  if (attached && !l->eps->attached)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "expert-parallel forward before glmrt_b200_ep_attach");
  return GLMRT_STATUS_OK;
}

void local_ep_buffers(Layer* l, glmrt_b200_ep_buffers_t* out) {
  out->act_codes = l->act1_codes;
  out->act_sf = l->act1_sf;
  out->slot_out = l->slot_out;
  out->route_rows = l->route_rows;
  out->control = l->ep_ctrl;
  out->act_sf_rows = l->act1_sf_rows;
}

glmrt_status_t ep_phase(Layer* l, uint32_t phase, const uint16_t* hidden, size_t rows, uint16_t* out,
                        cudaStream_t s) {
  const auto& c = l->cfg;
  // Work-item size of the step: every rank must choose the same (it fixes the slot layout), so it
  // follows the size of the whole batch where the caller has stated it, else the layer's capacity.
  const uint32_t batch = l->eps->global_rows != 0 ? l->eps->global_rows : c.max_tokens;
  const int chunk_tokens = batch <= 256 ? 32 : 128;
  EpArgs a = l->eps->args;
  a.epoch = l->eps->epoch;
  a.chunk_tokens = chunk_tokens;
  switch (phase) {
    case 0: {
      // router; the tail of its selection kernel publishes this rank's routes-per-expert histogram
      mark(l, GLMRT_B200_STAGE_ROUTER, s);
      if (rows > 0) {
        RouterCountTail tail = ep_count_tail(a);
        tail.route_pos = l->route_slot;   // positions now, slots once the push kernel has placed the routes
        GLMRT_RETURN_IF_ERROR(run_router(l, hidden, rows, s, &tail));
      } else {
        GLMRT_RETURN_IF_ERROR(launch_ep_count(a, l->topk_idx, 0, s));
      }
      mark(l, GLMRT_B200_STAGE_QUANTIZE, s);
      return GLMRT_STATUS_OK;
    }
    case 1: {
      // wait for every histogram, derive the layout, quantise the rows and push them to their owners
      mark(l, GLMRT_B200_STAGE_PLAN, s);
      const PlanArgs p = plan_args(l, rows, chunk_tokens);
      mark(l, GLMRT_B200_STAGE_DISPATCH, s);
      return launch_ep_plan_dispatch(a, p, hidden, l->payload, static_cast<int>(rows), static_cast<int>(c.top_k),
                                     static_cast<int>(c.hidden_dim), s);
    }
    case 2: {
      // expert FFN on what arrived: FC1 waits for the peers' rows, FC2 stores each result row into
      // its home rank and raises the "combine" flag when the last CTA is done
      FfnArgs f = ffn_args(l, chunk_tokens, batch);
      mark(l, GLMRT_B200_STAGE_FC1, s);
      if (c.flags & GLMRT_B200_LAYER_ENGINE_SIMT) {
        if (chunk_tokens >= 128)
          GLMRT_RETURN_IF_ERROR(launch_ep_retile_scales(a, l->act1_sf_rows, l->act1_sf, static_cast<int>(c.hidden_dim / 16),
                                                        l->counters, l->counters + kCntError, l->counters + kCntChunks, s));
        GLMRT_RETURN_IF_ERROR(launch_ep_wait(ep_wait_dispatch(a), l->counters + kCntError, l->counters + kCntChunks, s));
        GLMRT_RETURN_IF_ERROR(launch_fc1_simt(f, s));
        mark(l, GLMRT_B200_STAGE_FC2, s);
        GLMRT_RETURN_IF_ERROR(launch_fc2_simt(f, s));
        mark(l, GLMRT_B200_STAGE_COMBINE, s);
        return launch_ep_signal(ep_signal_combine(a), l->counters + kCntError, s);
      }
      f.wait = ep_wait_dispatch(a);
      f.signal = ep_signal_combine(a);
      if (chunk_tokens >= 128)   // prefill-sized push: scale rows arrive row-major, re-tile what this rank owns
        GLMRT_RETURN_IF_ERROR(launch_ep_retile_scales(a, l->act1_sf_rows, l->act1_sf, static_cast<int>(c.hidden_dim / 16),
                                                      l->counters, l->counters + kCntError, l->counters + kCntChunks, s));
      if (!l->have_maps) GLMRT_RETURN_IF_ERROR(build_maps(l));
      const TensorMaps& maps = chunk_tokens == 32 ? l->maps32 : l->maps128;
      GLMRT_RETURN_IF_ERROR(chunk_tokens == 32 ? launch_fc1_tc(f, maps, l->sm_count, s)
                                               : launch_fc1_tc_prefill(f, maps, l->sm_count, s));
      mark(l, GLMRT_B200_STAGE_FC2, s);
      GLMRT_RETURN_IF_ERROR(chunk_tokens == 32 ? launch_fc2_tc(f, maps, l->sm_count, s)
                                               : launch_fc2_tc_prefill(f, maps, l->sm_count, s));
      mark(l, GLMRT_B200_STAGE_COMBINE, s);
      return GLMRT_STATUS_OK;
    }
    case 3: {
      if (rows > 0) {
        const EpWait w = ep_wait_combine(a);
        GLMRT_RETURN_IF_ERROR(launch_combine_routes(l->route_rows, l->topk_w, l->route_slot, out, static_cast<int>(rows),
                                                    static_cast<int>(c.top_k), static_cast<int>(c.hidden_dim), s,
                                                    nullptr, nullptr, &w, l->counters + kCntError));
      }
      mark(l, GLMRT_B200_STAGE_COUNT, s);
      l->stage_valid = l->profiling;
      return GLMRT_STATUS_OK;
    }
    default:
      return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_ep: phase must be 0..3");
  }
}

glmrt_status_t validate_ep_forward(Layer* l, glmrt_device_buffer_t hidden, size_t rows, glmrt_device_buffer_t out) {
  GLMRT_RETURN_IF_ERROR(require_ep(l, true));
  if (rows > l->cfg.max_tokens) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_ep: rows exceed max_tokens");
  if (rows > 0) {
    const size_t bytes = rows * static_cast<size_t>(l->cfg.hidden_dim) * 2;
    GLMRT_RETURN_IF_ERROR(check_buf(hidden, bytes, "forward_ep hidden"));
    GLMRT_RETURN_IF_ERROR(check_buf(out, bytes, "forward_ep output"));
    if (reinterpret_cast<uintptr_t>(hidden.ptr) % 16 != 0 || reinterpret_cast<uintptr_t>(out.ptr) % 16 != 0)
      return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_ep: hidden and output must be 16-byte aligned");
  }
  return GLMRT_STATUS_OK;
}

}  // namespace

extern "C" glmrt_status_t glmrt_b200_ep_local_buffers(void* layer, glmrt_b200_ep_buffers_t* out) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(require_ep(l, false));
  if (out == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "ep_local_buffers: null output");
  local_ep_buffers(l, out);
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_ep_ipc_export(void* layer, void* out_handles, size_t bytes) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(require_ep(l, false));
  if (out_handles == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "ep_ipc_export: null output");
  if (bytes < GLMRT_B200_EP_IPC_BYTES) return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "ep_ipc_export: need 384 bytes");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle size");
  glmrt_b200_ep_buffers_t b;
  local_ep_buffers(l, &b);
  void* ptrs[6] = {b.act_codes, b.act_sf, b.slot_out, b.route_rows, b.control, b.act_sf_rows};
  for (int i = 0; i < 6; ++i) {
    cudaIpcMemHandle_t h;
    cudaError_t err = cudaIpcGetMemHandle(&h, ptrs[i]);
    if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaIpcGetMemHandle", err);
    std::memcpy(static_cast<uint8_t*>(out_handles) + 64 * i, &h, 64);
  }
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_ep_ipc_open(void* layer, const void* handles, size_t bytes,
                                                 glmrt_b200_ep_buffers_t* out_mapped) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(require_ep(l, false));
  if (handles == nullptr || out_mapped == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "ep_ipc_open: null argument");
  if (bytes < GLMRT_B200_EP_IPC_BYTES) return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "ep_ipc_open: need 384 bytes");
  void* ptrs[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  for (int i = 0; i < 6; ++i) {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const uint8_t*>(handles) + 64 * i, 64);
    cudaError_t err = cudaIpcOpenMemHandle(&ptrs[i], h, cudaIpcMemLazyEnablePeerAccess);
    if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaIpcOpenMemHandle (peer access between the GPUs is required)", err);
    l->work_block->ipc_mappings.push_back(ptrs[i]);
  }
  out_mapped->act_codes = ptrs[0];
  out_mapped->act_sf = ptrs[1];
  out_mapped->slot_out = ptrs[2];
  out_mapped->route_rows = ptrs[3];
  out_mapped->control = ptrs[4];
  out_mapped->act_sf_rows = ptrs[5];
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_ep_attach(void* layer, const glmrt_b200_ep_buffers_t* peers, size_t world,
                                               const uint64_t* my_rows_in_peer) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(require_ep(l, false));
  if (peers == nullptr || my_rows_in_peer == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "ep_attach: null argument");
  if (world != l->cfg.ep_world) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "ep_attach: world differs from the layer's ep_world");
  EpArgs a{};
  a.world = static_cast<int>(world);
  a.rank = static_cast<int>(l->cfg.ep_rank);
  a.experts = static_cast<int>(l->cfg.experts);
  a.ctrl = l->ep_ctrl;
  a.counters = l->counters;
  for (size_t p = 0; p < world; ++p) {
    if (peers[p].act_codes == nullptr || peers[p].act_sf == nullptr || peers[p].slot_out == nullptr ||
        peers[p].control == nullptr || peers[p].act_sf_rows == nullptr || my_rows_in_peer[p] == 0)
      return fail(GLMRT_STATUS_INVALID_ARGUMENT, "ep_attach: a peer buffer is null");
    a.peer_ctrl[p] = static_cast<EpControl*>(peers[p].control);
    a.peer_act_codes[p] = static_cast<uint8_t*>(peers[p].act_codes);
    a.peer_act_sf[p] = static_cast<uint8_t*>(peers[p].act_sf);
    a.peer_act_sf_rows[p] = static_cast<uint8_t*>(peers[p].act_sf_rows);
    a.peer_slot_out[p] = static_cast<uint16_t**>(peers[p].slot_out);
    a.my_rows_in_peer[p] = reinterpret_cast<uint16_t*>(static_cast<uintptr_t>(my_rows_in_peer[p]));
  }
  if (a.peer_ctrl[a.rank] != l->ep_ctrl)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "ep_attach: the entry of this rank must be its own local buffers");
  l->eps->args = a;
  l->eps->attached = true;
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_ep_set_global_rows(void* layer, uint32_t global_rows) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(require_ep(l, false));
  if (static_cast<uint64_t>(global_rows) > static_cast<uint64_t>(l->cfg.max_tokens) * l->cfg.ep_world)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "ep_set_global_rows: more rows than the ranks can hold");
  l->eps->global_rows = global_rows;
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_forward_ep_phase_async(void* layer, uint32_t phase,
                                                                      glmrt_device_buffer_t hidden_bf16, size_t rows,
                                                                      glmrt_device_buffer_t output_bf16,
                                                                      void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(validate_ep_forward(l, hidden_bf16, rows, output_bf16));
  if (phase > 3) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_ep: phase must be 0..3");
  if (phase == 0) ++l->eps->epoch;
  const uint64_t before = launches_total();
  GLMRT_RETURN_IF_ERROR(ep_phase(l, phase, static_cast<const uint16_t*>(hidden_bf16.ptr), rows,
                                 static_cast<uint16_t*>(output_bf16.ptr), static_cast<cudaStream_t>(cuda_stream)));
  l->launches_last = (phase == 0 ? 0 : l->launches_last) + static_cast<uint32_t>(launches_total() - before);
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_forward_ep_async(void* layer, glmrt_device_buffer_t hidden_bf16,
                                                                size_t rows, glmrt_device_buffer_t output_bf16,
                                                                void* cuda_stream) {
  for (uint32_t phase = 0; phase < 4; ++phase)
    GLMRT_RETURN_IF_ERROR(glmrt_b200_moe_layer_forward_ep_phase_async(layer, phase, hidden_bf16, rows, output_bf16,
                                                                      cuda_stream));
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_moe_layer_forward_ep_host(void* layer, const void* hidden_host, size_t rows,
                                                               void* output_host, void* cuda_stream) {
  Layer* l = static_cast<Layer*>(layer);
  GLMRT_RETURN_IF_ERROR(require_ep(l, true));
  if (rows > l->cfg.max_tokens) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_ep_host: rows exceed max_tokens");
  if (rows > 0 && (hidden_host == nullptr || output_host == nullptr))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "forward_ep_host: null host pointer");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const size_t bytes = rows * static_cast<size_t>(l->cfg.hidden_dim) * 2;
  cudaError_t err = cudaSuccess;
  if (rows > 0) err = cudaMemcpyAsync(l->hidden_stage, hidden_host, bytes, cudaMemcpyHostToDevice, s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "forward_ep_host input copy", err);
  glmrt_device_buffer_t in{l->hidden_stage, bytes, l->device, 0}, out{l->out_stage, bytes, l->device, 0};
  GLMRT_RETURN_IF_ERROR(glmrt_b200_moe_layer_forward_ep_async(layer, in, rows, out, cuda_stream));
  if (rows > 0) err = cudaMemcpyAsync(output_host, l->out_stage, bytes, cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "forward_ep_host output copy", err);
  return ok();
}
