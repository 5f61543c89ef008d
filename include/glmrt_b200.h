/*
 * C ABI of libglmrt_b200.so: the routed-MoE expert FFN path of GLMRT, written for
 * NVIDIA B200 (sm_100a).
 *
 * The library is a drop-in for the hot-path subset of the reference's
 * libglmrt_native.so (reference header: native/include/glmrt_native.h).  Symbols
 * that keep a reference name keep the reference signature and error behaviour;
 * each declaration cites the reference declaration it replaces.  Entry points
 * named glmrt_b200_* are additions for what the reference's fixed-shape structs
 * cannot express (full-intermediate experts, fp32 router weights, expert-parallel
 * shards) and say so.
 *
 * Conventions (reference: native/include/glmrt_native.h:10-20,77-82,427;
 * native/src/glmrt_native.cc:30-49):
 *   - every function returns glmrt_status_t; on failure a thread-local message
 *     is readable with glmrt_last_error();
 *   - glmrt_device_buffer_t is passed by value, owned by the caller, never freed
 *     by the callee, and its `bytes` is validated before anything is launched;
 *   - *_async functions only enqueue work on `cuda_stream` (a cudaStream_t, NULL
 *     for the default stream); the twin without _async runs on the default
 *     stream and synchronises it;
 *   - no exception crosses the ABI; all validation happens before any launch;
 *   - there is no CPU fallback: without a CUDA device compute entry points
 *     return GLMRT_STATUS_CUDA_UNAVAILABLE.
 */
#pragma once

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* native/include/glmrt_native.h:10-20 */
typedef enum glmrt_status_t {
  GLMRT_STATUS_OK = 0,
  GLMRT_STATUS_INVALID_ARGUMENT = 1,
  GLMRT_STATUS_BUFFER_TOO_SMALL = 2,
  GLMRT_STATUS_CUDA_UNAVAILABLE = 3,
  GLMRT_STATUS_ALLOCATION_FAILED = 4,
  GLMRT_STATUS_COPY_FAILED = 5,
  GLMRT_STATUS_INTERNAL_ERROR = 6,
  GLMRT_STATUS_RDMA_UNAVAILABLE = 7,
  GLMRT_STATUS_NCCL_UNAVAILABLE = 8,
} glmrt_status_t;

/* native/include/glmrt_native.h:62-74 */
typedef struct glmrt_cuda_device_info_t {
  int device_id;
  int cuda_available;
  int compute_capability_major;
  int compute_capability_minor;
  int integrated;
  int can_map_host_memory;
  int unified_addressing;
  uint64_t total_memory_bytes;
  char name[128];
  char driver_version[64];
  char runtime_version[64];
} glmrt_cuda_device_info_t;

/* native/include/glmrt_native.h:77-82 */
typedef struct glmrt_device_buffer_t {
  void* ptr;
  size_t bytes;
  int device_id;
  uint64_t flags;
} glmrt_device_buffer_t;

/* ------------------------------------------------------------------------ */
/* Infrastructure (native/include/glmrt_native.h:296-313,415-427)             */
/* ------------------------------------------------------------------------ */
glmrt_status_t glmrt_native_version(char* out, size_t out_len);
glmrt_status_t glmrt_last_error(char* out, size_t out_len);
glmrt_status_t glmrt_cuda_device_info(int device_id, glmrt_cuda_device_info_t* out);
glmrt_status_t glmrt_alloc_device_buffer(size_t bytes, glmrt_device_buffer_t* out);
glmrt_status_t glmrt_free_device_buffer(glmrt_device_buffer_t* buf);
glmrt_status_t glmrt_cuda_stream_create(void** out_cuda_stream);
glmrt_status_t glmrt_cuda_stream_destroy(void* cuda_stream);
glmrt_status_t glmrt_cuda_stream_synchronize(void* cuda_stream);
glmrt_status_t glmrt_cuda_event_create(void** out_cuda_event);
glmrt_status_t glmrt_cuda_event_destroy(void* cuda_event);
glmrt_status_t glmrt_cuda_event_record(void* cuda_event, void* cuda_stream);
glmrt_status_t glmrt_cuda_event_synchronize(void* cuda_event);
glmrt_status_t glmrt_cuda_event_elapsed_ms(void* start_event, void* end_event, float* out_ms);
glmrt_status_t glmrt_copy_h2d(glmrt_device_buffer_t dst, const void* src, size_t bytes);
glmrt_status_t glmrt_copy_d2h(void* dst, glmrt_device_buffer_t src, size_t bytes);
glmrt_status_t glmrt_copy_d2d(glmrt_device_buffer_t dst, glmrt_device_buffer_t src, size_t bytes);
glmrt_status_t glmrt_copy_h2d_async(glmrt_device_buffer_t dst, const void* src, size_t bytes,
                                    void* cuda_stream);
glmrt_status_t glmrt_copy_d2h_async(void* dst, glmrt_device_buffer_t src, size_t bytes,
                                    void* cuda_stream);
glmrt_status_t glmrt_copy_d2d_async(glmrt_device_buffer_t dst, glmrt_device_buffer_t src,
                                    size_t bytes, void* cuda_stream);

/* ------------------------------------------------------------------------ */
/* Router (native/include/glmrt_native.h:1002-1018; kernels router.cu:7-180)  */
/* sigmoid(X W^T), selection = score + bias, top-k by selection (ties to the  */
/* lower expert id), weights = score / max(sum, 1e-12) * 2.5.                 */
/* rows, hidden_dim, experts > 0; 0 < top_k <= min(experts, 64).              */
/* ------------------------------------------------------------------------ */
glmrt_status_t glmrt_cuda_router_topk_f32(const float* hidden, const float* router_weight,
                                          const float* correction_bias, uint32_t* topk_indices,
                                          float* topk_scores, float* topk_weights, size_t rows,
                                          size_t hidden_dim, size_t experts, size_t top_k);
glmrt_status_t glmrt_cuda_router_topk_f32_async(
    const float* hidden, const float* router_weight, const float* correction_bias,
    uint32_t* topk_indices, float* topk_scores, float* topk_weights, size_t rows,
    size_t hidden_dim, size_t experts, size_t top_k, void* cuda_stream);
glmrt_status_t glmrt_cuda_router_topk_bf16(const uint16_t* hidden,
                                           const uint16_t* router_weight,
                                           const float* correction_bias, uint32_t* topk_indices,
                                           float* topk_scores, float* topk_weights, size_t rows,
                                           size_t hidden_dim, size_t experts, size_t top_k);
glmrt_status_t glmrt_cuda_router_topk_bf16_async(
    const uint16_t* hidden, const uint16_t* router_weight, const float* correction_bias,
    uint32_t* topk_indices, float* topk_scores, float* topk_weights, size_t rows,
    size_t hidden_dim, size_t experts, size_t top_k, void* cuda_stream);
/* glmrt_native.h:1019-1030: the variant whose scratch the caller owns (rows * experts floats in
 * corrected_scores and sorted_corrected_scores, rows * experts indices twice, rows + 1 offsets,
 * temporary storage), so that nothing is allocated.  Same results as the entry points above; the
 * logits live in corrected_scores, the other scratch arrays are only validated. */
glmrt_status_t glmrt_cuda_router_topk_bf16_cub(
    const uint16_t* hidden, const uint16_t* router_weight, const float* correction_bias,
    float* corrected_scores, float* sorted_corrected_scores, uint32_t* unsorted_indices,
    uint32_t* sorted_indices, int* segment_offsets, uint32_t* topk_indices, float* topk_scores,
    float* topk_weights, void* cub_temp_storage, size_t cub_temp_storage_bytes, size_t rows,
    size_t hidden_dim, size_t experts, size_t top_k);
glmrt_status_t glmrt_cuda_router_topk_bf16_cub_async(
    const uint16_t* hidden, const uint16_t* router_weight, const float* correction_bias,
    float* corrected_scores, float* sorted_corrected_scores, uint32_t* unsorted_indices,
    uint32_t* sorted_indices, int* segment_offsets, uint32_t* topk_indices, float* topk_scores,
    float* topk_weights, void* cub_temp_storage, size_t cub_temp_storage_bytes, size_t rows,
    size_t hidden_dim, size_t experts, size_t top_k, void* cuda_stream);
/* Addition: bf16 activations against float32 router weights, the operand types of
 * the Python oracle (python/reference/glmrt_reference/glm_moe_dsa_layer_ref.py:62-83).
 * `logits_scratch` holds rows * experts floats. */
glmrt_status_t glmrt_b200_router_topk_bf16_f32w_async(
    const uint16_t* hidden, const float* router_weight, const float* correction_bias,
    float* logits_scratch, uint32_t* topk_indices, float* topk_scores, float* topk_weights,
    size_t rows, size_t hidden_dim, size_t experts, size_t top_k, void* cuda_stream);

/* No counterpart in the reference.  Same computation as
 * glmrt_b200_router_topk_bf16_f32w_async, for callers that must not allocate device memory and
 * have no scratch buffer to lend: code running where cudaMalloc is off limits (inside a
 * latency-critical serving loop whose memory is fully pre-assigned, or after the process has
 * handed all remaining device memory to another component).  The rows * experts float logits
 * live in an array built into the library (1 MiB, held by every GPU that loads the library until
 * the process exits), so rows * experts must not exceed 262144; larger problems are rejected
 * with GLMRT_STATUS_BUFFER_TOO_SMALL.  The entry point calls no allocator.  The first call on a
 * device looks up the array's device address; make that first call outside any stream capture.
 * The address is cached per device for the life of the process, which assumes that the device's
 * primary context is not reset in between.
 * All calls on one device share the array: calls that may overlap on the GPU (different streams)
 * race on it and must be ordered by the caller. */
glmrt_status_t glmrt_b200_router_topk_bf16_f32w_static_async(
    const uint16_t* hidden, const float* router_weight, const float* correction_bias,
    uint32_t* topk_indices, float* topk_scores, float* topk_weights, size_t rows, size_t hidden_dim,
    size_t experts, size_t top_k, void* cuda_stream);

/* ------------------------------------------------------------------------ */
/* NVFP4 codecs                                                               */
/* ------------------------------------------------------------------------ */
/* native/include/glmrt_native.h:610-612 (kernel nvfp4_payload.cu:35-73): bf16 rows ->
 * row payload [hidden_dim/2 packed codes | hidden_dim/16 E4M3 scales], round-to-
 * nearest-even code thresholds on x * (1/scale).  hidden_dim % 16 == 0. */
glmrt_status_t glmrt_cuda_b12x_quantize_bf16_nvfp4_row_payload_async(
    glmrt_device_buffer_t input, glmrt_device_buffer_t payload, size_t rows, size_t hidden_dim,
    void* cuda_stream);
/* Addition: same payload layout with a selectable code rule. */
typedef enum glmrt_b200_fp4_rule_t {
  GLMRT_B200_FP4_RULE_RNE_PAYLOAD = 0, /* nvfp4_payload.cu:11-33,56-66 */
  GLMRT_B200_FP4_RULE_NEAREST_LOW = 1, /* quant_ref.py:41-46: x / scale, ties to lower magnitude */
} glmrt_b200_fp4_rule_t;
glmrt_status_t glmrt_b200_quantize_bf16_nvfp4_row_payload_async(
    glmrt_device_buffer_t input, glmrt_device_buffer_t payload, size_t rows, size_t hidden_dim,
    uint32_t rule, void* cuda_stream);
/* native/include/glmrt_native.h:627-630 (kernel mlp.cu:98-132): bf16 weights ->
 * packed codes + E4M3 block scales with a multiplicative global scale. */
glmrt_status_t glmrt_cuda_quantize_bf16_weight_nvfp4_async(
    glmrt_device_buffer_t input, glmrt_device_buffer_t packed, glmrt_device_buffer_t scales,
    size_t rows, size_t cols, float global_scale, void* cuda_stream);
/* Addition: float32 weights -> NVFP4 with scale_2 = amax / (6 * 448) (the benchmark's
 * weight recipe).  `scale_2_out` receives one float; `scratch` holds one uint32. */
glmrt_status_t glmrt_b200_quantize_f32_weight_nvfp4_async(
    glmrt_device_buffer_t input, glmrt_device_buffer_t packed, glmrt_device_buffer_t scales,
    glmrt_device_buffer_t scale_2_out, glmrt_device_buffer_t scratch, size_t rows, size_t cols,
    void* cuda_stream);
/* native/include/glmrt_native.h:631-634 (kernel b12x_direct.cu:269-290): gather payload
 * rows and expand them to bf16 (code * E4M3 scale, truncating bf16 store). */
glmrt_status_t glmrt_cuda_b12x_gather_nvfp4_rows_bf16_async(
    glmrt_device_buffer_t payload, size_t source_rows, size_t source_row_stride_bytes,
    glmrt_device_buffer_t row_indices, glmrt_device_buffer_t output, size_t rows,
    size_t hidden_dim, void* cuda_stream);

/* ------------------------------------------------------------------------ */
/* Combine (native/include/glmrt_native.h:679-681,843-846)                    */
/* ------------------------------------------------------------------------ */
/* The reference's float32 route MLP on bf16 activations and NVFP4 weights (W4A16; glmrt_native.h:
 * 114-127, 572-597; kernels native/cuda/kernels/mlp.cu:218-420).  For every route r with
 * row_indices[r] < rows: activation_workspace[r, m] = silu(x . gate[m]) * (x . up[m]) and
 * accumulator[row_indices[r], o] += route_weights[r] * (activation[r] . down[o]), all float32;
 * routes whose row index is out of range are skipped.  `grouped`: every route uses the one expert
 * given; `batched`: route r uses route_metadata[r] (device memory).  hidden_dim and the
 * intermediate sizes must be multiples of 16; hidden_row_stride counts bf16 elements. */
typedef struct glmrt_nvfp4_route_batched_metadata_t {
  uintptr_t gate_weight;
  uintptr_t gate_scale;
  uintptr_t up_weight;
  uintptr_t up_scale;
  uintptr_t down_weight;
  uintptr_t down_scale;
  size_t intermediate;
  size_t down_weight_row_stride_bytes;
  size_t down_scale_row_stride_bytes;
  float gate_scale_2;
  float up_scale_2;
  float down_scale_2;
} glmrt_nvfp4_route_batched_metadata_t;
glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_grouped_staged_accumulate_f32(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const uint8_t* gate_weight, const uint8_t* gate_scale, const uint8_t* up_weight,
    const uint8_t* up_scale, const uint8_t* down_weight, const uint8_t* down_scale,
    float* activation_workspace, float* accumulator, size_t rows, size_t routes,
    size_t hidden_dim, size_t hidden_row_stride, size_t intermediate, size_t output_dim,
    size_t down_weight_row_stride_bytes, size_t down_scale_row_stride_bytes,
    float gate_scale_2, float up_scale_2, float down_scale_2);
glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_grouped_staged_accumulate_f32_async(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const uint8_t* gate_weight, const uint8_t* gate_scale, const uint8_t* up_weight,
    const uint8_t* up_scale, const uint8_t* down_weight, const uint8_t* down_scale,
    float* activation_workspace, float* accumulator, size_t rows, size_t routes,
    size_t hidden_dim, size_t hidden_row_stride, size_t intermediate, size_t output_dim,
    size_t down_weight_row_stride_bytes, size_t down_scale_row_stride_bytes,
    float gate_scale_2, float up_scale_2, float down_scale_2, void* cuda_stream);
glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_accumulate_f32(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const glmrt_nvfp4_route_batched_metadata_t* route_metadata, float* activation_workspace,
    float* accumulator, size_t rows, size_t routes, size_t hidden_dim,
    size_t hidden_row_stride, size_t max_intermediate, size_t output_dim);
glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_accumulate_f32_async(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const glmrt_nvfp4_route_batched_metadata_t* route_metadata, float* activation_workspace,
    float* accumulator, size_t rows, size_t routes, size_t hidden_dim,
    size_t hidden_row_stride, size_t max_intermediate, size_t output_dim, void* cuda_stream);
/* The batched route MLP for a single token row (glmrt_native.h:598-607, mlp.cu:474-518, 1186-1231):
 * rows must be 1; out[o] = bf16(sum over the routes whose row index is 0, in route order, of
 * route_weight * (activation[route] . down[o])), truncated, written (not accumulated). */
glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_single_row_bf16(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const glmrt_nvfp4_route_batched_metadata_t* route_metadata, float* activation_workspace,
    uint16_t* out, size_t rows, size_t routes, size_t hidden_dim, size_t hidden_row_stride,
    size_t max_intermediate, size_t output_dim);
glmrt_status_t glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_single_row_bf16_async(
    const uint16_t* hidden, const uint32_t* row_indices, const float* route_weights,
    const glmrt_nvfp4_route_batched_metadata_t* route_metadata, float* activation_workspace,
    uint16_t* out, size_t rows, size_t routes, size_t hidden_dim, size_t hidden_row_stride,
    size_t max_intermediate, size_t output_dim, void* cuda_stream);
/* b12x_direct.cu:203-219: fixed-order float32 sum of the 8 per-route bf16 rows of width
 * 6144 per token, truncated to bf16.  routed_bf16 is [rows * 8, 6144]. */
glmrt_status_t glmrt_cuda_b12x_spark_sum_topk8_bf16_async(
    glmrt_device_buffer_t routed_bf16, glmrt_device_buffer_t output_bf16, size_t rows,
    void* cuda_stream);
/* residual.cu:666-678: dst[row_indices[r]] += row_weights[r] * src[r] (atomic). */
glmrt_status_t glmrt_cuda_scatter_add_rows_bf16_weighted_to_f32(
    const uint16_t* src, const uint32_t* row_indices, const float* row_weights, float* dst,
    size_t rows, size_t row_width);
glmrt_status_t glmrt_cuda_scatter_add_rows_bf16_weighted_to_f32_async(
    const uint16_t* src, const uint32_t* row_indices, const float* row_weights, float* dst,
    size_t rows, size_t row_width, void* cuda_stream);
/* residual.cu:133-158 */
glmrt_status_t glmrt_cuda_gather_rows_bf16_async(const uint16_t* src, const uint32_t* row_indices,
                                                 uint16_t* dst, size_t rows, size_t row_width,
                                                 void* cuda_stream);
/* The rest of the row gather / scatter-add family (glmrt_native.h:757-828; kernels residual.cu:
 * 133-158,409-535).  Scatter-adds decode each compact source row (float32, bf16, row-scaled FP8 =
 * row_width E4M3 bytes + a float32 scale, or NVFP4 = row_width/2 code bytes + row_width/16 E4M3
 * scale bytes) and add it to dst[row_indices[r]]; with at most 64 source rows the contributions
 * of an output value are added in source order (no atomics), above that with float32 atomics.
 * Empty work (rows or row_width 0) is accepted. */
glmrt_status_t glmrt_cuda_gather_rows_f32(const float* src, const uint32_t* row_indices, float* dst,
                                          size_t rows, size_t row_width);
glmrt_status_t glmrt_cuda_gather_rows_f32_async(const float* src, const uint32_t* row_indices,
                                                float* dst, size_t rows, size_t row_width,
                                                void* cuda_stream);
glmrt_status_t glmrt_cuda_gather_rows_bf16(const uint16_t* src, const uint32_t* row_indices,
                                           uint16_t* dst, size_t rows, size_t row_width);
glmrt_status_t glmrt_cuda_scatter_add_rows_f32(const float* src, const uint32_t* row_indices,
                                               float* dst, size_t rows, size_t row_width);
glmrt_status_t glmrt_cuda_scatter_add_rows_f32_async(const float* src, const uint32_t* row_indices,
                                                     float* dst, size_t rows, size_t row_width,
                                                     void* cuda_stream);
glmrt_status_t glmrt_cuda_scatter_add_rows_bf16_to_f32(const uint16_t* src,
                                                       const uint32_t* row_indices, float* dst,
                                                       size_t rows, size_t row_width);
glmrt_status_t glmrt_cuda_scatter_add_rows_bf16_to_f32_async(const uint16_t* src,
                                                             const uint32_t* row_indices, float* dst,
                                                             size_t rows, size_t row_width,
                                                             void* cuda_stream);
glmrt_status_t glmrt_cuda_scatter_add_rows_fp8_e4m3_row_scaled_to_f32(
    const uint8_t* src, size_t src_row_stride_bytes, const uint32_t* row_indices, float* dst,
    size_t rows, size_t row_width);
glmrt_status_t glmrt_cuda_scatter_add_rows_fp8_e4m3_row_scaled_to_f32_async(
    const uint8_t* src, size_t src_row_stride_bytes, const uint32_t* row_indices, float* dst,
    size_t rows, size_t row_width, void* cuda_stream);
glmrt_status_t glmrt_cuda_scatter_add_rows_nvfp4_e2m1_fp8_e4m3_to_f32(
    const uint8_t* src, size_t src_row_stride_bytes, const uint32_t* row_indices, float* dst,
    size_t rows, size_t row_width);
glmrt_status_t glmrt_cuda_scatter_add_rows_nvfp4_e2m1_fp8_e4m3_to_f32_async(
    const uint8_t* src, size_t src_row_stride_bytes, const uint32_t* row_indices, float* dst,
    size_t rows, size_t row_width, void* cuda_stream);
/* Sum of a local partial (float32 or bf16 rows) and one to three peers' wire rows into float32,
 * peers added in order (glmrt_native.h:90-105,829-836; kernel residual.cu:544-589). */
typedef enum glmrt_route_shard_wire_dtype_t {
  GLMRT_ROUTE_SHARD_WIRE_BF16 = 1,
  GLMRT_ROUTE_SHARD_WIRE_FP8_E4M3_ROW_SCALED = 2,
  GLMRT_ROUTE_SHARD_WIRE_NVFP4_E2M1_FP8_E4M3 = 3,
} glmrt_route_shard_wire_dtype_t;
typedef enum glmrt_route_shard_local_dtype_t {
  GLMRT_ROUTE_SHARD_LOCAL_F32 = 1,
  GLMRT_ROUTE_SHARD_LOCAL_BF16 = 2,
} glmrt_route_shard_local_dtype_t;
typedef struct glmrt_route_shard_reduction_buffers_t {
  glmrt_device_buffer_t local;
  glmrt_device_buffer_t peers[3];
  glmrt_device_buffer_t output_f32;
} glmrt_route_shard_reduction_buffers_t;
glmrt_status_t glmrt_cuda_reduce_route_shards_to_f32(
    const glmrt_route_shard_reduction_buffers_t* buffers, size_t rows, size_t row_width,
    size_t peer_row_stride_bytes, uint32_t local_dtype, uint32_t peer_dtype, uint32_t peer_count);
glmrt_status_t glmrt_cuda_reduce_route_shards_to_f32_async(
    const glmrt_route_shard_reduction_buffers_t* buffers, size_t rows, size_t row_width,
    size_t peer_row_stride_bytes, uint32_t local_dtype, uint32_t peer_dtype, uint32_t peer_count,
    void* cuda_stream);
/* Residual adds after the routed/shared MLP (native/include/glmrt_native.h:715-730, kernels
 * native/cuda/kernels/residual.cu:18-62): float32 adds, bf16 results stored by truncation, a
 * float32 delta truncated to bf16 first.  count == 0 is accepted and does nothing. */
glmrt_status_t glmrt_cuda_residual_add_bf16(const uint16_t* residual, const uint16_t* delta,
                                            uint16_t* out, size_t count);
glmrt_status_t glmrt_cuda_residual_add_bf16_async(const uint16_t* residual, const uint16_t* delta,
                                                  uint16_t* out, size_t count, void* cuda_stream);
glmrt_status_t glmrt_cuda_residual_add_f32_delta_bf16(const uint16_t* residual, const float* delta_f32,
                                                      uint16_t* out, size_t count);
glmrt_status_t glmrt_cuda_residual_add_f32_delta_bf16_async(const uint16_t* residual,
                                                            const float* delta_f32, uint16_t* out,
                                                            size_t count, void* cuda_stream);
/* bf16 rows -> E4M3 bytes + one float32 scale per row (glmrt_native.h:776-778, kernel residual.cu:
 * 245-277): scale = max |finite value| / 448 (1 for an all-zero row), byte = e4m3(value / scale),
 * saturating; dst_row_stride_bytes >= row_width + 4 and a multiple of 4. */
glmrt_status_t glmrt_cuda_bf16_rows_to_fp8_e4m3_row_scaled_async(const uint16_t* src, uint8_t* dst,
                                                                 size_t rows, size_t row_width,
                                                                 size_t dst_row_stride_bytes,
                                                                 void* cuda_stream);
/* The same encoding from float32 accumulator rows picked through row_indices (the response pack,
 * glmrt_native.h:766-771, kernel residual.cu:160-196). */
glmrt_status_t glmrt_cuda_gather_rows_f32_to_fp8_e4m3_row_scaled(const float* src,
                                                                 const uint32_t* row_indices,
                                                                 uint8_t* dst, size_t rows,
                                                                 size_t row_width,
                                                                 size_t dst_row_stride_bytes);
glmrt_status_t glmrt_cuda_gather_rows_f32_to_fp8_e4m3_row_scaled_async(
    const float* src, const uint32_t* row_indices, uint8_t* dst, size_t rows, size_t row_width,
    size_t dst_row_stride_bytes, void* cuda_stream);
/* float32 accumulator rows picked through row_indices -> NVFP4 wire rows [row_width/2 packed E2M1 |
 * row_width/16 E4M3 scales] at dst_row_stride_bytes (glmrt_native.h:787-792, kernel
 * nvfp4_payload.cu:75-115): scale = e4m3(amax/6), codes of clamp(x * (1/scale), -6, 6) with the
 * round-to-nearest-even thresholds.  src must be 16-byte aligned. */
glmrt_status_t glmrt_cuda_gather_rows_f32_to_nvfp4_e2m1_fp8_e4m3(const float* src,
                                                                 const uint32_t* row_indices,
                                                                 uint8_t* dst, size_t rows,
                                                                 size_t row_width,
                                                                 size_t dst_row_stride_bytes);
glmrt_status_t glmrt_cuda_gather_rows_f32_to_nvfp4_e2m1_fp8_e4m3_async(
    const float* src, const uint32_t* row_indices, uint8_t* dst, size_t rows, size_t row_width,
    size_t dst_row_stride_bytes, void* cuda_stream);
/* out = bf16(residual + bf16(shared_delta + bf16(routed_delta_f32))) */
glmrt_status_t glmrt_cuda_residual_add_shared_f32_delta_bf16(
    const uint16_t* residual, const uint16_t* shared_delta, const float* routed_delta_f32,
    uint16_t* out, size_t count);
glmrt_status_t glmrt_cuda_residual_add_shared_f32_delta_bf16_async(
    const uint16_t* residual, const uint16_t* shared_delta, const float* routed_delta_f32,
    uint16_t* out, size_t count, void* cuda_stream);

/* ------------------------------------------------------------------------ */
/* Layer-level entry points (additions).                                      */
/*                                                                            */
/* A layer object owns the NVFP4 weights of its local experts in tensor-core   */
/* layout plus all work buffers for up to max_tokens rows.  It replaces, for   */
/* one sparse layer, what the reference does in                                */
/* RealNvfp4ProtocolV2Executor::execute_protocol_v2_unordered                  */
/* (rust/crates/glmrt-daemon/src/commands/real_full/expert_probe/              */
/* protocol_v2_executor.rs:1882-2493) plus the coordinator-side router and     */
/* activation quantiser (sparse_mlp/router.rs:184-219,                         */
/* coordinator_kernels/activation.rs:34-92).                                   */
/* ------------------------------------------------------------------------ */
typedef struct glmrt_b200_moe_config_t {
  uint32_t hidden_dim;        /* H, multiple of 256 */
  uint32_t intermediate_dim;  /* I, multiple of 256 */
  uint32_t experts;           /* routed experts in the whole layer, <= 1024 */
  uint32_t top_k;             /* 1..16 */
  uint32_t max_tokens;        /* capacity in rows per forward call */
  uint32_t ep_world;          /* expert-parallel world size (1 = all experts local) */
  uint32_t ep_rank;           /* expert e is local iff e % ep_world == ep_rank
                                 (rust/crates/glmrt-core/src/placement.rs:25-42) */
  uint32_t flags;             /* GLMRT_B200_LAYER_* */
  float routed_scaling;       /* 2.5 for GLM-5.2 */
} glmrt_b200_moe_config_t;

enum {
  GLMRT_B200_LAYER_ENGINE_SIMT = 1u, /* run the expert FFN on the SIMT verification kernels */
  GLMRT_B200_LAYER_PAIR_FC1 = 2u,    /* batches above 192 routes per expert: plan 256-slot work items and run */
  GLMRT_B200_LAYER_PAIR_FC2 = 4u,    /* FC1 and/or FC2 on CTA pairs (tcgen05 cta_group::2) instead of one-CTA
                                        tiles; bit-identical results */
  GLMRT_B200_LAYER_PAIR_TILES = 6u,  /* both */
  GLMRT_B200_LAYER_ORDERED_COMBINE = 8u, /* batches above 256 rows: keep one bf16 row per route and sum them in
                                        route order in a pass of its own (bit-reproducible), instead of letting
                                        the down projection add weight * row into the output rows as the routes
                                        finish (the reference has both forms too: fixed-order top-k sum,
                                        native/cuda/kernels/b12x_direct.cu:203-219, and in-kernel accumulation,
                                        b12x_direct.cu:157-165,1291-1309, mlp.cu:275-314).  Batches of at most 256
                                        rows always use the ordered form. */
};

glmrt_status_t glmrt_b200_moe_layer_create(const glmrt_b200_moe_config_t* config, void** out_layer);
glmrt_status_t glmrt_b200_moe_layer_destroy(void* layer);
/* An execution lane: a handle that shares the expert weights and router of `layer` and owns a  */
/* workspace of its own, so that several host threads / streams can run the same experts at     */
/* once -- the reference executor keeps one route-tensor cache per lane behind a mutex and      */
/* serves up to 8 lanes (expert_probe/protocol_v2_executor.rs:123-126,674-690;                  */
/* rust/crates/glmrt-transport/src/host_batch_set.rs:52).  Every layer entry point accepts a    */
/* lane.  max_tokens: row capacity of the lane's workspace (0 = the layer's), e.g. a decode lane */
/* and a prefill lane on the same experts.  Weights may be (re)loaded through any handle, with   */
/* no forward in flight on the others.  The memory of the weights is released when the last     */
/* handle that shares it is destroyed.  The layer's device must be current.                      */
glmrt_status_t glmrt_b200_moe_layer_create_lane(void* layer, uint32_t max_tokens, void** out_lane);
/* A layer with weights of its own that shares the WORKSPACE of `workspace_layer` (same shape,  */
/* max_tokens and shard): the sparse layers of a model run one after the other                   */
/* (docs/balanced-path.md:53-66: 75 serially dependent sparse layers per cycle), so a stack     */
/* needs the expert weights of every layer but one workspace.  Handles that share a workspace   */
/* must run on one stream, in order; in the expert-parallel path the exchange buffers belong    */
/* to the workspace, so a stack attaches once (through any of its layers) and the epoch         */
/* counter of the exchange runs through all of them.                                             */
glmrt_status_t glmrt_b200_moe_layer_create_stacked(const glmrt_b200_moe_config_t* config, void* workspace_layer,
                                                   void** out_layer);
/* float32 router weight [experts, hidden_dim] and bias [experts] (device memory). */
glmrt_status_t glmrt_b200_moe_layer_set_router(void* layer, glmrt_device_buffer_t weight_f32,
                                               glmrt_device_buffer_t bias_f32, void* cuda_stream);
/* One expert's projections in the reference's tensor layout (route.rs:6732-6757):
 * gate/up codes [I, H/2], scales [I, H/16]; down codes [H, I/2], scales [H, I/16];
 * value = code * e4m3(scale) * scale_2.  Non-local experts are rejected. */
glmrt_status_t glmrt_b200_moe_layer_set_expert(
    void* layer, uint32_t expert_id, glmrt_device_buffer_t gate_codes,
    glmrt_device_buffer_t gate_scales, glmrt_device_buffer_t up_codes,
    glmrt_device_buffer_t up_scales, glmrt_device_buffer_t down_codes,
    glmrt_device_buffer_t down_scales, float gate_scale_2, float up_scale_2, float down_scale_2,
    void* cuda_stream);
/* Seeded synthetic expert weights generated and quantised on the device (benchmarks). */
glmrt_status_t glmrt_b200_moe_layer_fill_synthetic(void* layer, uint64_t seed, float weight_std,
                                                   void* cuda_stream);

/* One forward pass: router -> quantise -> plan/dispatch -> FC1+SwiGLU+requant -> FC2 ->
 * combine.  hidden_bf16 and output_bf16 are [rows, hidden_dim] bf16 in device memory.
 * topk_indices / topk_weights ([rows, top_k] uint32 / float) are optional (ptr may be
 * NULL).  ep_world must be 1 for this entry point. */
glmrt_status_t glmrt_b200_moe_layer_forward_async(
    void* layer, glmrt_device_buffer_t hidden_bf16, size_t rows, glmrt_device_buffer_t output_bf16,
    glmrt_device_buffer_t topk_indices, glmrt_device_buffer_t topk_weights, void* cuda_stream);
/* The same forward with the residual step of the sparse layer folded into the combine kernel
 * (python/reference/glmrt_reference/glm_moe_dsa_layer_ref.py:196-198 hidden + routed + shared, in
 * the arithmetic of native/cuda/kernels/residual.cu:47-58): output = bf16(residual +
 * bf16(shared_delta + routed)), truncating stores; shared_delta_bf16.ptr may be NULL (no shared
 * expert: output = bf16(residual + routed)).  hidden_bf16 is the normalised input of the router
 * and the experts, residual_bf16 the un-normalised layer input.  ep_world must be 1. */
glmrt_status_t glmrt_b200_moe_layer_forward_residual_async(
    void* layer, glmrt_device_buffer_t hidden_bf16, size_t rows, glmrt_device_buffer_t residual_bf16,
    glmrt_device_buffer_t shared_delta_bf16, glmrt_device_buffer_t output_bf16, void* cuda_stream);
/* Same with host buffers: copies the rows in from `hidden_host`, runs the layer, copies the
 * result out to `output_host` and synchronises the stream.  Host memory may be pageable;
 * pinned memory makes the copies asynchronous. */
glmrt_status_t glmrt_b200_moe_layer_forward_host(void* layer, const void* hidden_host, size_t rows,
                                                 void* output_host, void* cuda_stream);
/* Routed forward with caller-supplied routes (the expert worker's view of a request:
 * rows + (expert, weight) routes; protocol_v2.rs:236-310).  Skips the router.  An index entry
 * 0xFFFFFFFF means "no route" (a row with fewer than top_k experts on this worker) and is
 * skipped; any other id outside the layer is reported by glmrt_b200_moe_layer_check.  Routes of
 * experts that live on another shard (ep_world > 1) are skipped as well: the result is this
 * shard's partial. */
glmrt_status_t glmrt_b200_moe_layer_forward_routed_async(
    void* layer, glmrt_device_buffer_t hidden_bf16, size_t rows, glmrt_device_buffer_t topk_indices,
    glmrt_device_buffer_t topk_weights, glmrt_device_buffer_t output_bf16, void* cuda_stream);

/* Device-side error word of the last forward (0 = none): bounded waits that gave up and
 * capacity overflows are reported here instead of hanging or faulting.  Synchronises. */
glmrt_status_t glmrt_b200_moe_layer_check(void* layer, void* cuda_stream);

/* Introspection for tests and profiling. */
typedef enum glmrt_b200_debug_buffer_t {
  GLMRT_B200_DEBUG_PAYLOAD = 0,      /* [rows, H/2 + H/16] activation payload */
  GLMRT_B200_DEBUG_ROUTE_SLOT = 1,   /* int32 [rows * top_k] slot of each route (-1 = not local) */
  GLMRT_B200_DEBUG_ACT1_CODES = 2,   /* [slots, H/2] expert-sorted activation codes */
  GLMRT_B200_DEBUG_ACT1_SF = 3,      /* tiled scales of ACT1 */
  GLMRT_B200_DEBUG_ACT2_CODES = 4,   /* [slots, I/2] requantised SwiGLU output */
  GLMRT_B200_DEBUG_ACT2_SF = 5,
  GLMRT_B200_DEBUG_ROUTE_ROWS = 6,   /* bf16 [rows * top_k, H] per-route FC2 output */
  GLMRT_B200_DEBUG_COUNTERS = 7,     /* uint32 [8]: chunks, slots, error, ... */
  GLMRT_B200_DEBUG_CHUNKS = 8,       /* int32 [chunks][4]: expert, slot_base, tokens, 0 */
  GLMRT_B200_DEBUG_EXPERT_COUNTS = 9, /* int32 [local experts] routes per expert */
  GLMRT_B200_DEBUG_GATE_CODES = 10,   /* [local experts * I, H/2] */
  GLMRT_B200_DEBUG_UP_CODES = 11,
  GLMRT_B200_DEBUG_DOWN_CODES = 12,   /* [local experts * H, I/2] */
  GLMRT_B200_DEBUG_GATE_SF = 13,      /* tiled scales */
  GLMRT_B200_DEBUG_UP_SF = 14,
  GLMRT_B200_DEBUG_DOWN_SF = 15,
  GLMRT_B200_DEBUG_SCALE2 = 16,       /* float [local experts][3] = gate, up, down */
  GLMRT_B200_DEBUG_TOPK_IDX = 17,     /* uint32 [rows * top_k] */
  GLMRT_B200_DEBUG_TOPK_W = 18        /* float [rows * top_k] */
} glmrt_b200_debug_buffer_t;
glmrt_status_t glmrt_b200_moe_layer_debug_buffer(void* layer, uint32_t which,
                                                 glmrt_device_buffer_t* out);
/* Statistics of the last forward (after a stream synchronise): kernels launched by this
 * library, distinct experts touched, slots used. */
typedef struct glmrt_b200_layer_stats_t {
  uint64_t launches_total;
  uint32_t launches_last_forward;
  uint32_t chunks;
  uint32_t slots;
  uint32_t distinct_experts;
  uint32_t device_error;
  uint32_t reserved;
} glmrt_b200_layer_stats_t;
glmrt_status_t glmrt_b200_moe_layer_stats(void* layer, glmrt_b200_layer_stats_t* out);

/* ------------------------------------------------------------------------ */
/* NCCL wrappers (native/include/glmrt_native.h:428-444; implementation       */
/* native/src/glmrt_native.cc:1453-1757).  Same signatures and argument rules. */
/* NCCL is resolved at run time (GLMRT_NCCL_LIB or libnccl.so.2); without it    */
/* every entry point returns GLMRT_STATUS_NCCL_UNAVAILABLE.  Not on the data   */
/* path of the expert-parallel forward below; kept for callers of the          */
/* reference ABI and as its cross-check.                                       */
/* ------------------------------------------------------------------------ */
glmrt_status_t glmrt_nccl_unique_id_bytes(size_t* out_bytes);
glmrt_status_t glmrt_nccl_get_unique_id(void* out, size_t out_bytes);
glmrt_status_t glmrt_nccl_comm_init_rank(const void* unique_id, size_t unique_id_bytes, int world_size,
                                         int rank, void** out_handle);
glmrt_status_t glmrt_nccl_gather_u8_async(void* handle, glmrt_device_buffer_t send,
                                          glmrt_device_buffer_t recv, size_t bytes, int root,
                                          void* cuda_stream);
/* rows are split into world contiguous slices (the first rows % world one row longer); rank r
 * receives every peer's copy of slice r, back to back in peer order. */
glmrt_status_t glmrt_nccl_row_all_to_all_u8_async(void* handle, glmrt_device_buffer_t send,
                                                  glmrt_device_buffer_t recv, size_t rows,
                                                  size_t row_stride_bytes, void* cuda_stream);
glmrt_status_t glmrt_nccl_all_reduce_bf16_async(void* handle, glmrt_device_buffer_t send,
                                                glmrt_device_buffer_t recv, size_t values,
                                                void* cuda_stream);
glmrt_status_t glmrt_nccl_reduce_bf16_async(void* handle, glmrt_device_buffer_t send,
                                            glmrt_device_buffer_t recv, size_t values, int root,
                                            void* cuda_stream);
glmrt_status_t glmrt_nccl_comm_destroy(void* handle);

/* ------------------------------------------------------------------------ */
/* Expert-parallel forward over NVLink peer memory (additions).               */
/* Replaces the ExpertProtocolV2 TCP/RDMA transport between coordinator and    */
/* expert hosts (rust/crates/glmrt-transport/src/protocol_v2.rs:236-310) and   */
/* the NCCL row all-to-all between shards (native/src/glmrt_native.cc:         */
/* 1593-1659): rank r owns experts e % ep_world == r and is home to its own    */
/* rows; routed rows and results travel as in-kernel stores into the peer's    */
/* memory.  Set-up: every rank exports its buffers (ipc_export), opens every    */
/* peer's (ipc_open), tells the others where it sees their result rows, and    */
/* attaches.  A single process driving several layer objects on one device     */
/* may attach with glmrt_b200_ep_local_buffers pointers directly.              */
/* ------------------------------------------------------------------------ */
typedef struct glmrt_b200_ep_buffers_t {
  void* act_codes;   /* [slots, H/2] rows pushed by home ranks */
  void* act_sf;      /* tiled scales of the same */
  void* slot_out;    /* [slots] result-row address per slot */
  void* route_rows;  /* bf16 [rows * top_k, H] result rows pushed by owners */
  void* control;     /* histograms and epoch flags */
  void* act_sf_rows; /* [slots, H/16] row-major scale bytes of prefill-sized pushes (re-tiled by the owner) */
} glmrt_b200_ep_buffers_t;
#define GLMRT_B200_EP_IPC_BYTES 384 /* six 64-byte CUDA IPC handles */
glmrt_status_t glmrt_b200_ep_local_buffers(void* layer, glmrt_b200_ep_buffers_t* out);
glmrt_status_t glmrt_b200_ep_ipc_export(void* layer, void* out_handles, size_t bytes);
glmrt_status_t glmrt_b200_ep_ipc_open(void* layer, const void* handles, size_t bytes,
                                      glmrt_b200_ep_buffers_t* out_mapped);
/* peers[p] = rank p's buffers as addressable from this process (own rank: local buffers);
 * my_rows_in_peer[p] = the address under which rank p sees THIS rank's route_rows. */
glmrt_status_t glmrt_b200_ep_attach(void* layer, const glmrt_b200_ep_buffers_t* peers, size_t world,
                                    const uint64_t* my_rows_in_peer);
/* Collective: every rank calls it once per step with its own rows (rows may differ per rank and
 * may be 0).  Phases: 0 route + publish counts, 1 plan + push rows, 2 expert GEMMs + push results,
 * 3 combine.  forward_ep_async runs 0..3; the phase entry point lets one process step several
 * ranks that share a device (kernels that wait on one another must not be queued behind each
 * other).  Waits are bounded; expiry is reported by glmrt_b200_moe_layer_check. */
/* Optional: the row count of the whole batch over all ranks for the steps that follow (0 =     */
/* unknown).  All ranks must state the same value.  The exchange uses decode-sized work items    */
/* up to 256 rows and prefill-sized ones above; without this call it goes by max_tokens.         */
glmrt_status_t glmrt_b200_ep_set_global_rows(void* layer, uint32_t global_rows);
glmrt_status_t glmrt_b200_moe_layer_forward_ep_async(void* layer, glmrt_device_buffer_t hidden_bf16,
                                                     size_t rows, glmrt_device_buffer_t output_bf16,
                                                     void* cuda_stream);
glmrt_status_t glmrt_b200_moe_layer_forward_ep_phase_async(void* layer, uint32_t phase,
                                                           glmrt_device_buffer_t hidden_bf16, size_t rows,
                                                           glmrt_device_buffer_t output_bf16, void* cuda_stream);
glmrt_status_t glmrt_b200_moe_layer_forward_ep_host(void* layer, const void* hidden_host, size_t rows,
                                                    void* output_host, void* cuda_stream);

/* ------------------------------------------------------------------------ */
/* ExpertProtocolV2 frames and the expert executor (host side).               */
/* The wire format of rust/crates/glmrt-transport/src/protocol_v2.rs and its   */
/* protocol_v2/{request,response,view}.rs: little-endian, 96-byte headers      */
/* (128 with the debug checksum), 40-byte row descriptors, 10-byte route       */
/* entries (row, expert, bf16 gate weight), then the row payload.  Regular     */
/* request and response frames are encoded, parsed and validated with the      */
/* reference's rules; the executor also takes streamed ingress (a stream-plan  */
/* frame followed by stream-data frames); layer-block frames are recognised    */
/* and refused.  All functions are host-only and need no GPU except            */
/* glmrt_b200_pv2_execute.                                                     */
/* ------------------------------------------------------------------------ */
enum {                                     /* protocol_v2.rs:10-34 */
  GLMRT_B200_PV2_REQUEST_HEADER_LEN = 96,
  GLMRT_B200_PV2_RESPONSE_HEADER_LEN = 96,
  GLMRT_B200_PV2_DEBUG_HEADER_LEN = 128,
  GLMRT_B200_PV2_ROW_DESCRIPTOR_LEN = 40,
  GLMRT_B200_PV2_ROUTE_ENTRY_LEN = 10,
  GLMRT_B200_PV2_FLAG_DEBUG_CHECKSUM = 1u << 0,
  GLMRT_B200_PV2_FLAG_PRECOMPILE_WARMUP = 1u << 1,
  GLMRT_B200_PV2_FLAG_RESPONSE_ROW_INDICES = 1u << 2,
  GLMRT_B200_PV2_FLAG_RESPONSE_MORE_CHUNKS = 1u << 3,
  GLMRT_B200_PV2_FLAG_RESPONSE_FP8_E4M3_ROW_SCALED = 1u << 4,
  GLMRT_B200_PV2_FLAG_RESPONSE_NVFP4_E2M1_FP8_E4M3 = 1u << 5,
  GLMRT_B200_PV2_FLAG_STREAM_PLAN = 1u << 6,
  GLMRT_B200_PV2_FLAG_STREAM_DATA = 1u << 7,
  GLMRT_B200_PV2_FLAG_STREAM_FINAL = 1u << 8,
  GLMRT_B200_PV2_FLAG_SPARK_REDUCTION = 1u << 9,
  GLMRT_B200_PV2_FLAG_LAYER_BLOCK = 1u << 10,
  GLMRT_B200_PV2_FLAG_SPARK_ROW_SHARDED_REDUCTION = 1u << 11,
  GLMRT_B200_PV2_SPARK_COLLECTIVE_PART_COUNT_SHIFT = 12,   /* four bits */
};
enum {                                     /* ExpertV2Dtype, protocol_v2.rs:44-51 */
  GLMRT_B200_PV2_DTYPE_BF16 = 1,
  GLMRT_B200_PV2_DTYPE_F16 = 2,
  GLMRT_B200_PV2_DTYPE_FP8_DEBUG = 3,
  GLMRT_B200_PV2_DTYPE_NVFP4_E2M1_FP8_E4M3 = 4,   /* elements/2 code bytes + elements/16 scale bytes per row */
  GLMRT_B200_PV2_DTYPE_FP8_E4M3_ROW_SCALED = 5,   /* elements bytes + one float32 scale per row */
};
typedef struct glmrt_b200_pv2_request_header_t {   /* ExpertProtocolV2RequestHeader, protocol_v2.rs:236-250 */
  uint64_t request_id;
  uint64_t placement_version;
  uint32_t layer_id;
  uint32_t row_count;
  uint32_t hidden_dim;
  uint32_t hidden_dtype;
  uint32_t hidden_row_stride_bytes;
  uint32_t route_count;
  uint32_t row_descriptor_bytes;
  uint32_t route_bytes;
  uint64_t hidden_payload_bytes;
  uint32_t flags;
  uint32_t header_len;            /* 96 or 128; filled by parse and encode */
} glmrt_b200_pv2_request_header_t;
typedef struct glmrt_b200_pv2_row_t {               /* ExpertProtocolV2RowDescriptor, protocol_v2.rs:252-260 */
  uint64_t row_id;
  uint64_t source_request_id;
  uint64_t token_position;
  uint32_t route_offset;
  uint32_t route_count;
  uint32_t source_kind;           /* 1 decode, 2 prefill, 3 MTP verify, 4 benchmark */
  uint32_t reserved;
} glmrt_b200_pv2_row_t;
typedef struct glmrt_b200_pv2_route_t {             /* ExpertProtocolV2RouteEntry, protocol_v2.rs:262-267 */
  uint32_t row_index;
  uint32_t expert_id;
  float gate_weight;              /* travels as bf16 (truncated), protocol_v2.rs:584-608 */
} glmrt_b200_pv2_route_t;
typedef struct glmrt_b200_pv2_response_header_t {   /* ExpertProtocolV2ResponseHeader, protocol_v2.rs:269-282 */
  uint64_t request_id;
  uint64_t placement_version;
  uint32_t layer_id;
  uint32_t row_count;
  uint32_t output_dim;
  uint32_t output_dtype;
  uint32_t output_row_stride_bytes;
  uint32_t status;                /* 0 ok, 1 error */
  uint64_t output_payload_bytes;
  uint32_t flags;
  uint32_t header_len;
  uint64_t executor_id;
} glmrt_b200_pv2_response_header_t;
/* Where the sections of a parsed frame start (byte offsets into the frame). */
typedef struct glmrt_b200_pv2_sections_t {
  uint64_t rows_offset;           /* request: row descriptors; response: row-index table (or payload_offset) */
  uint64_t routes_offset;         /* request only */
  uint64_t payload_offset;
  uint64_t payload_bytes;
} glmrt_b200_pv2_sections_t;

/* ExpertV2Dtype::row_bytes (protocol_v2.rs:61-83). */
glmrt_status_t glmrt_b200_pv2_row_bytes(uint32_t dtype, size_t elements, size_t* out_bytes);
/* expert_protocol_v2_compact_id (protocol_v2.rs:229-232): first 8 bytes, little-endian, of SHA-256(name). */
glmrt_status_t glmrt_b200_pv2_compact_id(const char* name, uint64_t* out_id);
/* SHA-256 of a byte range (the digest behind the debug checksum and the compact id). */
glmrt_status_t glmrt_b200_pv2_sha256(const void* bytes, size_t len, uint8_t out_digest[32]);
/* ExpertProtocolV2Request::{validate, encode_into} (protocol_v2/request.rs:327-379, 516-633).  The
 * counts and byte sizes of `header` are taken from the arguments; request_id, placement_version,
 * layer_id, hidden_dim, hidden_dtype, hidden_row_stride_bytes (0 = the dtype's row size) and flags
 * from `header`.  Gate weights are made canonical (bf16) first.  *out_len receives the frame size
 * also when `out` is too small (BUFFER_TOO_SMALL). */
glmrt_status_t glmrt_b200_pv2_encode_request(const glmrt_b200_pv2_request_header_t* header,
                                             const glmrt_b200_pv2_row_t* rows, size_t row_count,
                                             const glmrt_b200_pv2_route_t* routes, size_t route_count,
                                             const void* hidden_payload, size_t hidden_payload_bytes,
                                             void* out, size_t out_capacity, size_t* out_len);
/* ExpertProtocolV2RequestView::parse (protocol_v2/view.rs:33-136): validates the frame and all
 * rows and routes like Request::decode, without copying and without checking the checksum. */
glmrt_status_t glmrt_b200_pv2_parse_request(const void* frame, size_t frame_bytes,
                                            glmrt_b200_pv2_request_header_t* out_header,
                                            glmrt_b200_pv2_sections_t* out_sections);
glmrt_status_t glmrt_b200_pv2_request_row(const void* frame, size_t frame_bytes, size_t index,
                                          glmrt_b200_pv2_row_t* out_row);
glmrt_status_t glmrt_b200_pv2_request_route(const void* frame, size_t frame_bytes, size_t index,
                                            glmrt_b200_pv2_route_t* out_route);
/* verify_checksum (protocol_v2/view.rs:299-330, :581-600): OK when the frame carries no checksum. */
glmrt_status_t glmrt_b200_pv2_verify_request_checksum(const void* frame, size_t frame_bytes);
glmrt_status_t glmrt_b200_pv2_verify_response_checksum(const void* frame, size_t frame_bytes);
/* ExpertProtocolV2Response::{validate, encode_into} (protocol_v2/response.rs:130-174, 577-642).
 * row_indices may be NULL unless the header's flags ask for the row-index table. */
glmrt_status_t glmrt_b200_pv2_encode_response(const glmrt_b200_pv2_response_header_t* header,
                                              const uint32_t* row_indices, const void* payload,
                                              size_t payload_bytes, void* out, size_t out_capacity,
                                              size_t* out_len);
glmrt_status_t glmrt_b200_pv2_parse_response(const void* frame, size_t frame_bytes,
                                             glmrt_b200_pv2_response_header_t* out_header,
                                             glmrt_b200_pv2_sections_t* out_sections);
/* The executor (ProtocolV2ExpertExecutor::execute_with_identity, glmrt-transport/src/synthetic.rs:
 * 51-66, in the role of RealNvfp4ProtocolV2Executor, protocol_v2_executor.rs:1882-2493): parses a
 * regular request frame, runs its rows through the experts of `layer` that its routes name
 * (hidden dtype bf16 or NVFP4 payload rows; at most top_k routes per row; routes of experts that
 * do not live on this layer's shard are refused) and writes a response frame with one partial
 * output row per request row: bf16, or NVFP4 payload rows (native rounding rule) or row-scaled
 * FP8 rows when the request's flags negotiate them.  The executor id is the compact
 * id of "b200-nvfp4-tcgen05-executor".  Synchronises `cuda_stream`.
 * Streamed ingress (protocol_v2/stream.rs:9-27, protocol_v2_executor.rs:1936-1945): a frame with
 * GLMRT_B200_PV2_FLAG_STREAM_PLAN carries the request's rows and routes and a "GLMSTRM2" plan
 * (an ordering of the rows in route groups) as its payload and opens a stream on `layer`; the
 * frames with GLMRT_B200_PV2_FLAG_STREAM_DATA that follow carry the payload rows named in their
 * row table.  Those calls return OK with *response_len = 0; the call that brings the frame with
 * GLMRT_B200_PV2_FLAG_STREAM_FINAL runs the request and writes the response a regular request
 * with the same rows would get.  One stream per layer handle at a time: a new plan frame replaces
 * the stream in progress, and a final frame that comes before every row has arrived ends it. */
glmrt_status_t glmrt_b200_pv2_execute(void* layer, const void* request_frame, size_t request_bytes,
                                      void* response_out, size_t response_capacity,
                                      size_t* response_len, void* cuda_stream);

/* Per-stage device times of the last forward, measured with CUDA events recorded on the
 * caller's stream between the kernels (reference precedent: the CUDA-event timeline behind
 * GLMRT_REAL_FULL_NVFP4_ROUTE_CUDA_EVENT_TIMING, sparse_mlp/route.rs:1010-1062). */
typedef enum glmrt_b200_stage_t {
  GLMRT_B200_STAGE_ROUTER = 0,
  GLMRT_B200_STAGE_QUANTIZE = 1,     /* 0 when quantise and dispatch run as one kernel (the usual case) */
  GLMRT_B200_STAGE_PLAN = 2,
  GLMRT_B200_STAGE_DISPATCH = 3,     /* dispatch, or the fused quantise + dispatch kernel */
  GLMRT_B200_STAGE_FC1 = 4,
  GLMRT_B200_STAGE_FC2 = 5,
  GLMRT_B200_STAGE_COMBINE = 6,
  GLMRT_B200_STAGE_COUNT = 7
} glmrt_b200_stage_t;
glmrt_status_t glmrt_b200_moe_layer_set_profiling(void* layer, int enable);
/* out_ms receives GLMRT_B200_STAGE_COUNT floats; waits for the last forward to finish. */
glmrt_status_t glmrt_b200_moe_layer_stage_times(void* layer, float* out_ms, size_t count);

/* Measurement aid (no counterpart in the reference): the rate at which all SMs together can bring
 * operand tiles into shared memory with the copy shapes of the prefill FC1 kernel (per stage three
 * 128-row x 128-byte TMA boxes and three 2 KB scale copies, `stages` stages of 54 KB in flight per
 * SM, nothing consumed).  working_set_bytes well below the L2 size measures L2 -> shared memory,
 * far above it HBM -> shared memory.  Allocates and frees its own buffers; synchronises the stream. */
glmrt_status_t glmrt_b200_probe_operand_delivery(size_t working_set_bytes, uint32_t stages, uint32_t tiles_per_cta,
                                                 float* out_gb_per_s, float* out_ms, void* cuda_stream);

#ifdef __cplusplus
}
#endif
