// Measurement probe: how fast can the SMs pull operand tiles out of L2 (or HBM) into shared memory
// with the copy shapes of the prefill expert GEMM and nothing else to do?
//
// The token-major FC1 kernel (gemm_tc_prefill.cu) brings 54 KB into shared memory per 256-element
// K stage: three 128-row x 128-byte TMA boxes (token rows, gate rows, up rows) and three 2 KB bulk
// copies of scales, four stages in flight per SM.  This kernel issues exactly those copies, from a
// buffer laid out like the weights (rows of `row_bytes`), and frees every stage the moment it has
// landed: no tensor-core work, no epilogue.  With a working set that fits the L2 it measures the
// L2 -> shared-memory delivery rate that bounds that kernel once its weights are L2 hits; with a
// working set far above the L2 it measures the HBM -> shared-memory rate of the same access shape.
// It has no counterpart in the reference (a measurement aid of this library).
#include <cuda.h>

#include "common.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace glmrt {
namespace {

using namespace tc;

constexpr int kProbeStageBytes = 3 * 128 * kStageBytesK + 3 * kSfStageBytes;   // 55296, as FC1's stage
constexpr int kProbeThreads = 64;

template <int kStages>
__global__ void __launch_bounds__(kProbeThreads, 1)
l2_probe_kernel(const __grid_constant__ CUtensorMap map, const uint8_t* __restrict__ scales, int row_blocks,
                int k_stages, int tiles_per_cta, uint32_t* error_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kStages) * kProbeStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(bars + 2 * kStages);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int warp = threadIdx.x / 32;
  if (warp == 0) {
    // producer: the copies of one FC1 stage per slot
    const uint64_t pol = policy_evict_last();
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int t = 0; t < tiles_per_cta && alive; ++t) {
      // three different row blocks per tile (token rows, gate rows, up rows), walked over the working set
      const long long tile = static_cast<long long>(blockIdx.x) + static_cast<long long>(t) * gridDim.x;
      const int rb0 = static_cast<int>((tile * 3) % row_blocks), rb1 = static_cast<int>((tile * 3 + 1) % row_blocks),
                rb2 = static_cast<int>((tile * 3 + 2) % row_blocks);
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_warp(&empty_bar[stage], phase ^ 1u, abort_flag)) { alive = false; break; }
        if (elect_one()) {
          const uint32_t s0 = smem_u32(smem + static_cast<size_t>(stage) * kProbeStageBytes);
          mbar_expect_tx(&full_bar[stage], kProbeStageBytes);
          tma_load_2d(s0, &map, &full_bar[stage], ks * kStageBytesK, rb0 * 128, pol);
          tma_load_2d(s0 + 128 * kStageBytesK, &map, &full_bar[stage], ks * kStageBytesK, rb1 * 128, pol);
          tma_load_2d(s0 + 256 * kStageBytesK, &map, &full_bar[stage], ks * kStageBytesK, rb2 * 128, pol);
          const uint32_t ssf = s0 + 384 * kStageBytesK;
          const size_t sf0 = (static_cast<size_t>(rb0) * k_stages + ks) * kSfStageBytes;
          const size_t sf1 = (static_cast<size_t>(rb1) * k_stages + ks) * kSfStageBytes;
          const size_t sf2 = (static_cast<size_t>(rb2) * k_stages + ks) * kSfStageBytes;
          bulk_load(ssf, scales + sf0, kSfStageBytes, &full_bar[stage], pol);
          bulk_load(ssf + kSfStageBytes, scales + sf1, kSfStageBytes, &full_bar[stage], pol);
          bulk_load(ssf + 2 * kSfStageBytes, scales + sf2, kSfStageBytes, &full_bar[stage], pol);
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // consumer: a stage is free again as soon as it has landed
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int t = 0; t < tiles_per_cta && alive; ++t) {
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag)) { alive = false; break; }
        if (elect_one()) mbar_arrive(&empty_bar[stage]);
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
  }
  __syncthreads();
  if (*abort_flag != 0u) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);   // let copies in flight land
    if (threadIdx.x == 0) atomicOr(error_word, static_cast<uint32_t>(kErrWaitTimeout));
  }
}

}  // namespace
}  // namespace glmrt

using namespace glmrt;

extern "C" glmrt_status_t glmrt_b200_probe_operand_delivery(size_t working_set_bytes, uint32_t stages,
                                                            uint32_t tiles_per_cta, float* out_gb_per_s,
                                                            float* out_ms, void* cuda_stream) {
  if (out_gb_per_s == nullptr || out_ms == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "operand-delivery probe: null output");
  if (stages != 2 && stages != 3 && stages != 4)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "operand-delivery probe: stages must be 2, 3 or 4");
  if (tiles_per_cta == 0 || tiles_per_cta > 4096)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "operand-delivery probe: tiles_per_cta must be 1..4096");
  constexpr size_t kRowBytes = 3072, kStagesK = kRowBytes / tc::kStageBytesK;   // a hidden-6144 FP4 row, 24 stages
  const size_t block_bytes = 128 * kRowBytes;
  if (working_set_bytes < 3 * block_bytes || working_set_bytes > (size_t(16) << 30))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "operand-delivery probe: working set must be 1.2 MB .. 16 GB");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const int row_blocks = static_cast<int>(working_set_bytes / block_bytes);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  uint8_t *codes = nullptr, *scales = nullptr;
  uint32_t* err_word = nullptr;
  const size_t code_bytes = static_cast<size_t>(row_blocks) * block_bytes;
  const size_t scale_bytes = static_cast<size_t>(row_blocks) * kStagesK * tc::kSfStageBytes;
  cudaError_t err = cudaMalloc(&codes, code_bytes);
  if (err == cudaSuccess) err = cudaMalloc(&scales, scale_bytes);
  if (err == cudaSuccess) err = cudaMalloc(&err_word, 4);
  if (err != cudaSuccess) {
    cudaFree(codes); cudaFree(scales); cudaFree(err_word);
    cudaGetLastError();
    return fail_cuda(GLMRT_STATUS_ALLOCATION_FAILED, "operand-delivery probe: cudaMalloc", err);
  }
  cudaMemsetAsync(codes, 0x11, code_bytes, s);
  cudaMemsetAsync(scales, 0x38, scale_bytes, s);
  cudaMemsetAsync(err_word, 0, 4, s);
  CUtensorMap map;
  glmrt_status_t st = make_codes_tensor_map(&map, codes, static_cast<uint64_t>(row_blocks) * 128, kRowBytes, 128);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  float ms = 0.0f;
  uint32_t device_error = 0;
  if (st == GLMRT_STATUS_OK) {
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    auto launch = [&](int tiles) {
      const size_t smem = static_cast<size_t>(stages) * kProbeStageBytes + 1024 + 256;
      const int k_stages = static_cast<int>(kStagesK);
      if (stages == 4) {
        cudaFuncSetAttribute(l2_probe_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        l2_probe_kernel<4><<<sms, kProbeThreads, smem, s>>>(map, scales, row_blocks, k_stages, tiles, err_word);
      } else if (stages == 3) {
        cudaFuncSetAttribute(l2_probe_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        l2_probe_kernel<3><<<sms, kProbeThreads, smem, s>>>(map, scales, row_blocks, k_stages, tiles, err_word);
      } else {
        cudaFuncSetAttribute(l2_probe_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        l2_probe_kernel<2><<<sms, kProbeThreads, smem, s>>>(map, scales, row_blocks, k_stages, tiles, err_word);
      }
      count_launch();
    };
    launch(static_cast<int>(tiles_per_cta));   // warm-up: brings the working set into the L2 where it fits
    cudaEventRecord(e0, s);
    launch(static_cast<int>(tiles_per_cta));
    cudaEventRecord(e1, s);
    err = cudaStreamSynchronize(s);
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
    if (err == cudaSuccess) err = cudaMemcpy(&device_error, err_word, 4, cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) st = fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "operand-delivery probe", err);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  cudaFree(codes);
  cudaFree(scales);
  cudaFree(err_word);
  if (st != GLMRT_STATUS_OK) return st;
  if (device_error != 0) return fail(GLMRT_STATUS_INTERNAL_ERROR, "operand-delivery probe: a bounded wait expired");
  const double bytes = static_cast<double>(sms) * tiles_per_cta * kStagesK * kProbeStageBytes;
  *out_ms = ms;
  *out_gb_per_s = static_cast<float>(bytes / (static_cast<double>(ms) * 1e-3) / 1e9);
  return ok();
}
