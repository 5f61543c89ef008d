// Router logits on the tensor core for prefill-sized batches.
//
// logits = X W^T with bf16 X and float32 W (python/reference/glmrt_reference/
// glm_moe_dsa_layer_ref.py:62-66) is a [T x 6144] x [6144 x 256] GEMM: 25.8 GFLOP at T = 8192, far
// too much for the SIMT kernel (the reference's own kernels use one CTA per (expert, row) dot
// product, native/cuda/kernels/router.cu:78-117).  The float32 weight is split once, exactly, into
// three bf16 terms (w = hi + mid + lo); every product x * term is exact in float32, so a
// kind::f16 UMMA over the concatenated reduction dimension [hi | mid | lo] accumulates the same
// exact products as the float32 reference, only in another order.
//
// Batches of a few hundred to a few thousand rows have fewer output tiles than the GPU has SMs, so
// the reduction dimension is cut into 2, 4 or 8 equal ranges: one CTA per (tile, range) writes a
// partial tile and the selection kernel adds the partials of a logit in range order.
//
// Tile = 128 rows x 128 experts, K stage = 64 elements (128-byte swizzled rows for both operands),
// accumulators double-buffered in tensor memory, epilogue = one thread per row writing 512
// contiguous bytes of logits.  Roles, bounded waits and teardown as in the expert GEMM kernels.
#include <cuda.h>

#include "common.cuh"
#include "internal.h"
#include "tc_ptx.cuh"

namespace glmrt {
namespace {

using namespace tc;

constexpr int kRtStages = 6;
constexpr int kRtTile = 128 * 128;                 // bytes: 128 rows x 64 bf16
constexpr int kRtStageBytes = 2 * kRtTile;         // A + B
constexpr size_t kRtSmemBytes = static_cast<size_t>(kRtStages) * kRtStageBytes + 1024 + 256;
constexpr int kRtTmemCols = 256;                   // two accumulator buffers of 128 columns

__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_load32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
// bf16 x bf16 -> f32, K-major A and B, M = 128, N = 128
__device__ __forceinline__ uint32_t idesc_bf16_128x128() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
}

// w (float32) -> [hi | mid | lo] bf16 by successive truncation: the three terms sum to w exactly.
__global__ void __launch_bounds__(256) split_weight_kernel(const float* __restrict__ w, uint16_t* __restrict__ w3,
                                                           int experts, int hidden) {
  const size_t n = static_cast<size_t>(experts) * hidden;
  const size_t i = blockIdx.x * static_cast<size_t>(256) + threadIdx.x;
  if (i >= n) return;
  const size_t e = i / hidden, k = i % hidden;
  const float v = w[i];
  const uint16_t hi = f32_to_bf16_trunc(v);
  const float r1 = v - bf16_bits_to_f32(hi);
  const uint16_t mid = f32_to_bf16_trunc(r1);
  const float r2 = r1 - bf16_bits_to_f32(mid);
  const uint16_t lo = f32_to_bf16_trunc(r2);
  uint16_t* row = w3 + e * 3 * static_cast<size_t>(hidden);
  row[k] = hi;
  row[hidden + k] = mid;
  row[2 * static_cast<size_t>(hidden) + k] = lo;
}

__global__ void __launch_bounds__(kThreadsTC, 1)
router_logits_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                        float* __restrict__ logits, int rows, int hidden, int experts, int splits,
                        uint32_t* error_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kRtStages) * kRtStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kRtStages;
  uint64_t* acc_full = bars + 2 * kRtStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int x_stages = hidden / 64;            // 64-element steps over one copy of X
  const int k_stages = 3 * x_stages / splits;  // [hi | mid | lo], this work item's share of it
  const int n_tiles = experts / 128;
  const int m_tiles = (rows + 127) / 128;
  const int num_tiles = m_tiles * n_tiles * splits;   // work item -> (row tile, expert tile, K range), K range fastest
  const size_t split_stride = static_cast<size_t>(rows) * experts;

  if (threadIdx.x == 0) {
    if (blockIdx.x == 0 && error_word != nullptr) *error_word = 0u;   // any expiry comes seconds later
    for (int s = 0; s < kRtStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) tmem_alloc(tmem_slot, kRtTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    const uint64_t pol = policy_evict_last();
    int stage = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      const int sp = tile % splits, mn = tile / splits;
      const int mt = mn / n_tiles, nt = mn % n_tiles;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_warp(&empty_bar[stage], phase ^ 1u, abort_flag)) { alive = false; break; }
        if (elect_one()) {
          const uint32_t s_a = smem_u32(smem + static_cast<size_t>(stage) * kRtStageBytes);
          const int kg = sp * k_stages + ks;   // step in the concatenated reduction dimension
          mbar_expect_tx(&full_bar[stage], kRtStageBytes);
          tma_load_2d(s_a, &map_x, &full_bar[stage], (kg % x_stages) * 128, mt * 128, pol);
          tma_load_2d(s_a + kRtTile, &map_w, &full_bar[stage], kg * 128, nt * 128, pol);
        }
        __syncwarp();
        if (++stage == kRtStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    int stage = 0;
    uint32_t phase = 0;
    int abuf = 0;
    uint32_t aphase = 0;
    bool alive = true;
    const uint32_t idesc = idesc_bf16_128x128();
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      if (!mbar_wait_warp(&acc_empty[abuf], aphase ^ 1u, abort_flag)) { alive = false; break; }
      tc_fence_after();
      const uint32_t d0 = tmem_base + abuf * 128;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag)) { alive = false; break; }
        tc_fence_after();
        if (elect_one()) {
          const uint32_t s_a = smem_u32(smem + static_cast<size_t>(stage) * kRtStageBytes);
          const uint32_t s_b = s_a + kRtTile;
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)   // 16 bf16 = 32 bytes per UMMA
            tc_mma_bf16(d0, desc_sw128(s_a + kb * 32), desc_sw128(s_b + kb * 32), idesc, (ks | kb) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == kRtStages) { stage = 0; phase ^= 1u; }
      }
      if (!alive) break;
      if (elect_one()) tc_commit(&acc_full[abuf]);
      __syncwarp();
      abuf ^= 1;
      if (abuf == 0) aphase ^= 1u;
    }
  } else {
    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    int abuf = 0;
    uint32_t aphase = 0;
    bool alive = true;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      const int sp = tile % splits, mn = tile / splits;
      const int mt = mn / n_tiles, nt = mn % n_tiles;
      const int row = mt * 128 + quad * 32 + lane;
      if (!mbar_wait_warp(&acc_full[abuf], aphase, abort_flag)) { alive = false; break; }
      tc_fence_after();
      const uint32_t t_acc = tmem_base + lane_base + abuf * 128;
#pragma unroll
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t v[32];
        tc_load32(t_acc + c0, v);
        tc_wait_ld();
        if (row < rows) {
          uint4* dst = reinterpret_cast<uint4*>(logits + sp * split_stride + static_cast<size_t>(row) * experts +
                                                nt * 128 + c0);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[abuf]);
      abuf ^= 1;
      if (abuf == 0) aphase ^= 1u;
    }
  }

  __syncwarp();
  if (*abort_flag != 0u) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && error_word != nullptr) atomicOr(error_word, static_cast<uint32_t>(kErrWaitTimeout));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kRtTmemCols);
}

}  // namespace

glmrt_status_t launch_split_router_weight(const float* w, uint16_t* w3, size_t experts, size_t hidden,
                                          cudaStream_t stream) {
  const size_t n = experts * hidden;
  split_weight_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(w, w3, static_cast<int>(experts),
                                                                                 static_cast<int>(hidden));
  GLMRT_LAUNCH_CHECK("split_weight_kernel");
  return GLMRT_STATUS_OK;
}

bool router_tc_supported(size_t rows, size_t hidden, size_t experts, const void* x) {
  return rows > 128 && hidden % 64 == 0 && experts % 128 == 0 && experts >= 128 &&
         reinterpret_cast<uintptr_t>(x) % 16 == 0;
}

// K ranges for a batch: the largest of 8, 4, 2, 1 that divides the reduction steps and keeps the
// number of work items within the SM count.
int router_tc_splits(size_t rows, size_t hidden, size_t experts, int sm_count) {
  const size_t tiles = ((rows + 127) / 128) * (experts / 128);
  const size_t steps = 3 * hidden / 64;
  for (int s = 8; s > 1; s >>= 1)
    if (steps % s == 0 && tiles * s <= static_cast<size_t>(sm_count)) return s;
  return 1;
}

glmrt_status_t launch_router_logits_tc(const uint16_t* x, const CUtensorMap& map_w3, float* logits, size_t rows,
                                       size_t hidden, size_t experts, uint32_t* error_word, int sm_count,
                                       cudaStream_t stream, int splits) {
  CUtensorMap map_x;
  GLMRT_RETURN_IF_ERROR(make_codes_tensor_map(&map_x, x, rows, hidden * 2, 128));
  static std::atomic<uint64_t> configured{0};
  GLMRT_RETURN_IF_ERROR(ensure_smem_limit(configured, router_logits_tc_kernel, kRtSmemBytes, "cudaFuncSetAttribute(router_logits_tc_kernel)"));
  const int tiles = static_cast<int>(((rows + 127) / 128) * (experts / 128)) * splits;
  router_logits_tc_kernel<<<std::min(sm_count, tiles), kThreadsTC, kRtSmemBytes, stream>>>(
      map_x, map_w3, logits, static_cast<int>(rows), static_cast<int>(hidden), static_cast<int>(experts), splits,
      error_word);
  GLMRT_LAUNCH_CHECK("router_logits_tc_kernel");
  return GLMRT_STATUS_OK;
}

}  // namespace glmrt
