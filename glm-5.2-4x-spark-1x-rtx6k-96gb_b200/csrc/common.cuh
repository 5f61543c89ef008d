// Shared host/device helpers for libglmrt_b200: status + last-error plumbing and the
// numeric formats of the routed-MoE path (E2M1 codes, E4M3 scales, bf16).
#pragma once
#include <atomic>

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <limits>
#include <string>

#include "../../include/glmrt_b200.h"

namespace glmrt {

// ---- status / last error (reference convention: native/src/glmrt_native.cc:30-49) ----
glmrt_status_t fail(glmrt_status_t status, const std::string& message);
glmrt_status_t ok();
glmrt_status_t fail_cuda(glmrt_status_t status, const char* action, cudaError_t err);
// Every CUDA launch error maps to COPY_FAILED as in native/cuda/kernels/common.h:96-102.
glmrt_status_t status_from_cuda(cudaError_t err, const char* action);
// CUDA_UNAVAILABLE unless a device is present.
glmrt_status_t require_cuda();
void count_launch(uint64_t n = 1);
uint64_t launches_total();

inline bool checked_mul(size_t a, size_t b, size_t* out) {
  if (a != 0 && b > std::numeric_limits<size_t>::max() / a) return false;
  *out = a * b;
  return true;
}

#define GLMRT_RETURN_IF_ERROR(expr)                   \
  do {                                                \
    glmrt_status_t _st = (expr);                      \
    if (_st != GLMRT_STATUS_OK) return _st;           \
  } while (0)

#define GLMRT_LAUNCH_CHECK(what)                                                  \
  do {                                                                            \
    cudaError_t _e = cudaGetLastError();                                          \
    if (_e != cudaSuccess) return ::glmrt::status_from_cuda(_e, what);            \
    ::glmrt::count_launch();                                                      \
  } while (0)

// Raises a kernel's dynamic shared-memory limit once per device.  `done` is a static of the call
// site (one bit per device ordinal); the attribute belongs to the device, so a process that drives
// several GPUs sets it on each.  Racing first calls both set it, which is harmless.
template <typename Kernel>
inline glmrt_status_t ensure_smem_limit(std::atomic<uint64_t>& done, Kernel kernel, size_t bytes, const char* what) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return status_from_cuda(err, "cudaGetDevice");
  const uint64_t bit = 1ull << (dev & 63);
  if (done.load(std::memory_order_acquire) & bit) return GLMRT_STATUS_OK;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  if (err != cudaSuccess) return status_from_cuda(err, what);
  done.fetch_or(bit, std::memory_order_release);
  return GLMRT_STATUS_OK;
}

// ---- programmatic dependent launch ----
// The kernels of a forward pass are launched so that each may begin while its predecessor on the
// stream is still running: a kernel raises pdl_launch_dependents() as its first statement (its
// successor's CTAs may then take free SM resources and run their own set-up: barrier
// initialisation, tensor-memory allocation), and calls pdl_wait() before its first access to
// global memory that an earlier kernel may still be producing (or still reading).  pdl_wait()
// returns once every earlier kernel has completed and its writes are visible; both are no-ops in
// a kernel launched the ordinary way, and an ordinary launch after such a kernel waits for its
// completion as always.  GLMRT_B200_NO_PDL=1 in the environment turns the launch attribute off.
bool pdl_enabled();
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

// ---- optional timeline of the kernels of a forward pass (trace builds only) ----
// A library built with -DGLMRT_B200_TRACE (build.py --trace) stamps, per kernel of the chain and
// per launch, the global timer when the first and the last CTA start, when the first CTA is past
// its pdl_wait(), and when the last warp leaves.  A kernel never overlaps its own next launch
// (the other kernels of the pass lie between, each waiting for its predecessor to complete), so
// the launch number is the count of CTA arrivals divided by the grid size.  Every translation unit
// with chain kernels keeps its own table (GLMRT_CHAIN_TRACE_TU defines it and a C accessor);
// trace_chain.py merges them.  The product library has none of this.
enum ChainKernel : int {
  kChainLogits = 0, kChainSelect, kChainQuantDispatch, kChainFc1, kChainFc2, kChainCombine,
  kChainEpPlanDispatch, kChainEpCount, kChainEpRetile, kChainPlan, kChainKernels
};
#if defined(GLMRT_B200_TRACE) && defined(__CUDACC__)
constexpr int kChainLaunches = 16;   // ring over launches
constexpr int kChainStamps = 12;     // first CTA start, last CTA start, first CTA past its wait, last warp out, 8 marks
#define GLMRT_CHAIN_TRACE_TU(name)                                                                              \
  namespace glmrt { namespace {                                                                                \
  __device__ unsigned long long g_chain_table[kChainLaunches * kChainKernels * kChainStamps];                   \
  __device__ unsigned int g_chain_arrivals[kChainKernels];                                                      \
  } }                                                                                                           \
  extern "C" int glmrt_b200_trace_chain_##name(unsigned long long* out, int reset) {                            \
    if (out != nullptr &&                                                                                       \
        cudaMemcpyFromSymbol(out, glmrt::g_chain_table, sizeof(glmrt::g_chain_table)) != cudaSuccess) return 1; \
    if (reset) {                                                                                                \
      static unsigned long long init[glmrt::kChainLaunches * glmrt::kChainKernels * glmrt::kChainStamps];       \
      for (int i = 0; i < glmrt::kChainLaunches * glmrt::kChainKernels; ++i) {                                  \
        unsigned long long* r = init + i * glmrt::kChainStamps;                                                 \
        for (int j = 0; j < glmrt::kChainStamps; ++j) r[j] = 0ull;                                              \
        r[0] = ~0ull; r[2] = ~0ull;                                                                             \
      }                                                                                                         \
      static unsigned int zeros[glmrt::kChainKernels];                                                          \
      if (cudaMemcpyToSymbol(glmrt::g_chain_table, init, sizeof(init)) != cudaSuccess) return 1;                \
      if (cudaMemcpyToSymbol(glmrt::g_chain_arrivals, zeros, sizeof(zeros)) != cudaSuccess) return 1;           \
    }                                                                                                           \
    return 0;                                                                                                   \
  }
#define GLMRT_CHAIN_SCOPE(id) ChainScope chain_scope__(id, g_chain_table, g_chain_arrivals)
#define GLMRT_CHAIN_READY() chain_scope__.ready()
#define GLMRT_CHAIN_MARK(i) chain_mark(i)   /* latest time any CTA's thread 0 passed mark i (0..7) */
#define GLMRT_CHAIN_MARK_HERE(i) chain_mark_here(i)   /* the same, stamped by the calling thread */
static __shared__ unsigned long long* s_chain_row;   // set by the kernel's ChainScope; device functions mark through it
struct ChainScope {
  unsigned long long* row;
  __device__ __forceinline__ static unsigned long long now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
  }
  __device__ __forceinline__ ChainScope(int id, unsigned long long* table, unsigned int* arrivals) {
    __shared__ unsigned int launch_index;
    if (threadIdx.x == 0 && threadIdx.y == 0) {
      const unsigned int ctas = gridDim.x * gridDim.y * gridDim.z;
      launch_index = atomicAdd(&arrivals[id], 1u) / ctas;
    }
    __syncthreads();
    row = table + (static_cast<size_t>(launch_index % kChainLaunches) * kChainKernels + id) * kChainStamps;
    s_chain_row = row;   // every thread stores the same value
    if (threadIdx.x == 0 && threadIdx.y == 0) {
      const unsigned long long t = now();
      atomicMin(row + 0, t);
      atomicMax(row + 1, t);
    }
  }
  __device__ __forceinline__ void ready() const {
    if (threadIdx.x == 0 && threadIdx.y == 0) atomicMin(row + 2, now());
  }
  __device__ __forceinline__ ~ChainScope() {
    if ((threadIdx.x & 31) == 0) atomicMax(row + 3, now());
  }
};
__device__ __forceinline__ void chain_mark(int i) {
  if (threadIdx.x == 0 && threadIdx.y == 0) atomicMax(s_chain_row + 4 + i, ChainScope::now());
}
__device__ __forceinline__ void chain_mark_here(int i) { atomicMax(s_chain_row + 4 + i, ChainScope::now()); }
#else
#define GLMRT_CHAIN_TRACE_TU(name)
#define GLMRT_CHAIN_SCOPE(id) do { } while (0)
#define GLMRT_CHAIN_READY() do { } while (0)
#define GLMRT_CHAIN_MARK(i) do { } while (0)
#define GLMRT_CHAIN_MARK_HERE(i) do { } while (0)
#endif

// ---- device-side formats ----
#ifdef __CUDACC__

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t v) {
  return __uint_as_float(static_cast<uint32_t>(v) << 16);
}
// Round-to-nearest-even (torch semantics; the Python oracle's rounding): one cvt.rn.bf16.f32.
__device__ __forceinline__ uint16_t f32_to_bf16_rne(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
// Truncation (the reference's native kernels: native/cuda/kernels/common.h:64-66).
__device__ __forceinline__ uint16_t f32_to_bf16_trunc(float f) {
  return static_cast<uint16_t>(__float_as_uint(f) >> 16);
}

// E4M3 byte -> float, no NaN handling (0x7f -> 480), native/cuda/kernels/common.h:40-50.
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
  const uint32_t mag = b & 0x7fu;
  const uint32_t e = mag >> 3, m = mag & 7u;
  float v = e == 0 ? static_cast<float>(m) * 0.001953125f /* 2^-9 */
                   : __uint_as_float(((e + 120u) << 23) | (m << 20));
  return (b & 0x80u) ? -v : v;
}
// float -> E4M3 byte, round-to-nearest-even, saturating (nvfp4_payload.cu:57-58).
__device__ __forceinline__ uint32_t f32_to_e4m3_satfinite(float v) {
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3)) & 0xffu;
}

__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  // 0, .5, 1, 1.5, 2, 3, 4, 6 with the sign in bit 3; code 8 is +0 as in the reference's
  // codebook (native/cuda/kernels/common.h:32-38)
  const uint32_t m = code & 7u;
  if (m == 0u) return 0.0f;
  const float mag = m < 2 ? 0.5f * static_cast<float>(m)
                          : __uint_as_float((((m >> 1) + 126u) << 23) | ((m & 1u) << 22));
  return (code & 8u) ? -mag : mag;
}

// Nearest E2M1 code of an already scaled value, exact ties to the LOWER magnitude,
// a value that rounds to zero (and NaN) -> code 0.  Same result as the argmin over
// |x - codebook| of python/reference/glmrt_reference/quant_ref.py:41-46.
__device__ __forceinline__ uint32_t fp4_code_nearest_low(float q) {
  const float m = fabsf(q);
  const uint32_t mag = (m > 0.25f) + (m > 0.75f) + (m > 1.25f) + (m > 1.75f) + (m > 2.5f) +
                       (m > 3.5f) + (m > 5.0f);
  return mag | ((q < 0.0f && mag != 0u) ? 8u : 0u);
}
// Round-to-nearest-even thresholds with the sign taken from signbit()
// (native/cuda/kernels/nvfp4_payload.cu:11-33).
__device__ __forceinline__ uint32_t fp4_code_rne_payload(float q) {
  const float m = fabsf(q);
  uint32_t code;
  if (m <= 0.25f) code = 0;
  else if (m < 0.75f) code = 1;
  else if (m <= 1.25f) code = 2;
  else if (m < 1.75f) code = 3;
  else if (m <= 2.5f) code = 4;
  else if (m < 3.5f) code = 5;
  else if (m <= 5.0f) code = 6;
  else code = 7;
  return code | ((__float_as_uint(q) >> 31) ? 8u : 0u);
}

// Stable float32 sigmoid (native/cuda/kernels/common.h:23-30).
__device__ __forceinline__ float sigmoid_f32(float v) {
  if (v >= 0.0f) {
    return 1.0f / (1.0f + expf(-v));
  }
  const float e = expf(v);
  return e / (1.0f + e);
}

// The weights of one 128-row tile of a projection (codes and tiled scales) are asked into the L2,
// one 128-byte line per thread and pass, by all `threads` threads of a CTA; nothing waits for them.
__device__ __forceinline__ void l2_prefetch_lines(const uint8_t* p, size_t bytes, int threads) {
  for (size_t off = static_cast<size_t>(threadIdx.x) * 128; off < bytes; off += static_cast<size_t>(threads) * 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p + off) : "memory");
}
// Quarter `part` (0..3) of a 128-row weight tile: 32 rows of codes and a quarter of its scale tiles.
// The CTAs that only prefetch share their SMs with the CTAs that quantise rows, whose few loads
// would queue behind the thousands of prefetch requests (measured: a row's quantisation 2.6 -> 4-6 us);
// the prefetch CTAs therefore let the rows go first.
constexpr int kPrefetchParts = 4;
__device__ __forceinline__ void prefetch_cta_yield() {
  for (int i = 0; i < 3; ++i) __nanosleep(1000);
}
__device__ __forceinline__ void l2_prefetch_weight_tile_part(const uint8_t* codes, const uint8_t* sf, size_t first_row,
                                                             int row_bytes, int part, int threads) {
  l2_prefetch_lines(codes + (first_row + 32 * static_cast<size_t>(part)) * row_bytes, 32 * static_cast<size_t>(row_bytes),
                    threads);
  // scale tiles: 512 bytes per (128 rows, 64 elements of K)
  const size_t sf_bytes = static_cast<size_t>(row_bytes / 32) * 512;
  l2_prefetch_lines(sf + (first_row / 128) * sf_bytes + part * (sf_bytes / kPrefetchParts), sf_bytes / kPrefetchParts, threads);
}

// Byte offset of the scale of (row r, 16-element block j) in the tiled scale layout the
// tensor-core kernels consume: 512-byte tiles of 128 rows x 4 blocks, row-tile major.
__device__ __host__ __forceinline__ size_t sf_tile_offset(size_t r, size_t j, size_t kblocks) {
  return ((r >> 7) * (kblocks >> 2) + (j >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 +
         (j & 3);
}

#endif  // __CUDACC__

}  // namespace glmrt
