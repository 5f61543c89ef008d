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

// Byte offset of the scale of (row r, 16-element block j) in the tiled scale layout the
// tensor-core kernels consume: 512-byte tiles of 128 rows x 4 blocks, row-tile major.
__device__ __host__ __forceinline__ size_t sf_tile_offset(size_t r, size_t j, size_t kblocks) {
  return ((r >> 7) * (kblocks >> 2) + (j >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 +
         (j & 3);
}

#endif  // __CUDACC__

}  // namespace glmrt
