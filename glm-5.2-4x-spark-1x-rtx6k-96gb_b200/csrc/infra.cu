// Status plumbing and the infrastructure part of the C ABI: version, device info,
// device buffers, copies, streams and events.  Semantics follow the reference's
// native/src/glmrt_native.cc (alloc/copy/stream section) with one deliberate
// difference: there is no host fallback -- without a CUDA device these entry points
// return GLMRT_STATUS_CUDA_UNAVAILABLE.
#include <atomic>
#include <cstdio>
#include <cstring>

#include <cstdlib>

#include "common.cuh"

namespace glmrt {

namespace {
thread_local std::string g_last_error;
std::atomic<uint64_t> g_launches{0};
}  // namespace

glmrt_status_t fail(glmrt_status_t status, const std::string& message) {
  g_last_error = message;
  return status;
}
glmrt_status_t ok() {
  g_last_error.clear();
  return GLMRT_STATUS_OK;
}
glmrt_status_t fail_cuda(glmrt_status_t status, const char* action, cudaError_t err) {
  return fail(status, std::string(action) + ": " + cudaGetErrorString(err));
}
glmrt_status_t status_from_cuda(cudaError_t err, const char* action) {
  if (err == cudaSuccess) return ok();
  return fail_cuda(GLMRT_STATUS_COPY_FAILED, action, err);
}
glmrt_status_t require_cuda() {
  int n = 0;
  cudaError_t err = cudaGetDeviceCount(&n);
  if (err != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return fail(GLMRT_STATUS_CUDA_UNAVAILABLE, "no CUDA device is available");
  }
  return GLMRT_STATUS_OK;
}
bool pdl_enabled() {
  static const bool on = []() {
    const char* v = std::getenv("GLMRT_B200_NO_PDL");
    return !(v != nullptr && v[0] != '\0' && v[0] != '0');
  }();
  return on;
}
void count_launch(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
uint64_t launches_total() { return g_launches.load(std::memory_order_relaxed); }

namespace {
glmrt_status_t write_c_string(const std::string& value, char* out, size_t out_len) {
  if (out == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "output buffer is null");
  if (out_len == 0) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "output buffer length is zero");
  if (value.size() + 1 > out_len) {
    std::memcpy(out, value.data(), out_len - 1);
    out[out_len - 1] = '\0';
    return GLMRT_STATUS_BUFFER_TOO_SMALL;
  }
  std::memcpy(out, value.c_str(), value.size() + 1);
  return GLMRT_STATUS_OK;
}
}  // namespace
}  // namespace glmrt

using namespace glmrt;

extern "C" glmrt_status_t glmrt_native_version(char* out, size_t out_len) {
  return write_c_string("glmrt-b200 0.1.0 (sm_100a; routed-MoE expert path)", out, out_len);
}

extern "C" glmrt_status_t glmrt_last_error(char* out, size_t out_len) {
  // Reading the message must not clear or replace it.
  if (out == nullptr || out_len == 0) return GLMRT_STATUS_INVALID_ARGUMENT;
  const std::string copy = g_last_error;
  if (copy.size() + 1 > out_len) {
    std::memcpy(out, copy.data(), out_len - 1);
    out[out_len - 1] = '\0';
    return GLMRT_STATUS_BUFFER_TOO_SMALL;
  }
  std::memcpy(out, copy.c_str(), copy.size() + 1);
  return GLMRT_STATUS_OK;
}

extern "C" glmrt_status_t glmrt_cuda_device_info(int device_id, glmrt_cuda_device_info_t* out) {
  if (out == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "device info output pointer is null");
  if (device_id < 0) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "device id must be non-negative");
  std::memset(out, 0, sizeof(*out));
  out->device_id = device_id;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
    cudaGetLastError();
    return fail(GLMRT_STATUS_CUDA_UNAVAILABLE, "no CUDA device is available");
  }
  if (device_id >= count) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "device id out of range");
  cudaDeviceProp prop;
  cudaError_t err = cudaGetDeviceProperties(&prop, device_id);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaGetDeviceProperties", err);
  out->cuda_available = 1;
  out->compute_capability_major = prop.major;
  out->compute_capability_minor = prop.minor;
  out->integrated = prop.integrated;
  out->can_map_host_memory = prop.canMapHostMemory;
  out->unified_addressing = prop.unifiedAddressing;
  out->total_memory_bytes = prop.totalGlobalMem;
  std::snprintf(out->name, sizeof(out->name), "%s", prop.name);
  int drv = 0, rt = 0;
  cudaDriverGetVersion(&drv);
  cudaRuntimeGetVersion(&rt);
  std::snprintf(out->driver_version, sizeof(out->driver_version), "%d.%d", drv / 1000, (drv % 1000) / 10);
  std::snprintf(out->runtime_version, sizeof(out->runtime_version), "%d.%d", rt / 1000, (rt % 1000) / 10);
  return ok();
}

extern "C" glmrt_status_t glmrt_alloc_device_buffer(size_t bytes, glmrt_device_buffer_t* out) {
  if (out == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "device buffer output pointer is null");
  std::memset(out, 0, sizeof(*out));
  if (bytes == 0) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "device buffer size is zero");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  void* p = nullptr;
  cudaError_t err = cudaMalloc(&p, bytes);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return fail_cuda(GLMRT_STATUS_ALLOCATION_FAILED, "cudaMalloc", err);
  }
  int dev = 0;
  cudaGetDevice(&dev);
  out->ptr = p;
  out->bytes = bytes;
  out->device_id = dev;
  out->flags = 0;
  return ok();
}

extern "C" glmrt_status_t glmrt_free_device_buffer(glmrt_device_buffer_t* buf) {
  if (buf == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "device buffer pointer is null");
  if (buf->ptr != nullptr) {
    cudaError_t err = cudaFree(buf->ptr);
    if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaFree", err);
  }
  std::memset(buf, 0, sizeof(*buf));
  return ok();
}

extern "C" glmrt_status_t glmrt_cuda_stream_create(void** out_cuda_stream) {
  if (out_cuda_stream == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "stream output pointer is null");
  *out_cuda_stream = nullptr;
  GLMRT_RETURN_IF_ERROR(require_cuda());
  cudaStream_t s;
  cudaError_t err = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaStreamCreate", err);
  *out_cuda_stream = s;
  return ok();
}
extern "C" glmrt_status_t glmrt_cuda_stream_destroy(void* cuda_stream) {
  if (cuda_stream == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "stream is null");
  return status_from_cuda(cudaStreamDestroy(static_cast<cudaStream_t>(cuda_stream)), "cudaStreamDestroy");
}
extern "C" glmrt_status_t glmrt_cuda_stream_synchronize(void* cuda_stream) {
  GLMRT_RETURN_IF_ERROR(require_cuda());
  return status_from_cuda(cudaStreamSynchronize(static_cast<cudaStream_t>(cuda_stream)),
                          "cudaStreamSynchronize");
}
extern "C" glmrt_status_t glmrt_cuda_event_create(void** out_cuda_event) {
  if (out_cuda_event == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "event output pointer is null");
  *out_cuda_event = nullptr;
  GLMRT_RETURN_IF_ERROR(require_cuda());
  cudaEvent_t e;
  cudaError_t err = cudaEventCreate(&e);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_INTERNAL_ERROR, "cudaEventCreate", err);
  *out_cuda_event = e;
  return ok();
}
extern "C" glmrt_status_t glmrt_cuda_event_destroy(void* cuda_event) {
  if (cuda_event == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "event is null");
  return status_from_cuda(cudaEventDestroy(static_cast<cudaEvent_t>(cuda_event)), "cudaEventDestroy");
}
extern "C" glmrt_status_t glmrt_cuda_event_record(void* cuda_event, void* cuda_stream) {
  if (cuda_event == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "event is null");
  return status_from_cuda(
      cudaEventRecord(static_cast<cudaEvent_t>(cuda_event), static_cast<cudaStream_t>(cuda_stream)),
      "cudaEventRecord");
}
extern "C" glmrt_status_t glmrt_cuda_event_synchronize(void* cuda_event) {
  if (cuda_event == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "event is null");
  return status_from_cuda(cudaEventSynchronize(static_cast<cudaEvent_t>(cuda_event)), "cudaEventSynchronize");
}
extern "C" glmrt_status_t glmrt_cuda_event_elapsed_ms(void* start_event, void* end_event, float* out_ms) {
  if (start_event == nullptr || end_event == nullptr || out_ms == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "event or output pointer is null");
  return status_from_cuda(cudaEventElapsedTime(out_ms, static_cast<cudaEvent_t>(start_event),
                                               static_cast<cudaEvent_t>(end_event)),
                          "cudaEventElapsedTime");
}

namespace {
glmrt_status_t copy_impl(void* dst, const void* src, size_t bytes, size_t dst_cap, size_t src_cap,
                         cudaMemcpyKind kind, cudaStream_t stream, bool async) {
  if (dst == nullptr || src == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "copy pointer is null");
  if (bytes > dst_cap || bytes > src_cap) return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "copy exceeds buffer size");
  if (bytes == 0) return ok();
  GLMRT_RETURN_IF_ERROR(require_cuda());
  cudaError_t err = async ? cudaMemcpyAsync(dst, src, bytes, kind, stream) : cudaMemcpy(dst, src, bytes, kind);
  if (err != cudaSuccess) return fail_cuda(GLMRT_STATUS_COPY_FAILED, "cudaMemcpy", err);
  return ok();
}
constexpr size_t kNoCap = std::numeric_limits<size_t>::max();
}  // namespace

extern "C" glmrt_status_t glmrt_copy_h2d(glmrt_device_buffer_t dst, const void* src, size_t bytes) {
  return copy_impl(dst.ptr, src, bytes, dst.bytes, kNoCap, cudaMemcpyHostToDevice, nullptr, false);
}
extern "C" glmrt_status_t glmrt_copy_d2h(void* dst, glmrt_device_buffer_t src, size_t bytes) {
  return copy_impl(dst, src.ptr, bytes, kNoCap, src.bytes, cudaMemcpyDeviceToHost, nullptr, false);
}
extern "C" glmrt_status_t glmrt_copy_d2d(glmrt_device_buffer_t dst, glmrt_device_buffer_t src, size_t bytes) {
  return copy_impl(dst.ptr, src.ptr, bytes, dst.bytes, src.bytes, cudaMemcpyDeviceToDevice, nullptr, false);
}
extern "C" glmrt_status_t glmrt_copy_h2d_async(glmrt_device_buffer_t dst, const void* src, size_t bytes,
                                               void* cuda_stream) {
  return copy_impl(dst.ptr, src, bytes, dst.bytes, kNoCap, cudaMemcpyHostToDevice,
                   static_cast<cudaStream_t>(cuda_stream), true);
}
extern "C" glmrt_status_t glmrt_copy_d2h_async(void* dst, glmrt_device_buffer_t src, size_t bytes,
                                               void* cuda_stream) {
  return copy_impl(dst, src.ptr, bytes, kNoCap, src.bytes, cudaMemcpyDeviceToHost,
                   static_cast<cudaStream_t>(cuda_stream), true);
}
extern "C" glmrt_status_t glmrt_copy_d2d_async(glmrt_device_buffer_t dst, glmrt_device_buffer_t src,
                                               size_t bytes, void* cuda_stream) {
  return copy_impl(dst.ptr, src.ptr, bytes, dst.bytes, src.bytes, cudaMemcpyDeviceToDevice,
                   static_cast<cudaStream_t>(cuda_stream), true);
}
