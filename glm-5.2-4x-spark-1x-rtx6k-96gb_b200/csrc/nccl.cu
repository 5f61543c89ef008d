// NCCL entry points of the reference ABI (native/include/glmrt_native.h:428-444, implementation
// native/src/glmrt_native.cc:1453-1757): unique id, communicator, gather to root, row all-to-all,
// bf16 all-reduce and reduce-to-root.
//
// On this path NCCL is not the data plane (rows and results move as in-kernel peer stores, see
// ep.cu); the wrappers exist so that a caller written against the reference ABI keeps working and
// as the cross-check for the peer-store exchange.  The NCCL library is resolved at run time
// (dlopen of GLMRT_NCCL_LIB or libnccl.so.2, e.g. the copy PyTorch ships): the shared library has
// no link-time dependency on it, and without it every entry point returns
// GLMRT_STATUS_NCCL_UNAVAILABLE as the reference's non-NCCL build does.
#include <dlfcn.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace glmrt {
namespace {

struct UniqueId { char bytes[128]; };          // ncclUniqueId
using Comm = void*;                            // ncclComm_t
constexpr int kNcclUint8 = 1, kNcclBfloat16 = 9, kNcclSum = 0;

struct Api {
  void* lib = nullptr;
  int (*GetUniqueId)(UniqueId*) = nullptr;
  int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
  int (*CommDestroy)(Comm) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*Send)(const void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*Reduce)(const void*, void*, size_t, int, int, int, Comm, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
};

Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {std::getenv("GLMRT_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      if (n == nullptr || *n == '\0') continue;
      a.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (a.lib != nullptr) break;
    }
    if (a.lib == nullptr) return;
    auto sym = [&](const char* s) { return dlsym(a.lib, s); };
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
    a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
    a.Send = reinterpret_cast<decltype(a.Send)>(sym("ncclSend"));
    a.Recv = reinterpret_cast<decltype(a.Recv)>(sym("ncclRecv"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
    a.Reduce = reinterpret_cast<decltype(a.Reduce)>(sym("ncclReduce"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.GroupStart && a.GroupEnd && a.Send && a.Recv &&
           a.AllReduce && a.Reduce;
  });
  return a;
}

glmrt_status_t unavailable() {
  return fail(GLMRT_STATUS_NCCL_UNAVAILABLE, "NCCL is unavailable: libnccl.so.2 could not be loaded (set GLMRT_NCCL_LIB)");
}
glmrt_status_t fail_nccl(const char* what, int code) {
  const char* msg = api().GetErrorString != nullptr ? api().GetErrorString(code) : "?";
  return fail(GLMRT_STATUS_INTERNAL_ERROR, std::string(what) + ": " + msg);
}

struct CommHandle {
  Comm comm = nullptr;
  int world = 0;
  int rank = 0;
};

}  // namespace
}  // namespace glmrt

using namespace glmrt;

extern "C" glmrt_status_t glmrt_nccl_unique_id_bytes(size_t* out_bytes) {
  if (out_bytes == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL unique ID byte output is null");
  if (!api().ok) {
    *out_bytes = 0;
    return unavailable();
  }
  *out_bytes = sizeof(UniqueId);
  return ok();
}

extern "C" glmrt_status_t glmrt_nccl_get_unique_id(void* out, size_t out_bytes) {
  if (!api().ok) return unavailable();
  if (out == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL unique ID output is null");
  if (out_bytes != sizeof(UniqueId)) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL unique ID output has an unexpected byte size");
  UniqueId id{};
  const int r = api().GetUniqueId(&id);
  if (r != 0) return fail_nccl("ncclGetUniqueId failed", r);
  std::memcpy(out, &id, sizeof(id));
  return ok();
}

extern "C" glmrt_status_t glmrt_nccl_comm_init_rank(const void* unique_id, size_t unique_id_bytes, int world_size,
                                                    int rank, void** out_handle) {
  if (out_handle == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL communicator output is null");
  *out_handle = nullptr;
  if (!api().ok) return unavailable();
  if (unique_id == nullptr || unique_id_bytes != sizeof(UniqueId) || world_size <= 0 || rank < 0 || rank >= world_size)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL communicator arguments are invalid");
  GLMRT_RETURN_IF_ERROR(require_cuda());
  UniqueId id{};
  std::memcpy(&id, unique_id, sizeof(id));
  Comm comm = nullptr;
  const int r = api().CommInitRank(&comm, world_size, id, rank);
  if (r != 0) return fail_nccl("ncclCommInitRank failed", r);
  CommHandle* h = new CommHandle();
  h->comm = comm;
  h->world = world_size;
  h->rank = rank;
  *out_handle = h;
  return ok();
}

extern "C" glmrt_status_t glmrt_nccl_comm_destroy(void* handle) {
  if (!api().ok) return unavailable();
  CommHandle* h = static_cast<CommHandle*>(handle);
  if (h == nullptr) return ok();
  const int r = api().CommDestroy(h->comm);
  delete h;
  if (r != 0) return fail_nccl("ncclCommDestroy failed", r);
  return ok();
}

// Every non-root rank sends `bytes`; the root receives them back to back in rank order.
extern "C" glmrt_status_t glmrt_nccl_gather_u8_async(void* handle, glmrt_device_buffer_t send,
                                                     glmrt_device_buffer_t recv, size_t bytes, int root,
                                                     void* cuda_stream) {
  if (!api().ok) return unavailable();
  CommHandle* h = static_cast<CommHandle*>(handle);
  if (h == nullptr || h->comm == nullptr || cuda_stream == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL gather handle or CUDA stream is null");
  if (root < 0 || root >= h->world || bytes == 0 || send.ptr == nullptr || send.bytes < bytes)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL gather send contract is invalid");
  const size_t peers = static_cast<size_t>(h->world - 1);
  size_t need = 0;
  if (h->rank == root && peers > 0 && (!checked_mul(bytes, peers, &need) || recv.ptr == nullptr || recv.bytes < need))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL gather receive buffer is too small");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  int r = api().GroupStart();
  if (r != 0) return fail_nccl("ncclGroupStart failed", r);
  if (h->rank == root) {
    size_t slot = 0;
    for (int p = 0; p < h->world && r == 0; ++p) {
      if (p == root) continue;
      r = api().Recv(static_cast<uint8_t*>(recv.ptr) + slot * bytes, bytes, kNcclUint8, p, h->comm, s);
      ++slot;
    }
  } else {
    r = api().Send(send.ptr, bytes, kNcclUint8, root, h->comm, s);
  }
  const int g = api().GroupEnd();
  if (r != 0) return fail_nccl("NCCL gather operation failed", r);
  if (g != 0) return fail_nccl("ncclGroupEnd failed", g);
  return ok();
}

// Rows are split into `world` contiguous slices (the first rows % world slices one row longer);
// rank r keeps slice r and receives every peer's copy of it, back to back in peer order.
extern "C" glmrt_status_t glmrt_nccl_row_all_to_all_u8_async(void* handle, glmrt_device_buffer_t send,
                                                             glmrt_device_buffer_t recv, size_t rows,
                                                             size_t row_stride_bytes, void* cuda_stream) {
  if (!api().ok) return unavailable();
  CommHandle* h = static_cast<CommHandle*>(handle);
  if (h == nullptr || h->comm == nullptr || cuda_stream == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL row all-to-all handle or CUDA stream is null");
  const size_t world = static_cast<size_t>(h->world), rank = static_cast<size_t>(h->rank);
  size_t send_bytes = 0;
  if (rows < world || row_stride_bytes == 0 || !checked_mul(rows, row_stride_bytes, &send_bytes))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL row all-to-all shape is invalid");
  const size_t base = rows / world, extra = rows % world;
  const size_t local_bytes = (base + (rank < extra ? 1 : 0)) * row_stride_bytes;
  size_t recv_need = 0;
  if (send.ptr == nullptr || send.bytes < send_bytes || !checked_mul(local_bytes, world - 1, &recv_need) ||
      (world > 1 && (recv.ptr == nullptr || recv.bytes < recv_need)))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL row all-to-all device buffer is too small");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  int r = api().GroupStart();
  if (r != 0) return fail_nccl("ncclGroupStart failed", r);
  size_t slot = 0;
  for (size_t p = 0; p < world && r == 0; ++p) {
    if (p == rank) continue;
    const size_t p_rows = base + (p < extra ? 1 : 0);
    const size_t p_start = p * base + std::min(p, extra);
    r = api().Send(static_cast<const uint8_t*>(send.ptr) + p_start * row_stride_bytes, p_rows * row_stride_bytes,
                   kNcclUint8, static_cast<int>(p), h->comm, s);
    if (r != 0) break;
    r = api().Recv(static_cast<uint8_t*>(recv.ptr) + slot * local_bytes, local_bytes, kNcclUint8, static_cast<int>(p),
                   h->comm, s);
    ++slot;
  }
  const int g = api().GroupEnd();
  if (r != 0) return fail_nccl("NCCL row all-to-all operation failed", r);
  if (g != 0) return fail_nccl("ncclGroupEnd failed", g);
  return ok();
}

extern "C" glmrt_status_t glmrt_nccl_all_reduce_bf16_async(void* handle, glmrt_device_buffer_t send,
                                                           glmrt_device_buffer_t recv, size_t values,
                                                           void* cuda_stream) {
  if (!api().ok) return unavailable();
  CommHandle* h = static_cast<CommHandle*>(handle);
  if (h == nullptr || h->comm == nullptr || cuda_stream == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL BF16 all-reduce handle or CUDA stream is null");
  size_t bytes = 0;
  if (values == 0 || !checked_mul(values, 2, &bytes))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL BF16 all-reduce value count is invalid");
  if (send.ptr == nullptr || send.bytes < bytes || recv.ptr == nullptr || recv.bytes < bytes)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL BF16 all-reduce device buffer is too small");
  const int r = api().AllReduce(send.ptr, recv.ptr, values, kNcclBfloat16, kNcclSum, h->comm,
                                static_cast<cudaStream_t>(cuda_stream));
  if (r != 0) return fail_nccl("NCCL BF16 all-reduce failed", r);
  return ok();
}

extern "C" glmrt_status_t glmrt_nccl_reduce_bf16_async(void* handle, glmrt_device_buffer_t send,
                                                       glmrt_device_buffer_t recv, size_t values, int root,
                                                       void* cuda_stream) {
  if (!api().ok) return unavailable();
  CommHandle* h = static_cast<CommHandle*>(handle);
  if (h == nullptr || h->comm == nullptr || cuda_stream == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL BF16 reduce handle or CUDA stream is null");
  size_t bytes = 0;
  if (root < 0 || root >= h->world || values == 0 || !checked_mul(values, 2, &bytes))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL BF16 reduce contract is invalid");
  if (send.ptr == nullptr || send.bytes < bytes || (h->rank == root && (recv.ptr == nullptr || recv.bytes < bytes)))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "NCCL BF16 reduce device buffer is too small");
  const int r = api().Reduce(send.ptr, recv.ptr, values, kNcclBfloat16, kNcclSum, root, h->comm,
                             static_cast<cudaStream_t>(cuda_stream));
  if (r != 0) return fail_nccl("NCCL BF16 reduce failed", r);
  return ok();
}
