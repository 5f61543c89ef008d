// Epoch flags of the expert-parallel exchange: device-side wait and publish helpers.
//
// A flag is a 32-bit epoch counter in the receiving rank's memory that only grows; the sender
// stores the step's epoch with release semantics at system scope after a system-wide fence, the
// receiver polls with acquire loads.  Every wait is bounded (2 s on %globaltimer) and reports
// failure instead of spinning forever.  These take the place of the reference's transport-level
// completion (ExpertProtocolV2 responses, rust/crates/glmrt-transport/src/protocol_v2_tcp.rs:375-420)
// between GPUs of one NVSwitch box.
#pragma once

#include <stdint.h>

#include "internal.h"

namespace glmrt {

constexpr uint64_t kFlagWaitLimitNs = 2000000000ull;

__device__ __forceinline__ uint64_t ep_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *flag >= epoch.  Returns false on expiry.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = ep_timer_ns();
  while (true) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (ep_timer_ns() - t0 > kFlagWaitLimitNs) return false;
    __nanosleep(100);
  }
}

// One thread waits for every rank's flag in turn.  0 = all arrived, else the DeviceError bits to
// report (a wait that ran out, or a sender that declared it had nothing valid to send).
__device__ __forceinline__ uint32_t ep_wait_all_serial(const EpWait& w) {
  uint32_t err = 0;
  for (int r = 0; r < w.world; ++r) {
    if (!wait_flag(&w.flags[r], w.epoch)) return kErrWaitTimeout;
    if (w.poison != nullptr && ld_acquire_sys(&w.poison[r]) == w.epoch) err |= kErrPeerFailed;
  }
  return err;
}

// Called by every thread of a CTA after a __syncthreads() that follows the CTA's last store to
// peer memory.  One thread fences for the whole CTA (the barrier orders the other threads' stores
// before its fence, and fences are cumulative) and takes a ticket; the last CTA of the grid fences
// again on the acquiring side, resets the ticket and raises this rank's flag at every rank.  A
// system-scope fence by every thread of every CTA measured about 15 us at the end of FC2 on two
// GPUs; this form costs one fence per CTA.
__device__ __forceinline__ void ep_signal_last_cta(const EpSignal& s) {
  __shared__ int s_is_last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    s_is_last = atomicAdd(s.ticket, 1) == static_cast<int>(total) - 1;
    if (s_is_last) {
      __threadfence_system();
      *s.ticket = 0;
    }
  }
  __syncthreads();
  if (s_is_last && threadIdx.x < static_cast<unsigned>(s.world)) st_release_sys(s.peer_flags[threadIdx.x], s.epoch);
}

}  // namespace glmrt
