// Device-side helpers for kernels that talk to other GPUs of the NVSwitch domain through peer
// pointers: system-scope loads/stores, epoch flags and their bounded waits.
//
// Flags are 32-bit epochs that only grow. Slot s of a rank's flag buffer holds MAX_PEERS words;
// word r is written by rank r ("rank r has reached epoch e on slot s"). A wait compares in
// wrap-around arithmetic and gives up after `timeout_ns`, reporting ERR_WAIT_PEER through the status
// word, so a missing peer never hangs the GPU.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "fmb_api.h"
#include "ptx_sm100.cuh"

namespace fmb {

constexpr int MAX_PEERS = FMB_MAX_PEERS;

struct Peers {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_peer_f(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_peer_i(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool wait_epoch(const uint32_t* flag, uint32_t want, unsigned long long timeout_ns,
                                           int* status) {
  const uint64_t t0 = globaltimer_ns();
  int spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - want) < 0) {
    if (++spins > 64) {
      __nanosleep(64);
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (status != nullptr) atomicCAS(status, 0, ERR_WAIT_PEER);
        return false;
      }
    }
  }
  return true;
}

// Threads 0..world-1 of the calling block tell every rank that this rank reached `epoch` on `slot`.
__device__ __forceinline__ void signal_all(const Peers& flags, int slot, int rank, int world, uint32_t epoch) {
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(flags.p[threadIdx.x]) + slot * MAX_PEERS + rank, epoch);
  }
}
// Threads 0..world-1 wait for one source each; the whole block gets the result (contains __syncthreads).
__device__ __forceinline__ bool wait_all(const Peers& flags, int slot, int rank, int world, uint32_t epoch,
                                         unsigned long long timeout_ns, int* status) {
  int ok = 1;
  if (threadIdx.x < world)
    ok = wait_epoch(static_cast<const uint32_t*>(flags.p[rank]) + slot * MAX_PEERS + threadIdx.x, epoch, timeout_ns,
                    status) ? 1 : 0;
  return __syncthreads_and(ok) != 0;
}

}  // namespace fmb
