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

// ------------------------------------------------------------------ debug build: bounds on every peer access
// With -DFMB_DEBUG_BOUNDS (python -m forgeminds_b200.csrc.build --debug-bounds -> _C_debug.so) every load
// and store that goes through the helpers below is first checked against a table of registered buffers
// (the symmetric allocations and whatever else the host registers: base address, length). An address that
// lies in none of them is not touched: a load yields zeros, a store is dropped, and ERR_BOUNDS goes to the
// status word, which the host reads where it reads the wait errors. Nothing traps. This is the stand-in
// for a memory checker on machines where none may be run; in the normal build the checks compile away.
struct FmbExtent {
  unsigned long long lo, hi;     // [lo, hi) in this process's address space
};
#ifdef FMB_DEBUG_BOUNDS
static __device__ const FmbExtent* g_fmb_tab = nullptr;      // one copy per translation unit, bound by the host
static __device__ int g_fmb_ntab = 0;
static __device__ int* g_fmb_dbg_status = nullptr;
__device__ __forceinline__ bool addr_ok(const void* p, unsigned bytes) {
  const unsigned long long a = reinterpret_cast<unsigned long long>(p);
  const FmbExtent* tab = g_fmb_tab;
  const int n = g_fmb_ntab;
  for (int i = 0; i < n; ++i)
    if (a >= tab[i].lo && a + bytes <= tab[i].hi) return true;
  if (g_fmb_dbg_status != nullptr) atomicCAS(g_fmb_dbg_status, 0, ERR_BOUNDS);
  return false;
}
static int fmb_debug_bind_this_tu(const FmbExtent* tab, int n, int* status) {
  if (cudaMemcpyToSymbol(g_fmb_tab, &tab, sizeof(tab)) != cudaSuccess) return -3;
  if (cudaMemcpyToSymbol(g_fmb_ntab, &n, sizeof(n)) != cudaSuccess) return -3;
  if (cudaMemcpyToSymbol(g_fmb_dbg_status, &status, sizeof(status)) != cudaSuccess) return -3;
  return 0;
}
#define FMB_DEBUG_BIND(name) \
  extern "C" int fmb_debug_bind_##name(const void* tab, int n, int* status) { \
    return fmb::fmb_debug_bind_this_tu(static_cast<const fmb::FmbExtent*>(tab), n, status); \
  }
#else
__device__ __forceinline__ constexpr bool addr_ok(const void*, unsigned) { return true; }
#define FMB_DEBUG_BIND(name) \
  extern "C" int fmb_debug_bind_##name(const void*, int, int*) { return 0; }
#endif

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
  if (!addr_ok(p, 16)) return make_float4(0.f, 0.f, 0.f, 0.f);
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer_u4(const void* p) {
  uint4 v;
  if (!addr_ok(p, 16)) return make_uint4(0u, 0u, 0u, 0u);
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_peer_f(const float* p) {
  float v;
  if (!addr_ok(p, 4)) return 0.f;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_peer_i(const int* p) {
  int v;
  if (!addr_ok(p, 4)) return -1;
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
