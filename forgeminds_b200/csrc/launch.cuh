// Programmatic dependent launch. A kernel launched through launch_pdl() may have its blocks placed
// on the SMs while the previous kernel of the stream is still draining; such a kernel must call
// pdl_wait() before its first access to global memory (the wait returns when the previous grid has
// finished and its writes are visible) and should call pdl_launch_dependents() right after it, so
// that its own successor can be set up early in turn. What is gained is the launch latency and the
// prologue (barrier set-up, TMEM allocation, descriptor prefetch) of every kernel in a long stream
// of short ones.
#pragma once
#include <cuda_runtime.h>

#include <utility>

namespace fmb {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... P, typename... A>
inline cudaError_t launch_pdl(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(std::forward<A>(args))...);
}

// The same with thread-block clusters of `cluster_x` CTAs along x (the grid must be a multiple of it).
template <typename... P, typename... A>
inline cudaError_t launch_pdl_cluster(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, int cluster_x,
                                      cudaStream_t stream, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = static_cast<unsigned>(cluster_x);
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(std::forward<A>(args))...);
}

}  // namespace fmb
