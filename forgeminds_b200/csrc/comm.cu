// Collectives written as kernels over peer memory (NVLink / NVSwitch), fused with the work that
// follows them. One process drives one GPU; every rank launches the same kernels in the same order.
//
// Peers are addressed through a table of base pointers (one per rank) of a buffer that was
// allocated at the same size on every rank and mapped into every rank's address space
// ("symmetric" memory). A kernel here never waits without a limit: a flag that does not arrive in
// `timeout_ns` makes the kernel write ERR_WAIT_PEER to the status word and return, so the context
// stays usable and the host can report which step gave up.
//
//   rs_reduce_kernel     reduce-scatter by pulling: this rank's shard of a gradient bucket is summed
//                        over all ranks' buffers (fixed rank order), scaled, written back in place,
//                        and its sum of squares goes to per-block partials
//   step_reduce_kernel   one CTA: sums the partials, exchanges {sum of squares, loss} with the peers,
//                        and leaves norm, mean loss, the finite flag and the clip coefficient on
//                        the device for the optimizer kernel
//   adamw_push_kernel    AdamW on this rank's shard (chunk table: any mix of decay / no-decay runs)
//                        whose bf16 result is stored straight into every rank's working weights
//   push_cast_kernel     fp32 -> bf16 of a list of ranges into every rank's working weights (updates that
//                        were computed by other kernels, e.g. Muon on the matrices this rank owns)
//   barrier_kernel       all ranks have reached this point of their streams
//
// The reference gets these steps from FSDP2's NCCL reduce-scatter / all-gather, a foreach norm, a
// host read of the norm and torch's fused AdamW (forgemind/parallel/native.py:52-79,
// forgemind/trainer.py:213-250,124).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "peer.cuh"

namespace fmb {

// ------------------------------------------------------------------ reduce-scatter (pull) + sum of squares
__global__ void __launch_bounds__(256)
rs_reduce_kernel(Peers grads, long long lo, long long n, float scale, float* __restrict__ dst,
                 float* __restrict__ partial, Peers flags, int slot, uint32_t epoch, int rank, int world,
                 unsigned long long timeout_ns, int* status) {
  __shared__ float red[8];
  if (blockIdx.x == 0) signal_all(flags, slot, rank, world, epoch);     // my bucket is complete (stream order)
  if (!wait_all(flags, slot, rank, world, epoch, timeout_ns, status)) {
    if (threadIdx.x == 0) partial[blockIdx.x] = 0.f;
    return;
  }
  float s = 0.f;
  const long long nvec = n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // `dst` (a compact buffer of n floats) takes the result when several ranks reduce the SAME range (the replicas
  // of a hybrid-sharded group): storing in place would change what the other replica is still reading
  float* mine = dst != nullptr ? dst : static_cast<float*>(grads.p[rank]) + lo;
  const bool store = dst != nullptr || world > 1 || scale != 1.f;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (world <= 2) {
    // few sources: four vectors per source in flight per thread, or the loads cannot cover the latency
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      float4 v[4][2];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int r = 0; r < 2; ++r)
          if (r < world) v[u][r] = ld_peer_f4(static_cast<const float*>(grads.p[r]) + lo + ((i + u * stride) << 2));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float4 a = v[u][0];
        if (world > 1) { a.x += v[u][1].x; a.y += v[u][1].y; a.z += v[u][1].z; a.w += v[u][1].w; }
        a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
        if (store && addr_ok(reinterpret_cast<float4*>(mine) + i + u * stride, 16)) reinterpret_cast<float4*>(mine)[i + u * stride] = a;
        s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      }
    }
  }
  for (; i < nvec; i += stride) {
    float4 v[MAX_PEERS];
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r)
      if (r < world) v[r] = ld_peer_f4(static_cast<const float*>(grads.p[r]) + lo + (i << 2));
    float4 a = v[0];
#pragma unroll
    for (int r = 1; r < MAX_PEERS; ++r)
      if (r < world) { a.x += v[r].x; a.y += v[r].y; a.z += v[r].z; a.w += v[r].w; }
    a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
    if (store && addr_ok(reinterpret_cast<float4*>(mine) + i, 16)) reinterpret_cast<float4*>(mine)[i] = a;
    s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}

// ------------------------------------------------------------------ end-of-step scalars
// xchg: symmetric float buffer, [MAX_PEERS][4] per rank; slot r of a rank holds what rank r sent.
// stats out: [0] gradient norm, [1] mean loss, [2] 1 if both are finite on every rank.
// ctl out:   [0] clip coefficient, [1] apply flag (stats[2], or 1 when skipping is off).
__global__ void __launch_bounds__(256)
step_reduce_kernel(const float* __restrict__ partial, int n_partial, const float* __restrict__ extra_sq,
                   const float* __restrict__ loss, Peers xchg, Peers flags, int slot, uint32_t epoch, int rank,
                   int world, float max_norm, int skip_nonfinite, float* __restrict__ stats, float* __restrict__ ctl,
                   unsigned long long timeout_ns, int* status) {
  __shared__ float red[256];
  float s = 0.f;
  for (int i = threadIdx.x; i < n_partial; i += 256) s += partial[i];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  const float local_sq = red[0] + (extra_sq != nullptr ? extra_sq[0] : 0.f);
  const float local_loss = loss != nullptr ? loss[0] : 0.f;
  if (threadIdx.x < world) {
    float* dst = static_cast<float*>(xchg.p[threadIdx.x]) + rank * 4;
    dst[0] = local_sq;
    dst[1] = local_loss;
  }
  signal_all(flags, slot, rank, world, epoch);
  if (!wait_all(flags, slot, rank, world, epoch, timeout_ns, status)) {
    if (threadIdx.x == 0) { stats[0] = 0.f; stats[1] = 0.f; stats[2] = 0.f; ctl[0] = 1.f; ctl[1] = 0.f; }
    return;
  }
  if (threadIdx.x == 0) {
    const float* mine = static_cast<const float*>(xchg.p[rank]);
    float sq = 0.f, ls = 0.f;
    for (int r = 0; r < world; ++r) { sq += ld_peer_f(mine + r * 4); ls += ld_peer_f(mine + r * 4 + 1); }
    const float norm = sqrtf(fmaxf(sq, 0.f));
    const float mean_loss = ls / static_cast<float>(world);
    const bool finite = isfinite(sq) && isfinite(ls);
    stats[0] = finite ? norm : sq;               // keep inf / nan visible to the host
    stats[1] = mean_loss;
    stats[2] = finite ? 1.f : 0.f;
    ctl[0] = (max_norm > 0.f && finite) ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
    ctl[1] = (finite || !skip_nonfinite) ? 1.f : 0.f;
  }
}

// ------------------------------------------------------------------ AdamW on a shard + push of the bf16 weights
// Work is described by a chunk table (built once on the host): chunk c covers `len[c]` elements
// (a multiple of 8, at most ADAM_CHUNK) starting at flat offset `off[c]` of the parameter / gradient
// buffers and at `soff[c]` of this rank's moment buffers; `wd[c]` is that run's weight decay.
constexpr int ADAM_CHUNK = 4096;

__global__ void __launch_bounds__(256)
adamw_push_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m,
                  float* __restrict__ v, Peers shadows, int world, const long long* __restrict__ off,
                  const long long* __restrict__ soff, const int* __restrict__ len, const float* __restrict__ wd,
                  float lr, float beta1, float beta2, float eps, float bc1, float bc2,
                  const float* __restrict__ ctl, int grad_compact) {
  const float clip = ctl[0];
  if (!(ctl[1] > 0.5f)) return;
  const int c = blockIdx.x;
  const long long o = off[c], so = soff[c];
  const long long go = grad_compact ? so : o;      // reduced gradients laid out like the moments (see rs_reduce dst)
  const int n = len[c];
  const float step = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - lr * wd[c];
  for (int i = threadIdx.x * 8; i < n; i += 256 * 8) {
    float pe[8], ge[8], me[8], ve[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 pv = *reinterpret_cast<const float4*>(master + o + i + h * 4);
      const float4 gv = *reinterpret_cast<const float4*>(grad + go + i + h * 4);
      const float4 mv = *reinterpret_cast<const float4*>(m + so + i + h * 4);
      const float4 vv = *reinterpret_cast<const float4*>(v + so + i + h * 4);
      pe[h * 4 + 0] = pv.x; pe[h * 4 + 1] = pv.y; pe[h * 4 + 2] = pv.z; pe[h * 4 + 3] = pv.w;
      ge[h * 4 + 0] = gv.x * clip; ge[h * 4 + 1] = gv.y * clip; ge[h * 4 + 2] = gv.z * clip; ge[h * 4 + 3] = gv.w * clip;
      me[h * 4 + 0] = mv.x; me[h * 4 + 1] = mv.y; me[h * 4 + 2] = mv.z; me[h * 4 + 3] = mv.w;
      ve[h * 4 + 0] = vv.x; ve[h * 4 + 1] = vv.y; ve[h * 4 + 2] = vv.z; ve[h * 4 + 3] = vv.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      me[j] = me[j] + (ge[j] - me[j]) * (1.f - beta1);
      ve[j] = ve[j] * beta2 + ge[j] * ge[j] * (1.f - beta2);
      const float denom = sqrtf(ve[j]) * inv_sqrt_bc2 + eps;
      pe[j] = pe[j] * decay - step * me[j] / denom;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      *reinterpret_cast<float4*>(master + o + i + h * 4) = make_float4(pe[h * 4], pe[h * 4 + 1], pe[h * 4 + 2], pe[h * 4 + 3]);
      *reinterpret_cast<float4*>(m + so + i + h * 4) = make_float4(me[h * 4], me[h * 4 + 1], me[h * 4 + 2], me[h * 4 + 3]);
      *reinterpret_cast<float4*>(v + so + i + h * 4) = make_float4(ve[h * 4], ve[h * 4 + 1], ve[h * 4 + 2], ve[h * 4 + 3]);
    }
    uint4 w;
    w.x = pack_bf16(pe[0], pe[1]); w.y = pack_bf16(pe[2], pe[3]);
    w.z = pack_bf16(pe[4], pe[5]); w.w = pack_bf16(pe[6], pe[7]);
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r)
      if (r < world && addr_ok(static_cast<__nv_bfloat16*>(shadows.p[r]) + o + i, 16))
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(shadows.p[r]) + o + i) = w;
  }
}

// ------------------------------------------------------------------ push of updated weights (no optimizer math)
// For updates computed elsewhere (Muon's orthogonalised step on the matrices this rank owns): chunk c covers
// `len[c]` fp32 master elements (a multiple of 8) from flat offset `off[c]`; they are rounded to bf16 once and
// stored at the same offset of every rank's working weights.
__global__ void __launch_bounds__(256)
push_cast_kernel(const float* __restrict__ master, Peers shadows, int world, const long long* __restrict__ off,
                 const int* __restrict__ len) {
  const long long o = off[blockIdx.x];
  const int n = len[blockIdx.x];
  for (int i = threadIdx.x * 8; i < n; i += 256 * 8) {
    const float4 a = *reinterpret_cast<const float4*>(master + o + i);
    const float4 b = *reinterpret_cast<const float4*>(master + o + i + 4);
    uint4 w;
    w.x = pack_bf16(a.x, a.y); w.y = pack_bf16(a.z, a.w);
    w.z = pack_bf16(b.x, b.y); w.w = pack_bf16(b.z, b.w);
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r)
      if (r < world && addr_ok(static_cast<__nv_bfloat16*>(shadows.p[r]) + o + i, 16))
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(shadows.p[r]) + o + i) = w;
  }
}

__global__ void barrier_kernel(Peers flags, int slot, uint32_t epoch, int rank, int world,
                               unsigned long long timeout_ns, int* status) {
  signal_all(flags, slot, rank, world, epoch);
  wait_all(flags, slot, rank, world, epoch, timeout_ns, status);
}

// out = sum of the `world` bf16 slices of a staging buffer (+ residual), fp32 accumulation in slice order
__global__ void __launch_bounds__(256)
sum_partials_kernel(const uint4* __restrict__ staging, const uint4* __restrict__ residual, uint4* __restrict__ out,
                    long long nvec, int world) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) {
      const uint4 u = staging[static_cast<long long>(r) * nvec + i];
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    if (residual != nullptr) {
      const uint4 u = residual[i];
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    out[i] = o;
  }
}

__global__ void signal_kernel(Peers flags, int slot, uint32_t epoch, int rank, int world) {
  signal_all(flags, slot, rank, world, epoch);
}

static bool fill(Peers& t, const void* const* ptrs, int world) {
  if (world < 1 || world > MAX_PEERS) return false;
  for (int r = 0; r < MAX_PEERS; ++r) t.p[r] = r < world ? const_cast<void*>(ptrs[r]) : nullptr;
  for (int r = 0; r < world; ++r)
    if (t.p[r] == nullptr || (reinterpret_cast<uintptr_t>(t.p[r]) & 15)) return false;
  return true;
}

}  // namespace fmb

using namespace fmb;

extern "C" int fmb_comm_rs_reduce(const void* const* grad_ptrs, long long lo, long long n, float scale, float* dst,
                                  float* partial, int n_partial, const void* const* flag_ptrs, int slot,
                                  unsigned epoch, int rank, int world, unsigned long long timeout_ns, int* status,
                                  cudaStream_t stream) {
  Peers g, f;
  if (!fill(g, grad_ptrs, world) || !fill(f, flag_ptrs, world) || rank < 0 || rank >= world) return -2;
  if ((lo & 3) || (n & 3) || n_partial < 1 || slot < 0 || (reinterpret_cast<uintptr_t>(dst) & 15)) return -2;
  rs_reduce_kernel<<<n_partial, 256, 0, stream>>>(g, lo, n, scale, dst, partial, f, slot, epoch, rank, world,
                                                  timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_comm_step_reduce(const float* partial, int n_partial, const float* extra_sq, const float* loss,
                                    const void* const* xchg_ptrs, const void* const* flag_ptrs, int slot,
                                    unsigned epoch, int rank, int world, float max_norm, int skip_nonfinite,
                                    float* stats, float* ctl, unsigned long long timeout_ns, int* status,
                                    cudaStream_t stream) {
  Peers x, f;
  if (!fill(x, xchg_ptrs, world) || !fill(f, flag_ptrs, world) || rank < 0 || rank >= world) return -2;
  step_reduce_kernel<<<1, 256, 0, stream>>>(partial, n_partial, extra_sq, loss, x, f, slot, epoch, rank, world,
                                            max_norm, skip_nonfinite, stats, ctl, timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_comm_adamw_push(float* master, const float* grad, float* m, float* v,
                                   const void* const* shadow_ptrs, int world, const long long* off,
                                   const long long* soff, const int* len, const float* wd, int n_chunks, float lr,
                                   float beta1, float beta2, float eps, float bc1, float bc2, const float* ctl,
                                   int grad_compact, cudaStream_t stream) {
  Peers s;
  if (!fill(s, shadow_ptrs, world) || ctl == nullptr) return -2;
  if (n_chunks <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return -2;
  adamw_push_kernel<<<n_chunks, 256, 0, stream>>>(master, grad, m, v, s, world, off, soff, len, wd, lr, beta1, beta2,
                                                  eps, bc1, bc2, ctl, grad_compact);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_comm_push_cast(const float* master, const void* const* shadow_ptrs, int world, const long long* off,
                                  const int* len, int n_chunks, cudaStream_t stream) {
  Peers s;
  if (!fill(s, shadow_ptrs, world) || master == nullptr) return -2;
  if (n_chunks <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(master) & 15) return -2;
  push_cast_kernel<<<n_chunks, 256, 0, stream>>>(master, s, world, off, len);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_comm_adam_chunk(void) { return ADAM_CHUNK; }

// ------------------------------------------------------------------ debug build: the table of registered buffers
FMB_DEBUG_BIND(comm)
extern "C" int fmb_debug_bind_moe_ep(const void* tab, int n, int* status);
extern "C" int fmb_debug_bind_gemm(const void* tab, int n, int* status);

extern "C" int fmb_debug_bounds_enabled(void) {
#ifdef FMB_DEBUG_BOUNDS
  return 1;
#else
  return 0;
#endif
}

// Adds [base, base + bytes) to the buffers that the checked accesses accept on the current device and points
// the kernels' status reports at `status` (an int in device memory). Synchronises the device. No-op (returns 0)
// in the normal build. At most 1024 buffers per process.
extern "C" int fmb_debug_register_extent(const void* base, unsigned long long bytes, int* status) {
#ifdef FMB_DEBUG_BOUNDS
  constexpr int CAP = 1024;
  static FmbExtent host_tab[CAP];
  static int n = 0;
  static FmbExtent* dev_tab = nullptr;
  if (base == nullptr || bytes == 0) return -2;
  if (n >= CAP) return -5;
  if (dev_tab == nullptr && cudaMalloc(reinterpret_cast<void**>(&dev_tab), sizeof(FmbExtent) * CAP) != cudaSuccess) return -3;
  const unsigned long long lo = reinterpret_cast<unsigned long long>(base);
  host_tab[n].lo = lo;
  host_tab[n].hi = lo + bytes;
  ++n;
  if (cudaDeviceSynchronize() != cudaSuccess) return -3;
  if (cudaMemcpy(dev_tab, host_tab, sizeof(FmbExtent) * n, cudaMemcpyHostToDevice) != cudaSuccess) return -3;
  int rc = fmb_debug_bind_comm(dev_tab, n, status);
  if (rc == 0) rc = fmb_debug_bind_moe_ep(dev_tab, n, status);
  if (rc == 0) rc = fmb_debug_bind_gemm(dev_tab, n, status);
  return rc;
#else
  (void)base; (void)bytes; (void)status;
  return 0;
#endif
}

extern "C" int fmb_comm_barrier(const void* const* flag_ptrs, int slot, unsigned epoch, int rank, int world,
                                unsigned long long timeout_ns, int* status, cudaStream_t stream) {
  Peers f;
  if (!fill(f, flag_ptrs, world) || rank < 0 || rank >= world) return -2;
  barrier_kernel<<<1, 32, 0, stream>>>(f, slot, epoch, rank, world, timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// "Everything this rank enqueued before this call is done": posts `epoch` on `slot` of every rank.
extern "C" int fmb_comm_signal(const void* const* flag_ptrs, int slot, unsigned epoch, int rank, int world,
                               cudaStream_t stream) {
  Peers f;
  if (!fill(f, flag_ptrs, world) || rank < 0 || rank >= world) return -2;
  signal_kernel<<<1, 32, 0, stream>>>(f, slot, epoch, rank, world);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_comm_sum_partials(const void* staging, const void* residual, void* out, long long rows, int cols,
                                     int world, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8 || world < 1 || world > MAX_PEERS) return -2;
  const long long nvec = rows * (cols / 8);
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  sum_partials_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const uint4*>(staging),
                                                                         static_cast<const uint4*>(residual),
                                                                         static_cast<uint4*>(out), nvec, world);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
