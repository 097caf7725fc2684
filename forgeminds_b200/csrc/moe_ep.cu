// Expert parallelism over peer memory: the dispatch and combine all-to-alls are folded into the
// permutation kernels that a single-GPU mixture-of-experts layer runs anyway.
//
// Every rank routes its own N tokens (top-k expert ids over all E experts) and publishes, in
// symmetric memory, its token rows, expert ids and routing weights. Rank r owns experts
// [r * E_local, (r + 1) * E_local). Then, without any collective call:
//
//   ep_collect_idx    every rank reads ALL ranks' expert ids and renumbers them for its own plan:
//                     local expert id, or E_local ("somebody else's") for the rest;
//   (moe.cu plan)     the usual device-side slot plan over the W * N * k global entries;
//   ep_gather         slot rows are pulled straight from the token's rank (dispatch all-to-all + gather);
//   (grouped GEMMs)   gemm_sm100.cu, grouped by expert;
//   ep_combine        every token pulls its k expert outputs from the owners' buffers, using the owners'
//                     slot tables, and mixes them (combine all-to-all + scatter-add);
//   ep_combine_bwd    owner side of the backward: pulls the output gradient row and the routing weight
//                     of every slot from the token's rank, writes the scaled row for the expert
//                     backward and pushes d(loss)/d(weight) back to the token's rank.
//
// All waits are on epoch flags with a time limit (peer.cuh). The reference does this with two
// all_to_all_single calls per direction, a host read of the split sizes, a sort and index_add_
// (forgemind/moe.py:62-79, 227-287).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "peer.cuh"

namespace fmb {

__device__ __forceinline__ bool block_wait(const uint32_t* flags, int slot, int world, uint32_t epoch,
                                           unsigned long long timeout_ns, int* status) {
  int ok = 1;
  if (slot >= 0 && threadIdx.x < world)
    ok = wait_epoch(flags + slot * MAX_PEERS + threadIdx.x, epoch, timeout_ns, status) ? 1 : 0;
  return __syncthreads_and(ok) != 0;
}

// out[r * n + i] = local id of peer r's expert choice i, or e_local when another rank owns it
__global__ void __launch_bounds__(256)
ep_collect_idx_kernel(Peers idx, int* __restrict__ out, long long n, int world, int rank, int e_local,
                      const uint32_t* flags, int slot, uint32_t epoch, unsigned long long timeout_ns, int* status) {
  if (!block_wait(flags, slot, world, epoch, timeout_ns, status)) return;
  const long long total = n * world;
  const int lo = rank * e_local;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / n);
    const int e = ld_peer_i(static_cast<const int*>(idx.p[r]) + (i - r * n)) - lo;
    out[i] = (e >= 0 && e < e_local) ? e : e_local;
  }
}

// out[s, :] = x_of_rank[token / tokens_per_rank][token % tokens_per_rank, :] for s < *limit, zero rows for padding
__global__ void __launch_bounds__(256)
ep_gather_kernel(Peers x, const int* __restrict__ token_of_slot, const int* __restrict__ limit_ptr,
                 uint4* __restrict__ out, int dvec, long long tokens_per_rank, int world, const uint32_t* flags,
                 int slot, uint32_t epoch, unsigned long long timeout_ns, int* status) {
  if (!block_wait(flags, slot, world, epoch, timeout_ns, status)) return;
  const long long total = static_cast<long long>(*limit_ptr) * dvec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long s = i / dvec;
    const int c = static_cast<int>(i % dvec);
    const int t = token_of_slot[s];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t >= 0) {
      const int r = static_cast<int>(t / tokens_per_rank);
      v = ld_peer_u4(static_cast<const uint4*>(x.p[r]) + (t - r * tokens_per_rank) * dvec + c);
    }
    out[i] = v;
  }
}

// out[t, :] = sum_j w[t, j] * ys_of_owner[slot_of_owner[rank * n + t * k + j], :]; owner = idx[t, j] / e_local
__global__ void __launch_bounds__(256)
ep_combine_kernel(Peers ys, Peers slots, const int* __restrict__ idx, const float* __restrict__ w,
                  uint4* __restrict__ out, long long tokens, int k, int dvec, int e_local, int rank, int world,
                  const uint32_t* flags, int slot, uint32_t epoch, unsigned long long timeout_ns, int* status) {
  if (!block_wait(flags, slot, world, epoch, timeout_ns, status)) return;
  const long long total = tokens * dvec;
  const long long n = tokens * k;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / dvec;
    const int c = static_cast<int>(i % dvec);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int owner = idx[t * k + j] / e_local;
      const int s = ld_peer_i(static_cast<const int*>(slots.p[owner]) + rank * n + t * k + j);
      if (s < 0) continue;
      const float wj = w != nullptr ? w[t * k + j] : 1.f;
      const uint4 u = ld_peer_u4(static_cast<const uint4*>(ys.p[owner]) + static_cast<long long>(s) * dvec + c);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += wj * a.x; acc[1] += wj * a.y; acc[2] += wj * b.x; acc[3] += wj * b.y;
      acc[4] += wj * cc.x; acc[5] += wj * cc.y; acc[6] += wj * d.x; acc[7] += wj * d.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    out[i] = o;
  }
}

// Owner side of the combine backward, one warp per slot s < *limit with global entry en = entry_of_slot[s]:
//   dys[s, :] = w[en] * dout[token(en), :]      (dout and w live on the token's rank)
//   drw_of_rank[en_local] = <dout[token, :], ys[s, :]>   (stored on the token's rank)
__global__ void __launch_bounds__(256)
ep_combine_bwd_kernel(Peers dout, Peers w, Peers drw, const uint4* __restrict__ ys, const int* __restrict__ entry_of_slot,
                      const int* __restrict__ limit_ptr, uint4* __restrict__ dys, long long n, int k, int dvec, int world,
                      const uint32_t* flags, int slot, uint32_t epoch, unsigned long long timeout_ns, int* status) {
  if (!block_wait(flags, slot, world, epoch, timeout_ns, status)) return;
  const int lane = threadIdx.x & 31;
  const long long limit = *limit_ptr;
  for (long long s = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; s < limit;
       s += (static_cast<long long>(gridDim.x) * blockDim.x) >> 5) {
    const int en = entry_of_slot[s];
    if (en < 0) {
      for (int c = lane; c < dvec; c += 32) dys[s * dvec + c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int r = static_cast<int>(en / n);
    const long long el = en - r * n;
    const long long t = el / k;
    const float wj = ld_peer_f(static_cast<const float*>(w.p[r]) + el);
    float dot = 0.f;
    for (int c = lane; c < dvec; c += 32) {
      const uint4 g = ld_peer_u4(static_cast<const uint4*>(dout.p[r]) + t * dvec + c);
      const uint4 y = ys[s * dvec + c];
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, yw[4] = {y.x, y.y, y.z, y.w};
      uint32_t ow[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 gf = unpack_bf16(gw[q]), yf = unpack_bf16(yw[q]);
        dot += gf.x * yf.x + gf.y * yf.y;
        ow[q] = pack_bf16(gf.x * wj, gf.y * wj);
      }
      dys[s * dvec + c] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0 && addr_ok(static_cast<float*>(drw.p[r]) + el, 4)) static_cast<float*>(drw.p[r])[el] = dot;
  }
}

static bool fill_peers(Peers& t, const void* const* ptrs, int world) {
  if (world < 1 || world > MAX_PEERS) return false;
  for (int r = 0; r < MAX_PEERS; ++r) t.p[r] = r < world ? const_cast<void*>(ptrs[r]) : nullptr;
  for (int r = 0; r < world; ++r)
    if (t.p[r] == nullptr || (reinterpret_cast<uintptr_t>(t.p[r]) & 15)) return false;
  return true;
}

static int ep_grid(long long work) {
  long long b = (work + 255) / 256;
  const long long cap = 148ll * 16;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

// Cuts a slot plan down to `rows` buffer rows, in place: region[i] = {start, used, padded} of expert i (the
// last row is the region of the entries other ranks own; its start is the first row past the live ones). A plan
// that needed more rows leaves `code` in the status word (first error wins).
__global__ void ep_clamp_plan_kernel(int* __restrict__ region, int n, int rows, int* __restrict__ status, int code) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int start = region[3 * i], used = region[3 * i + 1], padded = region[3 * i + 2];
  if (i == n - 1 && start > rows && status != nullptr) atomicCAS(status, 0, code);
  const int s = min(start, rows);
  region[3 * i] = s;
  region[3 * i + 1] = max(min(start + used, rows) - s, 0);
  region[3 * i + 2] = max(min(start + padded, rows) - s, 0);
}

}  // namespace fmb

using namespace fmb;

extern "C" int fmb_ep_clamp_plan(int* region, int n, int rows, int* status, int code, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (region == nullptr || rows < 0) return -2;
  ep_clamp_plan_kernel<<<(n + 255) / 256, 256, 0, stream>>>(region, n, rows, status, code);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

FMB_DEBUG_BIND(moe_ep)

extern "C" int fmb_ep_collect_idx(const void* const* idx_ptrs, int* out, long long n, int world, int rank, int e_local,
                                  const unsigned* flags, int slot, unsigned epoch, unsigned long long timeout_ns,
                                  int* status, cudaStream_t stream) {
  Peers p;
  if (!fill_peers(p, idx_ptrs, world) || n <= 0 || e_local <= 0) return -2;
  ep_collect_idx_kernel<<<ep_grid(n * world), 256, 0, stream>>>(p, out, n, world, rank, e_local, flags, slot, epoch,
                                                               timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_ep_gather(const void* const* x_ptrs, const int* token_of_slot, const int* limit_ptr, void* out,
                             long long max_slots, int d, long long tokens_per_rank, int world, const unsigned* flags,
                             int slot, unsigned epoch, unsigned long long timeout_ns, int* status, cudaStream_t stream) {
  Peers p;
  if (!fill_peers(p, x_ptrs, world) || d % 8 || max_slots <= 0) return -2;
  ep_gather_kernel<<<ep_grid(max_slots * (d / 8)), 256, 0, stream>>>(p, token_of_slot, limit_ptr,
                                                                    static_cast<uint4*>(out), d / 8, tokens_per_rank,
                                                                    world, flags, slot, epoch, timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_ep_combine(const void* const* ys_ptrs, const void* const* slot_ptrs, const int* idx, const float* w,
                              void* out, long long tokens, int k, int d, int e_local, int rank, int world,
                              const unsigned* flags, int slot, unsigned epoch, unsigned long long timeout_ns,
                              int* status, cudaStream_t stream) {
  Peers y, s;
  if (!fill_peers(y, ys_ptrs, world) || !fill_peers(s, slot_ptrs, world) || d % 8 || tokens <= 0) return -2;
  ep_combine_kernel<<<ep_grid(tokens * (d / 8)), 256, 0, stream>>>(y, s, idx, w, static_cast<uint4*>(out), tokens, k,
                                                                  d / 8, e_local, rank, world, flags, slot, epoch,
                                                                  timeout_ns, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_ep_combine_bwd(const void* const* dout_ptrs, const void* const* w_ptrs, const void* const* drw_ptrs,
                                  const void* ys, const int* entry_of_slot, const int* limit_ptr, void* dys,
                                  long long max_slots, long long n, int k, int d, int world, const unsigned* flags,
                                  int slot, unsigned epoch, unsigned long long timeout_ns, int* status,
                                  cudaStream_t stream) {
  Peers g, w, dr;
  if (!fill_peers(g, dout_ptrs, world) || !fill_peers(w, w_ptrs, world) || !fill_peers(dr, drw_ptrs, world) || d % 8)
    return -2;
  ep_combine_bwd_kernel<<<ep_grid(max_slots * 32), 256, 0, stream>>>(g, w, dr, static_cast<const uint4*>(ys),
                                                                    entry_of_slot, limit_ptr, static_cast<uint4*>(dys),
                                                                    n, k, d / 8, world, flags, slot, epoch, timeout_ns,
                                                                    status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
