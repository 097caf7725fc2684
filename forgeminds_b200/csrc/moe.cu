// Mixture-of-experts routing kernels: softmax + top-k + renormalisation + load statistics in one
// pass over the router logits (no host read), the stable slot assignment that groups routed rows
// by expert, and the gather / weighted-combine that move token rows in and out of that layout.
#include "ptx_sm100.cuh"
#include "tensormap.h"
#include "fmb_api.h"
#include <math_constants.h>

namespace fmb {

constexpr int ROUTER_MAX_PER_LANE = 8;   // experts <= 256
constexpr int ROUTER_MAX_K = 8;

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// One warp per token. Outputs probs (saved for the backward), renormalised top-k weights, expert
// ids, logsumexp; per-block partial column sums of probs and of lse^2 (folded by a second kernel
// in a fixed order) and integer per-expert counts.
template <typename T>
__global__ void __launch_bounds__(256)
router_fwd_kernel(const T* __restrict__ logits, long long ld, float* __restrict__ probs, float* __restrict__ weights,
                  int* __restrict__ idx, float* __restrict__ lse_out, float* __restrict__ psum_partial,
                  int* __restrict__ counts, long long rows, int E, int k) {
  extern __shared__ float sm[];            // [E + 1] block partials, then [E] int counts
  float* s_psum = sm;
  int* s_cnt = reinterpret_cast<int*>(sm + E + 1);
  for (int i = threadIdx.x; i <= E; i += blockDim.x) s_psum[i] = 0.f;
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_cnt[i] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float acc_p[ROUTER_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) acc_p[i] = 0.f;
  float acc_z = 0.f;
  for (long long row = static_cast<long long>(blockIdx.x) * nwarps + warp; row < rows;
       row += static_cast<long long>(gridDim.x) * nwarps) {
    float v[ROUTER_MAX_PER_LANE];
    float m = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      v[i] = e < E ? static_cast<float>(logits[row * ld + e]) : -CUDART_INF_F;
      m = fmaxf(m, v[i]);
    }
    m = wmax(m);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      v[i] = e < E ? __expf(v[i] - m) : 0.f;
      s += v[i];
    }
    s = wsum(s);
    const float inv = 1.f / s;
    const float lse = m + __logf(s);
#pragma unroll
    for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      v[i] *= inv;
      if (e < E) { probs[row * E + e] = v[i]; acc_p[i] += v[i]; }
    }
    if (lane == 0) { lse_out[row] = lse; acc_z += lse * lse; }
    // k rounds of arg-max; ties go to the smaller expert id
    float sel_p[ROUTER_MAX_K];
    int sel_e[ROUTER_MAX_K];
    float tot = 0.f;
    for (int j = 0; j < k; ++j) {
      float bv = -1.f;
      int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        if (e < E && (v[i] > bv || (v[i] == bv && e < be))) { bv = v[i]; be = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
      }
      sel_p[j] = bv; sel_e[j] = be; tot += bv;
      if ((be & 31) == lane) v[be >> 5] = -2.f;     // remove from later rounds
    }
    if (lane == 0) {
      for (int j = 0; j < k; ++j) {
        weights[row * k + j] = sel_p[j] / tot;
        idx[row * k + j] = sel_e[j];
        atomicAdd(&s_cnt[sel_e[j]], 1);
      }
    }
  }
  // fold the per-warp column sums in warp order
  for (int turn = 0; turn < nwarps; ++turn) {
    if (warp == turn) {
#pragma unroll
      for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        if (e < E) s_psum[e] += acc_p[i];
      }
      if (lane == 0) s_psum[E] += acc_z;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i <= E; i += blockDim.x) psum_partial[static_cast<long long>(blockIdx.x) * (E + 1) + i] = s_psum[i];
  for (int i = threadIdx.x; i < E; i += blockDim.x)
    if (s_cnt[i]) atomicAdd(&counts[i], s_cnt[i]);
}

// dlogits for: renormalised top-k weights, the load-balance term (aux_grad[e] = dL/dp_e common to
// every token) and the z-loss (zc = dL/dz * 2 / rows).
template <typename T>
__global__ void __launch_bounds__(256)
router_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ idx, const float* __restrict__ weights,
                  const float* __restrict__ lse, const float* __restrict__ dweights, const float* __restrict__ aux_grad,
                  const float* __restrict__ zc_ptr, T* __restrict__ dlogits, long long ld, long long rows, int E, int k) {
  const int lane = threadIdx.x & 31;
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const float zc = zc_ptr != nullptr ? zc_ptr[0] : 0.f;
  float p[ROUTER_MAX_PER_LANE], dp[ROUTER_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? probs[row * E + e] : 0.f;
    dp[i] = (e < E && aux_grad != nullptr) ? aux_grad[e] : 0.f;
  }
  if (dweights != nullptr) {
    float S = 0.f, dot = 0.f;
    for (int j = 0; j < k; ++j) {
      const int e = idx[row * k + j];
      const float pe = probs[row * E + e];
      S += pe;
      dot += dweights[row * k + j] * weights[row * k + j];
    }
    for (int j = 0; j < k; ++j) {
      const int e = idx[row * k + j];
      if ((e & 31) == lane) dp[e >> 5] += (dweights[row * k + j] - dot) / S;
    }
  }
  float inner = 0.f;
#pragma unroll
  for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) inner += p[i] * dp[i];
  inner = wsum(inner);
  const float zl = zc * lse[row];
#pragma unroll
  for (int i = 0; i < ROUTER_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    if (e < E) dlogits[row * ld + e] = static_cast<T>(p[i] * (dp[i] - inner) + zl * p[i]);
  }
}

// ---- slot assignment -----------------------------------------------------------------------
// Routed entries (token t, choice j) are numbered n = t*k + j. Entries of one expert keep their
// order (stable), so results do not depend on scheduling. Three small kernels:
//   chunk_count: per chunk of CHUNK entries, per-expert counts
//   chunk_scan : exclusive scan over chunks per expert + expert base offsets (aligned regions)
//   chunk_place: local stable rank + base -> slot_of_entry, token_of_slot
constexpr int CHUNK = 1024;

__global__ void __launch_bounds__(256) chunk_count_kernel(const int* __restrict__ idx, int* __restrict__ chunk_counts,
                                                          long long n, int E) {
  extern __shared__ int s_c[];
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_c[i] = 0;
  __syncthreads();
  const long long base = static_cast<long long>(blockIdx.x) * CHUNK;
  for (int i = threadIdx.x; i < CHUNK; i += blockDim.x) {
    const long long e = base + i;
    if (e < n) atomicAdd(&s_c[idx[e]], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) chunk_counts[static_cast<long long>(blockIdx.x) * E + i] = s_c[i];
}

// mode 0 (dropless): expert regions start at multiples of `align` after the running total.
// mode 1 (capacity): expert e owns [e*cap, (e+1)*cap); entries past the capacity are dropped.
// region[e] = {start, used, padded_used}; meta[0] = total padded rows.
__global__ void chunk_scan_kernel(int* __restrict__ chunk_counts, int* __restrict__ region, int* __restrict__ meta,
                                  int nchunks, int E, int align, int cap, int mode) {
  const int e = threadIdx.x;
  __shared__ int s_tot[1024];
  int total = 0;
  if (e < E) {
    for (int c = 0; c < nchunks; ++c) {
      const int v = chunk_counts[static_cast<long long>(c) * E + e];
      chunk_counts[static_cast<long long>(c) * E + e] = total;   // exclusive prefix inside the expert
      total += v;
    }
  }
  s_tot[e] = e < E ? total : 0;
  __syncthreads();
  if (e == 0) {
    int run = 0;
    for (int i = 0; i < E; ++i) {
      const int used = mode == 1 ? min(s_tot[i], cap) : s_tot[i];
      const int start = mode == 1 ? i * cap : run;
      const int padded = mode == 1 ? cap : (used + align - 1) / align * align;
      region[3 * i + 0] = start;
      region[3 * i + 1] = used;
      region[3 * i + 2] = padded;
      run = start + padded;
    }
    meta[0] = run;
  }
}

__global__ void __launch_bounds__(256)
chunk_place_kernel(const int* __restrict__ idx, const int* __restrict__ chunk_prefix, const int* __restrict__ region,
                   int* __restrict__ slot_of_entry, int* __restrict__ token_of_slot, long long n, int E, int k) {
  // each warp walks its 128-entry strip in order; strips are ranked by a block-level prefix
  extern __shared__ int sm_i[];            // [8 warps][E] strip counts
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long base = static_cast<long long>(blockIdx.x) * CHUNK + warp * 128;
  int my_e[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long en = base + i * 32 + lane;
    my_e[i] = en < n ? idx[en] : -1;
  }
  for (int e = lane; e < E; e += 32) sm_i[warp * E + e] = 0;
  __syncwarp();
  // per-expert count inside the strip, and each entry's rank among equal experts before it
  int my_rank[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const unsigned peers = __match_any_sync(0xffffffffu, my_e[i]);
    const int before = __popc(peers & ((1u << lane) - 1u));
    int prior = 0;
    if (my_e[i] >= 0) prior = sm_i[warp * E + my_e[i]];
    __syncwarp();
    my_rank[i] = prior + before;
    if (my_e[i] >= 0 && before == 0) sm_i[warp * E + my_e[i]] = prior + __popc(peers);
    __syncwarp();
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long en = base + i * 32 + lane;
    if (en >= n) continue;
    const int e = my_e[i];
    int off = chunk_prefix[static_cast<long long>(blockIdx.x) * E + e];
    for (int w = 0; w < warp; ++w) off += sm_i[w * E + e];
    const int r = off + my_rank[i];
    const int start = region[3 * e], used = region[3 * e + 1];
    if (r < used) {
      slot_of_entry[en] = start + r;
      token_of_slot[start + r] = static_cast<int>(en / k);
    } else {
      slot_of_entry[en] = -1;     // dropped by the capacity limit
    }
  }
}

// out[s, :] = x[token_of_slot[s], :] (zero rows where the slot is unused)
__global__ void __launch_bounds__(256) moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ token_of_slot,
                                                         uint4* __restrict__ out, long long slots, int dvec) {
  const long long total = slots * dvec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long s = i / dvec;
    const int c = static_cast<int>(i % dvec);
    const int t = token_of_slot[s];
    out[i] = t >= 0 ? x[static_cast<long long>(t) * dvec + c] : make_uint4(0, 0, 0, 0);
  }
}

// out[t, :] = sum_j w[t, j] * ys[slot_of_entry[t*k + j], :]   (bf16 rows, fp32 accumulate)
__global__ void __launch_bounds__(256) moe_combine_kernel(const uint4* __restrict__ ys, const int* __restrict__ slot_of_entry,
                                                          const float* __restrict__ w, uint4* __restrict__ out,
                                                          long long tokens, int k, int dvec) {
  const long long total = tokens * dvec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / dvec;
    const int c = static_cast<int>(i % dvec);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int s = slot_of_entry[t * k + j];
      if (s < 0) continue;
      const float wj = w != nullptr ? w[t * k + j] : 1.f;
      const uint4 u = ys[static_cast<long long>(s) * dvec + c];
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

// dys[s, :] = w[entry] * dout[token, :]  and  dw[entry] = <dout[token, :], ys[s, :]>; one warp per entry
__global__ void __launch_bounds__(256) moe_combine_bwd_kernel(const uint4* __restrict__ dout, const uint4* __restrict__ ys,
                                                              const int* __restrict__ slot_of_entry, const float* __restrict__ w,
                                                              uint4* __restrict__ dys, float* __restrict__ dw,
                                                              long long entries, int k, int dvec) {
  const int lane = threadIdx.x & 31;
  const long long en = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (en >= entries) return;
  const int s = slot_of_entry[en];
  if (s < 0) { if (lane == 0 && dw != nullptr) dw[en] = 0.f; return; }
  const long long t = en / k;
  const float wj = w[en];
  float dot = 0.f;
  for (int c = lane; c < dvec; c += 32) {
    const uint4 g = dout[t * dvec + c];
    const uint4 y = ys[static_cast<long long>(s) * dvec + c];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, yw[4] = {y.x, y.y, y.z, y.w};
    uint32_t ow[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 gf = unpack_bf16(gw[q]), yf = unpack_bf16(yw[q]);
      dot += gf.x * yf.x + gf.y * yf.y;
      ow[q] = pack_bf16(gf.x * wj, gf.y * wj);
    }
    dys[static_cast<long long>(s) * dvec + c] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
  dot = wsum(dot);
  if (lane == 0 && dw != nullptr) dw[en] = dot;
}

// tile_group[t] = expert whose region holds row tile t (128 rows) and has live rows there, else -1
__global__ void tile_group_kernel(const int* __restrict__ region, int* __restrict__ tile_group, int n_tiles, int E) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tiles) return;
  const int row = t * 128;
  int g = -1;
  for (int e = 0; e < E; ++e) {
    const int start = region[3 * e], used = region[3 * e + 1];
    if (row >= start && row < start + used) { g = e; break; }
  }
  tile_group[t] = g;
}

static int grid_cap(long long items, int threads) {
  long long b = (items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace fmb

using namespace fmb;

extern "C" int fmb_router_blocks(long long rows) {
  long long b = (rows + 7) / 8;
  const long long cap = static_cast<long long>(sm_count()) * 2;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

extern "C" int fmb_router_fwd(const void* logits, long long ld, int dtype, float* probs, float* weights, int* idx,
                              float* lse, float* psum_partial, int* counts, long long rows, int E, int k, int nblocks,
                              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E > 32 * ROUTER_MAX_PER_LANE || k > ROUTER_MAX_K || k > E) return -2;
  const size_t sm = sizeof(float) * (E + 1) + sizeof(int) * E;
  if (dtype == FMB_BF16)
    router_fwd_kernel<__nv_bfloat16><<<nblocks, 256, sm, stream>>>(static_cast<const __nv_bfloat16*>(logits), ld, probs, weights, idx, lse, psum_partial, counts, rows, E, k);
  else if (dtype == FMB_F32)
    router_fwd_kernel<float><<<nblocks, 256, sm, stream>>>(static_cast<const float*>(logits), ld, probs, weights, idx, lse, psum_partial, counts, rows, E, k);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_router_bwd(const float* probs, const int* idx, const float* weights, const float* lse,
                              const float* dweights, const float* aux_grad, const float* zc, void* dlogits, long long ld,
                              int dtype, long long rows, int E, int k, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E > 32 * ROUTER_MAX_PER_LANE || k > ROUTER_MAX_K) return -2;
  const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
  if (dtype == FMB_BF16)
    router_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(probs, idx, weights, lse, dweights, aux_grad, zc, static_cast<__nv_bfloat16*>(dlogits), ld, rows, E, k);
  else if (dtype == FMB_F32)
    router_bwd_kernel<float><<<blocks, 256, 0, stream>>>(probs, idx, weights, lse, dweights, aux_grad, zc, static_cast<float*>(dlogits), ld, rows, E, k);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// chunk_counts: int[nchunks * E] scratch; region: int[3 * E]; meta: int[1]; token_of_slot must be
// pre-filled with -1 by the caller.
extern "C" int fmb_moe_plan(const int* idx, int* chunk_counts, int* region, int* meta, int* slot_of_entry,
                            int* token_of_slot, long long entries, int E, int k, int align, int cap, int mode,
                            cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (E > 1024) return -2;
  const int nchunks = static_cast<int>((entries + CHUNK - 1) / CHUNK);
  chunk_count_kernel<<<nchunks, 256, sizeof(int) * E, stream>>>(idx, chunk_counts, entries, E);
  chunk_scan_kernel<<<1, 1024, 0, stream>>>(chunk_counts, region, meta, nchunks, E, align, cap, mode);
  chunk_place_kernel<<<nchunks, 256, sizeof(int) * 8 * E, stream>>>(idx, chunk_counts, region, slot_of_entry, token_of_slot, entries, E, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_moe_gather(const void* x, const int* token_of_slot, void* out, long long slots, int d,
                              cudaStream_t stream) {
  if (slots <= 0) return 0;
  if (d % 8) return -2;
  moe_gather_kernel<<<grid_cap(slots * (d / 8), 256), 256, 0, stream>>>(static_cast<const uint4*>(x), token_of_slot, static_cast<uint4*>(out), slots, d / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_moe_combine(const void* ys, const int* slot_of_entry, const float* w, void* out, long long tokens,
                               int k, int d, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d % 8) return -2;
  moe_combine_kernel<<<grid_cap(tokens * (d / 8), 256), 256, 0, stream>>>(static_cast<const uint4*>(ys), slot_of_entry, w, static_cast<uint4*>(out), tokens, k, d / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_moe_combine_bwd(const void* dout, const void* ys, const int* slot_of_entry, const float* w, void* dys,
                                   float* dw, long long entries, int k, int d, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (d % 8) return -2;
  const unsigned blocks = static_cast<unsigned>((entries * 32 + 255) / 256);
  moe_combine_bwd_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(dout), static_cast<const uint4*>(ys), slot_of_entry, w, static_cast<uint4*>(dys), dw, entries, k, d / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_moe_tile_groups(const int* region, int* tile_group, int n_tiles, int E, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  tile_group_kernel<<<(n_tiles + 127) / 128, 128, 0, stream>>>(region, tile_group, n_tiles, E);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
