// Bandwidth-bound kernels: RMSNorm (+residual), SwiGLU, rotary embedding, per-head QK norm + RoPE,
// softmax and top-k. All of them move 16-byte vectors, accumulate in fp32 and round once at the
// store. Row reductions use one warp per row up to 2048 columns and one 256-thread block per row
// above that, so no row ever makes a second trip to HBM.
#include "ptx_sm100.cuh"
#include "tensormap.h"
#include "fmb_api.h"
#include "launch.cuh"
#include <math_constants.h>

namespace fmb {

// ------------------------------------------------------------------ 8-wide vector access
template <typename T> struct V8;
template <> struct V8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]); u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct V8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the TPR threads that share a row (TPR = 32: one warp ... 256: the whole block).
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* scratch) {
  v = warp_sum(v);
  if constexpr (TPR > 32) {
    const int w = threadIdx.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[w] = v;
    __syncthreads();
    v = 0.f;
    const int first = (w / (TPR / 32)) * (TPR / 32);      // first warp of this thread's row
#pragma unroll
    for (int i = 0; i < TPR / 32; ++i) v += scratch[first + i];
  }
  return v;
}

constexpr int ROW_THREADS = 256;

// ------------------------------------------------------------------ RMSNorm forward
template <typename T, typename WT, int TPR, int VPL, bool ADD>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ delta, const WT* __restrict__ w,
                   T* __restrict__ xn, T* __restrict__ y, float* __restrict__ rstd, long long rows, int d, float eps) {
  __shared__ float scratch[ROW_THREADS / 32];
  pdl_wait();
  pdl_launch_dependents();
  constexpr int RPB = ROW_THREADS / TPR;
  const int sub = threadIdx.x / TPR, t = threadIdx.x % TPR;
  const long long row = static_cast<long long>(blockIdx.x) * RPB + sub;
  const bool live = row < rows;
  const int nvec = d >> 3;
  float v[VPL][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = i * TPR + t;
    if (live && vi < nvec) {
      V8<T>::load(x + row * d + vi * 8, v[i]);
      if constexpr (ADD) {
        float dl[8];
        V8<T>::load(delta + row * d + vi * 8, dl);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += dl[j];
        // the residual stream is stored in T, and the norm is taken over the stored values
        V8<T>::store(xn + row * d + vi * 8, v[i]);
        if constexpr (sizeof(T) == 2) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16(v[i][j]));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  ss = row_sum<TPR>(ss, scratch);
  const float r = rsqrtf(ss / static_cast<float>(d) + eps);
  if (live && t == 0 && rstd != nullptr) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = i * TPR + t;
    if (live && vi < nvec) {
      float wv[8], o[8];
      V8<WT>::load(w + vi * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * r * wv[j];
      V8<T>::store(y + row * d + vi * 8, o);
    }
  }
}

// ------------------------------------------------------------------ RMSNorm backward
// dx = r * (dy*w) - x * r^3 / d * sum(dy*w*x) (+ dres);   dw += dy * x * r, reduced over rows in
// two deterministic stages (per-block partial rows, then a column sum).
template <typename T, typename WT, int TPR, int VPL>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const WT* __restrict__ w,
                   const float* __restrict__ rstd, const T* __restrict__ dres, T* __restrict__ dx,
                   float* __restrict__ dw_partial, long long rows, int d) {
  __shared__ float scratch[ROW_THREADS / 32];
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float dw_smem[];           // d floats, only used when several rows share a block
  constexpr int RPB = ROW_THREADS / TPR;
  const int sub = threadIdx.x / TPR, t = threadIdx.x % TPR;
  const int nvec = d >> 3;
  float wv[VPL][8], dwacc[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = i * TPR + t;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dwacc[i][j] = 0.f; wv[i][j] = 0.f; }
    if (vi < nvec) V8<WT>::load(w + vi * 8, wv[i]);
  }
  for (long long base = static_cast<long long>(blockIdx.x) * RPB; base < rows;
       base += static_cast<long long>(gridDim.x) * RPB) {
    const long long row = base + sub;
    const bool live = row < rows;
    const float r = live ? rstd[row] : 0.f;
    float g[VPL][8], xv[VPL][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = i * TPR + t;
      if (live && vi < nvec) {
        V8<T>::load(dy + row * d + vi * 8, g[i]);
        V8<T>::load(x + row * d + vi * 8, xv[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dwacc[i][j] += g[i][j] * xv[i][j] * r;
          g[i][j] *= wv[i][j];
          dot += g[i][j] * xv[i][j];
        }
      }
    }
    dot = row_sum<TPR>(dot, scratch);
    const float c = dot * r * r * r / static_cast<float>(d);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = i * TPR + t;
      if (live && vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = g[i][j] * r - xv[i][j] * c;
        if (dres != nullptr) {
          float rs[8];
          V8<T>::load(dres + row * d + vi * 8, rs);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += rs[j];
        }
        V8<T>::store(dx + row * d + vi * 8, o);
      }
    }
  }
  if (dw_partial == nullptr) return;
  if constexpr (RPB > 1) {
    // the RPB row groups of the block hold partial sums of the same columns: fold them in a fixed order
    for (int turn = 0; turn < RPB; ++turn) {
      if (sub == turn) {
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
          const int vi = i * TPR + t;
          if (vi < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float prev = turn == 0 ? 0.f : dw_smem[vi * 8 + j];
              dw_smem[vi * 8 + j] = prev + dwacc[i][j];
            }
          }
        }
      }
      __syncthreads();
    }
    for (int c = threadIdx.x; c < d; c += ROW_THREADS) dw_partial[static_cast<long long>(blockIdx.x) * d + c] = dw_smem[c];
  } else {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = i * TPR + t;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) dw_partial[static_cast<long long>(blockIdx.x) * d + vi * 8 + j] = dwacc[i][j];
      }
    }
  }
}

// Column sums of part[nrows, d] in a fixed order: block = 32 columns x 32 row groups.
__global__ void __launch_bounds__(1024)
colsum_kernel(const float* __restrict__ part, float* __restrict__ out, int nrows, int d, int accumulate) {
  __shared__ float red[32][33];
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < d)
    for (int r = threadIdx.y; r < nrows; r += 32) s += part[static_cast<long long>(r) * d + c];
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < d) {
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < 32; ++g) t += red[g][threadIdx.x];
    out[c] = accumulate ? out[c] + t : t;
  }
}

// ------------------------------------------------------------------ SwiGLU
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
                                  long long rows, int h, long long ld_in, const int* __restrict__ row_limit) {
  pdl_wait();
  pdl_launch_dependents();
  if (row_limit != nullptr) rows = min(rows, static_cast<long long>(*row_limit));   // rows known only on the device
  const int hv = h >> 3;
  const long long total = rows * hv;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / hv;
    const int c = static_cast<int>(i % hv) * 8;
    float g[8], u[8], o[8];
    V8<T>::load(gate + r * ld_in + c, g);
    V8<T>::load(up + r * ld_in + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    V8<T>::store(out + r * h + c, o);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, const T* __restrict__ dy,
                                  T* __restrict__ dgate, T* __restrict__ dup, long long rows, int h, long long ld_in,
                                  const int* __restrict__ row_limit) {
  pdl_wait();
  pdl_launch_dependents();
  if (row_limit != nullptr) rows = min(rows, static_cast<long long>(*row_limit));
  const int hv = h >> 3;
  const long long total = rows * hv;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / hv;
    const int c = static_cast<int>(i % hv) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    V8<T>::load(gate + r * ld_in + c, g);
    V8<T>::load(up + r * ld_in + c, u);
    V8<T>::load(dy + r * h + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      du[j] = d[j] * g[j] * s;
      dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
    }
    V8<T>::store(dgate + r * ld_in + c, dg);
    V8<T>::store(dup + r * ld_in + c, du);
  }
}

// ------------------------------------------------------------------ RoPE (half-split)
// Rotates the first n_rot heads of every row; the remaining heads are copied when dst != src.
// With q32 given, the first n_q32 heads are read from that packed fp32 tensor [rows, n_q32, hd] instead of
// src (the attention backward leaves dQ there as an fp32 sum; this pass is then also its conversion).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ src, T* __restrict__ dst, const float* __restrict__ cs,
                            const float* __restrict__ sn, long long rows, int T_len, int n_rot, int heads_total, int hd,
                            float sign, const float* __restrict__ q32, int n_q32) {
  pdl_wait();
  pdl_launch_dependents();
  const int half = hd >> 1;
  const int hv = half >> 3;
  const bool inplace = src == dst;
  const int heads = inplace ? n_rot : heads_total;
  const long long total = rows * heads * hv;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % hv) * 8;
    const long long rh = i / hv;
    const int head = static_cast<int>(rh % heads);
    const long long row = rh / heads;
    const long long off = (row * heads_total + head) * hd + c;
    float a[8], b[8], oa[8], ob[8];
    if (q32 != nullptr && head < n_q32) {
      const long long off32 = (row * n_q32 + head) * hd + c;
      V8<float>::load(q32 + off32, a);
      V8<float>::load(q32 + off32 + half, b);
    } else {
      V8<T>::load(src + off, a);
      V8<T>::load(src + off + half, b);
    }
    if (head < n_rot) {
      const int pos = static_cast<int>(row % T_len);
      float co[8], si[8];
      V8<float>::load(cs + static_cast<long long>(pos) * half + c, co);
      V8<float>::load(sn + static_cast<long long>(pos) * half + c, si);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float s = si[j] * sign;
        oa[j] = a[j] * co[j] - b[j] * s;
        ob[j] = a[j] * s + b[j] * co[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { oa[j] = a[j]; ob[j] = b[j]; }
    }
    V8<T>::store(dst + off, oa);
    V8<T>::store(dst + off + half, ob);
  }
}

// ------------------------------------------------------------------ per-head RMSNorm + RoPE
// Eight lanes per (row, head): lane l holds elements [8l, 8l+8) of each half (hd <= 128).
template <typename T, typename WT>
__global__ void qknorm_rope_fwd_kernel(const T* __restrict__ x, const WT* __restrict__ w, const float* __restrict__ cs,
                                       const float* __restrict__ sn, T* __restrict__ y, float* __restrict__ rstd,
                                       long long n_heads_rows, int T_len, int H, int hd, float eps) {
  const int half = hd >> 1;
  const int l = threadIdx.x & 7;
  const long long item = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
  const bool live = item < n_heads_rows;
  const bool has = live && (l * 8 < half);
  float a[8] = {0}, b[8] = {0};
  const long long off = item * hd + l * 8;
  if (has) { V8<T>::load(x + off, a); V8<T>::load(x + off + half, b); }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss += a[j] * a[j] + b[j] * b[j];
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  ss += __shfl_xor_sync(0xffffffffu, ss, 4);
  const float r = rsqrtf(ss / static_cast<float>(hd) + eps);
  if (live && l == 0 && rstd != nullptr) rstd[item] = r;
  if (!has) return;
  const int pos = static_cast<int>((item / H) % T_len);
  float wa[8], wb[8], co[8], si[8], oa[8], ob[8];
  V8<WT>::load(w + l * 8, wa);
  V8<WT>::load(w + half + l * 8, wb);
  V8<float>::load(cs + static_cast<long long>(pos) * half + l * 8, co);
  V8<float>::load(sn + static_cast<long long>(pos) * half + l * 8, si);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float y1 = a[j] * r * wa[j], y2 = b[j] * r * wb[j];
    oa[j] = y1 * co[j] - y2 * si[j];
    ob[j] = y1 * si[j] + y2 * co[j];
  }
  V8<T>::store(y + off, oa);
  V8<T>::store(y + off + half, ob);
}

template <typename T, typename WT>
__global__ void qknorm_rope_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const WT* __restrict__ w,
                                       const float* __restrict__ cs, const float* __restrict__ sn,
                                       const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_partial,
                                       long long n_heads_rows, int T_len, int H, int hd) {
  const int half = hd >> 1;
  const int l = threadIdx.x & 7;
  const bool col_ok = l * 8 < half;
  float wa[8] = {0}, wb[8] = {0}, dwa[8] = {0}, dwb[8] = {0};
  if (col_ok) { V8<WT>::load(w + l * 8, wa); V8<WT>::load(w + half + l * 8, wb); }
  const long long groups = (static_cast<long long>(gridDim.x) * blockDim.x) >> 3;
  for (long long item = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
       item < ((n_heads_rows + groups - 1) / groups) * groups; item += groups) {
    const bool live = item < n_heads_rows;
    const bool has = live && col_ok;
    float a[8] = {0}, b[8] = {0}, ga[8] = {0}, gb[8] = {0};
    const long long off = item * hd + l * 8;
    float r = 0.f;
    if (has) {
      float g1[8], g2[8], co[8], si[8];
      r = rstd[item];
      const int pos = static_cast<int>((item / H) % T_len);
      V8<T>::load(x + off, a); V8<T>::load(x + off + half, b);
      V8<T>::load(dy + off, g1); V8<T>::load(dy + off + half, g2);
      V8<float>::load(cs + static_cast<long long>(pos) * half + l * 8, co);
      V8<float>::load(sn + static_cast<long long>(pos) * half + l * 8, si);
#pragma unroll
      for (int j = 0; j < 8; ++j) {   // undo the rotation: gradient w.r.t. the normalised values
        ga[j] = g1[j] * co[j] + g2[j] * si[j];
        gb[j] = -g1[j] * si[j] + g2[j] * co[j];
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dwa[j] += ga[j] * a[j] * r; dwb[j] += gb[j] * b[j] * r;
      ga[j] *= wa[j]; gb[j] *= wb[j];
      dot += ga[j] * a[j] + gb[j] * b[j];
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    dot += __shfl_xor_sync(0xffffffffu, dot, 4);
    if (has) {
      const float c = dot * r * r * r / static_cast<float>(hd);
      float oa[8], ob[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { oa[j] = ga[j] * r - a[j] * c; ob[j] = gb[j] * r - b[j] * c; }
      V8<T>::store(dx + off, oa);
      V8<T>::store(dx + off + half, ob);
    }
  }
  // fold the lanes that share a column (same l) inside the block, in a fixed order
  __shared__ float acc[ROW_THREADS / 8][16];
  const int grp = threadIdx.x >> 3;
  float* mine = nullptr;
  for (int part = 0; part < 8; ++part) {       // 8 lanes x 16 values per group, staged through smem
    __syncthreads();
    if (l == part) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { acc[grp][j] = dwa[j]; acc[grp][8 + j] = dwb[j]; }
    }
    __syncthreads();
    if (threadIdx.x < 16 && part * 8 < half) {
      float s = 0.f;
      for (int g2 = 0; g2 < ROW_THREADS / 8; ++g2) s += acc[g2][threadIdx.x];
      const int col = threadIdx.x < 8 ? part * 8 + threadIdx.x : half + part * 8 + (threadIdx.x - 8);
      dw_partial[static_cast<long long>(blockIdx.x) * hd + col] = s;
    }
  }
  (void)mine;
}

// ------------------------------------------------------------------ softmax
template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int n) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * n;
  float m = -CUDART_INF_F;
  bool has_nan = false;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = static_cast<float>(xr[i]);
    has_nan |= (v != v);
    m = fmaxf(m, v);
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
  for (int i = 1; i < (blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
  __syncthreads();
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += __expf(static_cast<float>(xr[i]) - m);
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  s = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) s += red[i];
  const int any_nan = __syncthreads_or(has_nan ? 1 : 0);
  const float inv = 1.f / s;     // all -inf row: exp(nan) -> nan, like torch
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = __expf(static_cast<float>(xr[i]) - m) * inv;
    if (any_nan) v = CUDART_NAN_F;
    y[row * n + i] = static_cast<T>(v);
  }
}

// Rows of up to 1024 values: one warp per row, the row lives in registers (one read, one write).
template <typename T, int VPT>
__global__ void __launch_bounds__(256)
softmax_fwd_warp_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + row * n;
  float v[VPT];
  float m = -CUDART_INF_F;
  bool has_nan = false;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = j * 32 + lane;
    v[j] = i < n ? static_cast<float>(xr[i]) : -CUDART_INF_F;
    has_nan |= (v[j] != v[j]);
    m = fmaxf(m, v[j]);
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    v[j] = (j * 32 + lane) < n ? __expf(v[j] - m) : 0.f;
    s += v[j];
  }
  s = warp_sum(s);
  const bool any_nan = __any_sync(0xffffffffu, has_nan);
  const float inv = 1.f / s;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = j * 32 + lane;
    if (i < n) y[row * n + i] = static_cast<T>(any_nan ? CUDART_NAN_F : v[j] * inv);
  }
}

template <typename T, int VPT>
__global__ void __launch_bounds__(256)
softmax_bwd_warp_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, long long rows, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float yv[VPT], gv[VPT];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = j * 32 + lane;
    yv[j] = i < n ? static_cast<float>(y[row * n + i]) : 0.f;
    gv[j] = i < n ? static_cast<float>(dy[row * n + i]) : 0.f;
    s += yv[j] * gv[j];
  }
  s = warp_sum(s);
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = j * 32 + lane;
    if (i < n) dx[row * n + i] = static_cast<T>(yv[j] * (gv[j] - s));
  }
}

template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                                   long long rows, int n) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    s += static_cast<float>(y[row * n + i]) * static_cast<float>(dy[row * n + i]);
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  s = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) s += red[i];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float yv = static_cast<float>(y[row * n + i]);
    dx[row * n + i] = static_cast<T>((static_cast<float>(dy[row * n + i]) - s) * yv);
  }
}

// ------------------------------------------------------------------ top-k
// Exact selection in k rounds; order: value descending (NaN counts as largest), then index
// ascending, which also fixes which of several equal values at the boundary is kept.
__device__ __forceinline__ bool key_before(float va, int ia, float vb, int ib) {
  const bool na = va != va, nb = vb != vb;
  if (na != nb) return na;
  if (!na && va != vb) return va > vb;
  return ia < ib;
}

template <typename T>
__global__ void topk_kernel(const T* __restrict__ x, T* __restrict__ values, long long* __restrict__ indices,
                            long long rows, int n, int k) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float last_v;
  __shared__ int last_i;
  const long long row = blockIdx.x;
  const T* xr = x + row * n;
  for (int round = 0; round < k; ++round) {
    float bv = 0.f;
    int bi = -1;
    const float lv = last_v;
    const int li = last_i;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = static_cast<float>(xr[i]);
      if (round > 0 && !key_before(lv, li, v, i)) continue;      // already taken (or is the last pick)
      if (bi < 0 || key_before(v, i, bv, bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi >= 0 && (bi < 0 || key_before(ov, oi, bv, bi))) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = bv; s_idx[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int wq = 1; wq < (blockDim.x >> 5); ++wq) {
        if (s_idx[wq] >= 0 && (bi < 0 || key_before(s_val[wq], s_idx[wq], bv, bi))) { bv = s_val[wq]; bi = s_idx[wq]; }
      }
      last_v = bv;
      last_i = bi;
      values[row * k + round] = xr[bi];
      indices[row * k + round] = bi;
    }
    __syncthreads();
  }
}


// Top-k by radix selection, one CTA per row. The row is staged in shared memory as order-preserving
// integer keys (16 bits for bf16, 32 for fp32; NaN maps to the largest key); the k-th largest key is
// found digit by digit with 256-bin histograms, the winners are gathered (ties at the boundary by
// smallest index) and the k of them are sorted with a bitonic network. The row is read from global
// memory once, whatever k is. Used when the keys of a row fit in shared memory and k <= 1024.
template <typename T> struct TopkKey;
template <> struct TopkKey<float> {
  using Key = uint32_t;
  static constexpr int BITS = 32;
  static __device__ __forceinline__ Key of(float f) {
    if (f != f) return 0xFFFFFFFFu;
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  }
};
template <> struct TopkKey<__nv_bfloat16> {
  using Key = uint16_t;
  static constexpr int BITS = 16;
  static __device__ __forceinline__ Key of(__nv_bfloat16 b) {
    const uint16_t u = __bfloat16_as_ushort(b);
    if ((u & 0x7FFFu) > 0x7F80u) return 0xFFFFu;
    return (u & 0x8000u) ? static_cast<uint16_t>(~u) : static_cast<uint16_t>(u | 0x8000u);
  }
};

constexpr int TOPK_THREADS = 512;

template <typename T>
__global__ void __launch_bounds__(TOPK_THREADS)
topk_select_kernel(const T* __restrict__ x, T* __restrict__ values, long long* __restrict__ indices, long long rows,
                   int n, int k, int kpad) {
  using KT = TopkKey<T>;
  using Key = typename KT::Key;
  extern __shared__ __align__(16) uint8_t topk_smem[];
  uint32_t* sel_key = reinterpret_cast<uint32_t*>(topk_smem);          // [kpad]
  int* sel_idx = reinterpret_cast<int*>(sel_key + kpad);               // [kpad]
  int* hist = sel_idx + kpad;                                          // [256]
  int* misc = hist + 256;                                              // [8]: prefix, remaining, counters
  int* warp_cnt = misc + 8;                                            // [16]
  Key* keys = reinterpret_cast<Key*>(warp_cnt + 16);                   // [n]
  const long long row = blockIdx.x;
  const T* xr = x + row * n;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < n; i += TOPK_THREADS) keys[i] = KT::of(xr[i]);
  if (tid == 0) { misc[0] = 0; misc[1] = k; misc[2] = 0; misc[3] = 0; }
  __syncthreads();
  // ---- the k-th largest key, one byte at a time
  for (int shift = KT::BITS - 8; shift >= 0; shift -= 8) {
    for (int b = tid; b < 256; b += TOPK_THREADS) hist[b] = 0;
    __syncthreads();
    const uint32_t prefix = static_cast<uint32_t>(misc[0]);
    const int hi = shift + 8;
    for (int i = tid; i < n; i += TOPK_THREADS) {
      const uint32_t key = keys[i];
      if (hi >= KT::BITS || (key >> hi) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int remaining = misc[1], b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= remaining) break;
        remaining -= hist[b];
      }
      misc[0] = static_cast<int>((prefix << 8) | static_cast<uint32_t>(b));
      misc[1] = remaining;
    }
    __syncthreads();
  }
  const uint32_t thr = static_cast<uint32_t>(misc[0]);
  const int need_eq = misc[1];             // how many keys equal to the threshold belong to the result
  const int n_gt = k - need_eq;
  // ---- keys above the threshold: any order (sorted afterwards)
  for (int i = tid; i < n; i += TOPK_THREADS) {
    const uint32_t key = keys[i];
    if (key > thr) {
      const int pos = atomicAdd(&misc[2], 1);
      sel_key[pos] = key;
      sel_idx[pos] = i;
    }
  }
  // ---- keys equal to the threshold: the first need_eq of them in index order
  for (int base = 0; base < n; base += TOPK_THREADS) {
    __syncthreads();
    const int taken = misc[3];
    if (taken >= need_eq) break;
    const int i = base + tid;
    const bool eq = i < n && static_cast<uint32_t>(keys[i]) == thr;
    const unsigned ballot = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) warp_cnt[warp] = __popc(ballot);
    __syncthreads();
    int before = taken;
    for (int w = 0; w < warp; ++w) before += warp_cnt[w];
    const int rank = before + __popc(ballot & ((1u << lane) - 1u));
    if (eq && rank < need_eq) {
      sel_key[n_gt + rank] = thr;
      sel_idx[n_gt + rank] = i;
    }
    __syncthreads();
    if (tid == 0) {
      int total = 0;
      for (int w = 0; w < TOPK_THREADS / 32; ++w) total += warp_cnt[w];
      misc[3] = taken + total;
    }
  }
  __syncthreads();
  for (int i = k + tid; i < kpad; i += TOPK_THREADS) { sel_key[i] = 0; sel_idx[i] = 0x7FFFFFFF; }   // padding sorts last
  __syncthreads();
  // ---- bitonic sort: key descending, then index ascending
  for (int size = 2; size <= kpad; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < (kpad >> 1); t += TOPK_THREADS) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi2 = lo + stride;
        const bool up = (lo & size) == 0;
        const uint32_t ka = sel_key[lo], kb = sel_key[hi2];
        const int ia = sel_idx[lo], ib = sel_idx[hi2];
        const bool a_first = ka > kb || (ka == kb && ia < ib);
        if (a_first != up) { sel_key[lo] = kb; sel_key[hi2] = ka; sel_idx[lo] = ib; sel_idx[hi2] = ia; }
      }
      __syncthreads();
    }
  }
  for (int i = tid; i < k; i += TOPK_THREADS) {
    const int idx = sel_idx[i];
    values[row * k + i] = xr[idx];
    indices[row * k + i] = idx;
  }
}

// ------------------------------------------------------------------ dispatch helpers
template <typename F>
static int by_dtype(int dtype, F&& f) {
  if (dtype == FMB_BF16) return f(static_cast<__nv_bfloat16*>(nullptr));
  if (dtype == FMB_F32) return f(static_cast<float*>(nullptr));
  return -1;
}

static int grid_for(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

template <typename T, typename WT, bool ADD>
static int launch_rms_fwd(const void* x, const void* delta, const void* w, void* xn, void* y, float* rstd,
                          long long rows, int d, float eps, cudaStream_t st) {
  const int nvec = d / 8;
#define FMB_RMS_FWD(TPR, VPL)                                                                         \
  {                                                                                                   \
    constexpr int RPB = ROW_THREADS / TPR;                                                            \
    const unsigned blocks = static_cast<unsigned>((rows + RPB - 1) / RPB);                            \
    return launch_pdl(rmsnorm_fwd_kernel<T, WT, TPR, VPL, ADD>, dim3(blocks), dim3(ROW_THREADS), 0, st, \
        static_cast<const T*>(x), static_cast<const T*>(delta), static_cast<const WT*>(w),            \
        static_cast<T*>(xn), static_cast<T*>(y), rstd, rows, d, eps) == cudaSuccess ? 0 : -3;         \
  }
  if (nvec <= 32) FMB_RMS_FWD(32, 1)
  if (nvec <= 64) FMB_RMS_FWD(32, 2)
  if (nvec <= 128) FMB_RMS_FWD(32, 4)
  if (nvec <= 256) FMB_RMS_FWD(32, 8)
  if (nvec <= 512) FMB_RMS_FWD(256, 2)
  if (nvec <= 1024) FMB_RMS_FWD(256, 4)
  if (nvec <= 2048) FMB_RMS_FWD(256, 8)
#undef FMB_RMS_FWD
  return -2;
}

template <typename T, typename WT>
static int launch_rms_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                          float* dwp, long long rows, int d, int nblocks, cudaStream_t st) {
  const int nvec = d / 8;
#define FMB_RMS_BWD(TPR, VPL)                                                                         \
  {                                                                                                   \
    const size_t sm = TPR < ROW_THREADS ? sizeof(float) * d : 0;                                      \
    return launch_pdl(rmsnorm_bwd_kernel<T, WT, TPR, VPL>, dim3(nblocks), dim3(ROW_THREADS), sm, st,  \
        static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const WT*>(w), rstd,         \
        static_cast<const T*>(dres), static_cast<T*>(dx), dwp, rows, d) == cudaSuccess ? 0 : -3;      \
  }
  // few values per thread: the kernel keeps four of them (dy, x, w, dw) live per element
  if (nvec <= 32) FMB_RMS_BWD(32, 1)
  if (nvec <= 64) FMB_RMS_BWD(64, 1)
  if (nvec <= 128) FMB_RMS_BWD(128, 1)
  if (nvec <= 256) FMB_RMS_BWD(256, 1)
  if (nvec <= 512) FMB_RMS_BWD(256, 2)
  if (nvec <= 1024) FMB_RMS_BWD(256, 4)
  if (nvec <= 2048) FMB_RMS_BWD(256, 8)
#undef FMB_RMS_BWD
  return -2;
}

}  // namespace fmb

using namespace fmb;

extern "C" int fmb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int d, float eps,
                               int dtype, int w_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (d % 8) return -2;
  return by_dtype(dtype, [&](auto* tp) {
    using T = std::remove_pointer_t<decltype(tp)>;
    if (w_dtype == dtype) return launch_rms_fwd<T, T, false>(x, nullptr, w, nullptr, y, rstd, rows, d, eps, stream);
    if (w_dtype == FMB_F32) return launch_rms_fwd<T, float, false>(x, nullptr, w, nullptr, y, rstd, rows, d, eps, stream);
    return -1;
  });
}

extern "C" int fmb_add_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* xn, void* y, float* rstd,
                                   long long rows, int d, float eps, int dtype, int w_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (d % 8) return -2;
  return by_dtype(dtype, [&](auto* tp) {
    using T = std::remove_pointer_t<decltype(tp)>;
    if (w_dtype == dtype) return launch_rms_fwd<T, T, true>(x, delta, w, xn, y, rstd, rows, d, eps, stream);
    if (w_dtype == FMB_F32) return launch_rms_fwd<T, float, true>(x, delta, w, xn, y, rstd, rows, d, eps, stream);
    return -1;
  });
}

extern "C" int fmb_rmsnorm_bwd_blocks(long long rows, int d) {
  const int nvec = d / 8;
  const int tpr = nvec <= 32 ? 32 : nvec <= 64 ? 64 : nvec <= 128 ? 128 : 256;
  const int rpb = ROW_THREADS / tpr;
  long long need = (rows + rpb - 1) / rpb;
  long long cap = static_cast<long long>(sm_count()) * (nvec <= 256 ? 4 : 2);
  return static_cast<int>(need < 1 ? 1 : (need > cap ? cap : need));
}

extern "C" int fmb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                               void* dx, float* dw_partial, float* dw, int dw_accumulate, long long rows, int d,
                               int dtype, int w_dtype, int nblocks, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (d % 8) return -2;
  int rc = by_dtype(dtype, [&](auto* tp) {
    using T = std::remove_pointer_t<decltype(tp)>;
    if (w_dtype == dtype) return launch_rms_bwd<T, T>(dy, x, w, rstd, dres, dx, dw_partial, rows, d, nblocks, stream);
    if (w_dtype == FMB_F32) return launch_rms_bwd<T, float>(dy, x, w, rstd, dres, dx, dw_partial, rows, d, nblocks, stream);
    return -1;
  });
  if (rc != 0 || dw_partial == nullptr || dw == nullptr) return rc;
  return launch_pdl(colsum_kernel, dim3((d + 31) / 32), dim3(32, 32), 0, stream, dw_partial, dw, nblocks, d,
                    dw_accumulate) == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_swiglu_fwd(const void* gate, const void* up, void* out, long long rows, int h, long long ld_in,
                              int dtype, const int* row_limit, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (h % 8 || ld_in % 8) return -2;
  return by_dtype(dtype, [&](auto* tp) {
    using T = std::remove_pointer_t<decltype(tp)>;
    return launch_pdl(swiglu_fwd_kernel<T>, dim3(grid_for(rows * (h / 8), 256)), dim3(256), 0, stream,
                      static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<T*>(out), rows, h,
                      ld_in, row_limit) == cudaSuccess ? 0 : -3;
  });
}

extern "C" int fmb_swiglu_bwd(const void* gate, const void* up, const void* dy, void* dgate, void* dup, long long rows,
                              int h, long long ld_in, int dtype, const int* row_limit, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (h % 8 || ld_in % 8) return -2;
  return by_dtype(dtype, [&](auto* tp) {
    using T = std::remove_pointer_t<decltype(tp)>;
    return launch_pdl(swiglu_bwd_kernel<T>, dim3(grid_for(rows * (h / 8), 256)), dim3(256), 0, stream,
                      static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<const T*>(dy),
                      static_cast<T*>(dgate), static_cast<T*>(dup), rows, h, ld_in, row_limit) == cudaSuccess ? 0 : -3;
  });
}

extern "C" int fmb_rope(const void* src, void* dst, const float* cos, const float* sin, long long rows, int T,
                        int n_rot_heads, int heads_total, int hd, float sign, int dtype, const float* q32, int n_q32,
                        cudaStream_t stream) {
  if (rows <= 0 || n_rot_heads <= 0) return 0;
  if (hd % 16) return -2;
  if (q32 != nullptr && (n_q32 <= 0 || n_q32 > n_rot_heads || (reinterpret_cast<uintptr_t>(q32) & 15))) return -2;
  const int heads = src == dst ? n_rot_heads : heads_total;
  return by_dtype(dtype, [&](auto* tp) {
    using Tt = std::remove_pointer_t<decltype(tp)>;
    return launch_pdl(rope_kernel<Tt>, dim3(grid_for(rows * heads * (hd / 16), 256)), dim3(256), 0, stream,
                      static_cast<const Tt*>(src), static_cast<Tt*>(dst), cos, sin, rows, T, n_rot_heads, heads_total,
                      hd, sign, q32, q32 ? n_q32 : 0) == cudaSuccess ? 0 : -3;
  });
}

extern "C" int fmb_qk_norm_rope_fwd(const void* x, const void* w, const float* cos, const float* sin, void* y,
                                    float* rstd, long long rows, int T, int H, int hd, float eps, int dtype,
                                    int w_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hd % 16 || hd > 128) return -2;
  const long long items = rows * H;
  const unsigned blocks = static_cast<unsigned>((items * 8 + ROW_THREADS - 1) / ROW_THREADS);
  return by_dtype(dtype, [&](auto* tp) {
    using Tt = std::remove_pointer_t<decltype(tp)>;
    if (w_dtype == dtype)
      qknorm_rope_fwd_kernel<Tt, Tt><<<blocks, ROW_THREADS, 0, stream>>>(
          static_cast<const Tt*>(x), static_cast<const Tt*>(w), cos, sin, static_cast<Tt*>(y), rstd, items, T, H, hd, eps);
    else if (w_dtype == FMB_F32)
      qknorm_rope_fwd_kernel<Tt, float><<<blocks, ROW_THREADS, 0, stream>>>(
          static_cast<const Tt*>(x), static_cast<const float*>(w), cos, sin, static_cast<Tt*>(y), rstd, items, T, H, hd, eps);
    else return -1;
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  });
}

extern "C" int fmb_qk_norm_rope_bwd(const void* dy, const void* x, const void* w, const float* cos, const float* sin,
                                    const float* rstd, void* dx, float* dw_partial, float* dw, long long rows, int T,
                                    int H, int hd, int dtype, int w_dtype, int nblocks, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hd % 16 || hd > 128) return -2;
  const long long items = rows * H;
  int rc = by_dtype(dtype, [&](auto* tp) {
    using Tt = std::remove_pointer_t<decltype(tp)>;
    if (w_dtype == dtype)
      qknorm_rope_bwd_kernel<Tt, Tt><<<nblocks, ROW_THREADS, 0, stream>>>(
          static_cast<const Tt*>(dy), static_cast<const Tt*>(x), static_cast<const Tt*>(w), cos, sin, rstd,
          static_cast<Tt*>(dx), dw_partial, items, T, H, hd);
    else if (w_dtype == FMB_F32)
      qknorm_rope_bwd_kernel<Tt, float><<<nblocks, ROW_THREADS, 0, stream>>>(
          static_cast<const Tt*>(dy), static_cast<const Tt*>(x), static_cast<const float*>(w), cos, sin, rstd,
          static_cast<Tt*>(dx), dw_partial, items, T, H, hd);
    else return -1;
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  });
  if (rc != 0) return rc;
  launch_pdl(colsum_kernel, dim3((hd + 31) / 32), dim3(32, 32), 0, stream, dw_partial, dw, nblocks, hd, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_softmax_fwd(const void* x, void* y, long long rows, int n, int dtype, cudaStream_t stream) {
  if (rows <= 0 || n <= 0) return 0;
  const int threads = n >= 1024 ? 256 : (n >= 128 ? 128 : 32);
  return by_dtype(dtype, [&](auto* tp) {
    using T = std::remove_pointer_t<decltype(tp)>;
    if (n <= 1024) {
      const dim3 grid(static_cast<unsigned>((rows * 32 + 255) / 256));
      const T* xp = static_cast<const T*>(x);
      T* yp = static_cast<T*>(y);
      cudaError_t e;
      if (n <= 128) e = launch_pdl(softmax_fwd_warp_kernel<T, 4>, grid, dim3(256), 0, stream, xp, yp, rows, n);
      else if (n <= 256) e = launch_pdl(softmax_fwd_warp_kernel<T, 8>, grid, dim3(256), 0, stream, xp, yp, rows, n);
      else if (n <= 512) e = launch_pdl(softmax_fwd_warp_kernel<T, 16>, grid, dim3(256), 0, stream, xp, yp, rows, n);
      else e = launch_pdl(softmax_fwd_warp_kernel<T, 32>, grid, dim3(256), 0, stream, xp, yp, rows, n);
      return e == cudaSuccess ? 0 : -3;
    }
    softmax_fwd_kernel<T><<<static_cast<unsigned>(rows), threads, 0, stream>>>(static_cast<const T*>(x), static_cast<T*>(y), rows, n);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  });
}

extern "C" int fmb_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int n, int dtype,
                               cudaStream_t stream) {
  if (rows <= 0 || n <= 0) return 0;
  const int threads = n >= 1024 ? 256 : (n >= 128 ? 128 : 32);
  return by_dtype(dtype, [&](auto* tp) {
    using T = std::remove_pointer_t<decltype(tp)>;
    if (n <= 1024) {
      const dim3 grid(static_cast<unsigned>((rows * 32 + 255) / 256));
      const T* yp = static_cast<const T*>(y);
      const T* gp = static_cast<const T*>(dy);
      T* dp = static_cast<T*>(dx);
      cudaError_t e;
      if (n <= 128) e = launch_pdl(softmax_bwd_warp_kernel<T, 4>, grid, dim3(256), 0, stream, yp, gp, dp, rows, n);
      else if (n <= 256) e = launch_pdl(softmax_bwd_warp_kernel<T, 8>, grid, dim3(256), 0, stream, yp, gp, dp, rows, n);
      else if (n <= 512) e = launch_pdl(softmax_bwd_warp_kernel<T, 16>, grid, dim3(256), 0, stream, yp, gp, dp, rows, n);
      else e = launch_pdl(softmax_bwd_warp_kernel<T, 32>, grid, dim3(256), 0, stream, yp, gp, dp, rows, n);
      return e == cudaSuccess ? 0 : -3;
    }
    softmax_bwd_kernel<T><<<static_cast<unsigned>(rows), threads, 0, stream>>>(
        static_cast<const T*>(y), static_cast<const T*>(dy), static_cast<T*>(dx), rows, n);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  });
}

extern "C" int fmb_topk(const void* x, void* values, long long* indices, long long rows, int n, int k, int dtype,
                        cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (k < 1 || k > n) return -2;
  const int threads = n >= 4096 ? 512 : (n >= 512 ? 256 : 64);
  return by_dtype(dtype, [&](auto* tp) {
    using T = std::remove_pointer_t<decltype(tp)>;
    int kpad = 2;
    while (kpad < k) kpad <<= 1;
    const size_t smem = static_cast<size_t>(kpad) * 8 + (256 + 8 + 16) * 4 + static_cast<size_t>(n) * sizeof(typename TopkKey<T>::Key) + 16;
    if (k <= 1024 && n >= 1024 && smem <= 200 * 1024) {       // one pass over the row
      auto kern = topk_select_kernel<T>;
      static bool attr_set = false;
      if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return -6;
        attr_set = true;
      }
      kern<<<static_cast<unsigned>(rows), TOPK_THREADS, smem, stream>>>(static_cast<const T*>(x), static_cast<T*>(values),
                                                                       indices, rows, n, k, kpad);
      return cudaGetLastError() == cudaSuccess ? 0 : -3;
    }
    topk_kernel<T><<<static_cast<unsigned>(rows), threads, 0, stream>>>(static_cast<const T*>(x), static_cast<T*>(values), indices, rows, n, k);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  });
}

// ------------------------------------------------------------------ allocation-free RMSNorm backward
// See fmb_noalloc.h for who this is for and for the rules of use. The scratch for the per-block
// weight-gradient partial sums is this file-scope device array. Host code must not pass the symbol
// itself to a kernel: in host code the name is only a handle. Its device address is fetched once per
// device with cudaGetSymbolAddress and that pointer is what the launcher receives.
#include "fmb_noalloc.h"
#include <atomic>
#include <cstdio>

static __device__ __align__(256) float g_noalloc_scratch[FMB_NOALLOC_MAX_D * FMB_NOALLOC_MAX_BLOCKS];

extern "C" int fmb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                       float* dw, long long rows, int d, int dtype, int w_dtype, cudaStream_t stream) {
  // one slot per device; atomic because two host threads may make their first call at the same time
  // (both then look the address up and store the same value)
  static std::atomic<float*> scratch_of_device[64];
  if (rows <= 0) return 0;
  if (d <= 0 || d % 8) {
    std::fprintf(stderr, "fmb_rmsnorm_bwd_noalloc: row width %d is not a positive multiple of 8\n", d);
    return FMB_NOALLOC_BAD_WIDTH;
  }
  int nblocks = fmb_rmsnorm_bwd_blocks(rows, d);
  if (nblocks > FMB_NOALLOC_MAX_BLOCKS) nblocks = FMB_NOALLOC_MAX_BLOCKS;   // the kernel strides over the rows
  if (d > FMB_NOALLOC_MAX_D ||
      static_cast<long long>(nblocks) * d > static_cast<long long>(FMB_NOALLOC_MAX_D) * FMB_NOALLOC_MAX_BLOCKS) {
    std::fprintf(stderr, "fmb_rmsnorm_bwd_noalloc: row width %d (x %d blocks) exceeds the built-in scratch "
                         "(max width %d); use fmb_rmsnorm_bwd with your own buffer\n", d, nblocks, FMB_NOALLOC_MAX_D);
    return FMB_NOALLOC_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FMB_NOALLOC_SETUP_FAILED;
  float* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // first call on this device (it is the current one): resolve the array's device address
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      std::fprintf(stderr, "fmb_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return FMB_NOALLOC_SETUP_FAILED;
    }
    scratch_of_device[dev].store(ptr, std::memory_order_release);
    scratch = ptr;
  }
  // every block writes its whole row of partial sums before the column sum reads it: nothing to clear
  return fmb_rmsnorm_bwd(dy, x, w, rstd, nullptr, dx, scratch, dw, 0, rows, d, dtype, w_dtype, nblocks, stream);
}
