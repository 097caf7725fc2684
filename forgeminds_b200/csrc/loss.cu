// Cross-entropy and KL(teacher || student) over rows of logits, forward and gradient in one launch.
// A row is reduced with an online (max, sum-exp) pair per thread, merged across the block; the
// second sweep over the row (served by L2) turns the logits into gradients in place.
#include "ptx_sm100.cuh"
#include "fmb_api.h"
#include <math_constants.h>

namespace fmb {

struct MaxSum {
  float m, s;
};
__device__ __forceinline__ MaxSum ms_merge(MaxSum a, MaxSum b) {
  if (a.m == -CUDART_INF_F) return b;
  if (b.m == -CUDART_INF_F) return a;
  const float m = fmaxf(a.m, b.m);
  return {m, a.s * __expf(a.m - m) + b.s * __expf(b.m - m)};
}
__device__ __forceinline__ void ms_push(MaxSum& a, float v) {
  if (v > a.m) { a.s = a.s * __expf(a.m - v) + 1.f; a.m = v; }
  else a.s += __expf(v - a.m);
}
__device__ __forceinline__ MaxSum block_ms(MaxSum v, MaxSum* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other{__shfl_xor_sync(0xffffffffu, v.m, o), __shfl_xor_sync(0xffffffffu, v.s, o)};
    v = ms_merge(v, other);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  MaxSum r = scratch[0];
  for (int i = 1; i < (blockDim.x >> 5); ++i) r = ms_merge(r, scratch[i]);
  return r;
}
__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) r += scratch[i];
  return r;
}

__global__ void __launch_bounds__(256)
ce_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ row_loss,
          long long rows, int V, long long ld, float grad_scale_in, const float* __restrict__ grad_scale_ptr,
          long long ignore_index, int write_grad) {
  __shared__ MaxSum scratch[8];
  const float grad_scale = grad_scale_ptr != nullptr ? grad_scale_in * __ldg(grad_scale_ptr) : grad_scale_in;
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = label == ignore_index || label < 0 || label >= V;
  const int nvec = V >> 3;
  if (ignored) {
    if (threadIdx.x == 0) row_loss[row] = 0.f;
    if (write_grad) {
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) reinterpret_cast<uint4*>(lr)[i] = make_uint4(0, 0, 0, 0);
    }
    return;
  }
  MaxSum acc{-CUDART_INF_F, 0.f};
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(lr)[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16(w[j]);
      ms_push(acc, f.x);
      ms_push(acc, f.y);
    }
  }
  const MaxSum tot = block_ms(acc, scratch);
  const float lse = tot.m + __logf(tot.s);
  if (threadIdx.x == 0) row_loss[row] = lse - __bfloat162float(lr[label]);
  if (!write_grad) return;
  __syncthreads();   // the label logit has been read before anyone overwrites it
  const int lab_vec = static_cast<int>(label >> 3), lab_sub = static_cast<int>(label & 7);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(lr)[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float g[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16(w[j]);
      g[2 * j] = __expf(f.x - lse) * grad_scale;
      g[2 * j + 1] = __expf(f.y - lse) * grad_scale;
    }
    if (i == lab_vec) g[lab_sub] -= grad_scale;
    uint4 o;
    o.x = pack_bf16(g[0], g[1]); o.y = pack_bf16(g[2], g[3]); o.z = pack_bf16(g[4], g[5]); o.w = pack_bf16(g[6], g[7]);
    reinterpret_cast<uint4*>(lr)[i] = o;
  }
}

// KL(softmax(t) || softmax(s)) per row = sum p_t (log p_t - log p_s); grad wrt s = (p_s - p_t) * scale
template <typename T>
__global__ void __launch_bounds__(256)
kl_kernel(const T* __restrict__ s, const T* __restrict__ t, float* __restrict__ row_loss, T* __restrict__ grad,
          long long rows, int V, float grad_scale, int write_grad) {
  __shared__ MaxSum scratch[8];
  __shared__ float fscratch[8];
  const long long row = blockIdx.x;
  const T* sr = s + row * V;
  const T* tr = t + row * V;
  MaxSum as{-CUDART_INF_F, 0.f}, at{-CUDART_INF_F, 0.f};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    ms_push(as, static_cast<float>(sr[i]));
    ms_push(at, static_cast<float>(tr[i]));
  }
  const MaxSum ts = block_ms(as, scratch);
  const MaxSum tt = block_ms(at, scratch);
  const float lse_s = ts.m + __logf(ts.s), lse_t = tt.m + __logf(tt.s);
  float part = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float sv = static_cast<float>(sr[i]), tv = static_cast<float>(tr[i]);
    const float lpt = tv - lse_t, lps = sv - lse_s;
    const float pt = __expf(lpt);
    if (pt > 0.f) part += pt * (lpt - lps);
    if (write_grad) grad[row * V + i] = static_cast<T>((__expf(lps) - pt) * grad_scale);
  }
  part = block_sum(part, fscratch);
  if (threadIdx.x == 0) row_loss[row] = part;
}

// Deterministic sum of n floats by one block (n is a few thousand row losses).
__global__ void __launch_bounds__(1024) sum_kernel(const float* __restrict__ x, float* __restrict__ out, long long n,
                                                   float scale, int accumulate) {
  __shared__ float scratch[32];
  float v = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) v += x[i];
  v = block_sum(v, scratch);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + v * scale : v * scale;
}

}  // namespace fmb

using namespace fmb;

extern "C" int fmb_ce_fwd_bwd(void* logits, const long long* labels, float* row_loss, long long rows, int V,
                              long long ld, float grad_scale, const float* grad_scale_ptr, long long ignore_index,
                              int write_grad, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V % 8 || ld % 8 || (reinterpret_cast<uintptr_t>(logits) & 15)) return -2;
  ce_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(logits), labels, row_loss, rows,
                                                            V, ld, grad_scale, grad_scale_ptr, ignore_index, write_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_kl_fwd_bwd(const void* student, const void* teacher, float* row_loss, void* grad, long long rows,
                              int V, float grad_scale, int dtype, int write_grad, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dtype == FMB_BF16)
    kl_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(student), static_cast<const __nv_bfloat16*>(teacher), row_loss,
        static_cast<__nv_bfloat16*>(grad), rows, V, grad_scale, write_grad);
  else if (dtype == FMB_F32)
    kl_kernel<float><<<static_cast<unsigned>(rows), 256, 0, stream>>>(
        static_cast<const float*>(student), static_cast<const float*>(teacher), row_loss, static_cast<float*>(grad),
        rows, V, grad_scale, write_grad);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_sum_f32(const float* x, float* out, long long n, float scale, int accumulate, cudaStream_t stream) {
  sum_kernel<<<1, 1024, 0, stream>>>(x, out, n, scale, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
