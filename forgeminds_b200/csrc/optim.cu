// Optimizer-side kernels over flat buffers: fused AdamW (clip coefficient and skip flag read from
// device memory, bf16 shadow weights written in the same pass), squared-norm reduction, scaled
// casts, and the two elementwise steps of the Newton-Schulz iteration.
#include "ptx_sm100.cuh"
#include "tensormap.h"
#include "fmb_api.h"

namespace fmb {

__global__ void __launch_bounds__(256)
adamw_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                  __nv_bfloat16* __restrict__ shadow, long long n, float lr, float beta1, float beta2, float eps,
                  float wd, float bc1, float bc2, const float* __restrict__ ctl) {
  const float clip = ctl != nullptr ? ctl[0] : 1.f;
  const bool ok = ctl == nullptr || ctl[1] > 0.5f;
  if (!ok) return;
  const float step = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - lr * wd;
  const long long nvec = n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    const float4 gv = reinterpret_cast<const float4*>(g)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float pe[4] = {pv.x, pv.y, pv.z, pv.w};
    const float ge[4] = {gv.x * clip, gv.y * clip, gv.z * clip, gv.w * clip};
    float me[4] = {mv.x, mv.y, mv.z, mv.w};
    float ve[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      me[j] = me[j] + (ge[j] - me[j]) * (1.f - beta1);
      ve[j] = ve[j] * beta2 + ge[j] * ge[j] * (1.f - beta2);
      const float denom = sqrtf(ve[j]) * inv_sqrt_bc2 + eps;
      pe[j] = pe[j] * decay - step * me[j] / denom;
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(pe[0], pe[1], pe[2], pe[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(me[0], me[1], me[2], me[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(ve[0], ve[1], ve[2], ve[3]);
    if (shadow != nullptr) {
      uint2 o;
      o.x = pack_bf16(pe[0], pe[1]);
      o.y = pack_bf16(pe[2], pe[3]);
      reinterpret_cast<uint2*>(shadow)[i] = o;
    }
  }
  // tail (n not a multiple of 4)
  const long long tail0 = nvec << 2;
  for (long long i = tail0 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float ge = g[i] * clip;
    const float me = m[i] + (ge - m[i]) * (1.f - beta1);
    const float ve = v[i] * beta2 + ge * ge * (1.f - beta2);
    const float pe = p[i] * decay - step * me / (sqrtf(ve) * inv_sqrt_bc2 + eps);
    p[i] = pe; m[i] = me; v[i] = ve;
    if (shadow != nullptr) shadow[i] = __float2bfloat16(pe);
  }
}

constexpr int SQ_BLOCKS_MAX = 1024;

__global__ void __launch_bounds__(256) sqnorm_stage1(const float* __restrict__ x, float* __restrict__ partial, long long n) {
  __shared__ float scratch[8];
  float s = 0.f;
  const long long nvec = n >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const float4 a = reinterpret_cast<const float4*>(x)[i];
    s += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  for (long long i = (nvec << 2) + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    s += x[i] * x[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += scratch[i];
    partial[blockIdx.x] = t;
  }
}

__global__ void __launch_bounds__(1024) sqnorm_stage2(const float* __restrict__ partial, float* __restrict__ out, int nparts,
                                                      int accumulate) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 32; ++i) t += scratch[i];
    out[0] = accumulate ? out[0] + t : t;
  }
}

template <typename S, typename D>
__global__ void scale_cast_kernel(const S* __restrict__ src, D* __restrict__ dst, long long n, float scale) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = static_cast<D>(static_cast<float>(src[i]) * scale);
}

template <typename T>
__global__ void axpby_kernel(const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ out, long long n, float a,
                             float b) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = static_cast<T>(a * static_cast<float>(x[i]) + b * static_cast<float>(y[i]));
}

static int flat_grid(long long n, int per_thread) {
  long long b = (n / per_thread + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace fmb

using namespace fmb;

extern "C" int fmb_adamw_flat(float* p, const float* g, float* m, float* v, void* shadow, long long n, float lr,
                              float beta1, float beta2, float eps, float wd, float bc1, float bc2, const float* ctl,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return -2;
  if (shadow != nullptr && (reinterpret_cast<uintptr_t>(shadow) & 7)) return -2;
  adamw_flat_kernel<<<flat_grid(n, 4), 256, 0, stream>>>(p, g, m, v, static_cast<__nv_bfloat16*>(shadow), n, lr, beta1,
                                                         beta2, eps, wd, bc1, bc2, ctl);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// `partial` must hold at least 1024 floats.
extern "C" int fmb_sqnorm_f32_scratch(const float* x, float* partial, float* out, long long n, int accumulate,
                                      cudaStream_t stream) {
  if (reinterpret_cast<uintptr_t>(x) & 15) return -2;
  int blocks = flat_grid(n, 4);
  if (blocks > SQ_BLOCKS_MAX) blocks = SQ_BLOCKS_MAX;
  sqnorm_stage1<<<blocks, 256, 0, stream>>>(x, partial, n);
  sqnorm_stage2<<<1, 1024, 0, stream>>>(partial, out, blocks, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_scale_cast(const void* src, void* dst, long long n, float scale, int src_dtype, int dst_dtype,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  const int grid = flat_grid(n, 1);
  if (src_dtype == FMB_F32 && dst_dtype == FMB_BF16)
    scale_cast_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), n, scale);
  else if (src_dtype == FMB_BF16 && dst_dtype == FMB_F32)
    scale_cast_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), static_cast<float*>(dst), n, scale);
  else if (src_dtype == FMB_F32 && dst_dtype == FMB_F32)
    scale_cast_kernel<float, float><<<grid, 256, 0, stream>>>(static_cast<const float*>(src), static_cast<float*>(dst), n, scale);
  else if (src_dtype == FMB_BF16 && dst_dtype == FMB_BF16)
    scale_cast_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), n, scale);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int fmb_ns_axpby(const void* x, const void* y, void* out, long long n, float a, float b, int dtype,
                            cudaStream_t stream) {
  if (n <= 0) return 0;
  const int grid = flat_grid(n, 1);
  if (dtype == FMB_BF16)
    axpby_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(out), n, a, b);
  else if (dtype == FMB_F32)
    axpby_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<const float*>(y), static_cast<float*>(out), n, a, b);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
