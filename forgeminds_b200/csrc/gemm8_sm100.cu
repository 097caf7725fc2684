// 8-bit GEMMs for sm_100a: D[M,N] = scale_a * scale_b * sum_k A(m,k) * B(n,k), A and B K-major,
// int8 (tcgen05 kind::i8, int32 accumulation) or fp8 e4m3 (kind::f8f6f4, fp32 accumulation).
//
// Same machine as the bf16 kernel (gemm_sm100.cu): one persistent CTA per SM; warp 0 feeds a ring of
// 128B-swizzled shared-memory stages with TMA, warp 1 issues tcgen05.mma into TMEM, warps 2-5 drain
// TMEM. A stage holds 128 rows of A and BN rows of B, 128 bytes (= 128 elements of K) each: four MMAs of
// K = 32. At the 8-bit rate a 128 x 128 tile needs 32 KB of operands per 256 tensor cycles, which is all
// that shared memory delivers (128 B / clock); products with row scales therefore use 128 x 256 tiles
// (48 KB per 512 cycles) whenever the output is at least 256 columns wide.
//
// Two scaling schemes:
//   row scales      one fp32 scale per row of A and per row of B (per token / per output channel).
//                   The scales factor out of the sum, so the product accumulates in TMEM over all of
//                   K and is scaled once in the epilogue.
//   block scales    fp8 only: A has a scale per row and 128-wide K block, B a scale per 128 x 128
//                   block. They do not factor out, so every K block is multiplied into its own TMEM
//                   buffer (two alternate), and the epilogue warps add it, scaled, into fp32 registers
//                   while the tensor core works on the next block.
//
// The reference reaches these products through torchao / Transformer Engine when they are installed
// (forgemind/quant.py:93-154).
#include <cuda_fp8.h>

#include "ptx_sm100.cuh"
#include "launch.cuh"
#include "tensormap.h"
#include "fmb_api.h"

namespace fmb {

constexpr int G8_BM = 128, G8_BK = 128, G8_THREADS = 192;

struct G8Params {
  int M, N;
  int tiles_m, tiles_n, kblocks;
  void* D;
  long long ldd;
  int d_f32;
  const float* sa;      // row scales [M] or block scales [M, sa_ld]
  const float* sb;      // row scales [N] or block scales [ceil(N/128), sb_ld]
  int sa_ld, sb_ld;
  int* status;
};

template <int BN>
struct G8Smem {
  static constexpr int STAGES = BN == 128 ? 6 : 4;
  static constexpr uint32_t A_BYTES = G8_BM * G8_BK;
  static constexpr uint32_t B_BYTES = BN * G8_BK;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr uint32_t TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;
};

// KIND: 0 = int8, 1 = fp8 e4m3.  BLOCKED: per-K-block scales (fp8 only, BN = 128).  BN: 128 or 256 output columns.
template <int KIND, bool BLOCKED, int BN>
__global__ void __launch_bounds__(G8_THREADS, 1)
gemm8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, G8Params p) {
  using L = G8Smem<BN>;
  static_assert(!BLOCKED || BN == 128, "the block-scaled epilogue keeps a 128-column tile in registers");
  constexpr int BM = G8_BM, BK = G8_BK, STAGES = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::BAR_OFFSET + (2 * STAGES + 4) * 8);
  AbortState* ab = reinterpret_cast<AbortState*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(tfull_bar(s), 1); mbar_init(tempty_bar(s), 4); }
    ab->flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc<2 * BN>(smem_u32(tmem_slot)); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  const int total_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (elect_one()) {
      uint32_t stage = 0, phase = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int m_blk = tile % p.tiles_m, n_blk = tile / p.tiles_m;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, ab, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + stage * L::STAGE_BYTES, sB = sA + L::A_BYTES;
          mbar_expect_tx(full_bar(stage), L::STAGE_BYTES);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          tma_load_2d(sA, &tmA, full_bar(stage), kb * BK, m_blk * BM);
          tma_load_2d(sB, &tmB, full_bar(stage), kb * BK, n_blk * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok || ab->flag) {
        for (int s = 0; s < STAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          const uint32_t par = (armed_parity >> s) & 1u;
          for (int it = 0; it < 200000 && !mbar_try_wait(full_bar(s), par); ++it) {}
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = KIND == 0 ? umma_idesc(BM, BN, 1, 1, 2, false, false)
                                           : umma_idesc(BM, BN, 0, 0, 1, false, false);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        if constexpr (!BLOCKED) {
          if (!mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, ab, p.status, ERR_WAIT_TMEM_EMPTY)) break;
          tc_fence_after();
        }
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if constexpr (BLOCKED) {
            if (!mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, ab, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
            tc_fence_after();
          }
          if (!mbar_wait_bounded(full_bar(stage), phase, ab, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * L::STAGE_BYTES, sB = sA + L::A_BYTES;
          const uint32_t d_tmem = tmem_base + acc * BN;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            const uint64_t da = umma_smem_desc_sw128(sA + k * 32u, 16u, 1024u);
            const uint64_t db = umma_smem_desc_sw128(sB + k * 32u, 16u, 1024u);
            const uint32_t accumulate = BLOCKED ? (k > 0 ? 1u : 0u) : ((kb > 0 || k > 0) ? 1u : 0u);
            if constexpr (KIND == 0) umma_i8_ss(d_tmem, da, db, idesc, accumulate);
            else                     umma_f8_ss(d_tmem, da, db, idesc, accumulate);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if constexpr (BLOCKED) {
            umma_commit(tfull_bar(acc));
            acc ^= 1u;
            if (acc == 0) acc_phase ^= 1u;
          }
        }
        if (!ok) break;
        if constexpr (!BLOCKED) {
          umma_commit(tfull_bar(acc));
          acc ^= 1u;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    const long long d_es = p.d_f32 ? 4 : 2;
    const bool wide_d = (reinterpret_cast<uintptr_t>(p.D) & 31) == 0 && (p.ldd * d_es) % 32 == 0;   // 32-byte stores stay aligned
    // 32 finished output values of one row, columns [col0, col0 + 32)
    auto store32 = [&](int row, int col0, const float (&v)[32]) {
      if (col0 >= p.N) return;
      const bool full = col0 + 32 <= p.N;
      if (p.d_f32) {
        float* dp = reinterpret_cast<float*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
        if (full && wide_d) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            st_global_v8(dp + 8 * i, __float_as_uint(v[8 * i]), __float_as_uint(v[8 * i + 1]), __float_as_uint(v[8 * i + 2]),
                         __float_as_uint(v[8 * i + 3]), __float_as_uint(v[8 * i + 4]), __float_as_uint(v[8 * i + 5]),
                         __float_as_uint(v[8 * i + 6]), __float_as_uint(v[8 * i + 7]));
        } else if (full) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            reinterpret_cast<float4*>(dp)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) if (col0 + i < p.N) dp[i] = v[i];
        }
      } else {
        __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
        if (full && wide_d) {                     // one 32-byte sector per store
#pragma unroll
          for (int i = 0; i < 2; ++i)
            st_global_v8(dp + 16 * i, pack_bf16(v[16 * i + 0], v[16 * i + 1]), pack_bf16(v[16 * i + 2], v[16 * i + 3]),
                         pack_bf16(v[16 * i + 4], v[16 * i + 5]), pack_bf16(v[16 * i + 6], v[16 * i + 7]),
                         pack_bf16(v[16 * i + 8], v[16 * i + 9]), pack_bf16(v[16 * i + 10], v[16 * i + 11]),
                         pack_bf16(v[16 * i + 12], v[16 * i + 13]), pack_bf16(v[16 * i + 14], v[16 * i + 15]));
        } else if (full) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            o.x = pack_bf16(v[8 * i + 0], v[8 * i + 1]);
            o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
            o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]);
            o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
            reinterpret_cast<uint4*>(dp)[i] = o;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) if (col0 + i < p.N) dp[i] = __float2bfloat16(v[i]);
        }
      }
    };
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int m_blk = tile % p.tiles_m, n_blk = tile / p.tiles_m;
      const int row = m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      if constexpr (BLOCKED) {
        float out[BN / 32][32];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) out[c][i] = 0.f;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_bounded(tfull_bar(acc), acc_phase, ab, p.status, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
          tc_fence_after();
          const float s = (row_ok ? __ldg(p.sa + static_cast<long long>(row) * p.sa_ld + kb) : 0.f) *
                          __ldg(p.sb + static_cast<long long>(n_blk) * p.sb_ld + kb);
          const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_row + c * 32, r);
            tmem_ld_fence(r);
#pragma unroll
            for (int i = 0; i < 32; ++i) out[c][i] += __uint_as_float(r[i]) * s;
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(acc));
          acc ^= 1u;
          if (acc == 0) acc_phase ^= 1u;
        }
        if (!ok) break;
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) store32(row, n_blk * BN + c * 32, out[c]);
        }
      } else {
        if (!mbar_wait_bounded(tfull_bar(acc), acc_phase, ab, p.status, ERR_WAIT_TMEM_FULL)) break;
        tc_fence_after();
        const float sa = row_ok ? __ldg(p.sa + row) : 0.f;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
        const int cols_left = p.N - n_blk * BN;
        const int n_chunks = cols_left >= BN ? BN / 32 : (cols_left + 31) / 32;
        auto finish_chunk = [&](int c, const uint32_t (&r)[32]) {
          if (!row_ok) return;
          const int col0 = n_blk * BN + c * 32;
          float v[32];
          if (col0 + 32 <= p.N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 sb = __ldg(reinterpret_cast<const float4*>(p.sb + col0) + i);
              const float sc[4] = {sb.x, sb.y, sb.z, sb.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint32_t w = r[4 * i + q];
                const float x = KIND == 0 ? static_cast<float>(static_cast<int>(w)) : __uint_as_float(w);
                v[4 * i + q] = x * sa * sc[q];
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float x = KIND == 0 ? static_cast<float>(static_cast<int>(r[i])) : __uint_as_float(r[i]);
              v[i] = x * sa * (col0 + i < p.N ? __ldg(p.sb + col0 + i) : 0.f);
            }
          }
          store32(row, col0, v);
        };
        // TMEM reads run one chunk ahead of the stores; the accumulator goes back to the MMA warp as soon
        // as its last chunk is in registers.
        auto release_acc = [&]() {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_relaxed(tempty_bar(acc));
        };
        uint32_t ra[32], rb[32];
        if (n_chunks > 0) tmem_ld_32x32(t_row, ra);
#pragma unroll 1
        for (int c = 0; c < n_chunks; c += 2) {
          tmem_ld_fence(ra);
          if (c + 1 < n_chunks) tmem_ld_32x32(t_row + (c + 1) * 32, rb);
          else release_acc();
          finish_chunk(c, ra);
          if (c + 1 < n_chunks) {
            tmem_ld_fence(rb);
            if (c + 2 < n_chunks) tmem_ld_32x32(t_row + (c + 2) * 32, ra);
            else release_acc();
            finish_chunk(c + 1, rb);
          }
        }
        if (n_chunks <= 0) release_acc();
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2 * BN>(tmem_base);
  }
}

// ------------------------------------------------------------------ quantisers
// One warp per row: q[r, c] = round(x[r, c] / scale[r]) with scale = amax(row) / 127 (int8) or
// amax / 448 (e4m3). With `block` > 0 (fp8) there is one scale per row and `block`-wide column group.
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

template <typename T, int KIND>
__global__ void __launch_bounds__(256)
quant_rows_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, long long rows, int cols,
                  long long ldx, int block, int n_blocks) {
  pdl_wait();
  pdl_launch_dependents();
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + row * ldx;
  uint8_t* qr = q + row * cols;
  constexpr float QMAX = KIND == 0 ? 127.f : 448.f;
  const int groups = block > 0 ? n_blocks : 1;
  const int width = block > 0 ? block : cols;
  for (int g = 0; g < groups; ++g) {
    const int c0 = g * width, c1 = min(cols, c0 + width);
    float amax = 0.f;
    for (int c = c0 + lane; c < c1; c += 32) amax = fmaxf(amax, fabsf(static_cast<float>(xr[c])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = fmaxf(amax, 1e-12f) / QMAX;
    const float inv = 1.f / s;
    if (lane == 0) scale[row * groups + g] = s;
    for (int c = c0 + lane; c < c1; c += 32) {
      const float v = static_cast<float>(xr[c]) * inv;
      if constexpr (KIND == 0) qr[c] = static_cast<uint8_t>(static_cast<int8_t>(fminf(fmaxf(rintf(v), -127.f), 127.f)));
      else qr[c] = to_e4m3(v);
    }
  }
}

// fp8 weights with one scale per 128 x 128 block: one CTA per block.
template <typename T>
__global__ void __launch_bounds__(256)
quant_tiles_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, int rows, int cols,
                   long long ldx, int n_col_blocks) {
  __shared__ float red[8];
  pdl_wait();
  pdl_launch_dependents();
  const int br = blockIdx.y, bc = blockIdx.x;
  const int r0 = br * 128, c0 = bc * 128;
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = r0 + i / 128, c = c0 + i % 128;
    if (r < rows && c < cols) amax = fmaxf(amax, fabsf(static_cast<float>(x[static_cast<long long>(r) * ldx + c])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int w = 0; w < 8; ++w) amax = fmaxf(amax, red[w]);
  const float s = fmaxf(amax, 1e-12f) / 448.f;
  const float inv = 1.f / s;
  if (threadIdx.x == 0) scale[br * n_col_blocks + bc] = s;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = r0 + i / 128, c = c0 + i % 128;
    if (r < rows && c < cols)
      q[static_cast<long long>(r) * cols + c] = to_e4m3(static_cast<float>(x[static_cast<long long>(r) * ldx + c]) * inv);
  }
}

}  // namespace fmb

using namespace fmb;

template <int KIND, bool BLOCKED, int BN>
static int launch_gemm8(const CUtensorMap& ta, const CUtensorMap& tb, const G8Params& p, int grid, cudaStream_t stream) {
  auto kern = gemm8_kernel<KIND, BLOCKED, BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G8Smem<BN>::TOTAL) != cudaSuccess) return -6;
    attr_set = true;
  }
  return launch_pdl(kern, dim3(grid), dim3(G8_THREADS), G8Smem<BN>::TOTAL, stream, ta, tb, p) == cudaSuccess ? 0 : -3;
}

// kind: 0 int8, 1 fp8 e4m3. A [M, K] and B [N, K] are 1-byte, K-major with pitches lda / ldb (bytes = elements,
// multiples of 16). sa_ld == 0 selects row scales (sa[M], sb[N]); otherwise block scales (fp8): sa[M, sa_ld],
// sb[ceil(N / 128), sb_ld] with one column per 128 elements of K.
extern "C" int fmb_gemm8(const void* A, const void* B, void* D, int M, int N, int K, long long lda, long long ldb,
                         long long ldd, int d_f32, int kind, const float* sa, const float* sb, int sa_ld, int sb_ld,
                         int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 16) || (ldb % 16) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(D) & 15) || (ldd % (d_f32 ? 4 : 8)) || sa == nullptr || sb == nullptr)
    return -2;
  if (kind != 0 && kind != 1) return -1;
  const bool blocked = sa_ld > 0;
  if (blocked && kind != 1) return -1;
  G8Params p;
  p.M = M; p.N = N;
  p.tiles_m = (M + G8_BM - 1) / G8_BM;
  p.kblocks = (K + G8_BK - 1) / G8_BK;
  // wide tiles for row-scaled products unless they would leave most of the machine idle or mostly padded
  const int sms = sm_count();
  int bn = 128;
  if (!blocked && N >= 256) {
    const long long wide_tiles = static_cast<long long>(p.tiles_m) * ((N + 255) / 256);
    const double pad = static_cast<double>(N) / (((N + 255) / 256) * 256.0);
    if (wide_tiles >= sms / 2 && pad >= 0.8) bn = 256;
  }
  static const bool wide_env = [] { const char* v = getenv("FMB_GEMM8_WIDE"); return v == nullptr || v[0] != '0'; }();
  if (!wide_env) bn = 128;
  p.tiles_n = (N + bn - 1) / bn;
  if (blocked && (sa_ld < p.kblocks || sb_ld < p.kblocks)) return -2;
  p.D = D; p.ldd = ldd; p.d_f32 = d_f32;
  p.sa = sa; p.sb = sb; p.sa_ld = sa_ld; p.sb_ld = sb_ld;
  p.status = status;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, A, M, K, lda, G8_BM, G8_BK, 1, TmapSwizzle::B128) ||
      !make_tmap_2d(&tb, B, N, K, ldb, static_cast<uint32_t>(bn), G8_BK, 1, TmapSwizzle::B128))
    return -5;
  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n;
  const int grid = static_cast<int>(total < sms ? total : sms);
  if (blocked) return launch_gemm8<1, true, 128>(ta, tb, p, grid, stream);
  if (bn == 256) return kind == 0 ? launch_gemm8<0, false, 256>(ta, tb, p, grid, stream)
                                  : launch_gemm8<1, false, 256>(ta, tb, p, grid, stream);
  return kind == 0 ? launch_gemm8<0, false, 128>(ta, tb, p, grid, stream)
                   : launch_gemm8<1, false, 128>(ta, tb, p, grid, stream);
}

// Row quantiser. x: bf16 (dtype 0) or fp32 (1), [rows, cols] with pitch ldx. block > 0: fp8 scales per row and
// `block` columns, scale shape [rows, ceil(cols / block)]; block == 0: one scale per row.
// The same quantiser for rows whose width and pitch are multiples of 8 elements: every lane works on 8
// consecutive elements (16-byte loads of bf16, 8-byte stores). Without blocks a warp makes two passes
// over its row (maximum, then quantise); with 128-wide blocks a half warp owns one block and quantises
// it from registers.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16(w[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  } else {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}
template <int KIND>
__device__ __forceinline__ uint2 quant8(const float (&v)[8], float inv) {
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float x = v[i] * inv;
    uint32_t b;
    if constexpr (KIND == 0) b = static_cast<uint32_t>(static_cast<uint8_t>(static_cast<int8_t>(fminf(fmaxf(rintf(x), -127.f), 127.f))));
    else b = to_e4m3(x);
    w[i >> 2] |= b << (8 * (i & 3));
  }
  return make_uint2(w[0], w[1]);
}

template <typename T, int KIND>
__global__ void __launch_bounds__(256)
quant_rows_vec_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, long long rows, int cols,
                      long long ldx, int block, int n_blocks) {
  pdl_wait();
  pdl_launch_dependents();
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* xr = x + row * ldx;
  uint8_t* qr = q + row * cols;
  constexpr float QMAX = KIND == 0 ? 127.f : 448.f;
  if (block == 0) {
    float amax = 0.f;
    for (int c = lane * 8; c < cols; c += 256) {
      float v[8];
      load8(xr + c, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = fmaxf(amax, 1e-12f) / QMAX;
    const float inv = 1.f / s;
    if (lane == 0) scale[row] = s;
    for (int c = lane * 8; c < cols; c += 256) {
      float v[8];
      load8(xr + c, v);
      *reinterpret_cast<uint2*>(qr + c) = quant8<KIND>(v, inv);
    }
  } else {                                    // block == 128: 16 lanes x 8 elements
    const int half = lane >> 4, sub = lane & 15;
    for (int g0 = 0; g0 < n_blocks; g0 += 2) {
      const int g = g0 + half, c = g * 128 + sub * 8;
      const bool live = g < n_blocks && c < cols;
      float v[8];
      if (live) load8(xr + c, v);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float s = fmaxf(amax, 1e-12f) / QMAX;
      if (g < n_blocks && sub == 0) scale[row * n_blocks + g] = s;
      if (live) *reinterpret_cast<uint2*>(qr + c) = quant8<KIND>(v, 1.f / s);
    }
  }
}

extern "C" int fmb_quant_rows(const void* x, void* q, float* scale, long long rows, int cols, long long ldx, int dtype,
                              int kind, int block, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (block > 0 && kind != 1) return -1;
  const int n_blocks = block > 0 ? (cols + block - 1) / block : 1;
  const unsigned grid = static_cast<unsigned>((rows * 32 + 255) / 256);
  cudaError_t e;
  const bool vec = cols % 8 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(q) & 7) == 0 && (block == 0 || block == 128);
#define FMB_QR(T, KIND)                                                                                     \
  e = vec ? launch_pdl(quant_rows_vec_kernel<T, KIND>, dim3(grid), dim3(256), 0, stream, static_cast<const T*>(x), \
                       static_cast<uint8_t*>(q), scale, rows, cols, ldx, block, n_blocks)                    \
          : launch_pdl(quant_rows_kernel<T, KIND>, dim3(grid), dim3(256), 0, stream, static_cast<const T*>(x), \
                       static_cast<uint8_t*>(q), scale, rows, cols, ldx, block, n_blocks)
  if (dtype == FMB_BF16 && kind == 0) FMB_QR(__nv_bfloat16, 0);
  else if (dtype == FMB_BF16 && kind == 1) FMB_QR(__nv_bfloat16, 1);
  else if (dtype == FMB_F32 && kind == 0) FMB_QR(float, 0);
  else if (dtype == FMB_F32 && kind == 1) FMB_QR(float, 1);
  else return -1;
#undef FMB_QR
  return e == cudaSuccess ? 0 : -3;
}

// fp8 quantiser with one scale per 128 x 128 block; scale shape [ceil(rows/128), ceil(cols/128)].
extern "C" int fmb_quant_tiles_fp8(const void* x, void* q, float* scale, int rows, int cols, long long ldx, int dtype,
                                   cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const dim3 grid((cols + 127) / 128, (rows + 127) / 128);
  cudaError_t e;
  if (dtype == FMB_BF16)
    e = launch_pdl(quant_tiles_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x),
                   static_cast<uint8_t*>(q), scale, rows, cols, ldx, static_cast<int>(grid.x));
  else if (dtype == FMB_F32)
    e = launch_pdl(quant_tiles_kernel<float>, grid, dim3(256), 0, stream, static_cast<const float*>(x),
                   static_cast<uint8_t*>(q), scale, rows, cols, ldx, static_cast<int>(grid.x));
  else return -1;
  return e == cudaSuccess ? 0 : -3;
}
