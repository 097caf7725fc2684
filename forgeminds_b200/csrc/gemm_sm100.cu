// bf16 GEMM for sm_100a: D[M,N] = alpha * sum_k A(m,k) * B(n,k) + beta * C[M,N].
//
// One persistent CTA per SM, six warps with fixed roles:
//   warp 0    one elected thread issues TMA tile loads into a ring of 128B-swizzled smem stages;
//   warp 1    owns TMEM (two fp32 accumulators) and one elected thread issues tcgen05.mma;
//   warps 2-5 read the finished accumulator back with tcgen05.ld (one TMEM lane quarter each),
//             apply the epilogue and store, while the MMA warp already works on the other
//             accumulator.
// Operands may be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]); this covers
// the forward (K,K), input-gradient (K,MN) and weight-gradient (MN,MN) products of a linear layer
// without a transpose pass. Split-K (fp32 atomic accumulation) fills the machine when the output
// has fewer tiles than SMs, which is the usual case for weight gradients.
#include "ptx_sm100.cuh"
#include "tensormap.h"
#include "fmb_api.h"

namespace fmb {

constexpr int GEMM_BK_C = 64;

struct GemmParams {
  int M, N;
  int tiles_m, tiles_n, splits;
  int kblocks_total, kblocks_per_split;
  void* D;
  long long ldd;
  const void* C;
  long long ldc;
  int d_f32, c_f32, atomic;
  float alpha, beta;
  const float* alpha_ptr;   // optional device scalar multiplied into alpha
  int* status;
  // grouped modes (0 = plain)
  //   1: rows of A/D are partitioned into groups; `tile_group[m_blk]` names the B matrix (z coordinate of
  //      the 3-D B map) used by that row tile, or -1 for a tile that holds only padding (skipped).
  //   2: one output matrix per group, reduced over that group's rows: `region[3g] = {first row, used,
  //      padded rows}` gives the K range, `group_stride_d` the distance between output matrices.
  int mode;
  int n_groups;
  const int* tile_group;
  const int* region;
  long long group_stride_d;
};

struct TileInfo {
  int m_blk, n_blk, k0, k1, zb;
  long long d_off;
  bool valid;
};

__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, int tile) {
  TileInfo t;
  t.zb = 0;
  t.d_off = 0;
  t.valid = true;
  if (p.mode == 2) {
    const int per = p.tiles_m * p.tiles_n;
    const int g = tile / per, mn = tile % per;
    t.m_blk = mn % p.tiles_m;
    t.n_blk = mn / p.tiles_m;
    t.k0 = __ldg(p.region + 3 * g) / GEMM_BK_C;
    t.k1 = t.k0 + __ldg(p.region + 3 * g + 2) / GEMM_BK_C;
    t.d_off = static_cast<long long>(g) * p.group_stride_d;
    t.valid = t.k1 > t.k0;
    return t;
  }
  const int ks = tile % p.splits;
  const int mn = tile / p.splits;
  t.m_blk = mn % p.tiles_m;
  t.n_blk = mn / p.tiles_m;
  t.k0 = ks * p.kblocks_per_split;
  t.k1 = min(p.kblocks_total, t.k0 + p.kblocks_per_split);
  if (p.mode == 1) {
    t.zb = __ldg(p.tile_group + t.m_blk);
    t.valid = t.zb >= 0;
  }
  return t;
}

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr uint32_t A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr uint32_t B_BYTES = BN * GEMM_BK * 2;
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr uint32_t TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;  // + alignment slack
};

__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  using L = GemmSmem<BN, STAGES>;
  constexpr int BM = GEMM_BM, BK = GEMM_BK;
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

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 4);
    }
    ab->flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<2 * BN>(smem_u32(tmem_slot));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.tiles_m * p.tiles_n * (p.mode == 2 ? p.n_groups : p.splits);

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      uint32_t armed = 0, armed_parity = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileInfo ti = decode_tile(p, tile);
        if (!ti.valid) continue;
        const int m_blk = ti.m_blk, n_blk = ti.n_blk, k0 = ti.k0, k1 = ti.k1;
        for (int kb = k0; kb < k1; ++kb) {
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, ab, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sB = sA + L::A_BYTES;
          mbar_expect_tx(full_bar(stage), L::STAGE_BYTES);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          if constexpr (!A_MN) {
            tma_load_2d(sA, &tmA, full_bar(stage), kb * BK, m_blk * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sA + j * (BK * 128), &tmA, full_bar(stage), m_blk * BM + j * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_3d(sB, &tmB, full_bar(stage), kb * BK, n_blk * BN, ti.zb);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sB + j * (BK * 128), &tmB, full_bar(stage), n_blk * BN + j * 64, kb * BK, ti.zb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok || ab->flag) {
        // Leave no bulk copy in flight towards this CTA's shared memory before it exits.
        for (int s = 0; s < STAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          const uint32_t par = (armed_parity >> s) & 1u;
          for (int it = 0; it < 200000 && !mbar_try_wait(full_bar(s), par); ++it) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1, 1, A_MN, B_MN);
      constexpr uint32_t A_KSTEP = A_MN ? 16u * 128u : 32u;   // bytes per 16-wide K slice
      constexpr uint32_t B_KSTEP = B_MN ? 16u * 128u : 32u;
      constexpr uint32_t MN_LBO = BK * 128u;                  // next 64-wide block of an MN-major tile
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileInfo ti = decode_tile(p, tile);
        if (!ti.valid) continue;
        const int k0 = ti.k0, k1 = ti.k1;
        if (!mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, ab, p.status, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = k0; kb < k1; ++kb) {
          if (!mbar_wait_bounded(full_bar(stage), phase, ab, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sB = sA + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = umma_smem_desc_sw128(sA + k * A_KSTEP, A_MN ? MN_LBO : 16u, 1024u);
            const uint64_t db = umma_smem_desc_sw128(sB + k * B_KSTEP, B_MN ? MN_LBO : 16u, 1024u);
            umma_f16_ss(d_tmem, da, db, idesc, (kb > k0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;                 // TMEM lanes [32*quarter, 32*quarter + 32)
    uint32_t acc = 0, acc_phase = 0;
    const float alpha = p.alpha_ptr != nullptr ? p.alpha * __ldg(p.alpha_ptr) : p.alpha;
    const float beta = p.beta;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const TileInfo ti = decode_tile(p, tile);
      if (!ti.valid) continue;
      const int m_blk = ti.m_blk, n_blk = ti.n_blk;
      if (!mbar_wait_bounded(tfull_bar(acc), acc_phase, ab, p.status, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n_blk * BN + c * 32;
        if (col0 >= p.N) break;                   // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_wait_ld();
        if (!row_ok) continue;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
        const bool full = col0 + 32 <= p.N;
        if (p.C != nullptr && beta != 0.f) {
          if (p.c_f32) {
            const float* cp = reinterpret_cast<const float*>(p.C) + ti.d_off + static_cast<long long>(row) * p.ldc + col0;
            if (full) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float4 cv = reinterpret_cast<const float4*>(cp)[i];
                v[4 * i + 0] += beta * cv.x; v[4 * i + 1] += beta * cv.y;
                v[4 * i + 2] += beta * cv.z; v[4 * i + 3] += beta * cv.w;
              }
            } else {
              _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col0 + i < p.N) v[i] += beta * cp[i];
            }
          } else {
            const __nv_bfloat16* cp =
                reinterpret_cast<const __nv_bfloat16*>(p.C) + ti.d_off + static_cast<long long>(row) * p.ldc + col0;
            if (full) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 cv = reinterpret_cast<const uint4*>(cp)[i];
                float2 a0 = unpack_bf16(cv.x), a1 = unpack_bf16(cv.y), a2 = unpack_bf16(cv.z), a3 = unpack_bf16(cv.w);
                v[8 * i + 0] += beta * a0.x; v[8 * i + 1] += beta * a0.y;
                v[8 * i + 2] += beta * a1.x; v[8 * i + 3] += beta * a1.y;
                v[8 * i + 4] += beta * a2.x; v[8 * i + 5] += beta * a2.y;
                v[8 * i + 6] += beta * a3.x; v[8 * i + 7] += beta * a3.y;
              }
            } else {
              _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col0 + i < p.N) v[i] += beta * __bfloat162float(cp[i]);
            }
          }
        }
        if (p.d_f32) {
          float* dp = reinterpret_cast<float*>(p.D) + ti.d_off + static_cast<long long>(row) * p.ldd + col0;
          if (p.atomic) {
            if (full) {
#pragma unroll
              for (int i = 0; i < 8; ++i) red_add_f32x4(dp + 4 * i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
              _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col0 + i < p.N) atomicAdd(dp + i, v[i]);
            }
          } else if (full) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(dp)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else {
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col0 + i < p.N) dp[i] = v[i];
          }
        } else {
          __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + ti.d_off + static_cast<long long>(row) * p.ldd + col0;
          if (full) {
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
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col0 + i < p.N) dp[i] = __float2bfloat16(v[i]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2 * BN>(tmem_base);
  }
}

// ------------------------------------------------------------------------------------ host side
template <int BN, int STAGES, bool A_MN, bool B_MN>
static cudaError_t launch_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                              cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  static bool attr_set = false;
  constexpr int smem = GemmSmem<BN, STAGES>::TOTAL;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  kern<<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

static double wave_eff(long long work, int sms) {
  long long waves = (work + sms - 1) / sms;
  return static_cast<double>(work) / static_cast<double>(waves * sms);
}

}  // namespace fmb

namespace fmb {
struct GroupSpec {
  int mode = 0;                  // 0 plain, 1 row groups (B per group), 2 one output per group (K ranges)
  int n_groups = 1;
  const int* tile_group = nullptr;
  const int* region = nullptr;
  long long group_stride_b = 0;  // elements between the B matrices of consecutive groups (mode 1)
  long long group_stride_d = 0;  // elements between the D (and C) matrices of consecutive groups (mode 2)
};
}  // namespace fmb

static int run_gemm(const void* A, const void* B, void* D, const void* C, int M, int N, int K, int a_mn,
                    int b_mn, long long lda, long long ldb, long long ldd, long long ldc, int d_f32,
                    int c_f32, float alpha, float beta, const float* alpha_ptr, int allow_split, int* status,
                    int force_bn, const fmb::GroupSpec& gs, cudaStream_t stream) {
  using namespace fmb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (gs.mode != 0) allow_split = 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(D) & 15) || (ldd % (d_f32 ? 4 : 8)))
    return -2;   // TMA needs 16-byte aligned bases and pitches; the vector epilogue needs an aligned D
  if (C != nullptr && ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc % (c_f32 ? 4 : 8)))) return -2;
  const int sms = sm_count();
  const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int kblocks = (K + GEMM_BK - 1) / GEMM_BK;
  const bool can_split = allow_split && d_f32 && (C == nullptr || C == D);

  // Pick the N tile and the split count that fill the machine best.
  int best_bn = 256, best_split = 1;
  double best_score = -1.0;
  for (int bn : {256, 128}) {
    if (force_bn && bn != force_bn) continue;
    const int tn = (N + bn - 1) / bn;
    const long long tiles = static_cast<long long>(tiles_m) * tn;
    const int max_split = can_split ? 8 : 1;
    for (int s = 1; s <= max_split; ++s) {
      if (s > 1 && (kblocks / s) < 8) break;            // keep each split's K loop long enough
      double score = wave_eff(tiles * s, sms);
      score *= (bn == 256 ? 1.0 : 0.93);                // narrower tiles re-read A more often
      score *= 1.0 - 0.015 * (s - 1);                   // atomics and extra epilogues are not free
      const double pad = static_cast<double>(N) / (static_cast<double>(tn) * bn);
      score *= pad;
      if (score > best_score) { best_score = score; best_bn = bn; best_split = s; }
    }
  }
  int kbps = (kblocks + best_split - 1) / best_split;
  int splits = (kblocks + kbps - 1) / kbps;

  GemmParams p;
  p.M = M; p.N = N;
  p.tiles_m = tiles_m;
  p.tiles_n = (N + best_bn - 1) / best_bn;
  p.splits = splits;
  p.kblocks_total = kblocks;
  p.kblocks_per_split = kbps;
  p.D = D; p.ldd = ldd;
  p.C = C; p.ldc = ldc;
  p.d_f32 = d_f32; p.c_f32 = c_f32;
  p.atomic = splits > 1 ? 1 : 0;
  p.alpha = alpha; p.beta = beta;
  p.alpha_ptr = alpha_ptr;
  p.status = status;
  p.mode = gs.mode;
  p.n_groups = gs.n_groups;
  p.tile_group = gs.tile_group;
  p.region = gs.region;
  p.group_stride_d = gs.group_stride_d;
  if (splits > 1) {
    // Every split adds alpha*partial into D, which already holds the C term (C == D) or zeros.
    if (C == D && beta == 1.f) { p.C = nullptr; }
    else if (C == nullptr) { if (cudaMemsetAsync(D, 0, sizeof(float) * static_cast<size_t>(M) * ldd, stream) != cudaSuccess) return -3; }
    else return -4;
  }

  CUtensorMap ta, tb;
  bool ok = true;
  if (!a_mn) ok = ok && make_tmap_2d(&ta, A, M, K, lda, GEMM_BM, GEMM_BK, 2, TmapSwizzle::B128);
  else       ok = ok && make_tmap_2d(&ta, A, K, M, lda, GEMM_BK, 64, 2, TmapSwizzle::B128);
  {
    // B is always described by a 3-D map (inner, rows, group); plain products have one group.
    const int nb = gs.mode == 1 ? gs.n_groups : 1;
    const uint64_t gstride = gs.mode == 1 ? static_cast<uint64_t>(gs.group_stride_b)
                                          : static_cast<uint64_t>(b_mn ? K : N) * static_cast<uint64_t>(ldb);
    uint64_t dims[3], strides[3];
    uint32_t box[3];
    if (!b_mn) { dims[0] = K; dims[1] = N; box[0] = GEMM_BK; box[1] = best_bn; }
    else       { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = GEMM_BK; }
    dims[2] = nb; box[2] = 1;
    strides[0] = 2; strides[1] = static_cast<uint64_t>(ldb) * 2; strides[2] = gstride * 2;
    ok = ok && make_tmap_nd(&tb, B, 3, dims, strides, box, 2, TmapSwizzle::B128);
  }
  if (!ok) return -5;

  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * (gs.mode == 2 ? gs.n_groups : p.splits);
  const int grid = static_cast<int>(total < sms ? total : sms);
  cudaError_t e;
#define FMB_DISPATCH(BN, ST)                                                                   \
  if (a_mn && b_mn)       e = launch_cfg<BN, ST, true, true>(ta, tb, p, grid, stream);          \
  else if (a_mn)          e = launch_cfg<BN, ST, true, false>(ta, tb, p, grid, stream);         \
  else if (b_mn)          e = launch_cfg<BN, ST, false, true>(ta, tb, p, grid, stream);         \
  else                    e = launch_cfg<BN, ST, false, false>(ta, tb, p, grid, stream);
  if (best_bn == 256) { FMB_DISPATCH(256, 4) } else { FMB_DISPATCH(128, 6) }
#undef FMB_DISPATCH
  return e == cudaSuccess ? 0 : -10 - static_cast<int>(e);
}

extern "C" int fmb_gemm_bf16(const void* A, const void* B, void* D, const void* C, int M, int N, int K, int a_mn,
                             int b_mn, long long lda, long long ldb, long long ldd, long long ldc, int d_f32,
                             int c_f32, float alpha, float beta, const float* alpha_ptr, int allow_split, int* status,
                             int force_bn, cudaStream_t stream) {
  fmb::GroupSpec gs;
  return run_gemm(A, B, D, C, M, N, K, a_mn, b_mn, lda, ldb, ldd, ldc, d_f32, c_f32, alpha, beta, alpha_ptr,
                  allow_split, status, force_bn, gs, stream);
}

// Grouped products over rows that are partitioned into expert regions (see GemmParams::mode).
//   mode 1: D[rows, N] = A[rows, K] * B[g(row)]^T          (M = padded rows; K = reduction)
//   mode 2: D[g][M, N] (+)= A[rows_g, M]^T * B[rows_g, N]    (K = total padded rows; operands MN-major)
extern "C" int fmb_gemm_bf16_grouped(const void* A, const void* B, void* D, const void* C, int M, int N, int K,
                                     int a_mn, int b_mn, long long lda, long long ldb, long long ldd, long long ldc,
                                     int d_f32, int c_f32, float alpha, float beta, int mode, int n_groups,
                                     const int* tile_group, const int* region, long long group_stride_b,
                                     long long group_stride_d, int* status, cudaStream_t stream) {
  fmb::GroupSpec gs;
  gs.mode = mode;
  gs.n_groups = n_groups;
  gs.tile_group = tile_group;
  gs.region = region;
  gs.group_stride_b = group_stride_b;
  gs.group_stride_d = group_stride_d;
  if (mode != 1 && mode != 2) return -2;
  if (mode == 1 && tile_group == nullptr) return -2;
  if (mode == 2 && (region == nullptr || !a_mn || !b_mn)) return -2;
  return run_gemm(A, B, D, C, M, N, K, a_mn, b_mn, lda, ldb, ldd, ldc, d_f32, c_f32, alpha, beta, nullptr, 0,
                  status, 0, gs, stream);
}
