// Causal / full flash attention with grouped-query heads for sm_100a, forward and backward.
//
// Forward: one CTA per (batch, query head, 128-row query tile). Warp 0 streams K/V tiles with TMA,
// warp 1 issues tcgen05.mma (S = Q K^T into TMEM, then O += P V with P as a TMEM operand), eight row
// warps own half a query row per thread: they read S from TMEM, keep the running max / sum, write P
// (bf16) into its own TMEM columns and rescale the O accumulator in TMEM only when the row max moved.
// S and P have separate TMEM columns, so the CTA is software-pipelined: S(j+1) is issued as soon as the
// row warps have read S(j) and runs while they compute the exponentials of tile j; they only wait for
// P(j-1) V(j-1) before they overwrite P or touch O. Two CTAs fit on an SM for head_dim <= 64 (256 TMEM
// columns each), which hides the rest.
//
// Backward: one CTA per (batch, kv head, 128-row kv tile); it walks the query tiles of every query
// head of the group, keeps dK/dV in TMEM for the whole walk and hands each dQ tile to four
// writer warps that add it to an fp32 buffer with TMA reduce-add boxes. P and dS are written once to smem and serve both as
// the K-major operand of dQ = dS K and as the MN-major operand of dV = P^T dO, dK = dS^T Q.
//
// Head dims that are not a multiple of 64 are padded by TMA out-of-bounds fill (zeros).
#include "ptx_sm100.cuh"
#include "launch.cuh"
#include "tensormap.h"
#include "fmb_api.h"
#include <math_constants.h>

namespace fmb {

constexpr int ATT_BM = 128;          // query rows per tile
constexpr int ATT_BN = 128;          // kv rows per tile
constexpr uint32_t PANEL_BYTES = 128 * 128;   // 128 rows x 64 bf16, 128B-swizzled

struct AttnParams {
  int B, T, Hq, Hkv, hd;
  int n_tiles;                 // ceil(T / 128)
  float scale_log2;            // softmax scale * log2(e)
  float scale;
  int causal;
  void* o;
  long long o_stride_t;        // elements between consecutive tokens of o
  float* lse;                  // [B, Hq, T]
  int* status;
};

// Byte offset of the 16-byte chunk `chunk16` (0..15) of row `row` inside a [128 x 128] bf16 tile made
// of two 128B-swizzled panels of 64 columns.
__device__ __forceinline__ uint32_t swz_tile_offset(int row, int chunk16) {
  const int panel = chunk16 >> 3, c = chunk16 & 7;
  return panel * PANEL_BYTES + row * 128 + ((c ^ (row & 7)) << 4);
}

// Named barrier over `nthreads` threads that also ANDs a predicate: every participant gets the same
// answer, so a group of warps can agree to leave a loop together (one of them timing out must not
// strand the others at the next barrier).
__device__ __forceinline__ bool named_bar_and(int id, int nthreads, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %3, 0;\n\t"
      "bar.red.and.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(out)
      : "r"(id), "r"(nthreads), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return out != 0;
}

constexpr int ATT_ROW_WARPS = 8;      // two warps per TMEM lane quarter: each owns 64 of the 128 columns
constexpr int ATT_FWD_THREADS = 32 * (2 + ATT_ROW_WARPS);
constexpr int ATT_BWD_THREADS = 32 * (2 + ATT_ROW_WARPS + 4);

template <int HD_PAD>
struct FwdSmem {
  static constexpr int PANELS = HD_PAD / 64;
  static constexpr uint32_t TILE = PANELS * PANEL_BYTES;
  static constexpr uint32_t Q_OFF = 0;
  static constexpr uint32_t K_OFF = Q_OFF + TILE;           // two stages
  static constexpr uint32_t V_OFF = K_OFF + 2 * TILE;       // two stages
  static constexpr uint32_t P_OFF = V_OFF + 2 * TILE;
  static constexpr uint32_t BAR_OFF = P_OFF + 2 * PANEL_BYTES;
  static constexpr uint32_t TOTAL = BAR_OFF + 16 * 8 + 16;   // the dynamic segment is 1024-byte aligned
};

template <int HD_PAD>
__global__ void __launch_bounds__(ATT_FWD_THREADS, HD_PAD == 64 ? 2 : 1)   // head dim 64: two CTAs share an SM
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, AttnParams p) {
  using L = FwdSmem<HD_PAD>;
  constexpr int PANELS = L::PANELS;
  // P (bf16, two values per 32-bit column) is handed to the P.V product in TMEM, as its A operand: it
  // never goes through shared memory, whose bandwidth the operand reads of the MMAs already use up.
  constexpr uint32_t TMEM_COLS = HD_PAD == 64 ? 256 : 512;
  constexpr uint32_t S_COL = 0, O_COL = 128, P_COL = O_COL + HD_PAD;
  constexpr int OH = HD_PAD / 2;                 // output columns owned by one half
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + L::BAR_OFF;
  const uint32_t q_full = bars, kv_full0 = bars + 8, kv_empty0 = bars + 24, s_full = bars + 40, p_ready = bars + 48,
                 o_full = bars + 56, s_free = bars + 64, pv_done = bars + 72;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::BAR_OFF + 16 * 8);
  AbortState* ab = reinterpret_cast<AbortState*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles are scheduled first across the whole grid
  const int per_tile = p.Hq * p.B;
  const int q_tile = p.n_tiles - 1 - static_cast<int>(blockIdx.x) / per_tile;
  const int rem = static_cast<int>(blockIdx.x) % per_tile;
  const int h = rem % p.Hq, b = rem / p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int n_kv = p.causal ? q_tile + 1 : p.n_tiles;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
    mbar_init(s_full, 1);
    mbar_init(p_ready, ATT_ROW_WARPS);
    mbar_init(o_full, 1);
    mbar_init(s_free, ATT_ROW_WARPS);
    mbar_init(pv_done, 1);
    ab->flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) { tmem_alloc<TMEM_COLS>(smem_u32(tmem_slot)); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, L::TILE);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn)
        tma_load_4d(sbase + L::Q_OFF + pn * PANEL_BYTES, &tmQ, q_full, pn * 64, h, q_tile * ATT_BM, b);
      uint32_t phase = 0;
      bool ok = true;
      uint32_t armed = 0;
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait_bounded(kv_empty0 + 8 * st, phase ^ 1u, ab, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(kv_full0 + 8 * st, 2 * L::TILE);
        armed |= 1u << st;
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) {
          tma_load_4d(sbase + L::K_OFF + st * L::TILE + pn * PANEL_BYTES, &tmK, kv_full0 + 8 * st, pn * 64, hk, j * ATT_BN, b);
          tma_load_4d(sbase + L::V_OFF + st * L::TILE + pn * PANEL_BYTES, &tmV, kv_full0 + 8 * st, pn * 64, hk, j * ATT_BN, b);
        }
        if (st == 1) phase ^= 1u;
      }
      if (!ok || ab->flag) {   // drain: let every armed barrier see its bytes before the CTA exits
        for (int it = 0; it < 200000 && !mbar_try_wait(q_full, 0); ++it) {}
        for (int s = 0; s < 2; ++s)
          if (armed & (1u << s))
            for (int it = 0; it < 200000 && !(mbar_try_wait(kv_full0 + 8 * s, 0) || mbar_try_wait(kv_full0 + 8 * s, 1)); ++it) {}
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc(128, ATT_BN, 1, 1, 1, false, false);
      constexpr uint32_t idesc_pv = umma_idesc(128, HD_PAD, 1, 1, 1, false, true);
      auto issue_s = [&](int st) {
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = umma_smem_desc_sw128(sbase + L::Q_OFF + pn * PANEL_BYTES + k * 32, 16, 1024);
            const uint64_t db = umma_smem_desc_sw128(sbase + L::K_OFF + st * L::TILE + pn * PANEL_BYTES + k * 32, 16, 1024);
            umma_f16_ss(tmem + S_COL, da, db, idesc_s, (pn | k) ? 1u : 0u);
          }
      };
      bool ok = mbar_wait_bounded(q_full, 0, ab, p.status, ERR_WAIT_FULL) &&
                mbar_wait_bounded(kv_full0, 0, ab, p.status, ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        umma_commit(s_full);
      }
      // Software pipeline inside the CTA: the scores of tile j+1 are issued as soon as the row warps have
      // READ the scores of tile j (s_free), i.e. before P(j) exists, so S(j+1) runs on the tensor pipe while
      // the row warps are still busy with the exponentials of tile j, and their work on tile j+1 can start
      // the moment they have handed over P(j). P and the output accumulator are only touched by the row
      // warps again after P(j) V(j) has completed (pv_done).
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j & 1;
        if (j + 1 < n_kv) {
          const int nst = (j + 1) & 1;
          if (!mbar_wait_bounded(s_free, j & 1, ab, p.status, ERR_WAIT_MISC)) break;
          // stage nst holds tile j+1: it is the (j+1)/2-th use of that stage
          if (!mbar_wait_bounded(kv_full0 + 8 * nst, ((j + 1) >> 1) & 1, ab, p.status, ERR_WAIT_FULL)) break;
          tc_fence_after();
          issue_s(nst);
          umma_commit(s_full);
        }
        if (!mbar_wait_bounded(p_ready, j & 1, ab, p.status, ERR_WAIT_MISC)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < ATT_BN / 16; ++kk) {
          const uint64_t db = umma_smem_desc_sw128(sbase + L::V_OFF + st * L::TILE + kk * 2048, PANEL_BYTES, 1024);
          umma_f16_ts(tmem + O_COL, tmem + P_COL + kk * 8, db, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);   // 16 kv = 8 columns
        }
        umma_commit(kv_empty0 + 8 * st);
        umma_commit(pv_done);
        if (j + 1 == n_kv) umma_commit(o_full);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / epilogue warps
    // Row r of the tile is shared by two threads (same TMEM lane, different warps): `half` 0 owns
    // score columns [0,64) and the first half of the output columns, `half` 1 the rest. They
    // exchange the row maximum through the partner's own P row in smem (which only the partner
    // overwrites, after it has read the value), so no extra shared memory is needed.
    const int half = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                 // query row inside the tile
    const int q_idx = q_tile * ATT_BM + row;             // global query position
    const uint32_t t_lane = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    float* const put_slot = reinterpret_cast<float*>(smem + L::P_OFF + (half ^ 1) * PANEL_BYTES + row * 128);
    const float* const get_slot = reinterpret_cast<const float*>(smem + L::P_OFF + half * PANEL_BYTES + row * 128);
    float m_run = -CUDART_INF_F, l_run = 0.f;
    bool alive = true;
    for (int j = 0; j < n_kv; ++j) {
      bool ok = mbar_wait_bounded(s_full, j & 1, ab, p.status, ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      const bool diag = p.causal && j == q_tile;
      const bool ragged = (j + 1) * ATT_BN > p.T;
      // columns [0, limit) of the tile are visible to this row
      int limit = ATT_BN;
      if (diag) limit = row + 1;
      if (ragged) limit = min(limit, p.T - j * ATT_BN);
      const int c_lo = half * 64;                        // first column of this thread
      const bool masked = __any_sync(0xffffffffu, limit < c_lo + 64);
      uint32_t r0[32], r1[32];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(t_lane + S_COL + c_lo, r0);
        tmem_ld_32x32(t_lane + S_COL + c_lo + 32, r1);
        tmem_ld_fence(r0);
        tmem_ld_fence(r1);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);            // the scores are in registers: the next tile's may be written
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) { r0[i] = 0u; r1[i] = 0u; }
      }
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
      if (!masked) {
#pragma unroll
        for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(__uint_as_float(r0[i]), __uint_as_float(r1[i])));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (c_lo + i < limit) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r0[i]));
          if (c_lo + 32 + i < limit) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r1[i]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      *put_slot = mx;
      // only the two warps that share these 32 rows meet here (barrier 1 + quarter, 64 threads)
      if (!named_bar_and(1 + quarter, 64, ok)) { alive = false; break; }
      const float m_new = fmaxf(m_run, fmaxf(mx, *get_slot) * p.scale_log2);
      const float alpha = exp2f(m_run - m_new);          // 0 on the first tile (m_run = -inf)
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      // 32 columns at a time: exponentials, row sum, bf16 pairs (kept in registers until P(j-1) V(j-1) is done)
      uint32_t packed0[16], packed1[16];
      auto p_half = [&](const uint32_t (&r)[32], int c_first, uint32_t (&packed)[16]) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a0 = exp2f(fmaf(__uint_as_float(r[i]), p.scale_log2, -m_new));
          float a1 = exp2f(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -m_new));
          if (masked) {
            if (c_first + i >= limit) a0 = 0.f;
            if (c_first + i + 1 >= limit) a1 = 0.f;
          }
          sum4[(i >> 1) & 3] += a0 + a1;
          packed[i >> 1] = pack_bf16(a0, a1);
        }
      };
      p_half(r0, c_lo, packed0);
      p_half(r1, c_lo + 32, packed1);
      l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      m_run = m_new;
      if (j > 0) {          // P columns and the accumulator belong to the tensor pipe until the previous product is done
        bool done = mbar_wait_bounded(pv_done, (j - 1) & 1, ab, p.status, ERR_WAIT_TMEM_FULL);
        done = __all_sync(0xffffffffu, done);
        if (!done) { alive = false; break; }
        tc_fence_after();
      }
      tmem_st_32x16(t_lane + P_COL + half * 32, packed0);
      tmem_st_32x16(t_lane + P_COL + half * 32 + 16, packed1);
      // rescale this half's output columns only if some row of the warp moved its maximum
      if (j > 0 && !__all_sync(0xffffffffu, alpha == 1.f)) {
#pragma unroll 1
        for (int c = 0; c < OH / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_lane + O_COL + half * OH + c * 32, r);
          tmem_ld_fence(r);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32(t_lane + O_COL + half * OH + c * 32, r);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    if (alive) {
      bool ok = mbar_wait_bounded(o_full, 0, ab, p.status, ERR_WAIT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      *put_slot = l_run;                                  // P is no longer read: the last MMA has completed
      if (named_bar_and(1 + quarter, 64, ok)) {
        tc_fence_after();
        const float l_tot = l_run + *get_slot;
        const float inv_l = 1.f / l_tot;
        const bool live = q_idx < p.T;
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) +
                              (static_cast<long long>(b) * p.T + q_idx) * p.o_stride_t + static_cast<long long>(h) * p.hd;
#pragma unroll 1
        for (int c = 0; c < OH / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_lane + O_COL + half * OH + c * 32, r);
          tmem_ld_fence(r);
          if (!live) continue;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int col = half * OH + c * 32 + q4 * 8;
            if (col < p.hd) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(r[q4 * 8 + 0]) * inv_l, __uint_as_float(r[q4 * 8 + 1]) * inv_l);
              v.y = pack_bf16(__uint_as_float(r[q4 * 8 + 2]) * inv_l, __uint_as_float(r[q4 * 8 + 3]) * inv_l);
              v.z = pack_bf16(__uint_as_float(r[q4 * 8 + 4]) * inv_l, __uint_as_float(r[q4 * 8 + 5]) * inv_l);
              v.w = pack_bf16(__uint_as_float(r[q4 * 8 + 6]) * inv_l, __uint_as_float(r[q4 * 8 + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + col) = v;
            }
          }
        }
        if (live && half == 0)
          p.lse[(static_cast<long long>(b) * p.Hq + h) * p.T + q_idx] = m_run * 0.6931471805599453f + __logf(l_tot);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc<TMEM_COLS>(tmem); }
}

// =====================================================================================  backward
struct AttnBwdParams {
  int B, T, Hq, Hkv, hd;
  int n_tiles;
  float scale_log2, scale;
  int causal;
  const float* lse;            // [B, Hq, T]
  const float* delta;          // [B, Hq, T]
  float* dq_acc;               // [B, T, Hq, hd] fp32
  void* dk;
  void* dv;
  long long dkv_stride_t;
  int* status;
};

template <int HD_PAD>
struct BwdSmem {
  static constexpr int PANELS = HD_PAD / 64;
  static constexpr int STAGES = HD_PAD == 64 ? 2 : 1;
  static constexpr uint32_t TILE = PANELS * PANEL_BYTES;
  static constexpr uint32_t K_OFF = 0;
  static constexpr uint32_t V_OFF = K_OFF + TILE;
  static constexpr uint32_t Q_OFF = V_OFF + TILE;                  // STAGES tiles
  static constexpr uint32_t DO_OFF = Q_OFF + STAGES * TILE;        // STAGES tiles
  static constexpr uint32_t P_OFF = DO_OFF + STAGES * TILE;
  static constexpr uint32_t DS_OFF = P_OFF + 2 * PANEL_BYTES;
  // dQ staging: each of the four writer warps sends 32 x 32 fp32 boxes (4 KB, 128B-swizzled) with TMA reduce-add
  static constexpr int DQ_BUFS = HD_PAD == 64 ? 2 : 1;
  static constexpr uint32_t DQ_STG_OFF = DS_OFF + 2 * PANEL_BYTES;
  static constexpr uint32_t BAR_OFF = DQ_STG_OFF + 4 * DQ_BUFS * 4096;
  static constexpr uint32_t TOTAL = BAR_OFF + 16 * 8 + 16;
};

template <int HD_PAD>
__global__ void __launch_bounds__(ATT_BWD_THREADS)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmDQ, AttnBwdParams p) {
  using L = BwdSmem<HD_PAD>;
  constexpr int PANELS = L::PANELS;
  constexpr int STAGES = L::STAGES;
  constexpr bool ALIAS = HD_PAD > 64;              // dQ shares TMEM columns with S
  constexpr uint32_t S_COL = 0, DP_COL = 128;
  constexpr uint32_t DV_COL = 256, DK_COL = 256 + HD_PAD;
  constexpr uint32_t DQ_COL = ALIAS ? 0 : 256 + 2 * HD_PAD;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + L::BAR_OFF;
  const uint32_t kv_full = bars, qdo_full0 = bars + 8, qdo_empty0 = bars + 24, sdp_full = bars + 40,
                 pds_ready = bars + 48, pds_free = bars + 56, dq_full = bars + 64, dq_free = bars + 72,
                 dkv_full = bars + 80, sdp_read = bars + 88;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::BAR_OFF + 16 * 8);
  AbortState* ab = reinterpret_cast<AbortState*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // early kv tiles see the most query tiles under the causal mask: schedule them first
  const int per_tile = p.Hkv * p.B;
  const int j = static_cast<int>(blockIdx.x) / per_tile;                       // kv tile
  const int rem = static_cast<int>(blockIdx.x) % per_tile;
  const int hk = rem % p.Hkv, b = rem / p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int i0 = p.causal ? j : 0;
  const int n_i = p.n_tiles - i0;
  const int n_it = G * n_i;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(qdo_full0 + 8 * s, 1); mbar_init(qdo_empty0 + 8 * s, 1); }
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, ATT_ROW_WARPS);
    mbar_init(pds_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 4);
    mbar_init(dkv_full, 1);
    mbar_init(sdp_read, ATT_ROW_WARPS);
    ab->flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQ);
  }
  if (warp == 1) { tmem_alloc<512>(smem_u32(tmem_slot)); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(kv_full, 2 * L::TILE);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) {
        tma_load_4d(sbase + L::K_OFF + pn * PANEL_BYTES, &tmK, kv_full, pn * 64, hk, j * ATT_BN, b);
        tma_load_4d(sbase + L::V_OFF + pn * PANEL_BYTES, &tmV, kv_full, pn * 64, hk, j * ATT_BN, b);
      }
      bool ok = true;
      uint32_t armed = 0;
      for (int it = 0; it < n_it; ++it) {
        const int st = it % STAGES;
        const uint32_t use = it / STAGES;
        if (!mbar_wait_bounded(qdo_empty0 + 8 * st, (use & 1u) ^ 1u, ab, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
        const int g = it / n_i, i = i0 + it % n_i;
        const int h = hk * G + g;
        mbar_expect_tx(qdo_full0 + 8 * st, 2 * L::TILE);
        armed |= 1u << st;
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) {
          tma_load_4d(sbase + L::Q_OFF + st * L::TILE + pn * PANEL_BYTES, &tmQ, qdo_full0 + 8 * st, pn * 64, h, i * ATT_BM, b);
          tma_load_4d(sbase + L::DO_OFF + st * L::TILE + pn * PANEL_BYTES, &tmDO, qdo_full0 + 8 * st, pn * 64, h, i * ATT_BM, b);
        }
      }
      if (!ok || ab->flag) {
        for (int it = 0; it < 200000 && !mbar_try_wait(kv_full, 0); ++it) {}
        for (int s = 0; s < STAGES; ++s)
          if (armed & (1u << s))
            for (int it = 0; it < 200000 && !(mbar_try_wait(qdo_full0 + 8 * s, 0) || mbar_try_wait(qdo_full0 + 8 * s, 1)); ++it) {}
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc(128, 128, 1, 1, 1, false, false);        // S, dP: both K-major
      constexpr uint32_t idesc_kv = umma_idesc(128, HD_PAD, 1, 1, 1, true, true);       // dV, dK: A^T from smem, B MN-major
      constexpr uint32_t idesc_dq = umma_idesc(128, HD_PAD, 1, 1, 1, false, true);      // dQ: A K-major, B MN-major
      auto issue_sdp = [&](int st) {
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t off = pn * PANEL_BYTES + k * 32;
            umma_f16_ss(tmem + S_COL, umma_smem_desc_sw128(sbase + L::Q_OFF + st * L::TILE + off, 16, 1024),
                        umma_smem_desc_sw128(sbase + L::K_OFF + off, 16, 1024), idesc_s, (pn | k) ? 1u : 0u);
          }
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t off = pn * PANEL_BYTES + k * 32;
            umma_f16_ss(tmem + DP_COL, umma_smem_desc_sw128(sbase + L::DO_OFF + st * L::TILE + off, 16, 1024),
                        umma_smem_desc_sw128(sbase + L::V_OFF + off, 16, 1024), idesc_s, (pn | k) ? 1u : 0u);
          }
      };
      bool ok = mbar_wait_bounded(kv_full, 0, ab, p.status, ERR_WAIT_FULL);
      for (int it = 0; ok && it < n_it; ++it) {
        const int st = it % STAGES;
        if (ALIAS || it == 0) {
          if (ALIAS && it > 0 && !mbar_wait_bounded(dq_free, (it - 1) & 1, ab, p.status, ERR_WAIT_TMEM_EMPTY)) break;
          if (!mbar_wait_bounded(qdo_full0 + 8 * st, (it / STAGES) & 1, ab, p.status, ERR_WAIT_FULL)) break;
          tc_fence_after();
          issue_sdp(st);
          umma_commit(sdp_full);
        }
        if (!ALIAS && it + 1 < n_it) {
          // S and dP of the next query tile are issued as soon as the P / dS warps hold this tile's in
          // registers (sdp_read), so they run under those warps' exponentials and stores
          const int nst = (it + 1) % STAGES;
          if (!mbar_wait_bounded(sdp_read, it & 1, ab, p.status, ERR_WAIT_TMEM_EMPTY)) break;
          if (!mbar_wait_bounded(qdo_full0 + 8 * nst, ((it + 1) / STAGES) & 1, ab, p.status, ERR_WAIT_FULL)) break;
          tc_fence_after();
          issue_sdp(nst);
          umma_commit(sdp_full);
        }
        if (!mbar_wait_bounded(pds_ready, it & 1, ab, p.status, ERR_WAIT_MISC)) break;
        if (!ALIAS && it > 0 && !mbar_wait_bounded(dq_free, (it - 1) & 1, ab, p.status, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q ; dQ = dS K      (reduction over 128 rows in 8 slices of 16)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_p = umma_smem_desc_sw128(sbase + L::P_OFF + kk * 2048, PANEL_BYTES, 1024);
          const uint64_t b_do = umma_smem_desc_sw128(sbase + L::DO_OFF + st * L::TILE + kk * 2048, PANEL_BYTES, 1024);
          umma_f16_ss(tmem + DV_COL, a_p, b_do, idesc_kv, (it > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_ds = umma_smem_desc_sw128(sbase + L::DS_OFF + kk * 2048, PANEL_BYTES, 1024);
          const uint64_t b_q = umma_smem_desc_sw128(sbase + L::Q_OFF + st * L::TILE + kk * 2048, PANEL_BYTES, 1024);
          umma_f16_ss(tmem + DK_COL, a_ds, b_q, idesc_kv, (it > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a_ds = umma_smem_desc_sw128(sbase + L::DS_OFF + (kk >> 2) * PANEL_BYTES + (kk & 3) * 32, 16, 1024);
          const uint64_t b_k = umma_smem_desc_sw128(sbase + L::K_OFF + kk * 2048, PANEL_BYTES, 1024);
          umma_f16_ss(tmem + DQ_COL, a_ds, b_k, idesc_dq, kk > 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
        umma_commit(qdo_empty0 + 8 * st);
        umma_commit(pds_free);
        if (it + 1 == n_it) umma_commit(dkv_full);
      }
    }
  } else if (warp < 2 + ATT_ROW_WARPS) {
    // ---------------------------------------------------------------- P / dS warps
    // Two threads per query row (same TMEM lane, different warps); each owns 64 kv columns, i.e.
    // one 64-column panel of P and dS.
    const int half = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t t_lane = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    // row statistics of query tile `it`: fetched one iteration ahead, their latency would otherwise sit
    // between the arrival of S / dP and the first exponential
    auto row_stats = [&](int it, float& lse_v, float& dlt_v) {
      const int g = it / n_i, i = i0 + it % n_i;
      const int q_idx = i * ATT_BM + row;
      const long long stat = (static_cast<long long>(b) * p.Hq + (hk * G + g)) * p.T + q_idx;
      const bool live = it < n_it && q_idx < p.T;
      lse_v = live ? p.lse[stat] : 0.f;
      dlt_v = live ? p.delta[stat] : 0.f;
    };
    float lse_nxt, dlt_nxt;
    row_stats(0, lse_nxt, dlt_nxt);
    for (int it = 0; it < n_it; ++it) {
      const int i = i0 + it % n_i;
      const int q_idx = i * ATT_BM + row;
      const bool q_live = q_idx < p.T;
      const float lse_l2 = lse_nxt * LOG2E;
      const float dlt_s = dlt_nxt * p.scale;
      row_stats(it + 1, lse_nxt, dlt_nxt);
      ok = mbar_wait_bounded(sdp_full, it & 1, ab, p.status, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      tc_fence_after();
      const bool diag = p.causal && i == j;
      const bool ragged = (j + 1) * ATT_BN > p.T;
      int limit = ATT_BN;                      // visible kv columns of this row inside the tile
      if (diag) limit = row + 1;
      if (ragged) limit = min(limit, p.T - j * ATT_BN);
      if (!q_live) limit = 0;
      const int c_lo = half * 64;
      const bool masked = __any_sync(0xffffffffu, limit < c_lo + 64);
      // 32 columns of S and dP -> bf16 pairs of P and dS
      auto p_ds = [&](const uint32_t (&rs)[32], const uint32_t (&rd)[32], int c0, uint32_t (&pp)[16], uint32_t (&dd)[16]) {
        if (!masked) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(rs[e]), p.scale_log2, -lse_l2));
            const float p1 = exp2f(fmaf(__uint_as_float(rs[e + 1]), p.scale_log2, -lse_l2));
            const float d0 = p0 * fmaf(__uint_as_float(rd[e]), p.scale, -dlt_s);
            const float d1 = p1 * fmaf(__uint_as_float(rd[e + 1]), p.scale, -dlt_s);
            pp[e >> 1] = pack_bf16(p0, p1);
            dd[e >> 1] = pack_bf16(d0, d1);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const int col = c0 + e;
            float p0 = exp2f(fmaf(__uint_as_float(rs[e]), p.scale_log2, -lse_l2));
            float p1 = exp2f(fmaf(__uint_as_float(rs[e + 1]), p.scale_log2, -lse_l2));
            if (col >= limit) p0 = 0.f;
            if (col + 1 >= limit) p1 = 0.f;
            const float d0 = p0 * fmaf(__uint_as_float(rd[e]), p.scale, -dlt_s);
            const float d1 = p1 * fmaf(__uint_as_float(rd[e + 1]), p.scale, -dlt_s);
            pp[e >> 1] = pack_bf16(p0, p1);
            dd[e >> 1] = pack_bf16(d0, d1);
          }
        }
      };
      auto put = [&](int cc, const uint32_t (&pp)[16], const uint32_t (&dd)[16]) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t off = swz_tile_offset(row, half * 8 + cc * 4 + q4);
          *reinterpret_cast<uint4*>(smem + L::P_OFF + off) = make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]);
          *reinterpret_cast<uint4*>(smem + L::DS_OFF + off) = make_uint4(dd[4 * q4], dd[4 * q4 + 1], dd[4 * q4 + 2], dd[4 * q4 + 3]);
        }
      };
      uint32_t pp0[16], dd0[16];
      uint32_t rs[32], rd[32];
      tmem_ld_32x32(t_lane + S_COL + c_lo, rs);
      tmem_ld_32x32(t_lane + DP_COL + c_lo, rd);
      tmem_ld_fence(rs);
      tmem_ld_fence(rd);
      p_ds(rs, rd, c_lo, pp0, dd0);
      if (it > 0) {
        // P / dS of the previous iteration must have been consumed before they are overwritten
        ok = mbar_wait_bounded(pds_free, (it - 1) & 1, ab, p.status, ERR_WAIT_MISC);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      }
      put(0, pp0, dd0);
      tmem_ld_32x32(t_lane + S_COL + c_lo + 32, rs);
      tmem_ld_32x32(t_lane + DP_COL + c_lo + 32, rd);
      tmem_ld_fence(rs);
      tmem_ld_fence(rd);
      // S and dP of this tile are in registers: the tensor pipe may overwrite them with the next tile's
      // while this warp is still busy with the second half's exponentials and stores
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdp_read);
      p_ds(rs, rd, c_lo + 32, pp0, dd0);
      put(1, pp0, dd0);
      if (!ok) break;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);
    }
    // ---- final: half 0 stores dK, half 1 stores dV of this kv tile
    if (ok && mbar_wait_bounded(dkv_full, 0, ab, p.status, ERR_WAIT_TMEM_FULL)) {
      tc_fence_after();
      const int kv_idx = j * ATT_BN + row;
      const bool live = kv_idx < p.T;
      const long long base = (static_cast<long long>(b) * p.T + kv_idx) * p.dkv_stride_t + static_cast<long long>(hk) * p.hd;
      const uint32_t col_base = half == 0 ? DK_COL : DV_COL;
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(half == 0 ? p.dk : p.dv) + base;
#pragma unroll 1
      for (int c = 0; c < HD_PAD / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_lane + col_base + c * 32, r);
        tmem_ld_fence(r);
        if (!live) continue;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int col = c * 32 + q4 * 8;
          if (col < p.hd) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[q4 * 8 + 0]), __uint_as_float(r[q4 * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(r[q4 * 8 + 2]), __uint_as_float(r[q4 * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(r[q4 * 8 + 4]), __uint_as_float(r[q4 * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(r[q4 * 8 + 6]), __uint_as_float(r[q4 * 8 + 7]));
            *reinterpret_cast<uint4*>(out + col) = v;
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- dQ writer warps
    // Every kv tile contributes to the dQ rows of the query tiles it sees, so dQ is summed in an fp32 buffer.
    // The sum goes through TMA: a warp stages its 32 rows x 32 columns in 128B-swizzled shared memory and one
    // lane sends the box as a reduce-add ([B, T, Hq * hd] map: rows past T are clipped by the copy engine).
    // That is one instruction per 4 KB instead of 256 vector atomics per warp and chunk.
    const int quarter = warp & 3;
    const uint32_t stg_base = sbase + L::DQ_STG_OFF + static_cast<uint32_t>(quarter) * (L::DQ_BUFS * 4096u);
    const uint32_t t_lane = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    uint32_t stg_i = 0;
    for (int it = 0; it < n_it; ++it) {
      const int g = it / n_i, i = i0 + it % n_i;
      const int h = hk * G + g;
      bool ok = mbar_wait_bounded(dq_full, it & 1, ab, p.status, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, ok)) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < HD_PAD / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_lane + DQ_COL + c * 32, r);
        tmem_ld_fence(r);
        if (c == HD_PAD / 32 - 1) {
          // the accumulator is in registers now: let the MMA warp reuse it while the boxes drain
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(dq_free);
        }
        if (c * 32 >= p.hd) continue;                 // padding columns of a head dim below the tile width
        const uint32_t buf = stg_base + (stg_i % L::DQ_BUFS) * 4096u;
        ++stg_i;
        if (lane == 0) tma_store_wait_read<L::DQ_BUFS - 1>();     // the box sent from this buffer earlier has been read
        __syncwarp();
        const uint32_t row_addr = buf + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
        for (int q = 0; q < 8; ++q)                   // 16-byte piece q of row r sits at q ^ (r % 8)
          st_shared_v4(row_addr + (static_cast<uint32_t>(q ^ (lane & 7)) << 4), r[4 * q], r[4 * q + 1], r[4 * q + 2],
                       r[4 * q + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_3d(&tmDQ, buf, h * p.hd + c * 32, i * ATT_BM + quarter * 32, b);
          tma_store_commit();
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();           // shared memory must outlive the copies that read it
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc<512>(tmem); }
}

// delta[b, h, t] = sum_d dO * O. `lpr` lanes (a power of two, 8 elements each per pass) share one (b, t, h)
// row, so a warp reads 32 / lpr consecutive heads' rows as whole 16-byte pieces.
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                  int B, int T, int Hq, int hd, long long o_stride_t, int lpr) {
  pdl_wait();
  pdl_launch_dependents();
  const long long gtid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int sub = static_cast<int>(gtid % lpr);
  const long long item = gtid / lpr;                                   // (b, t, h)
  const bool live = item < static_cast<long long>(B) * T * Hq;
  const int h = live ? static_cast<int>(item % Hq) : 0;
  const long long bt = live ? item / Hq : 0;
  const __nv_bfloat16* orow = o + bt * o_stride_t + static_cast<long long>(h) * hd;
  const __nv_bfloat16* grow = d_o + bt * o_stride_t + static_cast<long long>(h) * hd;
  float s = 0.f;
  if (live) {
    for (int c = sub * 8; c < hd; c += lpr * 8) {
      const uint4 a = *reinterpret_cast<const uint4*>(orow + c), g = *reinterpret_cast<const uint4*>(grow + c);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 af = unpack_bf16(aw[q]), gf = unpack_bf16(gw[q]);
        s += af.x * gf.x + af.y * gf.y;
      }
    }
  }
  for (int ofs = lpr >> 1; ofs > 0; ofs >>= 1) s += __shfl_xor_sync(0xffffffffu, s, ofs);
  if (live && sub == 0) {
    const long long b = bt / T, t = bt % T;
    delta[(b * Hq + h) * T + t] = s;
  }
}

// dq (bf16, strided rows) = dq_acc (fp32 [B*T, Hq*hd])
__global__ void __launch_bounds__(256)
attn_dq_store_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long rows, int width,
                     long long dq_stride_t) {
  pdl_wait();
  pdl_launch_dependents();
  const int wv = width >> 3;
  const long long total = rows * wv;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / wv;
    const int c = static_cast<int>(i % wv) * 8;
    const float4 a = *reinterpret_cast<const float4*>(acc + r * width + c);
    const float4 b2 = *reinterpret_cast<const float4*>(acc + r * width + c + 4);
    uint4 v;
    v.x = pack_bf16(a.x, a.y); v.y = pack_bf16(a.z, a.w); v.z = pack_bf16(b2.x, b2.y); v.w = pack_bf16(b2.z, b2.w);
    *reinterpret_cast<uint4*>(dq + r * dq_stride_t + c) = v;
  }
}

static bool make_head_tmap(CUtensorMap* m, const void* base, int B, int T, int H, int hd, long long stride_t) {
  // dims innermost first: (hd, head, token, batch); heads are packed inside a token row
  uint64_t dims[4] = {static_cast<uint64_t>(hd), static_cast<uint64_t>(H), static_cast<uint64_t>(T),
                      static_cast<uint64_t>(B)};
  uint64_t strides[4] = {2, static_cast<uint64_t>(hd) * 2, static_cast<uint64_t>(stride_t) * 2,
                         static_cast<uint64_t>(stride_t) * 2 * static_cast<uint64_t>(T)};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_nd(m, base, 4, dims, strides, box, 2, TmapSwizzle::B128);
}

}  // namespace fmb

using namespace fmb;

extern "C" int fmb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int Hq,
                            int Hkv, int hd, long long q_stride_t, long long kv_stride_t, long long o_stride_t,
                            float scale, int causal, int* status, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (hd % 8 || hd > 128 || Hq % Hkv || (q_stride_t % 8) || (kv_stride_t % 8) || (o_stride_t % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return -2;
  CUtensorMap tq, tk, tv;
  if (!make_head_tmap(&tq, q, B, T, Hq, hd, q_stride_t) || !make_head_tmap(&tk, k, B, T, Hkv, hd, kv_stride_t) ||
      !make_head_tmap(&tv, v, B, T, Hkv, hd, kv_stride_t))
    return -5;
  AttnParams p;
  p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.hd = hd;
  p.n_tiles = (T + ATT_BM - 1) / ATT_BM;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.o = o; p.o_stride_t = o_stride_t; p.lse = lse; p.status = status;
  const unsigned grid = static_cast<unsigned>(p.n_tiles) * Hq * B;
  cudaError_t e;
  if (hd <= 64) {
    auto kern = attn_fwd_kernel<64>;
    constexpr int sm = FwdSmem<64>::TOTAL;
    static bool done = false;
    if (!done) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sm) != cudaSuccess) return -6; done = true; }
    e = launch_pdl(kern, dim3(grid), dim3(ATT_FWD_THREADS), sm, stream, tq, tk, tv, p);
  } else {
    auto kern = attn_fwd_kernel<128>;
    constexpr int sm = FwdSmem<128>::TOTAL;
    static bool done = false;
    if (!done) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sm) != cudaSuccess) return -6; done = true; }
    e = launch_pdl(kern, dim3(grid), dim3(ATT_FWD_THREADS), sm, stream, tq, tk, tv, p);
  }
  return e == cudaSuccess ? 0 : -10 - static_cast<int>(e);
}

extern "C" int fmb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, void* dq, void* dk, void* dv, float* delta, float* dq_acc, int B, int T,
                            int Hq, int Hkv, int hd, long long q_stride_t, long long kv_stride_t, long long o_stride_t,
                            long long dq_stride_t, long long dkv_stride_t, float scale, int causal, int delta_ready,
                            int* status, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (hd % 8 || hd > 128 || Hq % Hkv || (q_stride_t % 8) || (kv_stride_t % 8) || (o_stride_t % 8) ||
      (dq_stride_t % 8) || (dkv_stride_t % 8))
    return -2;
  CUtensorMap tq, tk, tv, tdo, tdq;
  if (!make_head_tmap(&tq, q, B, T, Hq, hd, q_stride_t) || !make_head_tmap(&tk, k, B, T, Hkv, hd, kv_stride_t) ||
      !make_head_tmap(&tv, v, B, T, Hkv, hd, kv_stride_t) || !make_head_tmap(&tdo, d_o, B, T, Hq, hd, o_stride_t))
    return -5;
  {
    // dq_acc [B, T, Hq * hd] fp32, reduce-added in boxes of 32 rows x 32 columns (x = h * hd + c * 32 is a
    // multiple of 4 elements because hd % 8 == 0)
    const uint64_t width = static_cast<uint64_t>(Hq) * hd;
    const uint64_t dims[3] = {width, static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
    const uint64_t strides[3] = {4, width * 4, width * 4 * static_cast<uint64_t>(T)};
    const uint32_t box[3] = {32, 32, 1};
    if ((reinterpret_cast<uintptr_t>(dq_acc) & 15) || !make_tmap_nd(&tdq, dq_acc, 3, dims, strides, box, 4, TmapSwizzle::B128))
      return -5;
  }
  if (!delta_ready) {     // else the caller computed delta[b, h, t] already (fused into the producer of dO)
    const long long items = static_cast<long long>(B) * T * Hq;
    int lpr = 1;
    while (lpr < 32 && lpr * 8 < hd) lpr <<= 1;
    launch_pdl(attn_delta_kernel, dim3(static_cast<unsigned>((items * lpr + 255) / 256)), dim3(256), 0, stream,
               static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, B, T, Hq, hd,
               o_stride_t, lpr);
  }
  AttnBwdParams p;
  p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.hd = hd;
  p.n_tiles = (T + ATT_BM - 1) / ATT_BM;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dk = dk; p.dv = dv; p.dkv_stride_t = dkv_stride_t; p.status = status;
  const unsigned grid = static_cast<unsigned>(p.n_tiles) * Hkv * B;
  if (hd <= 64) {
    auto kern = attn_bwd_kernel<64>;
    constexpr int sm = BwdSmem<64>::TOTAL;
    static bool done = false;
    if (!done) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sm) != cudaSuccess) return -6; done = true; }
    if (launch_pdl(kern, dim3(grid), dim3(ATT_BWD_THREADS), sm, stream, tq, tk, tv, tdo, tdq, p) != cudaSuccess) return -7;
  } else {
    auto kern = attn_bwd_kernel<128>;
    constexpr int sm = BwdSmem<128>::TOTAL;
    static bool done = false;
    if (!done) { if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, sm) != cudaSuccess) return -6; done = true; }
    if (launch_pdl(kern, dim3(grid), dim3(ATT_BWD_THREADS), sm, stream, tq, tk, tv, tdo, tdq, p) != cudaSuccess) return -7;
  }
  if (cudaGetLastError() != cudaSuccess) return -7;
  if (dq != nullptr) {   // a caller that consumes the fp32 sum itself (the RoPE backward) passes no dq
    const long long rows = static_cast<long long>(B) * T;
    const int width = Hq * hd;
    long long blocks = (rows * (width / 8) + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    launch_pdl(attn_dq_store_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, dq_acc,
               static_cast<__nv_bfloat16*>(dq), rows, width, dq_stride_t);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}
