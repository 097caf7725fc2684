// bf16 GEMM for sm_100a: D[M,N] = alpha * sum_k A(m,k) * B(n,k) + beta * C[M,N].
//
// Persistent, one CTA per SM, six warps with fixed roles:
//   warp 0    one elected thread issues TMA tile loads into a ring of 128B-swizzled smem stages;
//   warp 1    owns TMEM (two fp32 accumulators) and one elected thread issues tcgen05.mma;
//   warps 2-5 read the finished accumulator back with tcgen05.ld (one TMEM lane quarter each, the
//             loads one 32-column chunk ahead of the stores), apply the epilogue and store, while the
//             MMA warp already works on the other accumulator.
// Plain products run as CTA pairs (cta_group::2): two CTAs of a cluster share one 256 x BN tile, each
// loading its own 128 rows of A and half of B, so that every SM reads a third less from L2.
// Operands may be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]); this covers
// the forward (K,K), input-gradient (K,MN) and weight-gradient (MN,MN) products of a linear layer
// without a transpose pass. Split-K fills the machine when the output has fewer tiles than SMs, which
// is the usual case for weight gradients; fp32 outputs (split or accumulated into C == D) leave as
// TMA reduce-add boxes staged in shared memory. Peer instantiations gather an operand from the other
// GPUs of an NVSwitch domain with two extra warps, or scatter bf16 partial tiles to their owners.
#include <cstdlib>
#include <cstring>

#include "ptx_sm100.cuh"
#include "peer.cuh"
#include "launch.cuh"
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
  int tg_step;              // 128-row entries of tile_group per row tile of this launch (2 on CTA pairs)
  const int* tile_group;
  const int* region;
  long long group_stride_d;
  // peer modes (PEER instantiations only).
  // Gathered operand ("all-gather fused into the product"): the operand's rows (the y coordinate of its
  // TMA map: the M rows of a K-major A, the reduction rows of an MN-major A or B) are spread over the
  // ranks, `g_rows_per_src` (a multiple of 128) each, at the same offsets of one symmetric buffer per
  // rank. Two extra warps of every CTA pull the other ranks' rows into THIS rank's buffer -- each row
  // crosses NVLink exactly once -- and count finished rows per 128-row block in `g_ready`; the TMA
  // producer reads only local memory and waits for a block's count before its first load from it. The
  // copy of rank r's rows starts after flags[g_slot * MAX_PEERS + r] reached g_epoch (g_slot < 0: at once).
  // Row tiles of this rank's own rows are scheduled first, so the copy hides behind them.
  // Scattered output ("reduce-scatter fused into the epilogue"): with d_rows_per_rank > 0 the rows of the
  // output belong to the rank that owns them and every rank stores its bf16 partial product into the
  // owner's staging buffer [world, d_rows_per_rank, N] at slice `rank`; the owner sums the slices.
  int rank, world;
  int gather;               // 0 none, 1 operand A, 2 operand B
  int g_rows_per_src;
  long long g_ld;           // elements per row
  int g_row_bytes;          // bytes to copy per row (multiple of 16)
  void* g_local;
  const void* g_src[FMB_MAX_PEERS];
  int* g_ready;
  const uint32_t* flags;
  int g_slot;
  uint32_t g_epoch;
  unsigned long long timeout_ns;
  int own_m_tiles;          // > 0: row tiles [rot_m, rot_m + own_m_tiles) (all column tiles) come first
  int d_rows_per_rank;
  void* d_peer[FMB_MAX_PEERS];
  int rot_m;                // row tiles are visited starting from this one (own shard first / remote first)
  int rot_k;                // reduction blocks are visited starting from this one (own shard first)
  // fused epilogues (BN = 256, plain products only):
  //   1  SwiGLU forward. B is the stacked gate|up weight [2h, K]; a tile multiplies by rows [n0, n0+128)
  //      (gate) and [h+n0, h+n0+128) (up), D is the gate|up buffer [M, 2h] and aux_out[M, h] receives
  //      silu(gate) * up.
  //   2  SwiGLU backward. The accumulator is d(act) [M, h]; gate|up are read from aux_in [M, 2h] and
  //      d(gate)|d(up) are written to D [M, 2h]; d(act) itself is never stored.
  //   3  row dots. Besides D, rowdot[row, col / seg] = sum of D * aux_in over each seg-wide column group
  //      (aux_in has the layout of D). With epi_h = T > 0 the rows are (batch, t) pairs and the result is
  //      stored as [batch, group, t].
  int epi, epi_h, seg;
  // Output through TMA (plain fp32 products): 1 = D += alpha * product as 32 x 32 reduce-add boxes staged in
  // shared memory (replaces both "C == D, beta == 1" and the split-K atomics), 2 = the same as plain stores.
  int d_tma;
  int n_fast;               // tile order: column tiles vary fastest (default: row tiles)
  const void* aux_in;
  long long ld_aux_in;
  void* aux_out;
  long long ld_aux_out;
};

template <bool PEER>
struct MapSet {
  CUtensorMap m[1];
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
  if (p.own_m_tiles > 0) {            // this rank's own rows first (all column tiles), then the gathered ones
    const int own = p.own_m_tiles, first = own * p.tiles_n;
    if (mn < first) {
      t.m_blk = p.rot_m + mn % own;
      t.n_blk = mn / own;
    } else {
      const int rest = p.tiles_m - own, r = mn - first;
      t.m_blk = (p.rot_m + own + r % rest) % p.tiles_m;
      t.n_blk = r / rest;
    }
  } else if (p.n_fast) {              // consecutive CTAs share a row tile of A
    t.m_blk = mn / p.tiles_n;
    t.n_blk = mn - t.m_blk * p.tiles_n;
  } else {
    t.m_blk = mn % p.tiles_m;
    if (p.rot_m) t.m_blk = (t.m_blk + p.rot_m) % p.tiles_m;
    t.n_blk = mn / p.tiles_m;
  }
  t.k0 = ks * p.kblocks_per_split;
  t.k1 = min(p.kblocks_total, t.k0 + p.kblocks_per_split);
  if (p.mode == 1) {
    // on CTA pairs a 256-row tile starts a group or continues one (groups are 256-aligned then): its first
    // 128 rows name the group; a second half that holds only padding is computed and never read
    t.zb = __ldg(p.tile_group + t.m_blk * p.tg_step);
    t.valid = t.zb >= 0;
  }
  return t;
}

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

template <int BN, int STAGES, int CTAS = 1>
struct GemmSmem {
  static constexpr uint32_t A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr uint32_t B_BYTES = (BN / CTAS) * GEMM_BK * 2;   // a CTA pair splits the B tile
  static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t STG_OFFSET = STAGES * STAGE_BYTES;          // output staging: 4 warps x 2 boxes of 4 KB
  static constexpr uint32_t STG_BYTES = 4 * 2 * 4096;
  static constexpr uint32_t BAR_OFFSET = STG_OFFSET + STG_BYTES;
  static constexpr uint32_t TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;  // + alignment slack
};

__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Bounded wait for a counter in local memory (rows of a gathered block that have arrived).
__device__ __forceinline__ bool wait_count(const int* ctr, int want, unsigned long long timeout_ns, int* status) {
  const uint64_t t0 = globaltimer_ns();
  int spins = 0;
  for (;;) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= want) return true;
    if (++spins > 32) {
      __nanosleep(64);
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (status != nullptr) atomicCAS(status, 0, ERR_WAIT_PEER);
        return false;
      }
    }
  }
}

constexpr int GATHER_THREADS = 64;
constexpr int GATHER_DEPTH = 16;

// Executed by the two gather warps of every CTA: pull the other ranks' rows of the gathered operand into
// this rank's buffer, nearest rank first, 128-row block by block. The remote rows form one list that the
// CTAs share round robin; a CTA moves two rows at a time (up to 16 KB in flight: one NVLink round trip
// is several microseconds) and then adds the rows it finished to their blocks' counters.
__device__ __forceinline__ void gather_rows(const GemmParams& p, int tid) {
  const int vec_per_row = p.g_row_bytes >> 4;
  const int rps = p.g_rows_per_src;
  const int rows_total = (p.world - 1) * rps;
  uint32_t waited = 0;                           // sources whose flag has been seen
  auto locate = [&](int q, int& src, long long& off, int& blk) {
    const int step = q / rps + 1, lr = q - (step - 1) * rps;
    src = (p.rank + step) % p.world;
    const long long grow = static_cast<long long>(src) * rps + lr;      // row of the full operand
    off = grow * p.g_ld * 2;
    blk = static_cast<int>(grow >> 7);
  };
  for (int q = blockIdx.x; q < rows_total; q += 2 * gridDim.x) {
    int src0, src1 = 0, blk0, blk1 = 0;
    long long off0, off1 = 0;
    const bool two = q + static_cast<int>(gridDim.x) < rows_total;
    locate(q, src0, off0, blk0);
    if (two) locate(q + gridDim.x, src1, off1, blk1);
    if (p.g_slot >= 0) {
      if (!(waited & (1u << src0))) {
        if (!wait_epoch(p.flags + p.g_slot * MAX_PEERS + src0, p.g_epoch, p.timeout_ns, p.status)) return;
        waited |= 1u << src0;
      }
      if (two && !(waited & (1u << src1))) {
        if (!wait_epoch(p.flags + p.g_slot * MAX_PEERS + src1, p.g_epoch, p.timeout_ns, p.status)) return;
        waited |= 1u << src1;
      }
    }
    const uint4* sp0 = reinterpret_cast<const uint4*>(static_cast<const char*>(p.g_src[src0]) + off0);
    uint4* dp0 = reinterpret_cast<uint4*>(static_cast<char*>(p.g_local) + off0);
    const uint4* sp1 = reinterpret_cast<const uint4*>(static_cast<const char*>(p.g_src[src1]) + off1);
    uint4* dp1 = reinterpret_cast<uint4*>(static_cast<char*>(p.g_local) + off1);
    constexpr int HALF = GATHER_DEPTH / 2;
    for (int v0 = tid; v0 < vec_per_row; v0 += GATHER_THREADS * HALF) {
      uint4 a[HALF], b[HALF];
#pragma unroll
      for (int u = 0; u < HALF; ++u)
        if (v0 + u * GATHER_THREADS < vec_per_row) {
          a[u] = ld_peer_u4(sp0 + v0 + u * GATHER_THREADS);
          if (two) b[u] = ld_peer_u4(sp1 + v0 + u * GATHER_THREADS);
        }
#pragma unroll
      for (int u = 0; u < HALF; ++u)
        if (v0 + u * GATHER_THREADS < vec_per_row) {
          if (addr_ok(dp0 + v0 + u * GATHER_THREADS, 16)) dp0[v0 + u * GATHER_THREADS] = a[u];
          if (two && addr_ok(dp1 + v0 + u * GATHER_THREADS, 16)) dp1[v0 + u * GATHER_THREADS] = b[u];
        }
    }
    __threadfence();
    asm volatile("bar.sync 1, 64;" ::: "memory");
    if (tid == 0) {
      atomicAdd(p.g_ready + blk0, 1);
      if (two) atomicAdd(p.g_ready + blk1, 1);
    }
  }
}

// CTAS = 2: the CTAs 2i and 2i+1 of the grid form a cluster and work on one 256 x BN tile together. Each
// loads its own 128 rows of A and its own half (BN / 2 columns) of B; one thread of the even CTA issues
// cta_group::2 MMAs that read both CTAs' shared memory and write 128 accumulator rows into each CTA's
// TMEM; each CTA's epilogue warps store their own 128 rows. Per SM the B traffic from L2 is halved. All
// pipeline barriers that the MMA thread waits on live in the even CTA: loads of both CTAs count their
// bytes there and the epilogue warps of both arrive there; the MMA thread's commits arrive in both CTAs.
// p.tiles_m then counts 256-row tiles.
template <int BN, int STAGES, bool A_MN, bool B_MN, bool PEER, int CTAS = 1>
__global__ void __launch_bounds__(GEMM_THREADS + (PEER ? GATHER_THREADS : 0), 1)
gemm_bf16_kernel(const __grid_constant__ MapSet<PEER> tmA, const __grid_constant__ MapSet<PEER> tmB,
                 const __grid_constant__ CUtensorMap tmD, GemmParams p) {
  static_assert(CTAS == 1 || (CTAS == 2 && BN >= 128), "CTA pairs need BN >= 128");   // and no gathered operand
  using L = GemmSmem<BN, STAGES, CTAS>;
  constexpr int BM = GEMM_BM, BK = GEMM_BK;
  constexpr int BN_CTA = BN / CTAS;                  // columns of B that this CTA loads
  const uint32_t cta_rank = CTAS == 2 ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0u;
  const int unit = CTAS == 2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int n_units = CTAS == 2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
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
      mbar_init(tempty_bar(s), 4 * CTAS);
    }
    ab->flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA.m[0]);
    tma_prefetch_desc(&tmB.m[0]);
    if (p.d_tma) tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    if constexpr (CTAS == 2) {
      tmem_alloc_pair<2 * BN>(smem_u32(tmem_slot));
      tmem_relinquish_pair();
    } else {
      tmem_alloc<2 * BN>(smem_u32(tmem_slot));
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (CTAS == 2) {
    __syncwarp();
    cluster_sync_all();              // the other CTA's barriers are initialised before anything signals them
  } else {
    __syncthreads();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                      // everything above touched only this CTA's shared memory and TMEM
  pdl_launch_dependents();

  const int total_tiles = p.tiles_m * p.tiles_n * (p.mode == 2 ? p.n_groups : p.splits);

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      uint32_t armed = 0, armed_parity = 0;
      int ready_blk = -1;                       // last gathered 128-row block known to be complete
      bool ok = true;
      for (int tile = unit; ok && tile < total_tiles; tile += n_units) {
        const TileInfo ti = decode_tile(p, tile);
        if (!ti.valid) continue;
        const int m_blk = ti.m_blk * CTAS + static_cast<int>(cta_rank), n_blk = ti.n_blk, k0 = ti.k0, k1 = ti.k1;
        const int n_off = n_blk * BN + static_cast<int>(cta_rank) * BN_CTA;     // first B column of this CTA
        for (int kq = k0; kq < k1; ++kq) {
          int kb = kq;
          if (PEER && p.rot_k) { kb = kq + p.rot_k; if (kb >= k1) kb -= (k1 - k0); }
          const int a_y = A_MN ? kb * BK : m_blk * BM;
          const int b_y = B_MN ? kb * BK : n_off;
          if constexpr (PEER) {
            if (p.gather) {
              const int blk = (p.gather == 1 ? a_y : b_y) >> 7;
              if (blk != ready_blk) {
                const int owner = blk / (p.g_rows_per_src >> 7);
                if (owner != p.rank && !wait_count(p.g_ready + blk, 128, p.timeout_ns, p.status)) {
                  raise_abort(ab, p.status, ERR_WAIT_PEER);
                  ok = false;
                  break;
                }
                ready_blk = blk;
                fence_proxy_async_all();        // the rows were written by ordinary stores; TMA reads them next
              }
            }
          }
          if (!mbar_wait_bounded(empty_bar(stage), phase ^ 1u, ab, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sA = smem_base + stage * L::STAGE_BYTES;
          const uint32_t sB = sA + L::A_BYTES;
          if (leader) {                          // the even CTA's barrier counts the bytes of both CTAs
            mbar_expect_tx(full_bar(stage), CTAS * L::STAGE_BYTES);
            armed |= 1u << stage;
            armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          }
          const CUtensorMap* ma = &tmA.m[0];
          const CUtensorMap* mb = &tmB.m[0];
          if constexpr (CTAS == 2) {
            const uint32_t bar = mapa_shared(full_bar(stage), 0u);
            if constexpr (!A_MN) {
              tma_load_2d_pair(sA, ma, bar, kb * BK, a_y);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_2d_pair(sA + j * (BK * 128), ma, bar, m_blk * BM + j * 64, a_y);
            }
            if constexpr (!B_MN) {
              // SwiGLU forward: the even CTA holds the 128 gate rows of the stacked weight, the odd CTA the
              // 128 up rows, which makes accumulator columns [0,128) gate and [128,256) up
              const int b_row = (BN == 256 && p.epi == 1) ? (cta_rank ? p.epi_h + n_blk * 128 : n_blk * 128) : b_y;
              tma_load_3d_pair(sB, mb, bar, kb * BK, b_row, ti.zb);
            } else {
#pragma unroll
              for (int j = 0; j < BN_CTA / 64; ++j)
                tma_load_3d_pair(sB + j * (BK * 128), mb, bar, n_off + j * 64, b_y, ti.zb);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          if constexpr (!A_MN) {
            tma_load_2d(sA, ma, full_bar(stage), kb * BK, a_y);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sA + j * (BK * 128), ma, full_bar(stage), m_blk * BM + j * 64, a_y);
          }
          if constexpr (!B_MN) {
            if (BN == 256 && p.epi == 1) {       // gate rows and up rows of the stacked weight
              tma_load_3d(sB, mb, full_bar(stage), kb * BK, n_blk * 128, ti.zb);
              tma_load_3d(sB + 128u * 128u, mb, full_bar(stage), kb * BK, p.epi_h + n_blk * 128, ti.zb);
            } else {
              tma_load_3d(sB, mb, full_bar(stage), kb * BK, b_y, ti.zb);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sB + j * (BK * 128), mb, full_bar(stage), n_blk * BN + j * 64, b_y, ti.zb);
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
    if ((CTAS == 1 || leader) && elect_one()) {
      constexpr uint32_t idesc = umma_idesc(BM * CTAS, BN, 1, 1, 1, A_MN, B_MN);
      constexpr uint32_t A_KSTEP = A_MN ? 16u * 128u : 32u;   // bytes per 16-wide K slice
      constexpr uint32_t B_KSTEP = B_MN ? 16u * 128u : 32u;
      constexpr uint32_t MN_LBO = BK * 128u;                  // next 64-wide block of an MN-major tile
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = unit; ok && tile < total_tiles; tile += n_units) {
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
            if constexpr (CTAS == 2) umma_f16_ss_pair(d_tmem, da, db, idesc, (kb > k0 || k > 0) ? 1u : 0u);
            else                     umma_f16_ss(d_tmem, da, db, idesc, (kb > k0 || k > 0) ? 1u : 0u);
          }
          if constexpr (CTAS == 2) umma_commit_pair(empty_bar(stage), 3);   // frees the stage in both CTAs
          else                     umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if constexpr (CTAS == 2) umma_commit_pair(tfull_bar(acc), 3);
        else                     umma_commit(tfull_bar(acc));
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------- gather warps (PEER launches only)
    if constexpr (PEER) {
      if (p.gather) gather_rows(p, static_cast<int>(threadIdx.x) - GEMM_THREADS);
    }
  } else {
    // ------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;                 // TMEM lanes [32*quarter, 32*quarter + 32)
    uint32_t acc = 0, acc_phase = 0;
    const float alpha = p.alpha_ptr != nullptr ? p.alpha * __ldg(p.alpha_ptr) : p.alpha;
    const float beta = p.beta;
    const uint32_t stg_base = smem_base + L::STG_OFFSET + static_cast<uint32_t>(quarter) * 8192u;
    uint32_t stg_i = 0;                           // boxes issued so far by this warp (selects the staging buffer)
    const long long d_es = p.d_f32 ? 4 : 2;
    const bool wide_d = (reinterpret_cast<uintptr_t>(p.D) & 31) == 0 && (p.ldd * d_es) % 32 == 0 &&
                        (p.group_stride_d * d_es) % 32 == 0;          // 32-byte stores stay aligned
    for (int tile = unit; tile < total_tiles; tile += n_units) {
      const TileInfo ti = decode_tile(p, tile);
      if (!ti.valid) continue;
      const int m_blk = ti.m_blk * CTAS + static_cast<int>(cta_rank), n_blk = ti.n_blk;
      if (!mbar_wait_bounded(tfull_bar(acc), acc_phase, ab, p.status, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if (BN == 256 && p.epi == 1) {
        // SwiGLU forward: accumulator columns [0,128) are gate, [128,256) up, of hidden units n_blk*128 ...
        const bool wide1 = wide_d && (reinterpret_cast<uintptr_t>(p.aux_out) & 31) == 0 && (p.ld_aux_out * 2) % 32 == 0 &&
                           (p.epi_h * 2) % 32 == 0;
        auto swiglu_chunk = [&](int c, const uint32_t (&rg)[32], const uint32_t (&ru)[32]) {
          if (!row_ok) return;
          const int hc = n_blk * 128 + c * 32;                // hidden-unit column, < epi_h by construction
          __nv_bfloat16* gp = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + hc;
          __nv_bfloat16* up = gp + p.epi_h;
          __nv_bfloat16* ap = reinterpret_cast<__nv_bfloat16*>(p.aux_out) + static_cast<long long>(row) * p.ld_aux_out + hc;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint32_t og[8], ou[8], oa[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              // round gate and up to bf16 first: the activation is what a separate kernel would compute from them
              og[q] = pack_bf16(__uint_as_float(rg[16 * i + 2 * q]), __uint_as_float(rg[16 * i + 2 * q + 1]));
              ou[q] = pack_bf16(__uint_as_float(ru[16 * i + 2 * q]), __uint_as_float(ru[16 * i + 2 * q + 1]));
              const float2 g = unpack_bf16(og[q]), u = unpack_bf16(ou[q]);
              oa[q] = pack_bf16(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
            }
            if (wide1) {
              st_global_v8(gp + 16 * i, og[0], og[1], og[2], og[3], og[4], og[5], og[6], og[7]);
              st_global_v8(up + 16 * i, ou[0], ou[1], ou[2], ou[3], ou[4], ou[5], ou[6], ou[7]);
              st_global_v8(ap + 16 * i, oa[0], oa[1], oa[2], oa[3], oa[4], oa[5], oa[6], oa[7]);
            } else {
              reinterpret_cast<uint4*>(gp)[2 * i] = make_uint4(og[0], og[1], og[2], og[3]);
              reinterpret_cast<uint4*>(gp)[2 * i + 1] = make_uint4(og[4], og[5], og[6], og[7]);
              reinterpret_cast<uint4*>(up)[2 * i] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
              reinterpret_cast<uint4*>(up)[2 * i + 1] = make_uint4(ou[4], ou[5], ou[6], ou[7]);
              reinterpret_cast<uint4*>(ap)[2 * i] = make_uint4(oa[0], oa[1], oa[2], oa[3]);
              reinterpret_cast<uint4*>(ap)[2 * i + 1] = make_uint4(oa[4], oa[5], oa[6], oa[7]);
            }
          }
        };
        auto release1 = [&]() {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CTAS == 2) mbar_arrive_relaxed_cluster(mapa_shared(tempty_bar(acc), 0u));
            else                     mbar_arrive_relaxed(tempty_bar(acc));
          }
        };
        // gate / up chunk pairs are read one pair ahead of the stores
        uint32_t ga[32], ua[32], gb[32], ub[32];
        tmem_ld_32x32(t_row, ga);
        tmem_ld_32x32(t_row + 128, ua);
#pragma unroll 1
        for (int c = 0; c < 4; c += 2) {
          tmem_ld_fence(ga);
          tmem_ld_fence(ua);
          tmem_ld_32x32(t_row + (c + 1) * 32, gb);
          tmem_ld_32x32(t_row + 128 + (c + 1) * 32, ub);
          swiglu_chunk(c, ga, ua);
          tmem_ld_fence(gb);
          tmem_ld_fence(ub);
          if (c + 2 < 4) {
            tmem_ld_32x32(t_row + (c + 2) * 32, ga);
            tmem_ld_32x32(t_row + 128 + (c + 2) * 32, ua);
          } else {
            release1();
          }
          swiglu_chunk(c + 1, gb, ub);
        }
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
        continue;
      } else if (p.epi == 2) {
        // SwiGLU backward: v = d(act); d(gate) = v*u*s*(1+g*(1-s)), d(up) = v*g*s with s = sigmoid(g)
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n_blk * BN + c * 32;
          if (col0 >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_fence(r);
          if (!row_ok) continue;
          const __nv_bfloat16* gin = reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + static_cast<long long>(row) * p.ld_aux_in + col0;
          const __nv_bfloat16* uin = gin + p.epi_h;
          __nv_bfloat16* dg = reinterpret_cast<__nv_bfloat16*>(p.D) + static_cast<long long>(row) * p.ldd + col0;
          __nv_bfloat16* du = dg + p.epi_h;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 gv = reinterpret_cast<const uint4*>(gin)[i], uv = reinterpret_cast<const uint4*>(uin)[i];
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
            uint32_t og[4], ou[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 g = unpack_bf16(gw[q]), u = unpack_bf16(uw[q]);
              const float2 d = unpack_bf16(pack_bf16(__uint_as_float(r[8 * i + 2 * q]) * alpha,
                                                     __uint_as_float(r[8 * i + 2 * q + 1]) * alpha));
              const float s0 = 1.f / (1.f + __expf(-g.x)), s1 = 1.f / (1.f + __expf(-g.y));
              og[q] = pack_bf16(d.x * u.x * s0 * (1.f + g.x * (1.f - s0)), d.y * u.y * s1 * (1.f + g.y * (1.f - s1)));
              ou[q] = pack_bf16(d.x * g.x * s0, d.y * g.y * s1);
            }
            reinterpret_cast<uint4*>(dg)[i] = make_uint4(og[0], og[1], og[2], og[3]);
            reinterpret_cast<uint4*>(du)[i] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
          }
        }
      } else {
      float seg_dot = 0.f;
      const int cols_left = p.N - n_blk * BN;
      const int n_chunks = cols_left >= BN ? BN / 32 : (cols_left + 31) / 32;     // uniform across the warp
      // One 32-column chunk of this thread's row: scale, add C, store (and the row dots of epi 3).
      auto finish_chunk = [&](int c, const uint32_t (&r)[32]) {
        const int col0 = n_blk * BN + c * 32;
        if (p.d_tma) {                            // uniform: the whole warp stages its 32 x 32 box, one lane sends it
          const int row0 = m_blk * BM + quarter * 32;
          if (row0 >= p.M) return;
          const uint32_t buf = stg_base + ((stg_i & 1u) << 12);
          ++stg_i;
          if (lane == 0) tma_store_wait_read<1>();       // the box sent from this buffer two boxes ago has been read
          __syncwarp();
          const uint32_t row_addr = buf + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
          for (int j = 0; j < 8; ++j)                    // 128-byte swizzle: 16-byte chunk j of row r sits at j ^ (r % 8)
            st_shared_v4(row_addr + (static_cast<uint32_t>(j ^ (lane & 7)) << 4),
                         __float_as_uint(__uint_as_float(r[4 * j]) * alpha), __float_as_uint(__uint_as_float(r[4 * j + 1]) * alpha),
                         __float_as_uint(__uint_as_float(r[4 * j + 2]) * alpha), __float_as_uint(__uint_as_float(r[4 * j + 3]) * alpha));
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (p.d_tma == 1) tma_reduce_add_2d(&tmD, buf, col0, row0);
            else              tma_store_2d(&tmD, buf, col0, row0);
            tma_store_commit();
          }
          return;
        }
        if constexpr (PEER) {
          if (p.d_rows_per_rank > 0) {
            // Reduce-scatter output: two chunks (64 bf16 columns = 128 bytes per row) are staged in shared
            // memory, then eight lanes write one row's 128 contiguous bytes into slice `rank` of the
            // owner's staging buffer, so what crosses NVLink are whole lines, not 16-byte pieces.
            const int row0 = m_blk * BM + quarter * 32;
            if (row0 >= p.M) return;                       // uniform across the warp
            const uint32_t buf = stg_base + (((static_cast<uint32_t>(c) >> 1) & 1u) << 12);
            const uint32_t row_addr = buf + static_cast<uint32_t>(lane) * 128u;
            const int jb = (c & 1) * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q)
              st_shared_v4(row_addr + (static_cast<uint32_t>((jb + q) ^ (lane & 7)) << 4),
                           pack_bf16(__uint_as_float(r[8 * q]) * alpha, __uint_as_float(r[8 * q + 1]) * alpha),
                           pack_bf16(__uint_as_float(r[8 * q + 2]) * alpha, __uint_as_float(r[8 * q + 3]) * alpha),
                           pack_bf16(__uint_as_float(r[8 * q + 4]) * alpha, __uint_as_float(r[8 * q + 5]) * alpha),
                           pack_bf16(__uint_as_float(r[8 * q + 6]) * alpha, __uint_as_float(r[8 * q + 7]) * alpha));
            if (!(c & 1) && c + 1 < n_chunks) return;      // the other half of the pair follows
            __syncwarp();
            const int pair_col0 = n_blk * BN + (c & ~1) * 32;
            const int valid = min(64, p.N - pair_col0);    // existing columns of this pair (a multiple of 8)
            const int owner = row0 / p.d_rows_per_rank;
            __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.d_peer[owner]) +
                                  (static_cast<long long>(p.rank) * p.d_rows_per_rank + (row0 - owner * p.d_rows_per_rank)) * p.ldd +
                                  pair_col0;
            const int j = lane & 7, rsub = lane >> 3;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + rsub;
              if (row0 + rr < p.M && j * 8 < valid) {
                const uint4 val = ld_shared_v4(buf + static_cast<uint32_t>(rr) * 128u + (static_cast<uint32_t>(j ^ (rr & 7)) << 4));
                *reinterpret_cast<uint4*>(base + static_cast<long long>(rr) * p.ldd + j * 8) = val;
              }
            }
            __syncwarp();
            return;
          }
        }
        if (!row_ok) return;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
        const bool full = col0 + 32 <= p.N;
        if (p.epi == 3) {
          // dot of this chunk (as it will be stored, rounded to bf16) with the same chunk of aux_in
          const __nv_bfloat16* sp = reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + static_cast<long long>(row) * p.ld_aux_in + col0;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 sv = reinterpret_cast<const uint4*>(sp)[i];
            const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 a = unpack_bf16(sw[q]);
              const float2 d = unpack_bf16(pack_bf16(v[8 * i + 2 * q], v[8 * i + 2 * q + 1]));
              seg_dot += a.x * d.x + a.y * d.y;
            }
          }
          if (((col0 + 32) % p.seg) == 0) {
            const int g = (col0 + 32) / p.seg - 1;          // column group; ld_aux_out = number of groups
            long long at = static_cast<long long>(row) * p.ld_aux_out + g;
            if (p.epi_h > 0) {                             // rows are (batch, t) with t < epi_h: store as [batch, group, t]
              const int bb = row / p.epi_h, tt = row - bb * p.epi_h;
              at = (static_cast<long long>(bb) * p.ld_aux_out + g) * p.epi_h + tt;
            }
            reinterpret_cast<float*>(p.aux_out)[at] = seg_dot;
            seg_dot = 0.f;
          }
        }
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
          } else if (full && wide_d) {
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
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col0 + i < p.N) dp[i] = v[i];
          }
        } else {
          __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + ti.d_off + static_cast<long long>(row) * p.ldd + col0;
          const bool wide = wide_d;
          if (full && wide) {                     // one 32-byte sector per store
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
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (col0 + i < p.N) dp[i] = __float2bfloat16(v[i]);
          }
        }
      };
      // The accumulator is read two chunks ahead of the stores; the MMA warp gets it back as soon as the
      // last chunk is in registers.
      auto release_acc = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTAS == 2) mbar_arrive_relaxed_cluster(mapa_shared(tempty_bar(acc), 0u));
          else                     mbar_arrive_relaxed(tempty_bar(acc));
        }
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
      continue;
      }   // generic epilogue
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 2) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0u));
        else                     mbar_arrive(tempty_bar(acc));
      }
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (p.d_tma && lane == 0) tma_store_wait_all<0>();   // every box has been written before this CTA leaves
  }

  tc_fence_before();
  if constexpr (CTAS == 2) {
    // Neither CTA leaves (or frees TMEM) while the other may still read its shared memory, write its
    // TMEM or signal its barriers: every role of both CTAs has left its loop when this barrier opens.
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) {
      tc_fence_after();
      tmem_dealloc_pair<2 * BN>(tmem_base);
    }
  } else {
    __syncthreads();
    if (warp == 1) {
      tc_fence_after();
      tmem_dealloc<2 * BN>(tmem_base);
    }
  }
}

// ------------------------------------------------------------------------------------ host side
template <int BN, int STAGES, bool A_MN, bool B_MN, bool PEER, int CTAS = 1>
static cudaError_t launch_cfg(const MapSet<PEER>& ta, const MapSet<PEER>& tb, const CUtensorMap& td,
                              const GemmParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, PEER, CTAS>;
  static bool attr_set = false;
  constexpr int smem = GemmSmem<BN, STAGES, CTAS>::TOTAL;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  if constexpr (CTAS == 2)
    return launch_pdl_cluster(kern, dim3(grid), dim3(GEMM_THREADS), smem, 2, stream, ta, tb, td, p);
  return launch_pdl(kern, dim3(grid), dim3(GEMM_THREADS + (PEER ? GATHER_THREADS : 0)), smem, stream, ta, tb, td, p);
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
  int row_align = 128;           // mode 1: every group starts on a multiple of this many rows (256: CTA pairs may serve it)
  long long group_stride_b = 0;  // elements between the B matrices of consecutive groups (mode 1)
  long long group_stride_d = 0;  // elements between the D (and C) matrices of consecutive groups (mode 2)
};

// Fused epilogues (see GemmParams::epi).
struct EpiSpec {
  int epi = 0, h = 0, seg = 0;
  const void* aux_in = nullptr;
  long long ld_aux_in = 0;
  void* aux_out = nullptr;
  long long ld_aux_out = 0;
};

// Operands / output spread over the ranks of one NVSwitch domain (see GemmParams).
struct PeerSpec {
  int rank = 0, world = 1;
  int gather = 0;                        // 0 none, 1 operand A, 2 operand B (MN-major only)
  const void* const* gather_ptrs = nullptr;   // rank r's full-size buffer of the gathered operand, as mapped here
  int* ready = nullptr;                  // one counter per 128-row block of the gathered operand
  void* const* d_ptrs = nullptr;         // bf16 staging buffers [world, rows / world, N] (null: D is local)
  const uint32_t* flags = nullptr;       // this rank's flag words
  int slot = -1;
  uint32_t epoch = 0;
  unsigned long long timeout_ns = 2000000000ull;
};
}  // namespace fmb

static int run_gemm(const void* A, const void* B, void* D, const void* C, int M, int N, int K, int a_mn,
                    int b_mn, long long lda, long long ldb, long long ldd, long long ldc, int d_f32,
                    int c_f32, float alpha, float beta, const float* alpha_ptr, int allow_split, int* status,
                    int force_bn, const fmb::GroupSpec& gs, cudaStream_t stream,
                    const fmb::PeerSpec* ps = nullptr, const fmb::EpiSpec* es = nullptr) {
  using namespace fmb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (gs.mode != 0 || ps != nullptr) allow_split = 0;
  if (es != nullptr && es->epi != 0) {
    if (gs.mode != 0 || ps != nullptr || C != nullptr) return -2;
    allow_split = 0;
    force_bn = 256;
    if (es->epi == 1 && (b_mn || d_f32 || es->h <= 0 || es->h % 128 || N != 2 * es->h || es->aux_out == nullptr ||
                         (es->ld_aux_out % 8) || (reinterpret_cast<uintptr_t>(es->aux_out) & 15)))
      return -2;
    if (es->epi == 2 && (d_f32 || es->h <= 0 || es->h % 32 || N != es->h || es->aux_in == nullptr ||
                         (es->ld_aux_in % 8) || (reinterpret_cast<uintptr_t>(es->aux_in) & 15)))
      return -2;
    if (es->epi == 3 && (es->seg <= 0 || es->seg % 32 || 256 % es->seg || N % es->seg || es->aux_in == nullptr ||
                         es->aux_out == nullptr || (es->ld_aux_in % 8) || (reinterpret_cast<uintptr_t>(es->aux_in) & 15)))
      return -2;
    if (es->epi < 1 || es->epi > 3) return -2;
  }
  int g_rows = 0, g_rps = 0;
  if (ps != nullptr) {
    if (gs.mode != 0 || ps->world < 1 || ps->world > FMB_MAX_PEERS || ps->rank < 0 || ps->rank >= ps->world) return -2;
    if (ps->gather == 1) g_rows = a_mn ? K : M;
    else if (ps->gather == 2) { if (!b_mn) return -2; g_rows = K; }
    else if (ps->gather != 0) return -2;
    if (ps->gather) {
      if (ps->gather_ptrs == nullptr || ps->ready == nullptr || g_rows % (128 * ps->world)) return -2;
      g_rps = g_rows / ps->world;
      if (ps->slot >= 0 && ps->flags == nullptr) return -2;
    }
    if (ps->d_ptrs != nullptr && (d_f32 || C != nullptr || M % (128 * ps->world))) return -2;
  }
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(D) & 15) || (ldd % (d_f32 ? 4 : 8)))
    return -2;   // TMA needs 16-byte aligned bases and pitches; the vector epilogue needs an aligned D
  if (C != nullptr && ((reinterpret_cast<uintptr_t>(C) & 15) || (ldc % (c_f32 ? 4 : 8)))) return -2;
  const int sms = sm_count();
  const int kblocks = (K + GEMM_BK - 1) / GEMM_BK;
  const bool can_split = allow_split && d_f32 && (C == nullptr || C == D);
  // CTA pairs (256-row tiles over two SMs) serve plain products; FMB_GEMM_PAIR=0 turns them off.
  static const bool pair_env = [] { const char* v = getenv("FMB_GEMM_PAIR"); return v == nullptr || v[0] != '0'; }();
  static const bool gpair_env = [] { const char* v = getenv("FMB_GEMM_GROUP_PAIR"); return v == nullptr || v[0] != '0'; }();
  const bool rows_pair = gs.mode == 1 && gpair_env && gs.row_align % 256 == 0 && M % 256 == 0;
  const bool out_pair = gs.mode == 2 && gpair_env;          // one output per group: tiles are ordinary M x N tiles
  const bool pair_ok = pair_env && (ps == nullptr || ps->gather == 0) && (gs.mode == 0 || rows_pair || out_pair) &&
                       sms % 2 == 0;

  // Pick the N tile, the split count and the CTAs per tile that fill the machine best.
  int best_bn = 256, best_split = 1, best_ctas = 1;
  double best_score = -1.0;
  for (int ctas : {2, 1}) {
    if (ctas == 2 && !pair_ok) continue;
    const int tm = (M + GEMM_BM * ctas - 1) / (GEMM_BM * ctas);
    const double pad_m = static_cast<double>(M) / (static_cast<double>(tm) * GEMM_BM * ctas);
    for (int bn : {256, 128, 64}) {
      if (force_bn && bn != force_bn) continue;
      if (bn == 64 && (gs.mode != 0 || ps != nullptr || ctas == 2)) continue;   // narrow tiles: small plain products only
      const int tn = (N + bn - 1) / bn;
      const long long tiles = static_cast<long long>(tm) * tn;
      const int max_split = can_split ? 8 : 1;
      for (int s = 1; s <= max_split; ++s) {
        if (s > 1 && (kblocks / s) < 8) break;            // keep each split's K loop long enough
        double score = wave_eff(tiles * s, sms / ctas);
        score *= (bn == 256 ? 1.0 : bn == 128 ? 0.93 : 0.80);   // narrower tiles re-read A more often
        score *= 1.0 - 0.015 * (s - 1);                   // atomics and extra epilogues are not free
        score *= static_cast<double>(N) / (static_cast<double>(tn) * bn);
        score *= pad_m * (ctas == 2 ? 1.12 : 1.0);        // a pair reads half the B tile per SM
        if (score > best_score) { best_score = score; best_bn = bn; best_split = s; best_ctas = ctas; }
      }
    }
  }
  const int tiles_m = (M + GEMM_BM * best_ctas - 1) / (GEMM_BM * best_ctas);
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
  p.tg_step = best_ctas;
  p.tile_group = gs.tile_group;
  p.region = gs.region;
  p.group_stride_d = gs.group_stride_d;
  p.rank = 0; p.world = 1;
  p.gather = 0; p.g_rows_per_src = 0; p.g_ld = 0; p.g_row_bytes = 0; p.g_local = nullptr; p.g_ready = nullptr;
  p.flags = nullptr; p.g_slot = -1; p.g_epoch = 0; p.timeout_ns = 0;
  p.own_m_tiles = 0; p.d_rows_per_rank = 0;
  p.rot_m = p.rot_k = 0;
  for (int r = 0; r < FMB_MAX_PEERS; ++r) { p.d_peer[r] = nullptr; p.g_src[r] = nullptr; }
  if (ps != nullptr) {
    p.rank = ps->rank; p.world = ps->world;
    p.flags = ps->flags; p.g_slot = ps->slot; p.g_epoch = ps->epoch; p.timeout_ns = ps->timeout_ns;
    if (ps->gather) {
      const bool on_a = ps->gather == 1;
      p.gather = ps->gather;
      p.g_rows_per_src = g_rps;
      p.g_ld = on_a ? lda : ldb;
      p.g_row_bytes = 2 * (on_a ? (a_mn ? M : K) : N);
      if (p.g_row_bytes % 16) return -2;
      p.g_local = const_cast<void*>(on_a ? A : B);
      p.g_ready = ps->ready;
      for (int r = 0; r < ps->world; ++r) {
        if (ps->gather_ptrs[r] == nullptr || (reinterpret_cast<uintptr_t>(ps->gather_ptrs[r]) & 15)) return -2;
        p.g_src[r] = ps->gather_ptrs[r];
      }
      if (cudaMemsetAsync(ps->ready, 0, sizeof(int) * static_cast<size_t>(g_rows / 128), stream) != cudaSuccess) return -3;
      if (on_a && !a_mn) {              // row tiles: own rows first
        p.own_m_tiles = g_rps / GEMM_BM;
        p.rot_m = ps->rank * p.own_m_tiles;
      } else {                          // reduction blocks: start with the own ones
        p.rot_k = ps->rank * (g_rps / GEMM_BK);
      }
    }
    if (ps->d_ptrs != nullptr) {
      p.d_rows_per_rank = M / ps->world;
      for (int r = 0; r < ps->world; ++r) p.d_peer[r] = ps->d_ptrs[r];
      if (p.rot_m == 0 && p.own_m_tiles == 0 && p.d_rows_per_rank % (GEMM_BM * best_ctas) == 0)
        p.rot_m = ((ps->rank + 1) % ps->world) * (p.d_rows_per_rank / (GEMM_BM * best_ctas));   // remote rows first
    }
  }
  p.epi = 0; p.epi_h = 0; p.seg = 0;
  p.aux_in = nullptr; p.ld_aux_in = 0; p.aux_out = nullptr; p.ld_aux_out = 0;
  if (es != nullptr && es->epi != 0) {
    p.epi = es->epi; p.epi_h = es->h; p.seg = es->seg;
    p.aux_in = es->aux_in; p.ld_aux_in = es->ld_aux_in;
    p.aux_out = es->aux_out; p.ld_aux_out = es->ld_aux_out;
    if (es->epi == 1) p.tiles_n = es->h / 128;          // a tile = 128 hidden units = 128 gate + 128 up columns
  }
  if (splits > 1) {
    // Every split adds alpha*partial into D, which already holds the C term (C == D) or zeros.
    if (C == D && beta == 1.f) { p.C = nullptr; }
    else if (C == nullptr) { if (cudaMemsetAsync(D, 0, sizeof(float) * static_cast<size_t>(M) * ldd, stream) != cudaSuccess) return -3; }
    else return -4;
  }
  // Tile order. CTAs that run at the same time should share operand tiles, and an operand larger than the
  // L2 should be streamed from memory once: estimate the traffic of both orders and take the smaller.
  p.n_fast = 0;
  if (gs.mode == 0 && ps == nullptr) {
    const double l2_budget = 64.0 * (1 << 20);
    const double a_bytes = 2.0 * M * K, b_bytes = 2.0 * N * K;
    const int units_c = sms / best_ctas;
    const int tm_c = p.tiles_m, tn_c = p.tiles_n;
    auto passes = [&](int tiles_fast, int tiles_slow) {      // how often the operand of the fast dimension is streamed
      const int slow_per_wave = units_c / tiles_fast > 1 ? units_c / tiles_fast : 1;
      return (tiles_slow + slow_per_wave - 1) / slow_per_wave;
    };
    const double cost_m = (a_bytes > l2_budget ? a_bytes * passes(tm_c, tn_c) : a_bytes) + b_bytes;
    const double cost_n = (b_bytes > l2_budget ? b_bytes * passes(tn_c, tm_c) : b_bytes) + a_bytes;
    if (cost_n < 0.9 * cost_m) p.n_fast = 1;
  }
  // Plain fp32 outputs leave through TMA boxes (whole 128-byte lines, no per-thread scattered stores).
  static const bool dtma_env = [] { const char* v = getenv("FMB_GEMM_DTMA"); return v == nullptr || v[0] != '0'; }();
  p.d_tma = 0;
  CUtensorMap td;
  memset(&td, 0, sizeof(td));
  if (dtma_env && d_f32 && gs.mode == 0 && ps == nullptr && p.epi == 0) {
    const int want = (splits > 1 || (C == D && beta == 1.f)) ? 1 : (C == nullptr || beta == 0.f) ? 2 : 0;
    // an output that the driver refuses to describe (unusual pitch or extent) keeps the register path
    if (want && make_tmap_2d(&td, D, M, N, ldd, 32, 32, 4, TmapSwizzle::B128)) {
      p.d_tma = want;
      if (want == 1) { p.C = nullptr; p.atomic = 0; }
    }
  }

  MapSet<true> ta, tb;
  bool ok = true;
  if (!a_mn) ok = make_tmap_2d(&ta.m[0], A, M, K, lda, GEMM_BM, GEMM_BK, 2, TmapSwizzle::B128);
  else       ok = make_tmap_2d(&ta.m[0], A, K, M, lda, GEMM_BK, 64, 2, TmapSwizzle::B128);
  if (ok) {
    // B is always described by a 3-D map (inner, rows, group); plain products have one group.
    const int nb = gs.mode == 1 ? gs.n_groups : 1;
    const uint64_t gstride = gs.mode == 1 ? static_cast<uint64_t>(gs.group_stride_b)
                                          : static_cast<uint64_t>(b_mn ? K : N) * static_cast<uint64_t>(ldb);
    uint64_t dims[3], strides[3];
    uint32_t box[3];
    if (!b_mn) { dims[0] = K; dims[1] = N; box[0] = GEMM_BK; box[1] = (p.epi == 1) ? 128 : best_bn / best_ctas; }
    else       { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = GEMM_BK; }
    dims[2] = nb; box[2] = 1;
    strides[0] = 2; strides[1] = static_cast<uint64_t>(ldb) * 2; strides[2] = gstride * 2;
    ok = make_tmap_nd(&tb.m[0], B, 3, dims, strides, box, 2, TmapSwizzle::B128);
  }
  if (!ok) return -5;

  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * (gs.mode == 2 ? gs.n_groups : p.splits);
  const int units = sms / best_ctas;
  const int grid = best_ctas * static_cast<int>(total < units ? total : units);
  cudaError_t e;
  if (best_ctas == 2 && ps != nullptr) {
#define FMB_DISPATCH(BN, ST)                                                                         \
  if (a_mn && b_mn)       e = launch_cfg<BN, ST, true, true, true, 2>(ta, tb, td, p, grid, stream);   \
  else if (a_mn)          e = launch_cfg<BN, ST, true, false, true, 2>(ta, tb, td, p, grid, stream);  \
  else if (b_mn)          e = launch_cfg<BN, ST, false, true, true, 2>(ta, tb, td, p, grid, stream);  \
  else                    e = launch_cfg<BN, ST, false, false, true, 2>(ta, tb, td, p, grid, stream);
    if (best_bn == 256) { FMB_DISPATCH(256, 6) } else { FMB_DISPATCH(128, 8) }
#undef FMB_DISPATCH
  } else if (best_ctas == 2) {
    MapSet<false> sa, sb;
    sa.m[0] = ta.m[0];
    sb.m[0] = tb.m[0];
#define FMB_DISPATCH(BN, ST)                                                                         \
  if (a_mn && b_mn)       e = launch_cfg<BN, ST, true, true, false, 2>(sa, sb, td, p, grid, stream);      \
  else if (a_mn)          e = launch_cfg<BN, ST, true, false, false, 2>(sa, sb, td, p, grid, stream);     \
  else if (b_mn)          e = launch_cfg<BN, ST, false, true, false, 2>(sa, sb, td, p, grid, stream);     \
  else                    e = launch_cfg<BN, ST, false, false, false, 2>(sa, sb, td, p, grid, stream);
    if (best_bn == 256) { FMB_DISPATCH(256, 6) } else { FMB_DISPATCH(128, 8) }
#undef FMB_DISPATCH
  } else if (ps != nullptr) {
#define FMB_DISPATCH(BN, ST)                                                                         \
  if (a_mn && b_mn)       e = launch_cfg<BN, ST, true, true, true>(ta, tb, td, p, grid, stream);          \
  else if (a_mn)          e = launch_cfg<BN, ST, true, false, true>(ta, tb, td, p, grid, stream);         \
  else if (b_mn)          e = launch_cfg<BN, ST, false, true, true>(ta, tb, td, p, grid, stream);         \
  else                    e = launch_cfg<BN, ST, false, false, true>(ta, tb, td, p, grid, stream);
    if (best_bn == 256) { FMB_DISPATCH(256, 4) } else { FMB_DISPATCH(128, 6) }
#undef FMB_DISPATCH
  } else {
    MapSet<false> sa, sb;
    sa.m[0] = ta.m[0];
    sb.m[0] = tb.m[0];
#define FMB_DISPATCH(BN, ST)                                                                         \
  if (a_mn && b_mn)       e = launch_cfg<BN, ST, true, true, false>(sa, sb, td, p, grid, stream);         \
  else if (a_mn)          e = launch_cfg<BN, ST, true, false, false>(sa, sb, td, p, grid, stream);        \
  else if (b_mn)          e = launch_cfg<BN, ST, false, true, false>(sa, sb, td, p, grid, stream);        \
  else                    e = launch_cfg<BN, ST, false, false, false>(sa, sb, td, p, grid, stream);
    if (best_bn == 256) { FMB_DISPATCH(256, 4) } else if (best_bn == 128) { FMB_DISPATCH(128, 6) } else { FMB_DISPATCH(64, 8) }
#undef FMB_DISPATCH
  }
  return e == cudaSuccess ? 0 : -10 - static_cast<int>(e);
}

FMB_DEBUG_BIND(gemm)

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
  if (mode == 3) { mode = 1; gs.row_align = 256; }      // mode 1 whose groups all start on multiples of 256 rows
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

// Products whose operands or output are spread over the ranks of one NVSwitch domain.
//   gather        1: A, 2: B (MN-major) is the operand whose rows are spread over the ranks; A / B then points to
//                 THIS rank's full-size symmetric buffer, of which only the own rows need to be filled in
//   gather_ptrs   `world` device pointers: rank r's buffer as mapped into this process
//   ready         int counters, one per 128 rows of the gathered operand (cleared here)
//   d_ptrs        bf16 staging buffers [world, M / world, N] of every rank (null: D is an ordinary local output)
//   flags         this rank's flag words; rank r's rows are copied once flags[slot * 8 + r] reached epoch
extern "C" int fmb_gemm_bf16_peer(const void* A, const void* B, void* D, int M, int N, int K, int a_mn, int b_mn,
                                  long long lda, long long ldb, long long ldd, int d_f32, float alpha, int accumulate,
                                  int rank, int world, int gather, const void* const* gather_ptrs, int* ready,
                                  void* const* d_ptrs, const unsigned* flags, int slot, unsigned epoch,
                                  unsigned long long timeout_ns, int* status, cudaStream_t stream) {
  fmb::GroupSpec gs;
  fmb::PeerSpec ps;
  ps.rank = rank; ps.world = world;
  ps.gather = gather; ps.gather_ptrs = gather_ptrs; ps.ready = ready;
  ps.d_ptrs = d_ptrs;
  ps.flags = flags; ps.slot = slot; ps.epoch = epoch;
  ps.timeout_ns = timeout_ns;
  const bool acc = accumulate && d_ptrs == nullptr;      // D += product (local output only)
  return run_gemm(A, B, D, acc ? D : nullptr, M, N, K, a_mn, b_mn, lda, ldb, ldd, acc ? ldd : 0, d_f32,
                  acc ? d_f32 : 0, alpha, acc ? 1.f : 0.f, nullptr, 0, status, 0, gs, stream, &ps);
}

// Plain product with a fused epilogue (GemmParams::epi): 1 SwiGLU forward (N = 2h), 2 SwiGLU backward
// (N = h, D is [M, 2h]), 3 row dots against aux_in over seg-wide column groups.
extern "C" int fmb_gemm_bf16_epi(const void* A, const void* B, void* D, int M, int N, int K, int a_mn, int b_mn,
                                 long long lda, long long ldb, long long ldd, int d_f32, float alpha, int epi, int h,
                                 int seg, const void* aux_in, long long ld_aux_in, void* aux_out, long long ld_aux_out,
                                 int* status, cudaStream_t stream) {
  fmb::GroupSpec gs;
  fmb::EpiSpec es;
  es.epi = epi; es.h = h; es.seg = seg;
  es.aux_in = aux_in; es.ld_aux_in = ld_aux_in;
  es.aux_out = aux_out; es.ld_aux_out = ld_aux_out;
  return run_gemm(A, B, D, nullptr, M, N, K, a_mn, b_mn, lda, ldb, ldd, 0, d_f32, 0, alpha, 0.f, nullptr, 0, status, 256,
                  gs, stream, nullptr, &es);
}
