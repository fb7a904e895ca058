// Causal grouped-query attention, backward pass, on the 5th-generation tensor cores.
//
// One CTA owns one (batch, kv head, 128-key block) and walks over every query head of the
// group and every 64-query tile that can see the block.  Scores are formed transposed, keys on
// the TMEM lanes and queries on the columns, so every MMA has M = 128:
//
//   S^T  = K  Q^T            [keys x q]      A = K   (K-major)      B = Q   (K-major)
//   dP^T = V  dO^T           [keys x q]      A = V   (K-major)      B = dO  (K-major)
//   P^T  = exp2(c S^T - lse),  dS^T = scale * P^T (dP^T - delta)     (softmax warps)
//   dV  += P^T  dO           [keys x d]      A = P^T (K-major)      B = dO  (MN-major)
//   dK  += dS^T Q            [keys x d]      A = dS^T (K-major)     B = Q   (MN-major)
//   dQ^T = K^T  dS^T         [d x q]         A = K   (MN-major)     B = dS^T (MN-major)
//
// P^T and dS^T go back, as packed bf16, into the TMEM columns their scores came from and are the
// A operands of the dV and dK MMAs straight from tensor memory; dS^T is also written to shared
// memory (128-byte swizzle) as the MN-major B operand of the dQ^T MMA.  dK and dV stay in TMEM for the
// whole CTA; dQ^T is drained every tile and added to an fp32 accumulator in global memory with
// coalesced reductions (one query row, 32 consecutive head-dim elements per warp instruction).
//
// Warps: 0 = TMA (K, V once; Q, dO, lse, delta per tile, 3 stages), 1 = MMA issue, 2..17 =
// softmax and the final dK, dV store, 18..21 = dQ drain (so that the reductions of tile t-1 run
// beside the softmax of tile t).  The tail MMAs of tile t-1 are issued after S and dP
// of tile t, so the tensor cores work under the softmax of tile t.  All waits are bounded.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

#include "ftb200_common.cuh"
#include "tcgen05_helpers.cuh"

namespace {

using namespace ftb200::tc;

// Optional event trace for tuning (compiled in with -DFTB200_ATTN_TRACE): CTA 0 records clock64()
// at pipeline events of its first tiles into p.trace[role][tile][event].
#ifdef FTB200_ATTN_TRACE
#define TRACE(role, tile, ev)                                                                       \
  do {                                                                                              \
    if (p.trace != nullptr && blockIdx.x == 0 && (tile) < 32)                                       \
      p.trace[((role) * 32 + (tile)) * 8 + (ev)] = clock64();                                       \
  } while (0)
#else
#define TRACE(role, tile, ev) \
  do {                        \
  } while (0)
#endif

constexpr int BKV = 128;
constexpr int BQ = 64;
constexpr int NUM_THREADS = 704;
constexpr int SOFTMAX_THREADS = 512;
constexpr int DRAIN_THREADS = 128;
constexpr int GROUPS = 4;          // threads per key row
constexpr int CPT = BQ / GROUPS;   // query columns per thread
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DQ = 192, COL_DV = 256, COL_DK = 384;
constexpr uint32_t KV_SLAB = BKV * 128;        // 16 KB: [128 rows x 128 B], 64 head-dim elements per row
constexpr uint32_t Q_SLAB = BQ * 128;          // 8 KB: [64 rows x 128 B]
constexpr uint32_t PT_TILE = BKV * BQ * 2;     // 16 KB, one slab of [128 key rows x 64 q]
constexpr int QDO_STAGES = 3;  // a stage is held until the tile's dV/dK MMAs are done, two tiles after its load began
constexpr uint32_t PDS_BYTES = PT_TILE;        // dS^T only: P^T never leaves tensor memory
constexpr uint32_t STATS_BYTES = 2 * BQ * 4;   // per stage: lse[64], delta[64]

// Shared-memory layout for head dim D (64 or 128): K and V tiles of D/64 slabs each, then the Q/dO stages, the
// dS^T buffers, the statistics and the barriers.
template <int D>
struct Lay {
  static constexpr int SLABS = D / 64;
  static constexpr uint32_t KV_TILE = SLABS * KV_SLAB;
  static constexpr uint32_t Q_TILE = SLABS * Q_SLAB;
  static constexpr uint32_t OFF_K = 0, OFF_V = KV_TILE;
  static constexpr uint32_t OFF_STAGE = 2 * KV_TILE;    // per stage: Q, dO
  static constexpr uint32_t STAGE_BYTES = 2 * Q_TILE;
  static constexpr uint32_t OFF_PDS = OFF_STAGE + QDO_STAGES * STAGE_BYTES;  // per buffer: dS^T
  static constexpr uint32_t OFF_STATS = OFF_PDS + 2 * PDS_BYTES;
  static constexpr uint32_t OFF_MISC = OFF_STATS + QDO_STAGES * STATS_BYTES;
  static constexpr uint32_t SMEM_BYTES = OFF_MISC + 256 + 1024;
  static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

enum : int {
  BAR_KV = 0,
  BAR_QDO_FULL = 1,   // +stage (3)
  BAR_QDO_EMPTY = 4,  // +stage (3)
  BAR_S_FULL = 7,     // +buf
  BAR_S_EMPTY = 9,    // +buf
  BAR_DP_FULL = 11,
  BAR_DP_EMPTY = 12,
  BAR_PDS_FULL = 13,  // +buf
  BAR_PDS_EMPTY = 15, // +buf
  BAR_DQ_FULL = 17,
  BAR_DQ_EMPTY = 18,
  BAR_DKV_DONE = 19,
  NUM_BARS = 20,
};

struct BwdParams {
  int batch, seq, n_heads, n_kv_heads;
  int causal;
  float scale, scale_log2;
  const float* lse;    // [batch, n_heads, seq], natural log
  const float* delta;  // [batch, n_heads, seq]
  float* dq_acc;       // [batch*seq, n_heads*128] fp32, zeroed by the caller
  __nv_bfloat16* dK;   // rows batch*seq, row stride ld_dk
  __nv_bfloat16* dV;
  long long ld_dk, ld_dv;
  int* status;
  long long* trace;  // tuning aid, null unless built with FTB200_ATTN_TRACE
};

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const BwdParams p) {
  using Ly = Lay<D>;
  constexpr int SLABS = Ly::SLABS;
  constexpr uint32_t KV_TILE = Ly::KV_TILE, Q_TILE = Ly::Q_TILE, OFF_K = Ly::OFF_K, OFF_V = Ly::OFF_V;
  constexpr uint32_t OFF_STAGE = Ly::OFF_STAGE, STAGE_BYTES = Ly::STAGE_BYTES, OFF_PDS = Ly::OFF_PDS;
  constexpr uint32_t OFF_STATS = Ly::OFF_STATS, OFF_MISC = Ly::OFF_MISC;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_MISC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 196);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto bar = [&](int i) { return bar_base + 8u * i; };

  // early key blocks see the most queries under a causal mask: schedule them first
  const int per_block = p.batch * p.n_kv_heads;
  const int jb = static_cast<int>(blockIdx.x) / per_block;
  const int bh = static_cast<int>(blockIdx.x) % per_block;
  const int b = bh / p.n_kv_heads, hk = bh % p.n_kv_heads;
  const int rep = p.n_heads / p.n_kv_heads;
  const int n_qtiles = p.seq / BQ;
  const int first_q = (p.causal & 1) ? (jb * BKV) / BQ : 0;
  const int tiles_per_head = n_qtiles - first_q;
  const int T = rep * tiles_per_head;
  const int kv_row0 = b * p.seq + jb * BKV;
  auto tile_of = [&](int t, int& h, int& qt) {
    h = hk * rep + t / tiles_per_head;
    qt = first_q + t % tiles_per_head;
  };

  if (threadIdx.x == 0) {
    mbar_init(bar(BAR_KV), 1);
    for (int s = 0; s < QDO_STAGES; ++s) {
      mbar_init(bar(BAR_QDO_FULL + s), 1);
      mbar_init(bar(BAR_QDO_EMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(BAR_S_FULL + s), 1);
      mbar_init(bar(BAR_S_EMPTY + s), SOFTMAX_THREADS);
      mbar_init(bar(BAR_PDS_FULL + s), SOFTMAX_THREADS);
      mbar_init(bar(BAR_PDS_EMPTY + s), 1);
    }
    mbar_init(bar(BAR_DP_FULL), 1);
    mbar_init(bar(BAR_DP_EMPTY), SOFTMAX_THREADS);
    mbar_init(bar(BAR_DQ_FULL), 1);
    mbar_init(bar(BAR_DQ_EMPTY), DRAIN_THREADS);
    mbar_init(bar(BAR_DKV_DONE), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_expect_tx(bar(BAR_KV), 2 * KV_TILE);
#pragma unroll
      for (int sl = 0; sl < SLABS; ++sl) {
        tma_load_2d(smem_base + OFF_K + sl * KV_SLAB, &tmK, bar(BAR_KV), hk * D + 64 * sl, kv_row0);
        tma_load_2d(smem_base + OFF_V + sl * KV_SLAB, &tmV, bar(BAR_KV), hk * D + 64 * sl, kv_row0);
      }
      bool ok = true;
      for (int t = 0; t < T && ok; ++t) {
        const int st = t % QDO_STAGES;
        const uint32_t use = static_cast<uint32_t>(t / QDO_STAGES);
        if (!mbar_wait(bar(BAR_QDO_EMPTY + st), (use & 1u) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        int h, qt;
        tile_of(t, h, qt);
        const int q_row0 = b * p.seq + qt * BQ;
        const uint32_t sq = smem_base + OFF_STAGE + st * STAGE_BYTES;
        const uint32_t sdo = sq + Q_TILE;
        const uint32_t sst = smem_base + OFF_STATS + st * STATS_BYTES;
        const long long stat_off = (static_cast<long long>(b) * p.n_heads + h) * p.seq + qt * BQ;
        mbar_expect_tx(bar(BAR_QDO_FULL + st), 2 * Q_TILE + STATS_BYTES);
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          tma_load_2d(sq + sl * Q_SLAB, &tmQ, bar(BAR_QDO_FULL + st), h * D + 64 * sl, q_row0);
          tma_load_2d(sdo + sl * Q_SLAB, &tmDO, bar(BAR_QDO_FULL + st), h * D + 64 * sl, q_row0);
        }
        bulk_load_1d(sst, p.lse + stat_off, BQ * 4, bar(BAR_QDO_FULL + st));
        bulk_load_1d(sst + BQ * 4, p.delta + stat_off, BQ * 4, bar(BAR_QDO_FULL + st));
      }
      if (!ok) {
        const uint64_t t0 = ftb200::globaltimer_ns();
        while (ftb200::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t F = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(128 >> 4) << 24);
      const uint32_t idesc_st = F | (static_cast<uint32_t>(BQ >> 3) << 17);                             // N = 64, K-major both
      const uint32_t idesc_kv = F | (1u << 16) | (static_cast<uint32_t>(D >> 3) << 17);                 // N = D, B MN-major
      const uint32_t idesc_dq = F | (1u << 15) | (1u << 16) | (static_cast<uint32_t>(BQ >> 3) << 17);   // N = 64, both MN-major
      // descriptor bases: one per buffer and operand role, constants per K step (the issue loop
      // must stay short: these MMAs are too small to hide descriptor arithmetic)
      constexpr uint32_t HI = smem_desc_hi(1024);
      const uint32_t k_km = smem_desc_lo(smem_base + OFF_K, 16);        // K as K-major A (S^T)
      const uint32_t v_km = smem_desc_lo(smem_base + OFF_V, 16);        // V as K-major A (dP^T)
      // K as MN-major A (dQ^T): M = 128 runs over the head dim.  With head dim 64 the second 64 rows of that MMA
      // read the slab behind K's only one, which is V's: lanes 64..127 of dQ^T then hold a product nobody reads.
      const uint32_t k_mn = smem_desc_lo(smem_base + OFF_K, KV_SLAB);
      const uint32_t q_km0 = smem_desc_lo(smem_base + OFF_STAGE, 16);             // Q, stage 0, K-major B
      const uint32_t q_mn0 = smem_desc_lo(smem_base + OFF_STAGE, Q_SLAB);         // Q, stage 0, MN-major B
      const uint32_t ds_mn0 = smem_desc_lo(smem_base + OFF_PDS, PT_TILE);  // dS^T, buffer 0, MN-major B
      constexpr uint32_t STAGE16 = STAGE_BYTES >> 4, QT16 = Q_TILE >> 4, PDS16 = PDS_BYTES >> 4;
      bool ok = mbar_wait(bar(BAR_KV), 0, abort_flag);
      for (int t = 0; t <= T && ok; ++t) {
        if (t < T) {
          const int st = t & 1, qs = t % QDO_STAGES;
          const uint32_t use = static_cast<uint32_t>(t >> 1);
          if (!mbar_wait(bar(BAR_QDO_FULL + qs), static_cast<uint32_t>(t / QDO_STAGES) & 1u, abort_flag) ||
              !mbar_wait(bar(BAR_S_EMPTY + st), (use & 1u) ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          TRACE(0, t, 0);  // S inputs ready
          const uint32_t qb_km = q_km0 + qs * STAGE16;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t a_off = ((kk >> 2) * KV_SLAB + (kk & 3) * 32) >> 4, b_off = ((kk >> 2) * Q_SLAB + (kk & 3) * 32) >> 4;
            umma_bf16_lh(tmem_base + COL_S + st * BQ, k_km + a_off, HI, qb_km + b_off, HI, idesc_st, kk != 0);
          }
          umma_commit(bar(BAR_S_FULL + st));
          if (!mbar_wait(bar(BAR_DP_EMPTY), (static_cast<uint32_t>(t) & 1u) ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t a_off = ((kk >> 2) * KV_SLAB + (kk & 3) * 32) >> 4, b_off = ((kk >> 2) * Q_SLAB + (kk & 3) * 32) >> 4;
            umma_bf16_lh(tmem_base + COL_DP, v_km + a_off, HI, qb_km + QT16 + b_off, HI, idesc_st, kk != 0);
          }
          umma_commit(bar(BAR_DP_FULL));
          TRACE(0, t, 1);  // S, dP issued
        }
        if (t >= 1) {
          const int u = t - 1, pb = u & 1, qs = u % QDO_STAGES;
          const uint32_t use = static_cast<uint32_t>(u >> 1);
          if (!mbar_wait(bar(BAR_PDS_FULL + pb), use & 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          TRACE(0, u, 2);  // P, dS ready for the tail of tile u
          const uint32_t qb_mn = q_mn0 + qs * STAGE16;
          const uint32_t dsb_mn = ds_mn0 + pb * PDS16;
          // queries 16k..16k+15 of tile u: P^T in columns 16k..16k+7 of its score buffer, dS^T in 16k+8..16k+15
          const uint32_t pt_tmem = tmem_base + COL_S + pb * BQ;
#pragma unroll
          for (int kk = 0; kk < BQ / 16; ++kk) {  // dV += P^T dO
            umma_bf16_tmem_a(tmem_base + COL_DV, pt_tmem + kk * 16, qb_mn + QT16 + ((kk * 2048) >> 4), HI, idesc_kv, (u | kk) != 0);
          }
#pragma unroll
          for (int kk = 0; kk < BQ / 16; ++kk) {  // dK += dS^T Q
            umma_bf16_tmem_a(tmem_base + COL_DK, pt_tmem + kk * 16 + 8, qb_mn + ((kk * 2048) >> 4), HI, idesc_kv, (u | kk) != 0);
          }
          umma_commit(bar(BAR_QDO_EMPTY + qs));
          if (!mbar_wait(bar(BAR_DQ_EMPTY), (static_cast<uint32_t>(u) & 1u) ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk) {  // dQ^T = K^T dS^T
            umma_bf16_lh(tmem_base + COL_DQ, k_mn + ((kk * 2048) >> 4), HI, dsb_mn + ((kk * 2048) >> 4), HI, idesc_dq, kk != 0);
          }
          umma_commit(bar(BAR_PDS_EMPTY + pb));
          umma_commit(bar(BAR_DQ_FULL));
          TRACE(0, u, 3);  // tail issued
        }
      }
      if (ok) umma_commit(bar(BAR_DKV_DONE));
    }
    __syncwarp();
  } else if (warp >= 18) {
    // ---------------- dQ drain (warps 18..21): TMEM lane = head-dim index ----------------
    const int quarter = warp & 3;
    const int dcol = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const long long ldq = static_cast<long long>(p.n_heads) * D;
    for (int u = 0; u < T; ++u) {
      if (!mbar_wait(bar(BAR_DQ_FULL), static_cast<uint32_t>(u) & 1u, abort_flag)) break;
      tc_fence_after();
      uint32_t v[BQ];
      const bool mine = quarter * 32 < D;  // head dim 64: only lanes 0..63 of dQ^T are real
      if (mine) {
        tmem_ld32(tmem_base + COL_DQ + lane_addr, v);
        tmem_ld32(tmem_base + COL_DQ + 32 + lane_addr, v + 32);
        tmem_wait_ld();
      }
      tc_fence_before();
      mbar_arrive(bar(BAR_DQ_EMPTY));
      int h, qt;
      tile_of(u, h, qt);
      float* dst = p.dq_acc + (static_cast<long long>(b) * p.seq + qt * BQ) * ldq + h * D + dcol;
      if (mine && !(p.causal & 2))
#pragma unroll
        for (int c = 0; c < BQ; ++c) atomicAdd(dst + c * ldq, __uint_as_float(v[c]));
    }
  } else {
    // ---------------- softmax, dK/dV store (warps 2..17) ----------------
    const int quarter = warp & 3;
    const int g = (warp - 2) >> 2;  // which 16 of the tile's 64 queries (32 of 128 columns at the end)
    const int row = quarter * 32 + lane;  // key within the block; head-dim index when draining dQ^T
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float log2e = 1.4426950408889634f;
    bool ok = true;

    for (int t = 0; t < T; ++t) {
      const int st = t & 1;
      const uint32_t use = static_cast<uint32_t>(t >> 1);
      int h, qt;
      tile_of(t, h, qt);
      if (!mbar_wait(bar(BAR_S_FULL + st), use & 1u, abort_flag) ||
          !mbar_wait(bar(BAR_DP_FULL), static_cast<uint32_t>(t) & 1u, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (threadIdx.x == 64) TRACE(1, t, 0);  // S and dP complete
      uint32_t sv[CPT], dp[CPT];
      tmem_ld16(tmem_base + COL_S + st * BQ + g * CPT + lane_addr, sv);
      tmem_ld16(tmem_base + COL_DP + g * CPT + lane_addr, dp);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar(BAR_S_EMPTY + st));
      mbar_arrive(bar(BAR_DP_EMPTY));
      if (threadIdx.x == 64) TRACE(1, t, 1);  // scores in registers
      // the tile's statistics arrived with Q and dO
      const int qs = t % QDO_STAGES;
      if (!mbar_wait(bar(BAR_QDO_FULL + qs), static_cast<uint32_t>(t / QDO_STAGES) & 1u, abort_flag)) {
        ok = false;
        break;
      }
      const float4* stats4 = reinterpret_cast<const float4*>(smem + OFF_STATS + qs * STATS_BYTES);
      float lse_q[CPT], del_q[CPT];
#pragma unroll
      for (int c = 0; c < CPT / 4; ++c) {
        const float4 a = stats4[g * (CPT / 4) + c];
        const float4 d4 = stats4[BQ / 4 + g * (CPT / 4) + c];
        lse_q[4 * c] = a.x; lse_q[4 * c + 1] = a.y; lse_q[4 * c + 2] = a.z; lse_q[4 * c + 3] = a.w;
        del_q[4 * c] = d4.x; del_q[4 * c + 1] = d4.y; del_q[4 * c + 2] = d4.z; del_q[4 * c + 3] = d4.w;
      }
      const int key = jb * BKV + row;
      const int q0 = qt * BQ + g * CPT;
      const bool diag = (p.causal & 1) && (q0 < jb * BKV + BKV);
      uint32_t pk[CPT / 2], dk[CPT / 2];
#pragma unroll
      for (int c = 0; c < CPT / 2; ++c) {
        float pv[2], dv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int qi = 2 * c + e;
          float pe = exp2f(fmaf(__uint_as_float(sv[qi]), p.scale_log2, -lse_q[qi] * log2e));
          if (diag && key > q0 + qi) pe = 0.f;
          pv[e] = pe;
          dv[e] = pe * (__uint_as_float(dp[qi]) - del_q[qi]) * p.scale;
        }
        __nv_bfloat162 a = __floats2bfloat162_rn(pv[0], pv[1]);
        __nv_bfloat162 d2 = __floats2bfloat162_rn(dv[0], dv[1]);
        pk[c] = *reinterpret_cast<uint32_t*>(&a);
        dk[c] = *reinterpret_cast<uint32_t*>(&d2);
      }
      if (!mbar_wait(bar(BAR_PDS_EMPTY + st), (use & 1u) ^ 1u, abort_flag)) {
        ok = false;
        break;
      }
      if (threadIdx.x == 64) TRACE(1, t, 2);  // math done, P/dS buffer free
      // P^T and dS^T replace the scores this thread has just read (its own 16 columns)
      uint32_t pds[CPT];
#pragma unroll
      for (int c = 0; c < CPT / 2; ++c) {
        pds[c] = pk[c];
        pds[CPT / 2 + c] = dk[c];
      }
      tmem_st16(tmem_base + COL_S + st * BQ + g * CPT + lane_addr, pds);
      uint8_t* drow = smem + OFF_PDS + st * PDS_BYTES + row * 128;
#pragma unroll
      for (int c = 0; c < CPT / 8; ++c) {
        const int chunk = ((g * (CPT / 8) + c) ^ (row & 7)) << 4;
        *reinterpret_cast<uint4*>(drow + chunk) = make_uint4(dk[4 * c], dk[4 * c + 1], dk[4 * c + 2], dk[4 * c + 3]);
      }
      fence_async_smem();
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(BAR_PDS_FULL + st));
      if (threadIdx.x == 64) TRACE(1, t, 3);  // P/dS published
    }
    if (ok && mbar_wait(bar(BAR_DKV_DONE), 0, abort_flag)) {
      tc_fence_after();
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        constexpr int CW = D / GROUPS;  // head-dim columns per thread
        const uint32_t col = (which == 0 ? COL_DV : COL_DK) + g * CW;
        __nv_bfloat16* base = which == 0 ? p.dV : p.dK;
        const long long ld = which == 0 ? p.ld_dv : p.ld_dk;
        __nv_bfloat16* dst = base + static_cast<long long>(kv_row0 + row) * ld + hk * D + g * CW;
        uint32_t v[CW];
        if constexpr (CW == 32)
          tmem_ld32(tmem_base + col + lane_addr, v);
        else
          tmem_ld16(tmem_base + col + lane_addr, v);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < CW / 8; ++c) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[8 * c + e]);
          reinterpret_cast<ftb200::bf16x8*>(dst)[c] = ftb200::pack8(f);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, FTB200_ST_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (row, head)
template <int D>
__global__ void attention_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                       float* __restrict__ delta, int batch, int seq, int n_heads, long long ld_o,
                                       long long ld_do) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(batch) * seq * n_heads;
  if (w >= total) return;
  const long long r = w / n_heads;
  const int h = static_cast<int>(w % n_heads);
  constexpr int PAIRS = D / 64;  // bf16 pairs per lane
  __nv_bfloat162 a2[PAIRS], c2[PAIRS];
  if constexpr (PAIRS == 2) {
    *reinterpret_cast<uint2*>(a2) = *reinterpret_cast<const uint2*>(o + r * ld_o + h * D + lane * 4);
    *reinterpret_cast<uint2*>(c2) = *reinterpret_cast<const uint2*>(d_o + r * ld_do + h * D + lane * 4);
  } else {
    *reinterpret_cast<uint32_t*>(a2) = *reinterpret_cast<const uint32_t*>(o + r * ld_o + h * D + lane * 2);
    *reinterpret_cast<uint32_t*>(c2) = *reinterpret_cast<const uint32_t*>(d_o + r * ld_do + h * D + lane * 2);
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PAIRS; ++i) {
    const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(c2[i]);
    s += x.x * y.x + x.y * y.y;
  }
  s = ftb200::warp_sum(s);
  if (lane == 0) {
    const long long bb = r / seq, ss = r % seq;
    delta[(bb * n_heads + h) * seq + ss] = s;
  }
}

// dq[rows, cols] (bf16, row stride ld) = dq_acc[rows, cols] (fp32, dense)
__global__ void attention_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long rows,
                                         int cols, long long ld) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;  // one 8-element piece each
  const int per_row = cols / 8;
  if (i >= rows * per_row) return;
  const long long r = i / per_row;
  const int c = static_cast<int>(i % per_row) * 8;
  const float4 a = *reinterpret_cast<const float4*>(acc + r * cols + c);
  const float4 b2 = *reinterpret_cast<const float4*>(acc + r * cols + c + 4);
  const float f[8] = {a.x, a.y, a.z, a.w, b2.x, b2.y, b2.z, b2.w};
  *reinterpret_cast<ftb200::bf16x8*>(dq + r * ld + c) = ftb200::pack8(f);
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
    }
  }
  return fn;
}

int encode_rows(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  auto fn = encode_fn();
  if (fn == nullptr) return FTB200_E_DRIVER;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : FTB200_E_DRIVER;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// Scratch the backward pass needs, in bytes: fp32 dQ accumulator followed by delta.
// (sized for head dim 128; enough for 64 as well)
FTB200_API long long ftb200_attention_bwd_scratch_bytes(int batch, int seq, int n_heads) {
  const long long rows = static_cast<long long>(batch) * seq;
  return rows * n_heads * 128 * 4 + rows * n_heads * 4;
}

namespace {

template <int D>
int attention_bwd_impl(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                       void* dq, void* dk, void* dv, void* scratch, int batch, int seq, int n_heads, int n_kv_heads,
                       long long ld_q, long long ld_k, long long ld_v, long long ld_o, long long ld_do, long long ld_dq,
                       long long ld_dk, long long ld_dv, float scale, int causal, int* status, cudaStream_t stream) {
  constexpr uint32_t SMEM_BYTES = Lay<D>::SMEM_BYTES;
  const long long rows = static_cast<long long>(batch) * seq;
  float* dq_acc = reinterpret_cast<float*>(scratch);
  float* delta = dq_acc + rows * n_heads * D;
  CUtensorMap tq, tk, tv, tdo;
  int rc = encode_rows(&tq, q, rows, static_cast<long long>(n_heads) * D, ld_q, BQ);
  if (rc == 0) rc = encode_rows(&tdo, d_o, rows, static_cast<long long>(n_heads) * D, ld_do, BQ);
  if (rc == 0) rc = encode_rows(&tk, k, rows, static_cast<long long>(n_kv_heads) * D, ld_k, BKV);
  if (rc == 0) rc = encode_rows(&tv, v, rows, static_cast<long long>(n_kv_heads) * D, ld_v, BKV);
  if (rc != 0) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attention_bwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return FTB200_E_CUDA;
    attr_set = true;
  }
  if (cudaMemsetAsync(dq_acc, 0, rows * n_heads * D * 4, stream) != cudaSuccess) return FTB200_E_CUDA;
  {
    const long long warps = rows * n_heads;
    const long long blocks = (warps * 32 + 255) / 256;
    attention_delta_kernel<D><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(o), reinterpret_cast<const __nv_bfloat16*>(d_o), delta, batch, seq, n_heads,
        ld_o, ld_do);
  }
  BwdParams p;
  p.batch = batch; p.seq = seq; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.causal = causal;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dk); p.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  p.ld_dk = ld_dk; p.ld_dv = ld_dv; p.status = status;
  p.trace = nullptr;
#ifdef FTB200_ATTN_TRACE
  p.trace = reinterpret_cast<long long*>(delta + rows * n_heads);  // the caller sized the scratch for it
#endif
  const long long grid = static_cast<long long>(batch) * n_kv_heads * (seq / BKV);
  if (grid > 0x7fffffffLL) return FTB200_E_TOOBIG;
  attention_bwd_kernel<D><<<static_cast<unsigned>(grid), NUM_THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, tdo, p);
  {
    const long long pieces = rows * (static_cast<long long>(n_heads) * D / 8);
    attention_dq_cast_kernel<<<static_cast<unsigned>((pieces + 255) / 256), 256, 0, stream>>>(
        dq_acc, reinterpret_cast<__nv_bfloat16*>(dq), rows, n_heads * D, ld_dq);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

}  // namespace

// q, k, v, o, d_o as in the forward pass (2-D views, row strides in elements); dq, dk, dv are
// written (not accumulated).  lse is the forward's [batch, n_heads, seq].  scratch: at least
// ftb200_attention_bwd_scratch_bytes, 16-byte aligned.  Head dim 64 or 128.
FTB200_API int ftb200_attention_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                    const float* lse, void* dq, void* dk, void* dv, void* scratch, int batch, int seq,
                                    int n_heads, int n_kv_heads, int head_dim, long long ld_q, long long ld_k,
                                    long long ld_v, long long ld_o, long long ld_do, long long ld_dq, long long ld_dk,
                                    long long ld_dv, float scale, int causal, int* status, cudaStream_t stream) {
  if ((head_dim != 64 && head_dim != 128) || batch <= 0 || seq <= 0 || seq % BKV != 0 || n_heads <= 0 ||
      n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
    return FTB200_E_BADARG;
  const void* ptrs[] = {q, k, v, o, d_o, dq, dk, dv, scratch};
  for (const void* x : ptrs)
    if (!aligned16(x)) return FTB200_E_ALIGN;
  const long long lds[] = {ld_q, ld_k, ld_v, ld_o, ld_do, ld_dq, ld_dk, ld_dv};
  for (long long x : lds)
    if (x & 7) return FTB200_E_ALIGN;
  if (head_dim == 64)
    return attention_bwd_impl<64>(q, k, v, o, d_o, lse, dq, dk, dv, scratch, batch, seq, n_heads, n_kv_heads, ld_q, ld_k,
                                  ld_v, ld_o, ld_do, ld_dq, ld_dk, ld_dv, scale, causal, status, stream);
  return attention_bwd_impl<128>(q, k, v, o, d_o, lse, dq, dk, dv, scratch, batch, seq, n_heads, n_kv_heads, ld_q, ld_k,
                                 ld_v, ld_o, ld_do, ld_dq, ld_dk, ld_dv, scale, causal, status, stream);
}
