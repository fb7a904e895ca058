// bf16 GEMM with 2-SM tensor-core instructions (tcgen05.mma.cta_group::2).
//
// Same contract as the 1-CTA kernel in gemm_tcgen05.cu.  Two CTAs of a cluster share
// one 256x256 output tile: each stages its own 128 rows of A and its own 128 of the 256
// B columns (32 KiB per 64-deep K slab instead of 48 KiB), the pair's leader issues one
// M=256 MMA that reads both halves of B, and each CTA's TMEM receives the accumulator of
// its own 128 rows.  Per SM that is a third less shared-memory fill traffic per FLOP and
// room for a 6-stage ring, which is what the 1-CTA kernel lacks: its tensor pipe idles
// ~40% of the time waiting for operand tiles in flight.
//
// Synchronisation inside the pair:
//   full[s]   (leader)  both CTAs' TMA loads complete_tx on the leader's barrier
//   empty[s]  (each)    the leader's tcgen05.commit arrives on both CTAs' barriers
//   tfull[a]  (each)    likewise, after the last MMA of a tile
//   tempty[a] (leader)  the 2 x 128 epilogue threads of the pair arrive (remote arrive
//                       from the peer)
// All waits are bounded as in the 1-CTA kernel.
//
// All-gather fused into the GEMM (ftb200_gemm_bf16_gather): B is a weight whose rows lie
// spread over the ranks of a shard group, as one contiguous piece of a flat parameter unit
// that the ranks shard evenly.  Four extra warps per CTA pull the weight out of the owners'
// shard buffers over NVLink (plain 16-byte peer loads) into the local gathered unit, 16 KiB
// at a time in row order, and count the finished pieces per block of 128 B rows; the TMA
// producer of a tile waits (bounded) for the count of its 128 rows and then loads them from
// local memory, so the tensor cores work on the first tiles while the rest of the weight
// is still crossing the links, and every remote byte crosses them once.  The pieces are
// handed out through a counter, so the CTAs that are running pull everything whether or
// not the whole grid is resident.
#include <algorithm>
#include <cuda.h>
#include <cudaTypedefs.h>

#include "ftb200_common.cuh"
#include "tcgen05_helpers.cuh"

namespace {

constexpr int BM = 128;  // rows per CTA (256 per pair)
constexpr int BN = 256;  // columns per pair
constexpr int BNH = BN / 2;
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr uint32_t B_BYTES = BNH * BK * 2;
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int GATHER_WARPS = 4;  // only launched by the all-gather variant
constexpr int NUM_THREADS_GATHER = NUM_THREADS + 32 * GATHER_WARPS;
constexpr int GATHER_PIECE_V = 1024;  // 16-byte vectors per piece (16 KiB)
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr uint32_t SC_STAGE_WARP_BYTES = 32 * 256;  // scatter epilogue: 32 rows x 128 bf16 per warp
constexpr uint32_t SMEM_BYTES_SCATTER = SMEM_BYTES + 4 * SC_STAGE_WARP_BYTES;
constexpr int GROUP_M = 8;  // in 256-row pair tiles (the all-gather variant uses twice that)

using namespace ftb200::tc;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA tile load issued by one CTA of a pair; the completion bytes are signalled on a
// barrier that may live in the partner CTA (address in the cluster window).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive (once all MMAs issued so far have completed) on the barrier at the same
// shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;
  int out_fp32;
  int accumulate;
  long long ldc;
  void* C;
  int* status;
  // fused SwiGLU: output columns are (gate, up) pairs; aux[row, j] = silu(C[row,2j]) * C[row,2j+1]
  void* aux;
  long long ld_aux;
  // fused reduce-scatter epilogue: C is not written locally; every 16-byte piece of the
  // (contiguous, row-major) result goes to the rank that owns that slice of the flat
  // gradient unit, into that rank's staging area for source rank `sc_src`.
  int sc_world;                // 0 = off
  int sc_src;
  long long sc_shard;          // elements per shard (multiple of 8)
  long long sc_off;            // element offset of C inside the flat unit (multiple of 8)
  void* sc_peers[8];           // base of every rank's staging area (peer-mapped), [world][shard] elements
  int group_m;                 // tile order: this many 256-row tiles share a B tile before the next B tile
  // fused all-gather of B (see the head of the file); B points into the local gathered unit
  int ga_world;                // 0 = off
  long long ga_shard;          // elements per shard
  long long ga_off;            // element offset of B inside the flat unit (multiple of 8)
  const void* ga_peers[8];     // every rank's shard buffer (peer-mapped; [rank] is local)
  void* ga_dst;                // == B
  unsigned int* ga_sync;       // [0] next piece to hand out, [1 + c] pieces done of 128-row block c (zeroed per launch)
};

// Bounded wait until *p >= want (device-scope acquire).
__device__ __forceinline__ bool count_wait(const unsigned int* p, unsigned int want, volatile int* abort_flag) {
  const uint64_t t0 = ftb200::globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if (v >= want) return true;
    if ((++spins & 15u) == 0) {
      if (*abort_flag) return false;
      if (ftb200::globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        return false;
      }
      __nanosleep(64);
    }
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS_GATHER, 1)
gemm_bf16_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                              const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 256);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_k = (p.K + BK - 1) / BK;
  const int group_m = p.group_m;
  const int tiles_per_group = group_m * num_n;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  auto tile_coords = [&](int t, int& m0, int& n0) {
    const int g = t / tiles_per_group;
    const int first_m = g * group_m;
    const int gsz = min(num_m - first_m, group_m);
    const int r = t - g * tiles_per_group;
    m0 = (first_m + r % gsz) * (2 * BM) + static_cast<int>(rank) * BM;  // this CTA's rows
    n0 = (r / gsz) * BN;
  };

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int m0, n0;
        tile_coords(t, m0, n0);
        const int nb = n0 + static_cast<int>(rank) * BNH;  // this CTA's half of the B tile
        if (p.ga_world > 0 && nb < p.N) {
          // these 128 rows of B are local once all their pieces are counted; the loads below go through the
          // async proxy, the pieces were written through the generic one
          if (!count_wait(p.ga_sync + 1 + nb / BNH, static_cast<unsigned int>(p.K / 64), abort_flag)) {
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const int k0 = kb * BK;
          if (leader) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          const uint32_t fb = map_to_cta(full_bar(stage), 0);
          if (p.a_mn == 0) {
            tma_load_2d_pair(sa, &tmA, fb, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmA, fb, m0 + 64 * j, k0);
          }
          if (p.b_mn == 0) {
            tma_load_2d_pair(sb, &tmB, fb, k0, nb);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * (BK * 128), &tmB, fb, nb + 64 * j, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        const uint64_t t0 = ftb200::globaltimer_ns();
        while (ftb200::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(p.a_mn) << 15) |
                             (static_cast<uint32_t>(p.b_mn) << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                             (static_cast<uint32_t>((2 * BM) >> 4) << 24);
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, a_step = p.a_mn ? 2048 : 32;
      const uint32_t b_lbo = p.b_mn ? BK * 128 : 16, b_step = p.b_mn ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = make_smem_desc(sa + kk * a_step, a_lbo, 1024);
            const uint64_t bdesc = make_smem_desc(sb + kk * b_step, b_lbo, 1024);
            umma_bf16_pair(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(tfull_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ---------------- all-gather of B (warps 6..9 of both CTAs, all-gather variant only) ----------------
    if (p.ga_world > 0) {
      const long long total_v = static_cast<long long>(p.N) * p.K / 8;
      const long long pieces = (total_v + GATHER_PIECE_V - 1) / GATHER_PIECE_V;
      const unsigned int pieces_per_block = static_cast<unsigned int>(p.K / 64);  // 128 rows x K x 2 B / 16 KiB
      uint4* dstv = reinterpret_cast<uint4*>(p.ga_dst);
      for (;;) {
        unsigned int piece = 0;
        if (lane == 0) piece = atomicAdd(p.ga_sync, 1u);
        piece = __shfl_sync(0xffffffffu, piece, 0);
        if (piece >= pieces) break;
        const long long v0 = static_cast<long long>(piece) * GATHER_PIECE_V;
        const long long flat0 = p.ga_off + v0 * 8;
        const long long owner0 = flat0 / p.ga_shard;
        const long long rem0 = flat0 - owner0 * p.ga_shard;
#pragma unroll 1
        for (int b = 0; b < GATHER_PIECE_V / 256; ++b) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = b * 256 + u * 32 + lane;
            v[u] = make_uint4(0u, 0u, 0u, 0u);
            if (v0 + i < total_v) {
              long long rem = rem0 + static_cast<long long>(i) * 8;
              long long owner = owner0;
              if (rem >= p.ga_shard) {  // a piece is shorter than a shard: at most one boundary inside it
                rem -= p.ga_shard;
                ++owner;
              }
              if (FTB_IN_RANGE(owner, p.ga_world))
                v[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.ga_peers[owner]) + rem);
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = b * 256 + u * 32 + lane;
            if (v0 + i < total_v) dstv[v0 + i] = v[u];
          }
        }
        asm volatile("fence.proxy.async.global;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          atomicAdd(p.ga_sync + 1 + piece / pieces_per_block, 1u);
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = p.out_fp32 ? ((p.ldc & 3) == 0) : ((p.ldc & 7) == 0);
    for (int t = cluster_id; t < num_tiles; t += num_clusters) {
      int m0, n0;
      tile_coords(t, m0, n0);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr0 = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (p.sc_world > 0 || (!p.out_fp32 && !p.accumulate && vec_ok && (p.N & 7) == 0)) {
        // Staged epilogue (bf16 output, local or scattered to peers): the tile goes through a
        // per-warp staging area so that every store instruction covers two 256-byte row segments.
        // One 16-byte piece per thread and row would touch 32 rows per instruction: half-filled
        // sectors locally, and an NVLink packet each towards a peer, which throttles the kernel.
        uint8_t* stg = smem + STAGES * STAGE_BYTES + 256 + q * SC_STAGE_WARP_BYTES;
        const int half = lane >> 4, ch = lane & 15;
#pragma unroll 1
        for (int cg = 0; cg < BN / 128; ++cg) {
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t r[32];
            tmem_ld32(taddr0 + (cg * 4 + cc) * 32, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
              *reinterpret_cast<ftb200::bf16x8*>(stg + lane * 256 + (((cc * 4 + j) ^ (lane & 15)) << 4)) = ftb200::pack8(f);
            }
          }
          __syncwarp();
          const int gcol = n0 + cg * 128 + ch * 8;
#pragma unroll 4
          for (int it = 0; it < 16; ++it) {
            const int rr = it * 2 + half;
            const int grow = m0 + q * 32 + rr;
            const ftb200::bf16x8 v = *reinterpret_cast<const ftb200::bf16x8*>(stg + rr * 256 + ((ch ^ (rr & 15)) << 4));
            if (grow < p.M && gcol + 8 <= p.N) {
              if (p.sc_world > 0) {
                const long long flat = p.sc_off + static_cast<long long>(grow) * p.ldc + gcol;
                const long long owner = flat / p.sc_shard;
                const long long rem = flat - owner * p.sc_shard;
                if (!FTB_IN_RANGE(owner, p.sc_world)) continue;
                __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.sc_peers[owner]);
                *reinterpret_cast<ftb200::bf16x8*>(base + static_cast<long long>(p.sc_src) * p.sc_shard + rem) = v;
              } else {
                __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(grow) * p.ldc;
                *reinterpret_cast<ftb200::bf16x8*>(crow + gcol) = v;
                if (p.aux != nullptr) {
                  // activation of the rounded values, so that a later recompute from C agrees
                  float g[8];
                  ftb200::unpack8(v, g);
                  float sv[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) sv[e] = g[2 * e] / (1.f + __expf(-g[2 * e])) * g[2 * e + 1];
                  __nv_bfloat162 lo = __floats2bfloat162_rn(sv[0], sv[1]), hi = __floats2bfloat162_rn(sv[2], sv[3]);
                  uint2 o2;
                  o2.x = *reinterpret_cast<uint32_t*>(&lo);
                  o2.y = *reinterpret_cast<uint32_t*>(&hi);
                  *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.aux) + static_cast<long long>(grow) * p.ld_aux +
                                            (gcol >> 1)) = o2;
                }
              }
            }
          }
          __syncwarp();
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr0 + c * 32, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          const bool full = vec_ok && (col0 + 32 <= p.N);
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
            if (full) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                if (p.accumulate) {
                  const float4 o = reinterpret_cast<const float4*>(dst)[j];
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                reinterpret_cast<float4*>(dst)[j] = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.N) {
                  const float v = __uint_as_float(r[j]);
                  dst[j] = p.accumulate ? dst[j] + v : v;
                }
              }
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
            if (full) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]);
                if (p.accumulate) {
                  float o[8];
                  ftb200::unpack8(reinterpret_cast<const ftb200::bf16x8*>(dst)[j], o);
#pragma unroll
                  for (int e = 0; e < 8; ++e) f[e] += o[e];
                }
                const ftb200::bf16x8 packed = ftb200::pack8(f);
                reinterpret_cast<ftb200::bf16x8*>(dst)[j] = packed;
                if (p.aux != nullptr) {
                  // activation of the rounded values, so that a later recompute from C agrees
                  float g[8];
                  ftb200::unpack8(packed, g);
                  float sv[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) sv[e] = g[2 * e] / (1.f + __expf(-g[2 * e])) * g[2 * e + 1];
                  __nv_bfloat162 lo = __floats2bfloat162_rn(sv[0], sv[1]), hi = __floats2bfloat162_rn(sv[2], sv[3]);
                  uint2 o2;
                  o2.x = *reinterpret_cast<uint32_t*>(&lo);
                  o2.y = *reinterpret_cast<uint32_t*>(&hi);
                  __nv_bfloat16* adst =
                      reinterpret_cast<__nv_bfloat16*>(p.aux) + static_cast<long long>(row) * p.ld_aux + (col0 >> 1) + 4 * j;
                  *reinterpret_cast<uint2*>(adst) = o2;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.N) {
                  float v = __uint_as_float(r[j]);
                  if (p.accumulate) v += __bfloat162float(dst[j]);
                  dst[j] = __float2bfloat16(v);
                }
              }
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, FTB200_ST_TIMEOUT);
  cluster_sync_all();  // neither CTA retires while its partner may still touch its barriers or operands
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
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

int encode_2d(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_cols,
              int box_rows) {
  auto fn = get_encode_fn();
  if (fn == nullptr) return FTB200_E_DRIVER;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : FTB200_E_DRIVER;
}

}  // namespace

// Same arguments as ftb200_gemm_bf16; pairs of CTAs cooperate on 256x256 tiles.
struct ScatterSpec {
  int world = 0;
  int src = 0;
  long long shard = 0;
  long long off = 0;
  void* const* peers = nullptr;
};

struct GatherSpec {
  int world = 0;
  long long shard = 0;
  long long off = 0;
  const void* const* peers = nullptr;
  unsigned int* sync = nullptr;
};

static int gemm_2cta_impl(const void* A, const void* B, void* C, int M, int N, int K, int a_mn_major, int b_mn_major,
                          long long lda, long long ldb, long long ldc, int flags, int* status, int max_ctas, void* aux,
                          long long ld_aux, cudaStream_t stream, const ScatterSpec* sc = nullptr,
                          const GatherSpec* ga = nullptr) {
  if (M <= 0 || N <= 0 || K <= 0 || A == nullptr || B == nullptr || (C == nullptr && sc == nullptr)) return FTB200_E_BADARG;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7))
    return FTB200_E_ALIGN;
  if ((reinterpret_cast<uintptr_t>(C) & 15)) return FTB200_E_ALIGN;
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn_major)
    rc = encode_2d(&tmA, A, M, K, lda, BK, BM);
  else
    rc = encode_2d(&tmA, A, K, M, lda, 64, BK);
  if (rc) return rc;
  if (!b_mn_major)
    rc = encode_2d(&tmB, B, N, K, ldb, BK, BNH);
  else
    rc = encode_2d(&tmB, B, K, N, ldb, 64, BK);
  if (rc) return rc;

  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_bf16_tcgen05_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES_SCATTER) != cudaSuccess)
      return FTB200_E_CUDA;
    attr_set = true;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn_major ? 1 : 0;
  p.b_mn = b_mn_major ? 1 : 0;
  p.out_fp32 = flags & 1;
  p.accumulate = (flags >> 1) & 1;
  p.ldc = ldc;
  p.C = C;
  p.status = status;
  p.aux = aux;
  p.ld_aux = ld_aux;
  p.sc_world = 0;
  p.sc_src = 0;
  p.sc_shard = 0;
  p.sc_off = 0;
  for (int i = 0; i < 8; ++i) p.sc_peers[i] = nullptr;
  if (sc != nullptr) {
    p.sc_world = sc->world;
    p.sc_src = sc->src;
    p.sc_shard = sc->shard;
    p.sc_off = sc->off;
    for (int i = 0; i < sc->world && i < 8; ++i) p.sc_peers[i] = sc->peers[i];
  }
  p.group_m = GROUP_M;
  p.ga_world = 0;
  p.ga_shard = 0;
  p.ga_off = 0;
  p.ga_dst = nullptr;
  p.ga_sync = nullptr;
  for (int i = 0; i < 8; ++i) p.ga_peers[i] = nullptr;
  if (ga != nullptr) {
    p.ga_world = ga->world;
    p.ga_shard = ga->shard;
    p.ga_off = ga->off;
    p.ga_dst = const_cast<void*>(B);
    p.ga_sync = ga->sync;
    for (int i = 0; i < ga->world && i < 8; ++i) p.ga_peers[i] = ga->peers[i];
    // Sixteen row tiles share a B tile before the next B tile (eight without the gather).  The whole weight is
    // needed by the end of the first group of row tiles; with M = 8192 that group is half of the GEMM instead of
    // a quarter, which halves the link bandwidth the gather needs to stay ahead, and costs ~2.5 % of the GEMM's
    // speed in L2 locality (measured; all of M per B tile costs ~9 %).
    p.group_m = 2 * GROUP_M;
    if (cudaMemsetAsync(ga->sync, 0, sizeof(unsigned int) * (1 + static_cast<size_t>(N) / BNH), stream) != cudaSuccess)
      return FTB200_E_CUDA;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  int ctas = ftb200::sm_count() & ~1;
  if (max_ctas > 0 && max_ctas < ctas) ctas = std::max(2, max_ctas & ~1);
  if (2 * tiles < ctas) ctas = 2 * tiles;
  gemm_bf16_tcgen05_2cta_kernel<<<ctas, ga != nullptr ? NUM_THREADS_GATHER : NUM_THREADS, SMEM_BYTES_SCATTER, stream>>>(
      tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_gemm_bf16_2cta(const void* A, const void* B, void* C, int M, int N, int K, int a_mn_major,
                                     int b_mn_major, long long lda, long long ldb, long long ldc, int flags, int* status,
                                     int max_ctas, cudaStream_t stream) {
  return gemm_2cta_impl(A, B, C, M, N, K, a_mn_major, b_mn_major, lda, ldb, ldc, flags, status, max_ctas, nullptr, 0, stream);
}

// Forward GEMM of a gated MLP with the activation fused into the epilogue: B's rows are
// interleaved (gate_0, up_0, gate_1, up_1, ...), C [M,N] receives the pre-activations and
// aux [M,N/2] receives silu(gate) * up.  bf16 output, N a multiple of 32, no accumulate.
FTB200_API int ftb200_gemm_bf16_swiglu(const void* A, const void* B, void* C, void* aux, int M, int N, int K, long long lda,
                                       long long ldb, long long ldc, long long ld_aux, int* status, int max_ctas,
                                       cudaStream_t stream) {
  if (aux == nullptr || (N % 32) || (ldc & 7) || (ld_aux & 3) || (reinterpret_cast<uintptr_t>(aux) & 7)) return FTB200_E_ALIGN;
  return gemm_2cta_impl(A, B, C, M, N, K, 0, 0, lda, ldb, ldc, 0, status, max_ctas, aux, ld_aux, stream);
}

// GEMM whose epilogue is the reduce-scatter's transfer: the [M,N] result (row-major, row
// stride N) is one field of a flat gradient unit that `world` ranks shard evenly; each
// 16-byte piece is stored straight into the owner rank's staging area
// (peers[owner] + src_rank * shard_elems + offset-in-shard) over NVLink while the tensor
// cores work on the next tile.  A team round and a local sum over the `world` staging
// slices (ftb200_team_reduce_scatter on local pointers) finish the reduce-scatter.
// N must be a multiple of 32; shard_elems and unit_off multiples of 8.
FTB200_API int ftb200_gemm_bf16_scatter(const void* A, const void* B, int M, int N, int K, int a_mn_major, int b_mn_major,
                                        long long lda, long long ldb, void* const* peers, int world, int src_rank,
                                        long long shard_elems, long long unit_off, int* status, int max_ctas,
                                        cudaStream_t stream) {
  if (peers == nullptr || world < 1 || world > 8 || src_rank < 0 || src_rank >= world) return FTB200_E_BADARG;
  if ((N % 32) || (shard_elems % 8) || (unit_off % 8)) return FTB200_E_ALIGN;
  if (unit_off + static_cast<long long>(M) * N > shard_elems * world) return FTB200_E_TOOBIG;
  ScatterSpec sc;
  sc.world = world; sc.src = src_rank; sc.shard = shard_elems; sc.off = unit_off; sc.peers = peers;
  return gemm_2cta_impl(A, B, nullptr, M, N, K, a_mn_major, b_mn_major, lda, ldb, N, 0, status, max_ctas, nullptr, 0, stream, &sc);
}

// C[M,N] = A[M,K] . B[N,K]^T where B is still spread over the shard group: `B_local` points at the weight's place
// inside this rank's gathered copy of a flat parameter unit (`unit_off` elements from the unit's start, row stride
// K), `shard_peers[r]` at rank r's shard of that unit (`shard_elems` elements each; [rank] is local memory).  The
// kernel fills B_local from the shards while it multiplies (see the head of this file); after it, B_local is an
// ordinary gathered weight.  `sync_words`: 1 + N/128 32-bit words of scratch in local memory, zeroed here on
// `stream`; it may be shared by all calls on one stream.  aux / ld_aux: optional SwiGLU output as in
// ftb200_gemm_bf16_swiglu (then N must be a multiple of 32).  N a multiple of 128, K of 64, bf16 output.
// The caller orders the call after every rank's shard has been written (a team round) and keeps the shards
// unchanged until all ranks' calls have ended.
FTB200_API int ftb200_gemm_bf16_gather(const void* A, void* B_local, void* C, int M, int N, int K, long long lda,
                                       long long ldc, const void* const* shard_peers, int world, long long shard_elems,
                                       long long unit_off, unsigned int* sync_words, void* aux, long long ld_aux,
                                       int* status, int max_ctas, cudaStream_t stream) {
  if (shard_peers == nullptr || sync_words == nullptr || world < 1 || world > 8) return FTB200_E_BADARG;
  if ((N % BNH) || (K % 64) || (shard_elems % 8) || (unit_off % 8) || (ldc & 7)) return FTB200_E_ALIGN;
  if (shard_elems < 8LL * GATHER_PIECE_V) return FTB200_E_BADARG;  // a piece may cross one shard boundary, not two
  if (unit_off + static_cast<long long>(N) * K > shard_elems * world) return FTB200_E_TOOBIG;
  for (int r = 0; r < world; ++r)
    if (shard_peers[r] == nullptr || (reinterpret_cast<uintptr_t>(shard_peers[r]) & 15)) return FTB200_E_ALIGN;
  if (aux != nullptr && ((N % 32) || (ld_aux & 3) || (reinterpret_cast<uintptr_t>(aux) & 7))) return FTB200_E_ALIGN;
  GatherSpec ga;
  ga.world = world; ga.shard = shard_elems; ga.off = unit_off; ga.peers = shard_peers; ga.sync = sync_words;
  return gemm_2cta_impl(A, B_local, C, M, N, K, 0, 0, lda, K, ldc, 0, status, max_ctas, aux, ld_aux, stream, nullptr, &ga);
}

FTB_DEFINE_BOUNDS_QUERY(gemm_2cta)
