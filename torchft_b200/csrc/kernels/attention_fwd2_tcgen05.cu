// Causal grouped-query attention, forward pass, two query tiles per CTA.
//
//   O[b, s, h, :] = softmax(scale * Q[b, s, h, :] K[b, :, h / group, :]^T + causal mask) V[b, :, h / group, :]
//
// head_dim 64 or 128, bf16 in/out, fp32 accumulation and statistics.  Q, K and V are read in
// place from a packed [batch * seq, n_cols] activation (any row stride).
//
// One CTA owns one (batch, head) and 256 consecutive queries as two tiles of 128.  The loop over
// 128-key blocks is paced by two resources of the SM that cost about the same per tile and block:
// the tensor pipe (S = Q K^T and O += P V) and the exponential unit (128 x 128 exp2).  With two
// tiles in flight the tensor pipe works on one tile while the softmax of the other runs:
//
//   warp 0        TMA: Q tiles once, K and V blocks into a 2-stage ring
//   warp 1        tcgen05.mma, in the order  P0 V, S0', P1 V, S1'  (' = next block): the softmax of
//                 a tile has the two MMAs of the other tile to hide under
//   warps 2..5    softmax of tile 0, warps 6..9 softmax of tile 1: ONE thread per query row (the
//                 128 scores of a row sit in one TMEM lane), so the row maximum and sum need no
//                 exchange between threads.  P goes back as packed bf16 into the first 64 columns
//                 of the scores and is the A operand of P V straight from tensor memory.
//
// A share of the exponentials (POLY of every 8) is computed with a cubic polynomial on the FMA
// pipe instead of the exponential unit, which is the scarcer of the two; its relative error of
// 8e-5 disappears in the bf16 rounding of P.  The running maximum is only raised (and O in TMEM
// rescaled) when it grows by more than 2^8.
//
// Every mbarrier wait is bounded; on expiry the CTA records FTB200_ST_TIMEOUT in the caller's
// status word, frees its TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

#include "ftb200_common.cuh"
#include "tcgen05_helpers.cuh"

namespace {

using namespace ftb200::tc;

constexpr int BQ = 128;       // queries per tile
constexpr int TILES = 2;      // tiles per CTA
constexpr int BKV = 128;      // keys per block
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 320;
constexpr int ROW_THREADS = 128;  // softmax threads per tile
constexpr uint32_t TMEM_COLS = 512;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

template <int D>
struct Cfg {
  static constexpr uint32_t TILE_BYTES = 128 * D * 2;       // a 128-row operand tile
  static constexpr uint32_t SLAB_BYTES = 128 * 128;         // 128 rows x 64 elements (one swizzle atom wide)
  static constexpr int SLABS = D / 64;
  static constexpr uint32_t OFF_Q = 0;                      // Q0 Q1
  static constexpr uint32_t OFF_KV = TILES * TILE_BYTES;    // K0 V0 | K1 V1
  static constexpr uint32_t OFF_MISC = OFF_KV + KV_STAGES * 2 * TILE_BYTES;
  static constexpr uint32_t SMEM_BYTES = OFF_MISC + 256 + 1024;
  static constexpr uint32_t COL_S = 0;                      // S_t at COL_S + t * 128
  static constexpr uint32_t COL_O = 256;                    // O_t at COL_O + t * D
};

struct Attn2Params {
  int batch, seq, n_heads, n_kv_heads;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  __nv_bfloat16* O;
  long long ld_o;    // row stride of O in elements
  float* lse;        // [batch, n_heads, seq], natural log
  int* status;
};

enum : int {
  BAR_Q_FULL = 0,    // +tile
  BAR_K_FULL = 2,    // +stage
  BAR_V_FULL = 4,    // +stage
  BAR_K_EMPTY = 6,   // +stage
  BAR_V_EMPTY = 8,   // +stage
  BAR_S_FULL = 10,   // +tile
  BAR_P_FULL = 12,   // +tile
  BAR_O_DONE = 14,   // +tile
  NUM_BARS = 16,
};

// 2^x for x <= 8 on the FMA pipe: round to the nearest integer n with the magic-number trick,
// cubic in the remainder f in [-0.5, 0.5] (relative error 7.5e-5), n added to the exponent bits.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -125.f);
  const float xr = x + 12582912.f;  // 1.5 * 2^23: the integer lands in the low mantissa bits
  const float f = x - (xr - 12582912.f);
  float p = fmaf(f, 0.05517063f, 0.24260884f);
  p = fmaf(f, p, 0.69326095f);
  p = fmaf(f, p, 0.99992822f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(xr) << 23));
}

template <int D, int POLY>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attention_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const Attn2Params p) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_MISC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 196);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto bar = [&](int i) { return bar_base + 8u * i; };

  // heavy (late) query blocks first: with a causal mask their work is largest
  const int n_qpairs = p.seq / (BQ * TILES);
  const int per_block = p.batch * p.n_heads;
  const int qp = n_qpairs - 1 - static_cast<int>(blockIdx.x) / per_block;
  const int bh = static_cast<int>(blockIdx.x) % per_block;
  const int b = bh / p.n_heads, h = bh % p.n_heads;
  const int hk = h / (p.n_heads / p.n_kv_heads);
  // key blocks seen by tile 0 and tile 1
  const int n_kv1 = p.causal ? qp * TILES + 2 : p.seq / BKV;
  const int n_kv0 = p.causal ? n_kv1 - 1 : n_kv1;
  const int q_row0 = b * p.seq + qp * BQ * TILES;

  if (threadIdx.x == 0) {
    for (int t = 0; t < TILES; ++t) {
      mbar_init(bar(BAR_Q_FULL + t), 1);
      mbar_init(bar(BAR_S_FULL + t), 1);
      mbar_init(bar(BAR_P_FULL + t), ROW_THREADS);
      mbar_init(bar(BAR_O_DONE + t), 1);
    }
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(bar(BAR_K_FULL + s), 1);
      mbar_init(bar(BAR_V_FULL + s), 1);
      mbar_init(bar(BAR_K_EMPTY + s), 1);
      mbar_init(bar(BAR_V_EMPTY + s), 1);
    }
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
      for (int t = 0; t < TILES; ++t) {
        const uint32_t sq = smem_base + C::OFF_Q + t * C::TILE_BYTES;
        mbar_expect_tx(bar(BAR_Q_FULL + t), C::TILE_BYTES);
        for (int s = 0; s < C::SLABS; ++s)
          tma_load_2d(sq + s * C::SLAB_BYTES, &tmQ, bar(BAR_Q_FULL + t), h * D + s * 64, q_row0 + t * BQ);
      }
      bool ok = true;
      for (int j = 0; j < n_kv1 && ok; ++j) {
        const int st = j & 1;
        const uint32_t use = static_cast<uint32_t>(j >> 1);
        if (!mbar_wait(bar(BAR_K_EMPTY + st), (use & 1u) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        const uint32_t sk = smem_base + C::OFF_KV + st * 2 * C::TILE_BYTES;
        const uint32_t sv = sk + C::TILE_BYTES;
        const int kv_row0 = b * p.seq + j * BKV;
        mbar_expect_tx(bar(BAR_K_FULL + st), C::TILE_BYTES);
        for (int s = 0; s < C::SLABS; ++s) tma_load_2d(sk + s * C::SLAB_BYTES, &tmK, bar(BAR_K_FULL + st), hk * D + s * 64, kv_row0);
        if (!mbar_wait(bar(BAR_V_EMPTY + st), (use & 1u) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        mbar_expect_tx(bar(BAR_V_FULL + st), C::TILE_BYTES);
        for (int s = 0; s < C::SLABS; ++s) tma_load_2d(sv + s * C::SLAB_BYTES, &tmV, bar(BAR_V_FULL + st), hk * D + s * 64, kv_row0);
      }
      if (!ok) {
        // copies in flight land in this CTA's shared memory: give them time before the CTA exits
        const uint64_t t0 = ftb200::globaltimer_ns();
        while (ftb200::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // S = Q K^T: both operands K-major (head dim contiguous), M = N = 128
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BKV >> 3) << 17) |
                               (static_cast<uint32_t>(BQ >> 4) << 24);
      // O += P V: A = P from tensor memory (keys contiguous), B = V MN-major (stored [key][d]), N = D
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(D >> 3) << 17) |
                               (static_cast<uint32_t>(BQ >> 4) << 24);
      constexpr uint32_t HI = smem_desc_hi(1024);
      const uint32_t q_lo = smem_desc_lo(smem_base + C::OFF_Q, 16);
      const uint32_t k_lo = smem_desc_lo(smem_base + C::OFF_KV, 16);
      const uint32_t v_lo = smem_desc_lo(smem_base + C::OFF_KV + C::TILE_BYTES, C::SLAB_BYTES);
      constexpr uint32_t STAGE16 = (2 * C::TILE_BYTES) >> 4;
      constexpr uint32_t QTILE16 = C::TILE_BYTES >> 4;
      auto issue_s = [&](int t, int j) {
        const int st = j & 1;
        const uint32_t qb = q_lo + t * QTILE16;
        const uint32_t kb = k_lo + st * STAGE16;
        const uint32_t d_tmem = tmem_base + C::COL_S + t * 128;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * C::SLAB_BYTES + (kk & 3) * 32) >> 4;
          umma_bf16_lh(d_tmem, qb + off, HI, kb + off, HI, idesc_s, kk != 0);
        }
        umma_commit(bar(BAR_S_FULL + t));
      };
      auto issue_pv = [&](int t, int j) {
        const int st = j & 1;
        const uint32_t vb = v_lo + st * STAGE16;
        const uint32_t d_tmem = tmem_base + C::COL_O + t * D;
        const uint32_t p_tmem = tmem_base + C::COL_S + t * 128;  // P: keys 2k, 2k+1 in column k
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          umma_bf16_tmem_a(d_tmem, p_tmem + kk * 8, vb + ((kk * 2048) >> 4), HI, idesc_o, (j | kk) != 0);
        umma_commit(bar(BAR_O_DONE + t));
      };
      bool ok = mbar_wait(bar(BAR_Q_FULL + 0), 0, abort_flag) && mbar_wait(bar(BAR_K_FULL + 0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        ok = mbar_wait(bar(BAR_Q_FULL + 1), 0, abort_flag);
      }
      if (ok) {
        tc_fence_after();
        issue_s(1, 0);
        umma_commit(bar(BAR_K_EMPTY + 0));
      }
      for (int j = 0; j < n_kv1 && ok; ++j) {
        const int st = j & 1, st1 = st ^ 1;
        const uint32_t use = static_cast<uint32_t>(j >> 1), use1 = static_cast<uint32_t>((j + 1) >> 1);
        bool k_next = false;
        if (j < n_kv0) {
          if (!mbar_wait(bar(BAR_P_FULL + 0), static_cast<uint32_t>(j) & 1u, abort_flag) ||
              !mbar_wait(bar(BAR_V_FULL + st), use & 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_pv(0, j);
          if (j + 1 < n_kv0) {
            // S0 held P0 of block j: its P V was issued above and the tensor pipe runs in order
            if (!mbar_wait(bar(BAR_K_FULL + st1), use1 & 1u, abort_flag)) {
              ok = false;
              break;
            }
            k_next = true;
            tc_fence_after();
            issue_s(0, j + 1);
          }
        }
        if (!mbar_wait(bar(BAR_P_FULL + 1), static_cast<uint32_t>(j) & 1u, abort_flag) ||
            !mbar_wait(bar(BAR_V_FULL + st), use & 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        issue_pv(1, j);
        umma_commit(bar(BAR_V_EMPTY + st));
        if (j + 1 < n_kv1) {
          if (!k_next && !mbar_wait(bar(BAR_K_FULL + st1), use1 & 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_s(1, j + 1);
          umma_commit(bar(BAR_K_EMPTY + st1));
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax + epilogue: one thread per query row ----------------
    const int t = (warp - 2) >> 2;   // tile
    const int quarter = warp & 3;    // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + C::COL_S + t * 128 + lane_addr;
    const uint32_t o_addr = tmem_base + C::COL_O + t * D + lane_addr;
    const int n_kv = t == 0 ? n_kv0 : n_kv1;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(bar(BAR_S_FULL + t), static_cast<uint32_t>(j) & 1u, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sv[BKV];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) tmem_ld32(s_addr + c * 32, sv + c * 32);
      tmem_wait_ld();
      if (p.causal && j == n_kv - 1) {
        // the diagonal block: key c of the block is visible to query `row` of the tile iff c <= row
#pragma unroll
        for (int c = 0; c < BKV; ++c)
          if (c > row) sv[c] = __float_as_uint(-INFINITY);
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < BKV; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c]));
      const float m_new = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));

      // raise the maximum only when it moved far
      float alpha = 1.f;
      const bool raise = j > 0 && (m_new - m_used) * p.scale_log2 > RESCALE_THRESHOLD;
      const bool any_raise = __any_sync(0xffffffffu, raise);
      if (j == 0) {
        m_used = m_new;
      } else if (raise) {
        alpha = exp2f((m_used - m_new) * p.scale_log2);
        m_used = m_new;
        l_sum *= alpha;
      }
      if (any_raise) {
        // O may only be touched once P V of the previous block is done; P V of this block waits for P
        if (!mbar_wait(bar(BAR_O_DONE + t), static_cast<uint32_t>(j - 1) & 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t ov[32];
          tmem_ld32(o_addr + c * 32, ov);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
          tmem_st32(o_addr + c * 32, ov);
        }
      }
      const float neg_m = -m_used * p.scale_log2;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float x0 = fmaf(__uint_as_float(sv[c * 32 + 2 * e]), p.scale_log2, neg_m);
          const float x1 = fmaf(__uint_as_float(sv[c * 32 + 2 * e + 1]), p.scale_log2, neg_m);
          // POLY of every 8 exponentials go to the FMA pipe
          const float p0 = ((2 * e) & 7) < POLY ? exp2_poly(x0) : exp2f(x0);
          const float p1 = ((2 * e + 1) & 7) < POLY ? exp2_poly(x1) : exp2f(x1);
          sum4[e & 3] += p0 + p1;
          __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          packed[e] = *reinterpret_cast<uint32_t*>(&pk);
        }
        // P replaces the first half of the scores this thread has already taken into registers
        tmem_st16(s_addr + c * 16, packed);
      }
      l_sum += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(BAR_P_FULL + t));
    }

    if (ok && mbar_wait(bar(BAR_O_DONE + t), static_cast<uint32_t>(n_kv - 1) & 1u, abort_flag)) {
      tc_fence_after();
      const float inv = 1.f / l_sum;
      const long long grow = static_cast<long long>(q_row0 + t * BQ + row);
      __nv_bfloat16* dst = p.O + grow * p.ld_o + h * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t ov[32];
        tmem_ld32(o_addr + c * 32, ov);
        tmem_wait_ld();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(ov[8 * q4 + e]) * inv;
          reinterpret_cast<ftb200::bf16x8*>(dst + c * 32)[q4] = ftb200::pack8(f);
        }
      }
      if (p.lse != nullptr) {
        p.lse[(static_cast<long long>(b) * p.n_heads + h) * p.seq + qp * BQ * TILES + t * BQ + row] =
            (m_used * p.scale_log2 + log2f(l_sum)) * 0.6931471805599453f;
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

PFN_cuTensorMapEncodeTiled_v12000 encode_fn2() {
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

// [rows, cols] bf16 view with row stride ld (elements); box = 64 columns x 128 rows, 128-byte swizzle
int encode_rows2(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld) {
  auto fn = encode_fn2();
  if (fn == nullptr) return FTB200_E_DRIVER;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64u, 128u};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : FTB200_E_DRIVER;
}

template <int D, int POLY>
int launch_fwd2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const Attn2Params& p, long long grid,
                cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attention_fwd2_kernel<D, POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg<D>::SMEM_BYTES) != cudaSuccess)
      return FTB200_E_CUDA;
    attr_set = true;
  }
  attention_fwd2_kernel<D, POLY><<<static_cast<unsigned>(grid), NUM_THREADS, Cfg<D>::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

}  // namespace

// q: [batch*seq, n_heads*head_dim] view with row stride ld_q; k, v: [batch*seq, n_kv_heads*head_dim] views with
// row strides ld_k, ld_v; o: [batch*seq, n_heads*head_dim] with row stride ld_o.  lse (may be null):
// [batch, n_heads, seq] fp32.  head_dim 64 or 128; seq must be a multiple of 256.  poly: how many of every
// eight exponentials are computed on the FMA pipe (0, 2 or 4).
FTB200_API int ftb200_attention_fwd2(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq,
                                     int n_heads, int n_kv_heads, int head_dim, long long ld_q, long long ld_k,
                                     long long ld_v, long long ld_o, float scale, int causal, int poly, int* status,
                                     cudaStream_t stream) {
  if ((head_dim != 64 && head_dim != 128) || batch <= 0 || seq <= 0 || seq % (BQ * TILES) != 0 || n_heads <= 0 ||
      n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || (poly != 0 && poly != 2 && poly != 4))
    return FTB200_E_BADARG;
  auto aligned16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || (ld_q & 7) || (ld_k & 7) || (ld_v & 7) ||
      (ld_o & 7))
    return FTB200_E_ALIGN;
  CUtensorMap tq, tk, tv;
  const long long rows = static_cast<long long>(batch) * seq;
  int rc = encode_rows2(&tq, q, rows, static_cast<long long>(n_heads) * head_dim, ld_q);
  if (rc == 0) rc = encode_rows2(&tk, k, rows, static_cast<long long>(n_kv_heads) * head_dim, ld_k);
  if (rc == 0) rc = encode_rows2(&tv, v, rows, static_cast<long long>(n_kv_heads) * head_dim, ld_v);
  if (rc != 0) return rc;
  Attn2Params p;
  p.batch = batch; p.seq = seq; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.O = reinterpret_cast<__nv_bfloat16*>(o); p.ld_o = ld_o; p.lse = lse; p.status = status;
  const long long grid = static_cast<long long>(batch) * n_heads * (seq / (BQ * TILES));
  if (grid > 0x7fffffffLL) return FTB200_E_TOOBIG;
  if (head_dim == 128) {
    if (poly == 0) return launch_fwd2<128, 0>(tq, tk, tv, p, grid, stream);
    if (poly == 2) return launch_fwd2<128, 2>(tq, tk, tv, p, grid, stream);
    return launch_fwd2<128, 4>(tq, tk, tv, p, grid, stream);
  }
  if (poly == 0) return launch_fwd2<64, 0>(tq, tk, tv, p, grid, stream);
  if (poly == 2) return launch_fwd2<64, 2>(tq, tk, tv, p, grid, stream);
  return launch_fwd2<64, 4>(tq, tk, tv, p, grid, stream);
}
