// Causal grouped-query attention, forward pass, on the 5th-generation tensor cores.
//
//   O[b, s, h, :] = softmax(scale * Q[b, s, h, :] K[b, :, h / group, :]^T + causal mask) V[b, :, h / group, :]
//
// head_dim 128, bf16 in/out, fp32 accumulation and statistics.  Q, K and V are read in place
// from a packed [batch * seq, n_cols] activation (any row stride), the layout in which the
// QKV projection writes them, so no transposed copies exist on either side.
//
// One CTA owns one (batch, head, 128-query block).  Per 128-key block:
//   warp 0            TMA: K and V tiles into a 2-stage ring
//   (Q, stationary for the CTA, is loaded by the softmax warps straight into TMEM and is the A
//   operand of S = Q K^T from there: with both operands in shared memory the MMAs of tiles this
//   small are bound by operand fetch, not by the tensor pipe)
//   warp 1            tcgen05.mma: S = Q K^T into one of two TMEM buffers, O += P V
//   warps 2..17       softmax: four threads per query row (32 keys each); scores come from TMEM
//                     (tcgen05.ld) and P goes back into the same TMEM columns as packed bf16
//                     (tcgen05.st), from where the second MMA takes it as its A operand: P never
//                     touches shared memory, which halves the operand traffic of P V
// S of block j+1 is issued before P V of block j, so the tensor cores work on the next scores
// while the softmax of the current block runs.  The running maximum is only raised (and O in
// TMEM rescaled, tcgen05.ld/st) when it grows by more than 2^8, which keeps the accumulator
// read-modify-write off the common path.
//
// Every mbarrier wait is bounded; on expiry the CTA records FTB200_ST_TIMEOUT in the
// caller's status word, frees its TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

#include "ftb200_common.cuh"
#include "tcgen05_helpers.cuh"

namespace {

using namespace ftb200::tc;

// Optional event trace for tuning (compiled in with -DFTB200_ATTN_TRACE): the CTA with the most
// key blocks records clock64() at pipeline events of its first blocks into p.trace[role][block][event].
#ifdef FTB200_ATTN_TRACE
#define TRACE(role, blk, ev)                                                                        \
  do {                                                                                              \
    if (p.trace != nullptr && blockIdx.x == 0 && (blk) < 32)                                        \
      p.trace[((role) * 32 + (blk)) * 8 + (ev)] = clock64();                                        \
  } while (0)
#else
#define TRACE(role, blk, ev) \
  do {                       \
  } while (0)
#endif

constexpr int D = 128;       // head dim
constexpr int BQ = 128;      // queries per CTA
constexpr int BKV = 128;     // keys per block
constexpr uint32_t TILE_BYTES = 128 * 128 * 2;  // every operand tile: 128 x 128 bf16
constexpr uint32_t SLAB_BYTES = TILE_BYTES / 2;  // 128 rows x 64 elements, one swizzle atom wide
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 576;
constexpr int SOFTMAX_THREADS = 512;
constexpr int GROUPS = 4;   // threads per query row
constexpr int CPT = BKV / GROUPS;  // score columns per thread
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S = 0, COL_O = 256, COL_Q = 384;  // Q: 128 bf16 per row = 64 columns
// smem: K0 V0 | K1 V1 | barriers + exchange
constexpr uint32_t OFF_KV = 0;
constexpr uint32_t OFF_MISC = OFF_KV + KV_STAGES * 2 * TILE_BYTES;
constexpr uint32_t MISC_BYTES = 256 + 2 * GROUPS * BQ * 4;
constexpr uint32_t SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
constexpr float RESCALE_THRESHOLD = 8.0f;  // in log2 units

struct AttnParams {
  int batch, seq, n_heads, n_kv_heads;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  long long ld_o;    // row stride of O in elements
  const __nv_bfloat16* Q;
  long long ld_q;
  __nv_bfloat16* O;
  float* lse;        // [batch, n_heads, seq], natural log
  int* status;
  long long* trace;  // tuning aid, null unless built with FTB200_ATTN_TRACE
};

// barrier indices
enum : int {
  BAR_Q = 0,
  BAR_K_FULL = 1,    // +stage
  BAR_V_FULL = 3,    // +stage
  BAR_K_EMPTY = 5,   // +stage: K is free once its S MMA is done, long before V
  BAR_S_FULL = 7,    // +buf
  BAR_UNUSED = 9,    // (two slots kept so that the indices below stay put)
  BAR_P_FULL = 11,
  BAR_O_DONE = 12,
  BAR_XCHG = 13,     // +parity
  BAR_V_EMPTY = 15,  // +stage
  NUM_BARS = 17,
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_MISC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 196);
  float* xchg = reinterpret_cast<float*>(smem + OFF_MISC + 256);  // [parity][group][row]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto bar = [&](int i) { return bar_base + 8u * i; };

  // heavy (late) query blocks first: with a causal mask their work is largest
  const int n_qblocks = p.seq / BQ;
  const int per_block = p.batch * p.n_heads;
  const int qb = n_qblocks - 1 - static_cast<int>(blockIdx.x) / per_block;
  const int bh = static_cast<int>(blockIdx.x) % per_block;
  const int b = bh / p.n_heads, h = bh % p.n_heads;
  const int hk = h / (p.n_heads / p.n_kv_heads);
  const int n_kv = p.causal ? qb + 1 : p.seq / BKV;
  const int q_row0 = b * p.seq + qb * BQ;

  if (threadIdx.x == 0) {
    mbar_init(bar(BAR_Q), SOFTMAX_THREADS);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(bar(BAR_K_FULL + s), 1);
      mbar_init(bar(BAR_V_FULL + s), 1);
      mbar_init(bar(BAR_K_EMPTY + s), 1);
      mbar_init(bar(BAR_V_EMPTY + s), 1);
      mbar_init(bar(BAR_S_FULL + s), 1);
      mbar_init(bar(BAR_XCHG + s), SOFTMAX_THREADS);
    }
    mbar_init(bar(BAR_P_FULL), SOFTMAX_THREADS);
    mbar_init(bar(BAR_O_DONE), 1);
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
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t use = static_cast<uint32_t>(j >> 1);
        if (!mbar_wait(bar(BAR_K_EMPTY + st), (use & 1u) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        const uint32_t sk = smem_base + OFF_KV + st * 2 * TILE_BYTES;
        const uint32_t sv = sk + TILE_BYTES;
        const int kv_row0 = b * p.seq + j * BKV;
        mbar_expect_tx(bar(BAR_K_FULL + st), TILE_BYTES);
        tma_load_2d(sk, &tmK, bar(BAR_K_FULL + st), hk * D, kv_row0);
        tma_load_2d(sk + SLAB_BYTES, &tmK, bar(BAR_K_FULL + st), hk * D + 64, kv_row0);
        if (!mbar_wait(bar(BAR_V_EMPTY + st), (use & 1u) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        mbar_expect_tx(bar(BAR_V_FULL + st), TILE_BYTES);
        tma_load_2d(sv, &tmV, bar(BAR_V_FULL + st), hk * D, kv_row0);
        tma_load_2d(sv + SLAB_BYTES, &tmV, bar(BAR_V_FULL + st), hk * D + 64, kv_row0);
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
      // S = Q K^T: both operands K-major (head dim contiguous), M = N = 128
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BKV >> 3) << 17) |
                               (static_cast<uint32_t>(BQ >> 4) << 24);
      // O += P V: A = P K-major (keys contiguous), B = V MN-major (stored [key][d])
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(D >> 3) << 17) |
                               (static_cast<uint32_t>(BQ >> 4) << 24);
      // descriptor bases: one per buffer, constants per K step (the issue loop must stay short)
      constexpr uint32_t HI = smem_desc_hi(1024);
      const uint32_t k_lo = smem_desc_lo(smem_base + OFF_KV, 16);
      const uint32_t v_lo = smem_desc_lo(smem_base + OFF_KV + TILE_BYTES, SLAB_BYTES);
      constexpr uint32_t STAGE16 = (2 * TILE_BYTES) >> 4;
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t kb = k_lo + st * STAGE16;
        const uint32_t d_tmem = tmem_base + COL_S + st * BKV;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * SLAB_BYTES + (kk & 3) * 32) >> 4;
          umma_bf16_tmem_a(d_tmem, tmem_base + COL_Q + kk * 8, kb + off, HI, idesc_s, kk != 0);
        }
        umma_commit(bar(BAR_S_FULL + st));
        umma_commit(bar(BAR_K_EMPTY + st));
      };
      bool ok = mbar_wait(bar(BAR_Q), 0, abort_flag) && mbar_wait(bar(BAR_K_FULL + 0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t use = static_cast<uint32_t>(j >> 1);
        if (j + 1 < n_kv) {
          const int st1 = (j + 1) & 1;
          const uint32_t use1 = static_cast<uint32_t>((j + 1) >> 1);
          // S buffer st1 last held P of block j-1: its P V was issued above, and the tensor pipe runs in order
          if (!mbar_wait(bar(BAR_K_FULL + st1), use1 & 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          TRACE(0, j, 0);  // K of block j+1 present
          issue_s(j + 1);
          TRACE(0, j, 1);  // S of block j+1 issued
        }
        if (!mbar_wait(bar(BAR_P_FULL), static_cast<uint32_t>(j) & 1u, abort_flag) ||
            !mbar_wait(bar(BAR_V_FULL + st), use & 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        TRACE(0, j, 2);  // P of block j and V present
        const uint32_t vb = v_lo + st * STAGE16;
        const uint32_t d_tmem = tmem_base + COL_O;
        // P of keys 32g..32g+31 sits, two per column, in the first 16 of the 32 columns its thread group read S from
        const uint32_t p_tmem = tmem_base + COL_S + st * BKV;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          umma_bf16_tmem_a(d_tmem, p_tmem + (kk >> 1) * CPT + (kk & 1) * 8, vb + ((kk * 2048) >> 4), HI, idesc_o, (j | kk) != 0);
        }
        umma_commit(bar(BAR_V_EMPTY + st));
        umma_commit(bar(BAR_O_DONE));
        TRACE(0, j, 3);  // P V of block j issued
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax + epilogue (warps 2..17) ----------------
    const int sw = warp - 2;
    const int quarter = warp & 3;   // TMEM lane quarter this warp may touch
    const int g = sw >> 2;          // which 32 keys (and, in the epilogue, which 32 output columns)
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float m_used = -INFINITY, l_part = 0.f;
    bool ok = true;
    {
      // this thread's quarter of its query row -> TMEM (two head-dim elements per column)
      const uint4* src = reinterpret_cast<const uint4*>(p.Q + static_cast<long long>(q_row0 + row) * p.ld_q + h * D + g * 32);
      uint32_t qw[16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 v4 = src[c];
        qw[4 * c] = v4.x; qw[4 * c + 1] = v4.y; qw[4 * c + 2] = v4.z; qw[4 * c + 3] = v4.w;
      }
      tmem_st16(tmem_base + COL_Q + g * 16 + lane_addr, qw);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(BAR_Q));
    }
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      const uint32_t use = static_cast<uint32_t>(j >> 1);
      if (!mbar_wait(bar(BAR_S_FULL + st), use & 1u, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (threadIdx.x == 64) TRACE(1, j, 0);  // S complete
      uint32_t sv[CPT];
      tmem_ld32(tmem_base + COL_S + st * BKV + g * CPT + lane_addr, sv);
      tmem_wait_ld();
      if (threadIdx.x == 64) TRACE(1, j, 1);  // scores in registers

      if (p.causal && j == qb) {
        const int key0 = g * CPT;
#pragma unroll
        for (int c = 0; c < CPT; ++c)
          if (key0 + c > row) sv[c] = __float_as_uint(-INFINITY);
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < CPT; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sv[c]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float* xc = xchg + (st * GROUPS) * BQ;
      xc[g * BQ + row] = mx;
      mbar_arrive(bar(BAR_XCHG + st));
      if (!mbar_wait(bar(BAR_XCHG + st), use & 1u, abort_flag)) {
        ok = false;
        break;
      }
      const float m_new = fmaxf(fmaxf(xc[row], xc[BQ + row]), fmaxf(xc[2 * BQ + row], xc[3 * BQ + row]));
      if (threadIdx.x == 64) TRACE(1, j, 2);  // row maximum exchanged

      // raise the maximum only when it moved far; all threads of a row see the same numbers
      float alpha = 1.f;
      const bool raise = (m_new - m_used) * p.scale_log2 > RESCALE_THRESHOLD;
      const bool any_raise = __any_sync(0xffffffffu, raise) && j > 0;
      if (j == 0) {
        m_used = m_new;
      } else if (raise) {
        alpha = exp2f((m_used - m_new) * p.scale_log2);
        m_used = m_new;
        l_part *= alpha;
      }
      const float neg_m = -m_used * p.scale_log2;
      uint32_t packed[CPT / 2];
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < CPT / 2; ++c) {
        const float p0 = exp2f(fmaf(__uint_as_float(sv[2 * c]), p.scale_log2, neg_m));
        const float p1 = exp2f(fmaf(__uint_as_float(sv[2 * c + 1]), p.scale_log2, neg_m));
        sum4[c & 3] += p0 + p1;
        __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
        packed[c] = *reinterpret_cast<uint32_t*>(&pk);
      }
      l_part += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);

      if (threadIdx.x == 64) TRACE(1, j, 3);  // exponentials done
      // P replaces the scores this thread has just read (its own columns: nobody else touches them)
      tmem_st16(tmem_base + COL_S + st * BKV + g * CPT + lane_addr, packed);
      if (any_raise) {
        // O may only be touched once P V of the previous block is done
        if (!mbar_wait(bar(BAR_O_DONE), static_cast<uint32_t>(j - 1) & 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t o_addr = tmem_base + COL_O + g * 32 + lane_addr;
        uint32_t ov[32];
        tmem_ld32(o_addr, ov);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * alpha);
        tmem_st32(o_addr, ov);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(BAR_P_FULL));
      if (threadIdx.x == 64) TRACE(1, j, 4);  // P published
    }

    if (ok && mbar_wait(bar(BAR_O_DONE), static_cast<uint32_t>(n_kv - 1) & 1u, abort_flag)) {
      tc_fence_after();
      // total row sum: the threads of a row hold partial sums over their keys
      float* xc = xchg;  // both parities are free again
      xc[g * BQ + row] = l_part;
      const uint32_t xuse = static_cast<uint32_t>((n_kv + 1) >> 1);  // completed phases of XCHG+0 so far
      mbar_arrive(bar(BAR_XCHG + 0));
      if (mbar_wait(bar(BAR_XCHG + 0), xuse & 1u, abort_flag)) {
        const float l = (xc[row] + xc[BQ + row]) + (xc[2 * BQ + row] + xc[3 * BQ + row]);
        const float inv = 1.f / l;
        __nv_bfloat16* dst = p.O + static_cast<long long>(q_row0 + row) * p.ld_o + h * D + g * 32;
        uint32_t ov[32];
        tmem_ld32(tmem_base + COL_O + g * 32 + lane_addr, ov);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(ov[8 * c + e]) * inv;
          reinterpret_cast<ftb200::bf16x8*>(dst)[c] = ftb200::pack8(f);
        }
        if (g == 0 && p.lse != nullptr) {
          p.lse[(static_cast<long long>(b) * p.n_heads + h) * p.seq + qb * BQ + row] =
              (m_used * p.scale_log2 + log2f(l)) * 0.6931471805599453f;
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

// [rows, cols] bf16 view with row stride ld (elements); box = 64 columns x box_rows rows, 128-byte swizzle
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

// q: [batch*seq, n_heads*128] view with row stride ld_q; k, v: [batch*seq, n_kv_heads*128] views with row
// strides ld_k, ld_v; o: [batch*seq, n_heads*128] with row stride ld_o.  lse (may be null):
// [batch, n_heads, seq] fp32.  seq must be a multiple of 128.
FTB200_API int ftb200_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int seq,
                                    int n_heads, int n_kv_heads, int head_dim, long long ld_q, long long ld_k,
                                    long long ld_v, long long ld_o, float scale, int causal, int* status,
                                    cudaStream_t stream) {
  if (head_dim != D || batch <= 0 || seq <= 0 || seq % BQ != 0 || n_heads <= 0 || n_kv_heads <= 0 ||
      n_heads % n_kv_heads != 0)
    return FTB200_E_BADARG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || (ld_q & 7) || (ld_k & 7) || (ld_v & 7) ||
      (ld_o & 7))
    return FTB200_E_ALIGN;
  CUtensorMap tk, tv;
  const long long rows = static_cast<long long>(batch) * seq;
  int rc = encode_rows(&tk, k, rows, static_cast<long long>(n_kv_heads) * D, ld_k, BKV);
  if (rc == 0) rc = encode_rows(&tv, v, rows, static_cast<long long>(n_kv_heads) * D, ld_v, BKV);
  if (rc != 0) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return FTB200_E_CUDA;
    attr_set = true;
  }
  AttnParams p;
  p.batch = batch; p.seq = seq; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.Q = reinterpret_cast<const __nv_bfloat16*>(q); p.ld_q = ld_q;
  p.ld_o = ld_o; p.O = reinterpret_cast<__nv_bfloat16*>(o); p.lse = lse; p.status = status;
  p.trace = nullptr;
#ifdef FTB200_ATTN_TRACE
  p.trace = reinterpret_cast<long long*>(lse) + (static_cast<long long>(batch) * n_heads * seq + 1) / 2;  // caller over-allocates lse
#endif
  const long long grid = static_cast<long long>(batch) * n_heads * (seq / BQ);
  if (grid > 0x7fffffffLL) return FTB200_E_TOOBIG;
  attention_fwd_kernel<<<static_cast<unsigned>(grid), NUM_THREADS, SMEM_BYTES, stream>>>(tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}
