// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM,
// operands staged by TMA), written for sm_100a only.
//
//   C[M,N] (+)= A[M,K] * B[N,K]^T        fp32 accumulate, bf16 or fp32 output
//
// Either operand may be stored "K-major" (reduction dimension contiguous, i.e. the
// row-major [rows, K] matrix) or "MN-major" (the row-major [K, rows] matrix); the
// three GEMMs of a linear layer (forward, dgrad, wgrad) then run without any
// transposed copies:
//   forward  Y = X W^T      A = X  (K-major)   B = W  (K-major)
//   dgrad   dX = dY W       A = dY (K-major)   B = W  (MN-major)
//   wgrad   dW = dY^T X     A = dY (MN-major)  B = X  (MN-major)
//
// Kernel structure: persistent, one CTA per SM, 128x256 output tile, 64-deep K slabs
// in a 4-stage TMA ring.  Warp 0 is the TMA producer, warp 1 allocates TMEM and
// issues the MMAs (a single elected thread), warps 2..5 drain the accumulator
// (tcgen05.ld) and write C.  The accumulator is double-buffered in TMEM (2 x 256
// columns) so that the epilogue of tile i overlaps the main loop of tile i+1.
//
// Every mbarrier wait is bounded (wall-clock limit read from %globaltimer); when a
// wait expires the CTA raises a shared abort flag, records FTB200_ST_TIMEOUT in the
// caller's status word, drains, frees its TMEM and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "ftb200_common.cuh"
#include "tcgen05_helpers.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr uint32_t B_BYTES = BN * BK * 2;
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int GROUP_M = 16;

using namespace ftb200::tc;

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;      // operand storage: 0 = K-major, 1 = MN-major
  int out_fp32;        // 0: bf16 C, 1: fp32 C
  int accumulate;      // C += result (read-modify-write in the epilogue)
  long long ldc;
  void* C;
  int* status;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle atoms must sit on 1024-byte boundaries.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

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
      mbar_init(tempty_bar(s), 128);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_k = (p.K + BK - 1) / BK;
  const int tiles_per_group = GROUP_M * num_n;

  auto tile_coords = [&](int t, int& m0, int& n0) {
    const int g = t / tiles_per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(num_m - first_m, GROUP_M);
    const int r = t - g * tiles_per_group;
    m0 = (first_m + r % gsz) * BM;
    n0 = (r / gsz) * BN;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m0, n0;
        tile_coords(t, m0, n0);
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const int k0 = kb * BK;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          if (p.a_mn == 0) {
            tma_load_2d(sa, &tmA, full_bar(stage), k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * (BK * 128), &tmA, full_bar(stage), m0 + 64 * j, k0);
          }
          if (p.b_mn == 0) {
            tma_load_2d(sb, &tmB, full_bar(stage), k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &tmB, full_bar(stage), n0 + 64 * j, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // give copies that are still in flight time to land before the CTA retires
        const uint64_t t0 = ftb200::globaltimer_ns();
        while (ftb200::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(p.a_mn) << 15) |
                             (static_cast<uint32_t>(p.b_mn) << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                             (static_cast<uint32_t>(BM >> 4) << 24);
      // K-major: 8-row groups 1024 B apart, step 32 B along K inside the swizzle row.
      // MN-major: 64-element column blocks BK*128 B apart, 8-deep K groups 1024 B apart,
      //           step 16 K rows = 2048 B.
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, a_step = p.a_mn ? 2048 : 32;
      const uint32_t b_lbo = p.b_mn ? BK * 128 : 16, b_step = p.b_mn ? 2048 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
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
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = p.out_fp32 ? ((p.ldc & 3) == 0) : ((p.ldc & 7) == 0);
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int m0, n0;
      tile_coords(t, m0, n0);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr0 = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
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
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
                const float v = __uint_as_float(r[j]);
                dst[j] = p.accumulate ? dst[j] + v : v;
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
                reinterpret_cast<ftb200::bf16x8*>(dst)[j] = ftb200::pack8(f);
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
                float v = __uint_as_float(r[j]);
                if (p.accumulate) v += __bfloat162float(dst[j]);
                dst[j] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(tempty_bar(acc));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, FTB200_ST_TIMEOUT);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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

// rows x cols bf16 matrix, `cols` contiguous, row stride `ld` elements; box = box_cols x box_rows.
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

// C[M,N] (+)= A * B^T with A logical [M,K], B logical [N,K].
//   a_mn_major == 0: A stored row-major [M,K] (row stride lda); == 1: stored row-major [K,M].
//   b_mn_major == 0: B stored row-major [N,K] (row stride ldb); == 1: stored row-major [K,N].
//   flags bit0: fp32 output; bit1: accumulate into C.
// `status` may be null; otherwise a device int that receives FTB200_ST_TIMEOUT if a
// pipeline wait expired.  `max_ctas` <= 0 means one CTA per SM.
FTB200_API int ftb200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int a_mn_major,
                                int b_mn_major, long long lda, long long ldb, long long ldc, int flags, int* status,
                                int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || A == nullptr || B == nullptr || C == nullptr) return FTB200_E_BADARG;
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
    rc = encode_2d(&tmB, B, N, K, ldb, BK, BN);
  else
    rc = encode_2d(&tmB, B, K, N, ldb, 64, BK);
  if (rc) return rc;

  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
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
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int ctas = ftb200::sm_count();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (tiles < ctas) ctas = tiles;
  gemm_bf16_tcgen05_kernel<<<ctas, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}
