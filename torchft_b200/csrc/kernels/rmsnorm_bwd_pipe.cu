// RMSNorm backward with its rows streamed through shared memory by bulk asynchronous copies.
//
//   dx = dres + rstd * w * dy - x * rstd^3 / D * sum(dy * w * x);   dw partial sums per block
//
// The plain kernel (elementwise.cu) loads two rows, reduces, stores, and starts over: its loads
// are in flight only between two block-wide reductions, which leaves HBM idle half of the time
// (0.49 of the copy rate).  Here a producer warp keeps a ring of STAGES rows (dy, x and the
// residual gradient of one token each) in flight with cp.async.bulk, independent of what the
// consumer warps are doing; the consumers take a row's vectors from shared memory into
// registers, free the stage at once, and do the reduction and the store from registers.  One CTA
// per SM with a ring of eight rows keeps close to 200 KB of loads in flight per SM at all times.
//
// Every mbarrier wait is bounded; on expiry the CTA records FTB200_ST_TIMEOUT in the caller's
// status word and returns (the producer first gives its copies in flight time to land).
#include <algorithm>

#include "ftb200_common.cuh"
#include "tcgen05_helpers.cuh"

using ftb200::bf16x8;
using ftb200::pack8;
using ftb200::unpack8;

namespace {

using namespace ftb200::tc;

constexpr int STAGES = 8;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void consumer_sync(int n) { asm volatile("bar.sync 1, %0;" ::"r"(n) : "memory"); }

// blockDim.x = consumers + 32 (the last warp is the producer); consumers == D8 rounded up to a warp multiple.
__global__ void __launch_bounds__(544, 1)
rmsnorm_bwd_pipe_kernel(const bf16x8* __restrict__ dy, const bf16x8* __restrict__ x, const bf16x8* __restrict__ w,
                        const float* __restrict__ rstd, const bf16x8* __restrict__ dres, bf16x8* __restrict__ dx,
                        float* __restrict__ dw_partial, int T, int D8, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int consumers = blockDim.x - 32;
  const int ntens = dres != nullptr ? 3 : 2;
  const uint32_t row_bytes = static_cast<uint32_t>(D8) * 16u;
  const uint32_t stage_bytes = 3u * row_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * stage_bytes);
  float* scratch = reinterpret_cast<float*>(bars + 2 * STAGES);  // 66 floats
  volatile int* abort_flag = reinterpret_cast<volatile int*>(scratch + 66);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full = [&](int s) { return bar_base + 8u * s; };
  auto empty = [&](int s) { return bar_base + 8u * (STAGES + s); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), consumers / 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  __syncthreads();

  const int n_rows = (T - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (warp == consumers / 32) {
    // ---------------- producer ----------------
    if (lane == 0) {
      bool ok = true;
      for (int k = 0; k < n_rows && ok; ++k) {
        const int s = k % STAGES;
        const uint32_t use = static_cast<uint32_t>(k / STAGES);
        if (!mbar_wait(empty(s), (use & 1u) ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        const int64_t row = static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(k) * gridDim.x;
        const uint32_t dst = smem_base + s * stage_bytes;
        mbar_expect_tx(full(s), ntens * row_bytes);
        bulk_load(dst, dy + row * D8, row_bytes, full(s));
        bulk_load(dst + row_bytes, x + row * D8, row_bytes, full(s));
        if (dres != nullptr) bulk_load(dst + 2 * row_bytes, dres + row * D8, row_bytes, full(s));
      }
      if (!ok) {
        // copies in flight land in this CTA's shared memory: give them time before the CTA exits
        const uint64_t t0 = ftb200::globaltimer_ns();
        while (ftb200::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    return;
  }

  // ---------------- consumers: one 16-byte column group each ----------------
  const int i = threadIdx.x;
  const bool col_live = i < D8;
  float wc[8];
  {
    bf16x8 wv = {};
    if (col_live) wv = w[i];
    unpack8(wv, wc);
  }
  float dw_acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) dw_acc[e] = 0.f;

  for (int k0 = 0; k0 < n_rows; k0 += 2) {
    bf16x8 a[2] = {}, b[2] = {}, d[2] = {};
    float r[2] = {0.f, 0.f};
    bool live[2];
    int64_t rows[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int k = k0 + j;
      live[j] = k < n_rows;
      rows[j] = static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(k) * gridDim.x;
      if (!live[j]) continue;
      const int s = k % STAGES;
      const bool ok = mbar_wait(full(s), static_cast<uint32_t>(k / STAGES) & 1u, abort_flag);
      if (ok && col_live) {
        const bf16x8* srow = reinterpret_cast<const bf16x8*>(smem + s * stage_bytes);
        a[j] = srow[i];
        b[j] = srow[D8 + i];
        if (dres != nullptr) d[j] = srow[2 * D8 + i];
      }
      r[j] = rstd[rows[j]];
      __syncwarp();
      if (lane == 0) mbar_arrive(empty(s));  // the row is in registers: the stage can be refilled
    }
    float dot[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float fa[8], fb[8];
      unpack8(a[j], fa);
      unpack8(b[j], fb);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dot[j] += fa[e] * wc[e] * fb[e];
        dw_acc[e] += fa[e] * fb[e] * r[j];
      }
    }
    // two block-wide sums over the consumer warps (named barrier: the producer warp is not part of it)
    dot[0] = ftb200::warp_sum(dot[0]);
    dot[1] = ftb200::warp_sum(dot[1]);
    consumer_sync(consumers);
    if (lane == 0) {
      scratch[warp] = dot[0];
      scratch[33 + warp] = dot[1];
    }
    consumer_sync(consumers);
    if (*abort_flag) {  // read after a barrier that every consumer has passed: the same answer in all of them
      if (threadIdx.x == 0 && status != nullptr) atomicExch(status, FTB200_ST_TIMEOUT);
      return;
    }
    const int nw = consumers / 32;
    float ra = (lane < nw) ? scratch[lane] : 0.f;
    float rb = (lane < nw) ? scratch[33 + lane] : 0.f;
    ra = ftb200::warp_sum(ra);
    rb = ftb200::warp_sum(rb);
    const float coef[2] = {ra * r[0] * r[0] * r[0] / (8.f * D8), rb * r[1] * r[1] * r[1] / (8.f * D8)};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (live[j] && col_live) {
        float fa[8], fb[8], o[8];
        unpack8(a[j], fa);
        unpack8(b[j], fb);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = r[j] * wc[e] * fa[e] - fb[e] * coef[j];
        if (dres != nullptr) {
          float fd[8];
          unpack8(d[j], fd);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += fd[e];
        }
        dx[rows[j] * D8 + i] = pack8(o);
      }
    }
  }
  if (col_live) {
    float* dst = dw_partial + (static_cast<int64_t>(blockIdx.x) * D8 + i) * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) dst[e] = dw_acc[e];
  }
}

// dw[c] (+)= sum_b partial[b][c]: 32 columns per block, 8 warps striding over the rows
__global__ void colsum_partials_pipe_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw, int nblk,
                                            int D, int accumulate) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < D) {
#pragma unroll 4
    for (int b = ry; b < nblk; b += 8) s += partial[static_cast<int64_t>(b) * D + c];
  }
  red[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][cx];
    if (accumulate) t += __bfloat162float(dw[c]);
    dw[c] = __float2bfloat16(t);
  }
}

}  // namespace

// Same contract as ftb200_rmsnorm_bwd (dw_partial: at least 2 * SM count * D floats); rows of up to 4096 elements.
// Returns FTB200_E_TOOBIG for wider rows (use the plain kernel there).
FTB200_API int ftb200_rmsnorm_bwd_pipe(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                       void* dx, void* dw, float* dw_partial, int T, int D, int accumulate_dw, int* status,
                                       cudaStream_t st) {
  if (D % 8) return FTB200_E_ALIGN;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx) |
       reinterpret_cast<uintptr_t>(dres) | reinterpret_cast<uintptr_t>(w)) & 15)
    return FTB200_E_ALIGN;
  const int D8 = D / 8;
  if (D8 > 512) return FTB200_E_TOOBIG;
  if (T <= 0) return 0;
  const int consumers = std::max(32, (D8 + 31) / 32 * 32);
  const size_t smem = static_cast<size_t>(STAGES) * 3 * D8 * 16 + 2 * STAGES * 8 + 66 * 4 + 16 + 128;
  static size_t attr_bytes = 0;
  if (smem > attr_bytes) {
    if (cudaFuncSetAttribute(rmsnorm_bwd_pipe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return FTB200_E_CUDA;
    attr_bytes = smem;
  }
  const int nblk = std::min(T, ftb200::sm_count());
  rmsnorm_bwd_pipe_kernel<<<nblk, consumers + 32, smem, st>>>((const bf16x8*)dy, (const bf16x8*)x, (const bf16x8*)w, rstd,
                                                              (const bf16x8*)dres, (bf16x8*)dx, dw_partial, T, D8, status);
  colsum_partials_pipe_kernel<<<(D + 31) / 32, 256, 0, st>>>(dw_partial, (__nv_bfloat16*)dw, nblk, D, accumulate_dw);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}
