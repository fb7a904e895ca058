// Shared device/host helpers for the torchft_b200 sm_100a kernels.
//
// Conventions used by every kernel in this directory:
//  * the C ABI entry points return 0 on a successful launch and a negative
//    FTB200_E_* code when the arguments are rejected on the host;
//  * device-side waits are bounded: on expiry a kernel stores a FTB200_ST_* code
//    into the caller's status word and returns normally (no trap, no assert);
//  * nothing in here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FTB200_API extern "C" __attribute__((visibility("default")))

// host-side argument errors
#define FTB200_E_BADARG (-1)
#define FTB200_E_ALIGN (-2)
#define FTB200_E_DRIVER (-3)
#define FTB200_E_TOOBIG (-4)
#define FTB200_E_CUDA (-5)

// device-side status word values (0 == ok)
#define FTB200_ST_OK 0
#define FTB200_ST_TIMEOUT 1
#define FTB200_ST_ABORTED 2
#define FTB200_ST_EPOCH 3
#define FTB200_ST_BOUNDS 4

// Checked-index debug build (-DFT_BOUNDS_CHECK=1, FTB200_BOUNDS_CHECK=1 for the build driver):
// FTB_IN_RANGE(i, n) is true for 0 <= i < n; otherwise it records FTB200_ST_BOUNDS and the
// offending index in a per-translation-unit device word and is false, and the caller skips
// the access.  In the normal build it is the constant `true` and costs nothing.  Used where an
// index derives from data or from caller-supplied strides (token ids, targets, row strides,
// shard owners, copy tables); loops bounded by their own extent are not decorated.
// FTB_DEFINE_BOUNDS_QUERY(tag) exports `ftb200_bounds_status_<tag>(long long* index)`, which
// returns the recorded code and clears it.
#ifdef FT_BOUNDS_CHECK
namespace ftb200 {
namespace dbg {
static __device__ int g_bounds_status;
static __device__ long long g_bounds_index;
__device__ __forceinline__ bool in_range(long long i, long long n) {
  if (i >= 0 && i < n) return true;
  if (atomicCAS(&g_bounds_status, 0, FTB200_ST_BOUNDS) == 0) g_bounds_index = i;
  return false;
}
}  // namespace dbg
}  // namespace ftb200
#define FTB_IN_RANGE(i, n) ftb200::dbg::in_range(static_cast<long long>(i), static_cast<long long>(n))
#define FTB_DEFINE_BOUNDS_QUERY(tag)                                                                     \
  FTB200_API int ftb200_bounds_status_##tag(long long* index) {                                          \
    int st = 0;                                                                                          \
    long long idx = 0;                                                                                   \
    if (cudaMemcpyFromSymbol(&st, ftb200::dbg::g_bounds_status, sizeof(st)) != cudaSuccess) return -5;   \
    if (cudaMemcpyFromSymbol(&idx, ftb200::dbg::g_bounds_index, sizeof(idx)) != cudaSuccess) return -5;  \
    const int zero = 0;                                                                                  \
    if (cudaMemcpyToSymbol(ftb200::dbg::g_bounds_status, &zero, sizeof(zero)) != cudaSuccess) return -5; \
    if (index != nullptr) *index = idx;                                                                  \
    return st;                                                                                           \
  }
#else
#define FTB_IN_RANGE(i, n) true
#define FTB_DEFINE_BOUNDS_QUERY(tag)
#endif

namespace ftb200 {

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blocks whose size is a multiple of 32 (<= 1024 threads).
// `scratch` must hold 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) {
    r = warp_sum(r);
    if (lane == 0) scratch[32] = r;
  }
  __syncthreads();
  return scratch[32];
}

// Two block-wide sums for the price of one (same barriers).  `scratch` must hold 66 floats.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) {
    scratch[warp] = a;
    scratch[33 + warp] = b;
  }
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float ra = (threadIdx.x < nw) ? scratch[threadIdx.x] : 0.f;
  float rb = (threadIdx.x < nw) ? scratch[33 + threadIdx.x] : 0.f;
  if (warp == 0) {
    ra = warp_sum(ra);
    rb = warp_sum(rb);
    if (lane == 0) {
      scratch[32] = ra;
      scratch[65] = rb;
    }
  }
  __syncthreads();
  return make_float2(scratch[32], scratch[65]);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nw) ? scratch[threadIdx.x] : -INFINITY;
  if (warp == 0) {
    r = warp_max(r);
    if (lane == 0) scratch[32] = r;
  }
  __syncthreads();
  return scratch[32];
}

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace ftb200
