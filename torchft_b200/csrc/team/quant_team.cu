// Block-scaled fp8 (e4m3) quantisation and the quantised allreduce over peer memory.
//
// Format: the tensor is cut into blocks of 128 consecutive elements; each block stores 128
// e4m3 bytes and one fp32 scale s = absmax / 448 (value = s * decode(byte)).  A quantised
// buffer of n elements is laid out as [n bytes of codes][n/128 fp32 scales].  This is finer
// than the per-row scales of the reference's Triton kernels (torchft/quantization.py:53-162)
// and costs 1.03 bytes per element whatever the tensor's shape.
//
// Kernels:
//   quantize / dequantize / reduce      single-GPU building blocks (one warp per block)
//   allreduce_fp8                       ONE kernel per rank: [optional pseudo-gradient
//       g = a - b] -> quantise into the rank's arena -> ready round -> reduce own slice from
//       all peers (fp32), scale, requantise, write the slice into every peer's arena -> done
//       round -> dequantise everything into the output tensor.
//   diloco_outer_step                   fused Nesterov outer update + backup write + blend
//       with the local weights (runs after the commit vote, so it is not folded into the
//       allreduce kernel).
#include <cuda_fp8.h>

#include <algorithm>
#include <vector>

#include "ftb200_common.cuh"
#include "team_device.cuh"

using namespace ftb200::team;

namespace {

constexpr int QB = 128;  // elements per scale block
constexpr float FP8_MAX = 448.f;

template <typename T>
__device__ __forceinline__ void load4(const T* p, float* f);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float* f);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(f[0], f[1]), hi = __floats2bfloat162_rn(f[2], f[3]);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&lo);
  o.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = o;
}

__device__ __forceinline__ uint32_t encode4(const float* f, float inv_scale) {
  __nv_fp8x4_e4m3 q(make_float4(f[0] * inv_scale, f[1] * inv_scale, f[2] * inv_scale, f[3] * inv_scale));
  return q.__x;
}
__device__ __forceinline__ void decode4(uint32_t bits, float scale, float* f) {
  __nv_fp8x4_e4m3 q;
  q.__x = bits;
  const float4 v = static_cast<float4>(q);
  f[0] = v.x * scale; f[1] = v.y * scale; f[2] = v.z * scale; f[3] = v.w * scale;
}

// Eight lanes quantise one 128-element block (16 consecutive elements per lane), so a warp
// handles four blocks at a time and the abs-max needs three shuffles.
constexpr int EPL = 16;                 // elements per lane
constexpr int LPB = QB / EPL;           // lanes per block (8)
constexpr int BPW = 32 / LPB;           // blocks per warp iteration (4)

template <typename T>
__device__ __forceinline__ void load16(const T* p, float* f) {
#pragma unroll
  for (int k = 0; k < 4; ++k) load4<T>(p + 4 * k, f + 4 * k);
}
template <typename T>
__device__ __forceinline__ void store16(T* p, const float* f) {
#pragma unroll
  for (int k = 0; k < 4; ++k) store4<T>(p + 4 * k, f + 4 * k);
}
__device__ __forceinline__ float group8_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  return v;
}
__device__ __forceinline__ float absmax16(const float* f) {
  float m = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) m = fmaxf(m, fabsf(f[e]));
  return m;
}
__device__ __forceinline__ uint4 encode16(const float* f, float inv_scale) {
  uint4 q;
  q.x = encode4(f, inv_scale);
  q.y = encode4(f + 4, inv_scale);
  q.z = encode4(f + 8, inv_scale);
  q.w = encode4(f + 12, inv_scale);
  return q;
}
__device__ __forceinline__ void decode16(const uint4& q, float scale, float* f) {
  decode4(q.x, scale, f);
  decode4(q.y, scale, f + 4);
  decode4(q.z, scale, f + 8);
  decode4(q.w, scale, f + 12);
}

// Quantise the lane's 16 values of block `blk`; all 8 lanes of the block's group must call.
__device__ __forceinline__ void quantize_block16(const float* f, int sub, uint4* codes, float* scales, long long blk) {
  const float amax = group8_max(absmax16(f));
  const float scale = amax > 0.f ? amax / FP8_MAX : 1.f;
  codes[blk * LPB + sub] = encode16(f, 1.f / scale);
  if (sub == 0) scales[blk] = scale;
}

template <typename T>
__global__ void quantize_kernel(const T* __restrict__ a, const T* __restrict__ b, uint4* __restrict__ codes,
                                float* __restrict__ scales, long long nblocks) {
  const int lane = threadIdx.x & 31, sub = lane & (LPB - 1), bw = lane / LPB;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long blk0 = warp * BPW; blk0 < nblocks; blk0 += nwarps * BPW) {
    const long long blk = blk0 + bw;
    const bool live = blk < nblocks;
    float f[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) f[e] = 0.f;
    if (live) {
      load16<T>(a + blk * QB + sub * EPL, f);
      if (b != nullptr) {
        float g[EPL];
        load16<T>(b + blk * QB + sub * EPL, g);
#pragma unroll
        for (int e = 0; e < EPL; ++e) f[e] -= g[e];
      }
    }
    const float amax = group8_max(absmax16(f));
    if (live) {
      const float scale = amax > 0.f ? amax / FP8_MAX : 1.f;
      codes[blk * LPB + sub] = encode16(f, 1.f / scale);
      if (sub == 0) scales[blk] = scale;
    }
  }
}

template <typename T>
__global__ void dequantize_kernel(const uint4* __restrict__ codes, const float* __restrict__ scales,
                                  T* __restrict__ out, long long nblocks) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;  // one 16-element piece each
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = idx; i < nblocks * LPB; i += stride) {
    float f[EPL];
    decode16(codes[i], scales[i / LPB], f);
    store16<T>(out + i * EPL, f);
  }
}

struct QuantAllreduceArgs {
  uint8_t* arena[MAX_RANKS];  // every rank's quantised buffer: [n codes][n/128 scales]
  const void* in_a;           // local input (or the "global" operand of a pseudo-gradient)
  const void* in_b;           // optional: subtracted from in_a
  void* out;                  // local output, same dtype as the input
  long long n;                // elements, multiple of 128 * world
  float scale;                // applied to the reduced values (1/num_participants for AVG)
  int zero_contribution;
};

template <typename T>
__device__ __forceinline__ void allreduce_fp8_body(const TeamParams& tp, const QuantAllreduceArgs& a) {
  __shared__ int sh_code;
  const int lane = threadIdx.x & 31, sub = lane & (LPB - 1), bw = lane / LPB;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long nblocks = a.n / QB;
  uint4* my_codes = reinterpret_cast<uint4*>(a.arena[tp.rank]);
  float* my_scales = reinterpret_cast<float*>(a.arena[tp.rank] + a.n);

  // ---- quantise the local contribution into this rank's arena
  const T* ia = reinterpret_cast<const T*>(a.in_a);
  const T* ib = reinterpret_cast<const T*>(a.in_b);
  // two block groups per iteration so that twice as many loads are in flight per lane
  for (long long blk0 = warp * BPW; blk0 < nblocks; blk0 += 2 * nwarps * BPW) {
    float f[2][EPL];
    long long blk[2];
    bool live[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      blk[u] = blk0 + u * nwarps * BPW + bw;
      live[u] = blk[u] < nblocks;
#pragma unroll
      for (int e = 0; e < EPL; ++e) f[u][e] = 0.f;
      if (live[u] && !a.zero_contribution) load16<T>(ia + blk[u] * QB + sub * EPL, f[u]);
    }
    if (ib != nullptr && !a.zero_contribution) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (live[u]) {
          float g[EPL];
          load16<T>(ib + blk[u] * QB + sub * EPL, g);
#pragma unroll
          for (int e = 0; e < EPL; ++e) f[u][e] -= g[e];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float amax = group8_max(absmax16(f[u]));
      if (live[u]) {
        const float s = amax > 0.f ? amax / FP8_MAX : 1.f;
        my_codes[blk[u] * LPB + sub] = encode16(f[u], 1.f / s);
        if (sub == 0) my_scales[blk[u]] = s;
      }
    }
  }
  if (!grid_arrive(tp, 2, &sh_code)) return;
  if (!team_round(tp, 0, 0, &sh_code)) return;

  // ---- reduce this rank's slice over all peers, requantise, hand the slice to everybody
  const long long per = nblocks / tp.world;
  const long long lo = per * tp.rank;
  for (long long b0 = warp * BPW; b0 < per; b0 += nwarps * BPW) {
    const long long b = b0 + bw;
    const bool live = b < per;
    const long long blk = lo + (live ? b : 0);
    uint4 bits[MAX_RANKS];
    float sc[MAX_RANKS];
#pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      if (k < tp.world && live) {
        const int p = (tp.rank + k) % tp.world;
        bits[k] = reinterpret_cast<const uint4*>(a.arena[p])[blk * LPB + sub];
        sc[k] = reinterpret_cast<const float*>(a.arena[p] + a.n)[blk];
      }
    }
    float acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
#pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      if (k < tp.world && live) {
        float f[EPL];
        decode16(bits[k], sc[k], f);
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] += f[e];
      }
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] *= a.scale;
    const float amax = group8_max(absmax16(acc));
    if (live) {
      const float s = amax > 0.f ? amax / FP8_MAX : 1.f;
      const uint4 q = encode16(acc, 1.f / s);
      for (int k = 0; k < tp.world; ++k) {
        const int p = (tp.rank + k) % tp.world;
        reinterpret_cast<uint4*>(a.arena[p])[blk * LPB + sub] = q;
        if (sub == 0) reinterpret_cast<float*>(a.arena[p] + a.n)[blk] = s;
      }
    }
  }
  if (!grid_arrive(tp, 3, &sh_code)) return;
  if (!team_round(tp, 1, 1, &sh_code)) return;

  // ---- dequantise the complete result
  T* out = reinterpret_cast<T*>(a.out);
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  // four pieces in flight per thread: the loop is a pure stream and latency-bound otherwise
  const long long npieces = nblocks * LPB;
  for (long long i0 = tid; i0 < npieces; i0 += 4 * nthreads) {
    uint4 q[4];
    float sc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * nthreads;
      if (i < npieces) {
        q[u] = my_codes[i];
        sc[u] = my_scales[i / LPB];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * nthreads;
      if (i < npieces) {
        float f[EPL];
        decode16(q[u], sc[u], f);
        store16<T>(out + i * EPL, f);
      }
    }
  }
}

template <typename T>
__global__ void __maxnreg__(96) allreduce_fp8_kernel(const TeamParams tp, const QuantAllreduceArgs a) {
  allreduce_fp8_body<T>(tp, a);
}
template <typename T>
__global__ void __launch_bounds__(512) allreduce_fp8_emul_kernel(const TeamParams* tps, const QuantAllreduceArgs* as) {
  allreduce_fp8_body<T>(tps[blockIdx.y], as[blockIdx.y]);
}

// Outer (global) optimizer step of DiLoCo on flat buffers:
//   v = mu v + g ; u = nesterov ? g + mu v : v ; G = backup - lr u ; backup = G ;
//   param = G + alpha (param_local - G)
template <typename T>
__global__ void diloco_outer_kernel(const T* __restrict__ g, float* __restrict__ momentum, T* __restrict__ backup,
                                    T* __restrict__ param, long long n, float lr, float mu, float alpha, int nesterov,
                                    int first_step) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i + 4 <= n; i += stride) {
    float gg[4], bb[4], pp[4], vv[4];
    load4<T>(g + i, gg);
    load4<T>(backup + i, bb);
    load4<T>(param + i, pp);
    if (mu != 0.f) load4<float>(momentum + i, vv);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float u = gg[e];
      if (mu != 0.f) {
        vv[e] = first_step ? gg[e] : mu * vv[e] + gg[e];
        u = nesterov ? gg[e] + mu * vv[e] : vv[e];
      }
      const float G = bb[e] - lr * u;
      bb[e] = G;
      pp[e] = G + alpha * (pp[e] - G);
    }
    if (mu != 0.f) store4<float>(momentum + i, vv);
    store4<T>(backup + i, bb);
    store4<T>(param + i, pp);
  }
}

int grid_for_blocks(long long nblocks) {
  long long g = (nblocks * 8 + 511) / 512;
  return static_cast<int>(std::max<long long>(1, std::min<long long>(g, ftb200::sm_count() * 4LL)));
}

}  // namespace

// dtype: 0 bf16, 1 fp32.  codes: n bytes, scales: n/128 floats.  b (optional) is subtracted.
FTB200_API int ftb200_quantize_fp8(const void* a, const void* b, void* codes, float* scales, long long n, int dtype,
                                   cudaStream_t st) {
  if (n <= 0 || n % QB) return FTB200_E_ALIGN;
  const long long nb = n / QB;
  if (dtype == 0)
    quantize_kernel<__nv_bfloat16><<<grid_for_blocks(nb), 512, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                        (uint4*)codes, scales, nb);
  else
    quantize_kernel<float><<<grid_for_blocks(nb), 512, 0, st>>>((const float*)a, (const float*)b, (uint4*)codes, scales, nb);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_dequantize_fp8(const void* codes, const float* scales, void* out, long long n, int dtype,
                                     cudaStream_t st) {
  if (n <= 0 || n % QB) return FTB200_E_ALIGN;
  const long long nb = n / QB;
  if (dtype == 0)
    dequantize_kernel<__nv_bfloat16><<<grid_for_blocks(nb), 512, 0, st>>>((const uint4*)codes, scales, (__nv_bfloat16*)out, nb);
  else
    dequantize_kernel<float><<<grid_for_blocks(nb), 512, 0, st>>>((const uint4*)codes, scales, (float*)out, nb);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// arena[i]: rank i's quantised buffer (n + n/128*4 bytes, 16-byte aligned) inside its exported arena.
FTB200_API int ftb200_team_allreduce_fp8(const ftb200_team_desc* d, void* const* arena, const void* in_a, const void* in_b,
                                         void* out, long long n, int dtype, float scale, int zero_contribution, int ctas,
                                         cudaStream_t st) {
  if (d->world < 1 || d->world > MAX_RANKS || n <= 0) return FTB200_E_BADARG;
  if (n % (static_cast<long long>(QB) * d->world)) return FTB200_E_ALIGN;
  QuantAllreduceArgs a;
  for (int i = 0; i < MAX_RANKS; ++i) a.arena[i] = i < d->world ? reinterpret_cast<uint8_t*>(arena[i]) : nullptr;
  a.in_a = in_a; a.in_b = in_b; a.out = out; a.n = n; a.scale = scale; a.zero_contribution = zero_contribution;
  const int grid = ctas > 0 ? ctas : std::min(grid_for_blocks(n / QB), 96);
  if (dtype == 0)
    allreduce_fp8_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(to_params(d), a);
  else
    allreduce_fp8_kernel<float><<<grid, 512, 0, st>>>(to_params(d), a);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// Single-GPU emulation of all ranks (tests): one cooperative launch, blockIdx.y = rank.
FTB200_API int ftb200_team_allreduce_fp8_emulated(const ftb200_team_desc* descs, int launch_ranks, void* const* arena,
                                                  void* const* in_a, void* const* in_b, void* const* out, long long n,
                                                  int dtype, float scale, int ctas, cudaStream_t st) {
  const int world = descs[0].world;
  std::vector<TeamParams> tps;
  std::vector<QuantAllreduceArgs> as;
  for (int r = 0; r < launch_ranks; ++r) {
    tps.push_back(to_params(&descs[r]));
    QuantAllreduceArgs a;
    for (int i = 0; i < MAX_RANKS; ++i) a.arena[i] = i < world ? reinterpret_cast<uint8_t*>(arena[i]) : nullptr;
    a.in_a = in_a[r]; a.in_b = in_b ? in_b[r] : nullptr; a.out = out[r]; a.n = n; a.scale = scale; a.zero_contribution = 0;
    as.push_back(a);
  }
  TeamParams* d_tp = nullptr;
  QuantAllreduceArgs* d_a = nullptr;
  if (cudaMalloc(&d_tp, sizeof(TeamParams) * launch_ranks) != cudaSuccess ||
      cudaMalloc(&d_a, sizeof(QuantAllreduceArgs) * launch_ranks) != cudaSuccess)
    return FTB200_E_CUDA;
  cudaMemcpyAsync(d_tp, tps.data(), sizeof(TeamParams) * launch_ranks, cudaMemcpyHostToDevice, st);
  cudaMemcpyAsync(d_a, as.data(), sizeof(QuantAllreduceArgs) * launch_ranks, cudaMemcpyHostToDevice, st);
  void* args[2] = {&d_tp, &d_a};
  void* fn = dtype == 0 ? reinterpret_cast<void*>(allreduce_fp8_emul_kernel<__nv_bfloat16>)
                        : reinterpret_cast<void*>(allreduce_fp8_emul_kernel<float>);
  cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(ctas > 0 ? ctas : 4, launch_ranks, 1), dim3(512, 1, 1), args, 0, st);
  cudaStreamSynchronize(st);
  cudaFree(d_tp);
  cudaFree(d_a);
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_diloco_outer_step(const void* g, float* momentum, void* backup, void* param, long long n, int dtype,
                                        float lr, float mu, float alpha, int nesterov, int first_step, cudaStream_t st) {
  if (n <= 0 || n % 4) return FTB200_E_ALIGN;
  const int grid = static_cast<int>(std::min<long long>((n / 4 + 255) / 256, ftb200::sm_count() * 8LL));
  if (dtype == 0)
    diloco_outer_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)g, momentum, (__nv_bfloat16*)backup,
                                                             (__nv_bfloat16*)param, n, lr, mu, alpha, nesterov, first_step);
  else
    diloco_outer_kernel<float><<<grid, 256, 0, st>>>((const float*)g, momentum, (float*)backup, (float*)param, n, lr, mu,
                                                     alpha, nesterov, first_step);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}
