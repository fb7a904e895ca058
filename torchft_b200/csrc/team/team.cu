// Peer-memory team: collectives written as kernels that load and store other GPUs'
// memory directly over NVLink / NVSwitch (plain ld/st on IPC-mapped pointers).
//
// Memory model.  Every rank owns one exported *arena* (cudaMalloc + cudaIpcGetMemHandle)
// that peers map (cudaIpcOpenMemHandle).  All ranks sub-allocate in the same order, so a
// buffer sits at the same offset in every arena ("symmetric").  The first bytes of an
// arena are the rank's flag words: flag[slot][src] is written by rank `src` only.
//
// Synchronisation.  A collective is one launch per rank (each on its own GPU).  Inside,
// block 0 signals "ready" to every peer and waits for every peer's "ready"; the other
// blocks wait on a local go-word; data moves; then a "done" round keeps every rank's
// buffers valid until all readers/writers have finished.  Flag values are
// (epoch << 32 | sequence): stale values of an earlier quorum epoch or call never match.
//
// Never-hang contract.  Every wait polls (i) a host-mapped abort word, (ii) the flag,
// (iii) %globaltimer against a deadline.  On abort or expiry the kernel stores a
// FTB200_ST_* code in the team's status word, releases its local waiters and returns;
// the host reads the status after synchronising the stream.
#include <algorithm>
#include <cstring>
#include <vector>

#include "ftb200_common.cuh"
#include "team_device.cuh"

namespace {

using namespace ftb200::team;

struct AllreduceArgs {
  void* bufs[MAX_RANKS];  // symmetric staging / registered buffers (peer-mapped), element offset already applied
  const void* user_in;    // optional: copied into bufs[rank] first
  void* user_out;         // optional: receives the result (same dtype)
  long long n;            // elements, multiple of the vector width * world
  float scale;
  int zero_contribution;  // contribute zeros instead of the local data
};

// Two-shot allreduce in place on the symmetric buffers: rank r reduces slice r over all
// ranks (fp32 accumulation, fixed order starting at its own copy), scales, and writes the
// slice into every rank's buffer.
template <typename T>
__device__ __forceinline__ void allreduce_body(const TeamParams& tp, const AllreduceArgs& a) {
  __shared__ int sh_code;
  constexpr int V = Vec<T>::N;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  T* mine = reinterpret_cast<T*>(a.bufs[tp.rank]);

  if (a.user_in != nullptr || a.zero_contribution) {
    const T* src = reinterpret_cast<const T*>(a.user_in);
    for (long long i = tid * V; i < a.n; i += nthreads * V) {
      float f[V];
      if (a.zero_contribution) {
#pragma unroll
        for (int e = 0; e < V; ++e) f[e] = 0.f;
      } else {
        Vec<T>::load(src + i, f);
      }
      Vec<T>::store(mine + i, f);
    }
    if (!grid_arrive(tp, 2, &sh_code)) return;
  }
  if (!team_round(tp, /*slot=*/0, /*go=*/0, &sh_code)) return;

  const long long slice = a.n / tp.world;
  const long long lo = slice * tp.rank;
  // u positions x world peers = up to 8 independent 16-byte peer loads in flight per thread
  const int u = MAX_RANKS / tp.world;
  for (long long i0 = tid * V; i0 < slice; i0 += nthreads * V * u) {
    uint4 raw[MAX_RANKS];
#pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      const int pos = k / tp.world, pk = k - pos * tp.world;
      const long long i = i0 + pos * nthreads * V;
      if (pos < u && i < slice) {
        const int p = (tp.rank + pk) % tp.world;
        raw[k] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.bufs[p]) + lo + i);
      }
    }
    for (int pos = 0; pos < u; ++pos) {
      const long long i = i0 + pos * nthreads * V;
      if (i >= slice) break;
      float acc[V];
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] = 0.f;
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k / tp.world == pos) {
          float f[V];
          Vec<T>::load(reinterpret_cast<const T*>(&raw[k]), f);
#pragma unroll
          for (int e = 0; e < V; ++e) acc[e] += f[e];
        }
      }
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] *= a.scale;
      for (int k = 0; k < tp.world; ++k) {
        const int p = (tp.rank + k) % tp.world;
        Vec<T>::store(reinterpret_cast<T*>(a.bufs[p]) + lo + i, acc);
      }
    }
  }
  if (!grid_arrive(tp, 3, &sh_code)) return;
  if (!team_round(tp, /*slot=*/1, /*go=*/1, &sh_code)) return;

  if (a.user_out != nullptr) {
    T* dst = reinterpret_cast<T*>(a.user_out);
    for (long long i = tid * V; i < a.n; i += nthreads * V) {
      float f[V];
      Vec<T>::load(mine + i, f);
      Vec<T>::store(dst + i, f);
    }
  }
}

template <typename T>
__global__ void __maxnreg__(72) allreduce_kernel(const TeamParams tp, const AllreduceArgs a) {
  allreduce_body<T>(tp, a);
}
// Test vehicle: all ranks of a team emulated by ONE cooperative launch on one GPU
// (blockIdx.y selects the rank); separate launches that wait on each other must never
// share a GPU.
template <typename T>
__global__ void __launch_bounds__(512) allreduce_emul_kernel(const TeamParams* tps, const AllreduceArgs* as) {
  allreduce_body<T>(tps[blockIdx.y], as[blockIdx.y]);
}

struct GatherArgs {
  const void* src[MAX_RANKS];  // every rank's shard (peer-mapped)
  void* dst;                   // local full buffer: world * shard_bytes
  long long shard_bytes;       // multiple of 16
};

// All-gather by pulling: every rank copies all shards (its own included) into its full buffer.
__device__ __forceinline__ void allgather_body(const TeamParams& tp, const GatherArgs& a) {
  __shared__ int sh_code;
  if (!team_round(tp, 0, 0, &sh_code)) return;
  const long long v_per = a.shard_bytes / 16;
  const long long total = v_per * tp.world;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  uint4* dst = reinterpret_cast<uint4*>(a.dst);
  // eight independent 16-byte loads in flight per thread: NVLink latency is microseconds,
  // so bandwidth comes from bytes in flight
  constexpr int U = 8;
  for (long long i0 = tid; i0 < total; i0 += nthreads * U) {
    uint4 v[U];
    long long didx[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * nthreads;
      didx[u] = -1;
      if (i < total) {
        // start with the next rank's shard so that the ranks do not all hit the same peer at once
        const long long blk = i / v_per;
        const int p = static_cast<int>((blk + tp.rank + 1) % tp.world);
        const long long off = i - blk * v_per;
        v[u] = reinterpret_cast<const uint4*>(a.src[p])[off];
        didx[u] = p * v_per + off;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (didx[u] >= 0) dst[didx[u]] = v[u];
  }
  if (!grid_arrive(tp, 3, &sh_code)) return;
  team_round(tp, 1, 1, &sh_code);
}

__global__ void __maxnreg__(72) allgather_kernel(const TeamParams tp, const GatherArgs a) { allgather_body(tp, a); }
__global__ void __launch_bounds__(512) allgather_emul_kernel(const TeamParams* tps, const GatherArgs* as) {
  allgather_body(tps[blockIdx.y], as[blockIdx.y]);
}

struct ReduceScatterArgs {
  const void* src[MAX_RANKS];  // every rank's full buffer (peer-mapped), world * shard_elems
  void* dst;                   // local shard
  long long shard_elems;       // multiple of the vector width
  float scale;
};

// Reduce-scatter by pulling: rank r sums slice r of every rank's full buffer (fp32).
template <typename T>
__device__ __forceinline__ void reduce_scatter_body(const TeamParams& tp, const ReduceScatterArgs& a) {
  __shared__ int sh_code;
  constexpr int V = Vec<T>::N;
  if (!team_round(tp, 0, 0, &sh_code)) return;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long lo = a.shard_elems * tp.rank;
  T* dst = reinterpret_cast<T*>(a.dst);
  const int u = MAX_RANKS / tp.world;
  for (long long i0 = tid * V; i0 < a.shard_elems; i0 += nthreads * V * u) {
    uint4 raw[MAX_RANKS];
#pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      const int pos = k / tp.world, pk = k - pos * tp.world;
      const long long i = i0 + pos * nthreads * V;
      if (pos < u && i < a.shard_elems) {
        const int p = (tp.rank + pk) % tp.world;
        raw[k] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.src[p]) + lo + i);
      }
    }
    for (int pos = 0; pos < u; ++pos) {
      const long long i = i0 + pos * nthreads * V;
      if (i >= a.shard_elems) break;
      float acc[V];
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] = 0.f;
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k / tp.world == pos) {
          float f[V];
          Vec<T>::load(reinterpret_cast<const T*>(&raw[k]), f);
#pragma unroll
          for (int e = 0; e < V; ++e) acc[e] += f[e];
        }
      }
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] *= a.scale;
      Vec<T>::store(dst + i, acc);
    }
  }
  if (!grid_arrive(tp, 3, &sh_code)) return;
  team_round(tp, 1, 1, &sh_code);
}

template <typename T>
__global__ void __maxnreg__(72) reduce_scatter_kernel(const TeamParams tp, const ReduceScatterArgs a) {
  reduce_scatter_body<T>(tp, a);
}
template <typename T>
__global__ void __launch_bounds__(512) reduce_scatter_emul_kernel(const TeamParams* tps, const ReduceScatterArgs* as) {
  reduce_scatter_body<T>(tps[blockIdx.y], as[blockIdx.y]);
}

// Barrier only (also what a send/recv handshake uses).
__global__ void barrier_kernel(const TeamParams tp) {
  __shared__ int sh_code;
  team_round(tp, 0, 0, &sh_code);
}

struct CopySeg {
  const void* src;
  void* dst;
  long long bytes;  // multiple of 16
};

// Live-recovery copy: a table of (peer src, local dst, bytes) segments pulled with 16-byte
// vector loads; a bounds-free grid-stride loop per segment, all segments in one launch.
__global__ void __launch_bounds__(512) p2p_copy_kernel(const CopySeg* __restrict__ segs, int nsegs,
                                                       const volatile int* abort_word, int* status) {
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int s = 0; s < nsegs; ++s) {
    if (abort_word != nullptr && *abort_word != 0) {
      if (tid == 0 && status != nullptr) atomicMax(status, FTB200_ST_ABORTED);
      return;
    }
    const uint4* src = reinterpret_cast<const uint4*>(segs[s].src);
    uint4* dst = reinterpret_cast<uint4*>(segs[s].dst);
    const long long nv = segs[s].bytes / 16;
    for (long long i = tid; i < nv; i += nthreads) dst[i] = src[i];
  }
}

int grid_for_bytes(long long bytes) {
  // enough CTAs to saturate NVLink without starving concurrent compute of SMs
  long long g = bytes / (512 * 16 * 4);
  g = std::max<long long>(1, std::min<long long>(g, 128));
  return static_cast<int>(g);
}

}  // namespace

// ------------------------------------------------------------------------------------ C ABI

FTB200_API int ftb200_team_flag_bytes() { return FLAG_WORDS * 8; }
FTB200_API int ftb200_team_sync_bytes() { return 8 * 8; }
FTB200_API int ftb200_team_max_ranks() { return MAX_RANKS; }

FTB200_API int ftb200_arena_alloc(void** ptr, unsigned long long bytes) {
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return FTB200_E_CUDA;
  return 0;
}
FTB200_API int ftb200_arena_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : FTB200_E_CUDA; }

FTB200_API int ftb200_ipc_export(void* ptr, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return FTB200_E_CUDA;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
FTB200_API int ftb200_ipc_import(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  if (cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return FTB200_E_CUDA;
  }
  return 0;
}
FTB200_API int ftb200_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : FTB200_E_CUDA; }

// Host-mapped abort word: *host_ptr is written by the host, *dev_ptr read by kernels.
FTB200_API int ftb200_abort_word_create(int** host_ptr, void** dev_ptr) {
  if (cudaHostAlloc(reinterpret_cast<void**>(host_ptr), sizeof(int), cudaHostAllocMapped) != cudaSuccess) return FTB200_E_CUDA;
  **host_ptr = 0;
  if (cudaHostGetDevicePointer(dev_ptr, *host_ptr, 0) != cudaSuccess) return FTB200_E_CUDA;
  return 0;
}
FTB200_API int ftb200_abort_word_destroy(int* host_ptr) { return cudaFreeHost(host_ptr) == cudaSuccess ? 0 : FTB200_E_CUDA; }

// dtype: 0 = bf16, 1 = fp32.  bufs[i] already point at the buffer inside rank i's arena.
FTB200_API int ftb200_team_allreduce(const ftb200_team_desc* d, void* const* bufs, const void* user_in, void* user_out,
                                     long long n, int dtype, float scale, int zero_contribution, int ctas,
                                     cudaStream_t st) {
  if (d->world < 1 || d->world > MAX_RANKS || n <= 0) return FTB200_E_BADARG;
  const int V = dtype == 0 ? 8 : 4;
  if (n % (static_cast<long long>(V) * d->world)) return FTB200_E_ALIGN;
  AllreduceArgs a;
  for (int i = 0; i < MAX_RANKS; ++i) a.bufs[i] = i < d->world ? bufs[i] : nullptr;
  a.user_in = user_in;
  a.user_out = user_out;
  a.n = n;
  a.scale = scale;
  a.zero_contribution = zero_contribution;
  const TeamParams tp = to_params(d);
  const int grid = ctas > 0 ? ctas : grid_for_bytes(n * (dtype == 0 ? 2 : 4));
  if (dtype == 0)
    allreduce_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(tp, a);
  else
    allreduce_kernel<float><<<grid, 512, 0, st>>>(tp, a);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_team_allgather(const ftb200_team_desc* d, const void* const* src, void* dst, long long shard_bytes,
                                     int ctas, cudaStream_t st) {
  if (d->world < 1 || d->world > MAX_RANKS || shard_bytes <= 0) return FTB200_E_BADARG;
  if (shard_bytes % 16) return FTB200_E_ALIGN;
  GatherArgs a;
  for (int i = 0; i < MAX_RANKS; ++i) a.src[i] = i < d->world ? src[i] : nullptr;
  a.dst = dst;
  a.shard_bytes = shard_bytes;
  const int grid = ctas > 0 ? ctas : grid_for_bytes(shard_bytes * d->world);
  allgather_kernel<<<grid, 512, 0, st>>>(to_params(d), a);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_team_reduce_scatter(const ftb200_team_desc* d, const void* const* src, void* dst,
                                          long long shard_elems, int dtype, float scale, int ctas, cudaStream_t st) {
  if (d->world < 1 || d->world > MAX_RANKS || shard_elems <= 0) return FTB200_E_BADARG;
  const int V = dtype == 0 ? 8 : 4;
  if (shard_elems % V) return FTB200_E_ALIGN;
  ReduceScatterArgs a;
  for (int i = 0; i < MAX_RANKS; ++i) a.src[i] = i < d->world ? src[i] : nullptr;
  a.dst = dst;
  a.shard_elems = shard_elems;
  a.scale = scale;
  const int grid = ctas > 0 ? ctas : grid_for_bytes(shard_elems * (dtype == 0 ? 2 : 4) * d->world);
  if (dtype == 0)
    reduce_scatter_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(to_params(d), a);
  else
    reduce_scatter_kernel<float><<<grid, 512, 0, st>>>(to_params(d), a);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_team_barrier(const ftb200_team_desc* d, cudaStream_t st) {
  barrier_kernel<<<1, 32, 0, st>>>(to_params(d));
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// segs: device array of {src, dst, bytes}; the caller keeps it alive until the stream reaches the kernel.
FTB200_API int ftb200_p2p_copy(const void* segs_dev, int nsegs, long long total_bytes, const void* abort_word, int* status,
                               int ctas, cudaStream_t st) {
  if (nsegs <= 0) return 0;
  const int grid = ctas > 0 ? ctas : std::max(grid_for_bytes(total_bytes), 32);
  p2p_copy_kernel<<<grid, 512, 0, st>>>(reinterpret_cast<const CopySeg*>(segs_dev), nsegs,
                                        reinterpret_cast<const volatile int*>(abort_word), status);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// ---- single-GPU emulation of a whole team (tests) -----------------------------------------
// `descs` / `bufs` describe `world` ranks whose arenas all live on the current device.
// `launch_ranks` <= world ranks are launched (fewer than world makes the waits expire, which
// is how the timeout path is exercised without any peer).
namespace {
template <typename P, typename A>
int launch_emulated(void (*kernel)(const P*, const A*), const std::vector<P>& tps, const std::vector<A>& as, int grid_x,
                    cudaStream_t st) {
  const int n = static_cast<int>(tps.size());
  P* d_tp = nullptr;
  A* d_a = nullptr;
  if (cudaMalloc(&d_tp, sizeof(P) * n) != cudaSuccess || cudaMalloc(&d_a, sizeof(A) * n) != cudaSuccess) return FTB200_E_CUDA;
  cudaMemcpyAsync(d_tp, tps.data(), sizeof(P) * n, cudaMemcpyHostToDevice, st);
  cudaMemcpyAsync(d_a, as.data(), sizeof(A) * n, cudaMemcpyHostToDevice, st);
  void* args[2] = {&d_tp, &d_a};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(grid_x, n, 1), dim3(512, 1, 1), args, 0, st);
  cudaStreamSynchronize(st);
  cudaFree(d_tp);
  cudaFree(d_a);
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}
}  // namespace

FTB200_API int ftb200_team_allreduce_emulated(const ftb200_team_desc* descs, int launch_ranks, void* const* bufs,
                                              void* const* user_in, void* const* user_out, long long n, int dtype,
                                              float scale, const int* zero_contribution, int ctas, cudaStream_t st) {
  const int world = descs[0].world;
  std::vector<TeamParams> tps;
  std::vector<AllreduceArgs> as;
  for (int r = 0; r < launch_ranks; ++r) {
    tps.push_back(to_params(&descs[r]));
    AllreduceArgs a;
    for (int i = 0; i < MAX_RANKS; ++i) a.bufs[i] = i < world ? bufs[i] : nullptr;
    a.user_in = user_in ? user_in[r] : nullptr;
    a.user_out = user_out ? user_out[r] : nullptr;
    a.n = n;
    a.scale = scale;
    a.zero_contribution = zero_contribution ? zero_contribution[r] : 0;
    as.push_back(a);
  }
  if (dtype == 0) return launch_emulated(allreduce_emul_kernel<__nv_bfloat16>, tps, as, ctas > 0 ? ctas : 4, st);
  return launch_emulated(allreduce_emul_kernel<float>, tps, as, ctas > 0 ? ctas : 4, st);
}

FTB200_API int ftb200_team_allgather_emulated(const ftb200_team_desc* descs, int launch_ranks, const void* const* src,
                                              void* const* dst, long long shard_bytes, int ctas, cudaStream_t st) {
  const int world = descs[0].world;
  std::vector<TeamParams> tps;
  std::vector<GatherArgs> as;
  for (int r = 0; r < launch_ranks; ++r) {
    tps.push_back(to_params(&descs[r]));
    GatherArgs a;
    for (int i = 0; i < MAX_RANKS; ++i) a.src[i] = i < world ? src[i] : nullptr;
    a.dst = dst[r];
    a.shard_bytes = shard_bytes;
    as.push_back(a);
  }
  return launch_emulated(allgather_emul_kernel, tps, as, ctas > 0 ? ctas : 4, st);
}

FTB200_API int ftb200_team_reduce_scatter_emulated(const ftb200_team_desc* descs, int launch_ranks, const void* const* src,
                                                   void* const* dst, long long shard_elems, int dtype, float scale,
                                                   int ctas, cudaStream_t st) {
  const int world = descs[0].world;
  std::vector<TeamParams> tps;
  std::vector<ReduceScatterArgs> as;
  for (int r = 0; r < launch_ranks; ++r) {
    tps.push_back(to_params(&descs[r]));
    ReduceScatterArgs a;
    for (int i = 0; i < MAX_RANKS; ++i) a.src[i] = i < world ? src[i] : nullptr;
    a.dst = dst[r];
    a.shard_elems = shard_elems;
    a.scale = scale;
    as.push_back(a);
  }
  if (dtype == 0) return launch_emulated(reduce_scatter_emul_kernel<__nv_bfloat16>, tps, as, ctas > 0 ? ctas : 4, st);
  return launch_emulated(reduce_scatter_emul_kernel<float>, tps, as, ctas > 0 ? ctas : 4, st);
}

// Export the allocation that contains `ptr` (any device pointer obtained from cudaMalloc,
// e.g. a tensor of the framework's caching allocator) and report ptr's offset inside it.
FTB200_API int ftb200_ipc_export_any(const void* ptr, unsigned char* handle64, unsigned long long* offset,
                                     unsigned long long* alloc_bytes) {
  typedef int (*GetRangeFn)(unsigned long long*, size_t*, unsigned long long);
  static GetRangeFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return FTB200_E_DRIVER;
    fn = reinterpret_cast<GetRangeFn>(sym);
  }
  unsigned long long base = 0;
  size_t size = 0;
  if (fn(&base, &size, reinterpret_cast<unsigned long long>(ptr)) != 0) return FTB200_E_DRIVER;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
    cudaGetLastError();
    return FTB200_E_CUDA;
  }
  memcpy(handle64, &h, sizeof(h));
  *offset = reinterpret_cast<unsigned long long>(ptr) - base;
  *alloc_bytes = size;
  return 0;
}

// ---- pieces of the GEMM-fused reduce-scatter ------------------------------------------------
namespace {
struct StagePeers {
  void* p[MAX_RANKS];
};
// Small fields of a gradient unit (norm weights) that no GEMM produces: copy them into the
// owners' staging areas with the same addressing as the GEMM's scatter epilogue.
__global__ void scatter_to_stage_kernel(const ftb200::bf16x8* __restrict__ src, long long n8, long long unit_off,
                                        long long shard, int src_rank, StagePeers peers) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const long long flat = unit_off + i * 8;
  const long long owner = flat / shard;
  const long long rem = flat - owner * shard;
  if (!FTB_IN_RANGE(owner, MAX_RANKS)) return;
  __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(peers.p[owner]);
  *reinterpret_cast<ftb200::bf16x8*>(base + static_cast<long long>(src_rank) * shard + rem) = src[i];
}
}  // namespace

FTB200_API int ftb200_scatter_to_stage(const void* src, long long n, long long unit_off, long long shard_elems,
                                       void* const* peers, int world, int src_rank, cudaStream_t st) {
  if (n <= 0) return 0;
  if ((n % 8) || (unit_off % 8) || (shard_elems % 8) || (reinterpret_cast<uintptr_t>(src) & 15)) return FTB200_E_ALIGN;
  if (world < 1 || world > MAX_RANKS || unit_off + n > shard_elems * world) return FTB200_E_BADARG;
  StagePeers sp;
  for (int i = 0; i < MAX_RANKS; ++i) sp.p[i] = i < world ? peers[i] : nullptr;
  const long long n8 = n / 8;
  scatter_to_stage_kernel<<<static_cast<int>((n8 + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const ftb200::bf16x8*>(src), n8, unit_off, shard_elems, src_rank, sp);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB_DEFINE_BOUNDS_QUERY(team)
