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
// vector loads, eight in flight per thread (NVLink latency is microseconds: bandwidth comes
// from bytes in flight), all segments in one launch.  Every 16 rounds of a block (some tens
// of MB of the launch's traffic) thread 0 looks at the abort word and the deadline and the
// block agrees on going on, so an abort or an expired deadline ends the copy within a
// fraction of a millisecond instead of at the next segment.  With `sums`, the kernel also
// leaves a 64-bit additive checksum of the 32-bit words it moved per segment, which the
// caller compares with the source's own checksum of the same bytes.
__device__ __forceinline__ unsigned long long sum4(const uint4& v) {
  return static_cast<unsigned long long>(v.x) + v.y + v.z + v.w;
}

__global__ void __launch_bounds__(512) p2p_copy_kernel(const CopySeg* __restrict__ segs, int nsegs,
                                                       const volatile int* abort_word, int* status,
                                                       unsigned long long timeout_ns, unsigned long long* sums) {
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const uint64_t t0 = ftb200::globaltimer_ns();
  constexpr int U = 8;
  unsigned rounds = 0;
  for (int s = 0; s < nsegs; ++s) {
    const uint4* src = reinterpret_cast<const uint4*>(segs[s].src);
    uint4* dst = reinterpret_cast<uint4*>(segs[s].dst);
    const long long nv = segs[s].bytes / 16;
    unsigned long long acc = 0;
    // uniform trip count per block, so that the block-wide vote below is reached by all threads
    const long long first = static_cast<long long>(blockIdx.x) * blockDim.x;
    for (long long b0 = first; b0 < nv; b0 += nthreads * U) {
      if ((rounds++ & 15u) == 0) {
        int stop = 0;
        if (threadIdx.x == 0) {
          if (abort_word != nullptr && *abort_word != 0) stop = FTB200_ST_ABORTED;
          else if (timeout_ns != 0 && ftb200::globaltimer_ns() - t0 > timeout_ns) stop = FTB200_ST_TIMEOUT;
          if (stop != 0 && status != nullptr) atomicMax(status, stop);
        }
        if (__syncthreads_or(stop)) return;
      }
      const long long i0 = b0 + threadIdx.x;
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < nv) v[u] = src[i];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * nthreads;
        if (i < nv) {
          dst[i] = v[u];
          acc += sum4(v[u]);
        }
      }
    }
    if (sums != nullptr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if ((threadIdx.x & 31) == 0 && acc != 0) atomicAdd(sums + s, acc);
    }
  }
}

// The source's side of the end-to-end check: the same per-segment checksum over local memory.
__global__ void __launch_bounds__(512) checksum_kernel(const CopySeg* __restrict__ segs, int nsegs,
                                                       unsigned long long* sums) {
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int s = 0; s < nsegs; ++s) {
    const uint4* src = reinterpret_cast<const uint4*>(segs[s].src);
    const long long nv = segs[s].bytes / 16;
    unsigned long long acc = 0;
    for (long long i = tid; i < nv; i += nthreads) acc += sum4(src[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0 && acc != 0) atomicAdd(sums + s, acc);
  }
}

// One-shot allreduce for small messages: every rank publishes its data in a symmetric
// window, one ready round, then every rank sums all ranks' copies itself (same order on
// every rank, so the results are bit-identical) and writes only to its own output.  Nothing
// is written into a peer, so no done round is needed: the window has two halves that the
// caller alternates, and passing the ready round of call k proves that every peer has left
// call k-1, whose half is the one call k+1 overwrites.
struct OneShotArgs {
  void* bufs[MAX_RANKS];  // this call's half of the window in every rank's arena
  const void* user_in;
  void* user_out;
  long long n;  // elements, multiple of the vector width
  float scale;
  int zero_contribution;
};

template <typename T>
__device__ __forceinline__ void allreduce_oneshot_body(const TeamParams& tp, const OneShotArgs& a) {
  __shared__ int sh_code;
  constexpr int V = Vec<T>::N;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  T* mine = reinterpret_cast<T*>(a.bufs[tp.rank]);
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
  if (!team_round(tp, /*slot=*/0, /*go=*/0, &sh_code)) return;
  T* dst = reinterpret_cast<T*>(a.user_out);
  for (long long i = tid * V; i < a.n; i += nthreads * V) {
    uint4 raw[MAX_RANKS];
#pragma unroll
    for (int p = 0; p < MAX_RANKS; ++p)
      if (p < tp.world) raw[p] = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.bufs[p]) + i);
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = 0.f;
#pragma unroll
    for (int p = 0; p < MAX_RANKS; ++p) {
      if (p < tp.world) {
        float f[V];
        Vec<T>::load(reinterpret_cast<const T*>(&raw[p]), f);
#pragma unroll
        for (int e = 0; e < V; ++e) acc[e] += f[e];
      }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] *= a.scale;
    Vec<T>::store(dst + i, acc);
  }
}
template <typename T>
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const TeamParams tp, const OneShotArgs a) {
  allreduce_oneshot_body<T>(tp, a);
}
template <typename T>
__global__ void __launch_bounds__(512) allreduce_oneshot_emul_kernel(const TeamParams* tps, const OneShotArgs* as) {
  allreduce_oneshot_body<T>(tps[blockIdx.y], as[blockIdx.y]);
}

// Generic pull: after a ready round every rank copies up to MAX_RANKS segments (peer or local
// source, local destination); a done round keeps the sources valid until every reader is
// through.  Broadcast is one segment from the root's window, all-to-all is one segment per
// peer, a gather is `world` segments on the root and none elsewhere.
struct PullArgs {
  const void* src[MAX_RANKS];
  void* dst[MAX_RANKS];
  long long bytes[MAX_RANKS];  // multiples of 16
  int nsegs;
};

__device__ __forceinline__ void copy16(const void* src, void* dst, long long bytes, long long tid, long long nthreads) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  const long long nv = bytes / 16;
  constexpr int U = 8;  // independent 16-byte loads in flight per thread
  for (long long i0 = tid; i0 < nv; i0 += nthreads * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * nthreads;
      if (i < nv) v[u] = s[i];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * nthreads;
      if (i < nv) d[i] = v[u];
    }
  }
}

__device__ __forceinline__ void pull_body(const TeamParams& tp, const PullArgs& a) {
  __shared__ int sh_code;
  if (!team_round(tp, 0, 0, &sh_code)) return;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int s = 0; s < a.nsegs; ++s) {
    // start at a rank-dependent segment so that the ranks do not all read the same peer at once
    const int k = (s + tp.rank) % a.nsegs;
    copy16(a.src[k], a.dst[k], a.bytes[k], tid, nthreads);
  }
  if (!grid_arrive(tp, 3, &sh_code)) return;
  team_round(tp, 1, 1, &sh_code);
}
__global__ void __launch_bounds__(512) pull_kernel(const TeamParams tp, const PullArgs a) { pull_body(tp, a); }
__global__ void __launch_bounds__(512) pull_emul_kernel(const TeamParams* tps, const PullArgs* as) {
  pull_body(tps[blockIdx.y], as[blockIdx.y]);
}

// Point-to-point transfer between two ranks of a team, one launch on each side.  The sender
// has put the payload into its symmetric send window (stream-ordered before this kernel),
// tells the receiver so (flag slot 2) and waits until the receiver has taken it (slot 3);
// the receiver waits for the payload, pulls it over NVLink into its destination and says
// so.  Tokens count per ordered pair of ranks, so other ranks of the team are not involved.
// Local words 4 (go) and 5 (arrival counter) are this kernel's own: a transfer may run on
// another stream than the team's collectives.  All waits are bounded like the collectives'.
struct SendRecvArgs {
  int peer;
  int is_send;
  uint64_t token;
  const void* src;  // receiver: the sender's window (peer-mapped)
  void* dst;        // receiver: local destination
  long long bytes;  // multiple of 16
};

__device__ __forceinline__ void sendrecv_body(const TeamParams& tp, const SendRecvArgs& a) {
  __shared__ int sh_code;
  const uint64_t t0 = ftb200::globaltimer_ns();
  TeamParams tq = tp;
  tq.token = a.token;
  if (a.is_send) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      __threadfence_system();
      st_release_sys(tp.flags[a.peer] + 2 * MAX_RANKS + tp.rank, a.token);
      const int code = wait_equal<true>(tp.flags[tp.rank] + 3 * MAX_RANKS + a.peer, a.token, tq, t0);
      if (code != FTB200_ST_OK && tp.status != nullptr) atomicMax(tp.status, code);
    }
    return;
  }
  uint64_t* go = tp.local_sync + 4;
  uint64_t* ctr = tp.local_sync + 5;
  if (threadIdx.x == 0) {
    int code;
    if (blockIdx.x == 0) {
      code = wait_equal<true>(tp.flags[tp.rank] + 2 * MAX_RANKS + a.peer, a.token, tq, t0);
      if (code != FTB200_ST_OK && tp.status != nullptr) atomicMax(tp.status, code);
      st_release_gpu(go, code == FTB200_ST_OK ? a.token : GO_ABORT);
    } else {
      code = wait_equal<false>(go, a.token, tq, t0);
      if (code == FTB200_ST_TIMEOUT && tp.status != nullptr) atomicMax(tp.status, code);
    }
    sh_code = code;
  }
  __syncthreads();
  if (sh_code != FTB200_ST_OK) return;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  copy16(a.src, a.dst, a.bytes, tid, nthreads);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    atomicAdd(reinterpret_cast<unsigned long long*>(ctr), 1ull);
    if (blockIdx.x == 0) {
      uint32_t spins = 0;
      int code = FTB200_ST_OK;
      while (ld_acquire_gpu(ctr) < gridDim.x) {
        if ((++spins & 15u) == 0 && ftb200::globaltimer_ns() - t0 > tp.timeout_ns) { code = FTB200_ST_TIMEOUT; break; }
      }
      st_release_gpu(ctr, 0);
      if (code != FTB200_ST_OK && tp.status != nullptr) atomicMax(tp.status, code);
      // the sender may reuse its window now (also after a local failure: it must not wait for nothing)
      st_release_sys(tp.flags[a.peer] + 3 * MAX_RANKS + tp.rank, a.token);
    }
  }
}
__global__ void __launch_bounds__(512) sendrecv_kernel(const TeamParams tp, const SendRecvArgs a) { sendrecv_body(tp, a); }
__global__ void __launch_bounds__(512) sendrecv_emul_kernel(const TeamParams* tps, const SendRecvArgs* as) {
  sendrecv_body(tps[blockIdx.y], as[blockIdx.y]);
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

// One-shot allreduce of a small message (see allreduce_oneshot_body).  bufs[i] is this call's half
// of the small-message window in rank i's arena; user_in/user_out are local (may be the same tensor).
FTB200_API int ftb200_team_allreduce_oneshot(const ftb200_team_desc* d, void* const* bufs, const void* user_in,
                                             void* user_out, long long n, int dtype, float scale, int zero_contribution,
                                             cudaStream_t st) {
  if (d->world < 1 || d->world > MAX_RANKS || n <= 0 || user_out == nullptr) return FTB200_E_BADARG;
  if (user_in == nullptr && !zero_contribution) return FTB200_E_BADARG;
  const int V = dtype == 0 ? 8 : 4;
  if (n % V) return FTB200_E_ALIGN;
  if ((reinterpret_cast<uintptr_t>(user_in) | reinterpret_cast<uintptr_t>(user_out)) & 15) return FTB200_E_ALIGN;
  OneShotArgs a;
  for (int i = 0; i < MAX_RANKS; ++i) a.bufs[i] = i < d->world ? bufs[i] : nullptr;
  a.user_in = user_in;
  a.user_out = user_out;
  a.n = n;
  a.scale = scale;
  a.zero_contribution = zero_contribution;
  const long long vecs = n / V;
  const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(16, (vecs + 511) / 512)));
  if (dtype == 0)
    allreduce_oneshot_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(to_params(d), a);
  else
    allreduce_oneshot_kernel<float><<<grid, 512, 0, st>>>(to_params(d), a);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// Generic pull collective (see pull_body): src/dst/bytes describe this rank's nsegs copies.
FTB200_API int ftb200_team_pull(const ftb200_team_desc* d, const void* const* src, void* const* dst,
                                const long long* bytes, int nsegs, int ctas, cudaStream_t st) {
  if (d->world < 1 || d->world > MAX_RANKS || nsegs < 0 || nsegs > MAX_RANKS) return FTB200_E_BADARG;
  PullArgs a;
  long long total = 0;
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.src[i] = i < nsegs ? src[i] : nullptr;
    a.dst[i] = i < nsegs ? dst[i] : nullptr;
    a.bytes[i] = i < nsegs ? bytes[i] : 0;
    if (i < nsegs) {
      if (bytes[i] < 0 || (bytes[i] % 16)) return FTB200_E_ALIGN;
      if ((reinterpret_cast<uintptr_t>(src[i]) | reinterpret_cast<uintptr_t>(dst[i])) & 15) return FTB200_E_ALIGN;
      total += bytes[i];
    }
  }
  a.nsegs = nsegs;
  const int grid = ctas > 0 ? ctas : grid_for_bytes(total);
  pull_kernel<<<grid, 512, 0, st>>>(to_params(d), a);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// One side of a point-to-point transfer (see sendrecv_body).  pair_token = epoch << 32 | count of
// transfers from the sender to the receiver so far, the same on both sides.
FTB200_API int ftb200_team_sendrecv(const ftb200_team_desc* d, int peer, int is_send, unsigned long long pair_token,
                                    const void* src, void* dst, long long bytes, int ctas, cudaStream_t st) {
  if (d->world < 2 || d->world > MAX_RANKS || peer < 0 || peer >= d->world || peer == d->rank) return FTB200_E_BADARG;
  if (bytes < 0 || (bytes % 16)) return FTB200_E_ALIGN;
  if (!is_send && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return FTB200_E_ALIGN;
  SendRecvArgs a;
  a.peer = peer;
  a.is_send = is_send;
  a.token = pair_token;
  a.src = src;
  a.dst = dst;
  a.bytes = bytes;
  const int grid = is_send ? 1 : (ctas > 0 ? ctas : std::max(grid_for_bytes(bytes), 1));
  sendrecv_kernel<<<grid, is_send ? 32 : 512, 0, st>>>(to_params(d), a);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// segs: device array of {src, dst, bytes}; the caller keeps it alive until the stream reaches the kernel.
// abort_word (device pointer of a host-mapped word, may be null) and timeout_ns (0 = none) bound the copy;
// sums (may be null): nsegs zeroed 64-bit words that receive the per-segment checksums of the moved bytes.
FTB200_API int ftb200_p2p_copy(const void* segs_dev, int nsegs, long long total_bytes, const void* abort_word, int* status,
                               int ctas, cudaStream_t st) {
  if (nsegs <= 0) return 0;
  const int grid = ctas > 0 ? ctas : std::max(grid_for_bytes(total_bytes), 32);
  p2p_copy_kernel<<<grid, 512, 0, st>>>(reinterpret_cast<const CopySeg*>(segs_dev), nsegs,
                                        reinterpret_cast<const volatile int*>(abort_word), status, 0ull, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

FTB200_API int ftb200_p2p_copy_checked(const void* segs_dev, int nsegs, long long total_bytes, const void* abort_word,
                                       int* status, unsigned long long timeout_ns, unsigned long long* sums, int ctas,
                                       cudaStream_t st) {
  if (nsegs <= 0) return 0;
  const int grid = ctas > 0 ? ctas : std::max(grid_for_bytes(total_bytes), 32);
  p2p_copy_kernel<<<grid, 512, 0, st>>>(reinterpret_cast<const CopySeg*>(segs_dev), nsegs,
                                        reinterpret_cast<const volatile int*>(abort_word), status, timeout_ns, sums);
  return cudaGetLastError() == cudaSuccess ? 0 : FTB200_E_CUDA;
}

// Plain device-to-device copy (also from a peer-mapped source) for the ragged heads and tails that the
// 16-byte copy kernel leaves out.
FTB200_API int ftb200_memcpy_d2d(void* dst, const void* src, long long bytes, cudaStream_t st) {
  if (bytes <= 0) return 0;
  return cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, st) == cudaSuccess
             ? 0
             : FTB200_E_CUDA;
}

// Per-segment checksum of local memory (src and bytes of each segment; dst is ignored).
FTB200_API int ftb200_checksum(const void* segs_dev, int nsegs, long long total_bytes, unsigned long long* sums,
                               cudaStream_t st) {
  if (nsegs <= 0) return 0;
  const int grid = std::max(grid_for_bytes(total_bytes), 32) * 2;
  checksum_kernel<<<grid, 512, 0, st>>>(reinterpret_cast<const CopySeg*>(segs_dev), nsegs, sums);
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

FTB200_API int ftb200_team_allreduce_oneshot_emulated(const ftb200_team_desc* descs, int launch_ranks, void* const* bufs,
                                                      void* const* user_in, void* const* user_out, long long n,
                                                      int dtype, float scale, int ctas, cudaStream_t st) {
  const int world = descs[0].world;
  std::vector<TeamParams> tps;
  std::vector<OneShotArgs> as;
  for (int r = 0; r < launch_ranks; ++r) {
    tps.push_back(to_params(&descs[r]));
    OneShotArgs a;
    for (int i = 0; i < MAX_RANKS; ++i) a.bufs[i] = i < world ? bufs[i] : nullptr;
    a.user_in = user_in[r];
    a.user_out = user_out[r];
    a.n = n;
    a.scale = scale;
    a.zero_contribution = 0;
    as.push_back(a);
  }
  if (dtype == 0) return launch_emulated(allreduce_oneshot_emul_kernel<__nv_bfloat16>, tps, as, ctas > 0 ? ctas : 2, st);
  return launch_emulated(allreduce_oneshot_emul_kernel<float>, tps, as, ctas > 0 ? ctas : 2, st);
}

// src/dst/bytes: [launch_ranks][MAX_RANKS] row-major; nsegs: [launch_ranks].
FTB200_API int ftb200_team_pull_emulated(const ftb200_team_desc* descs, int launch_ranks, const void* const* src,
                                         void* const* dst, const long long* bytes, const int* nsegs, int ctas,
                                         cudaStream_t st) {
  std::vector<TeamParams> tps;
  std::vector<PullArgs> as;
  for (int r = 0; r < launch_ranks; ++r) {
    tps.push_back(to_params(&descs[r]));
    PullArgs a;
    for (int i = 0; i < MAX_RANKS; ++i) {
      a.src[i] = src[r * MAX_RANKS + i];
      a.dst[i] = dst[r * MAX_RANKS + i];
      a.bytes[i] = bytes[r * MAX_RANKS + i];
    }
    a.nsegs = nsegs[r];
    as.push_back(a);
  }
  return launch_emulated(pull_emul_kernel, tps, as, ctas > 0 ? ctas : 4, st);
}

// Both sides of one transfer in one cooperative launch: descs[0] sends, descs[1] receives
// (launch_ranks = 1 launches the receiver only, whose wait then runs out).
FTB200_API int ftb200_team_sendrecv_emulated(const ftb200_team_desc* send_desc, const ftb200_team_desc* recv_desc,
                                             int launch_sender, unsigned long long pair_token, const void* src, void* dst,
                                             long long bytes, int ctas, cudaStream_t st) {
  std::vector<TeamParams> tps;
  std::vector<SendRecvArgs> as;
  SendRecvArgs r;
  r.peer = send_desc->rank;
  r.is_send = 0;
  r.token = pair_token;
  r.src = src;
  r.dst = dst;
  r.bytes = bytes;
  tps.push_back(to_params(recv_desc));
  as.push_back(r);
  if (launch_sender) {
    SendRecvArgs s = r;
    s.peer = recv_desc->rank;
    s.is_send = 1;
    tps.push_back(to_params(send_desc));
    as.push_back(s);
  }
  return launch_emulated(sendrecv_emul_kernel, tps, as, ctas > 0 ? ctas : 4, st);
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
