// Device-side building blocks of the peer-memory team kernels: the launch parameters,
// system-scope flag accesses, the bounded cross-rank round and the in-launch arrival
// counter.  Shared by team.cu and quant_team.cu.
#pragma once

#include "ftb200_common.cuh"

namespace ftb200 {
namespace team {

constexpr int MAX_RANKS = 8;
constexpr int NUM_SLOTS = 4;  // ready, done, + 2 spare
constexpr int FLAG_WORDS = NUM_SLOTS * MAX_RANKS;
constexpr uint64_t GO_ABORT = ~0ull;

struct TeamParams {
  int rank;
  int world;
  uint64_t token;        // (epoch << 32) | sequence number of this call
  uint64_t timeout_ns;
  uint64_t* flags[MAX_RANKS];  // base of every rank's flag words (peer-mapped; [rank] is local)
  uint64_t* local_sync;        // local words: [0] go-ready, [1] go-done, [2] arrival counter a, [3] counter b
  const volatile int* abort_word;  // host-mapped; non-zero aborts
  int* status;                 // local status word
};

__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint64_t* p, uint64_t v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_gpu(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Bounded spin until *p == want.  Returns 0 on success, a FTB200_ST_* code otherwise.
// A cross-rank word (SYS) also passes when it already holds a LATER token of the same epoch: tokens of a team
// only grow, every word has one writer, and a peer that is one single-round call ahead (a barrier or a one-shot
// allreduce followed at once by the next collective) may overwrite its token before this rank has looked -- it
// has then certainly posted the one waited for.
// Only system-scope waits (block 0's per-peer threads) look at the host-mapped abort word,
// and only every 256 polls: it sits across PCIe and many concurrent readers are slow.
// Every other waiter learns of an abort through the GO_ABORT value of its go-word.
template <bool SYS>
__device__ __forceinline__ int wait_equal(const uint64_t* p, uint64_t want, const TeamParams& tp, uint64_t t0) {
  uint32_t spins = 0;
  for (;;) {
    const uint64_t v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if (v == want) return FTB200_ST_OK;
    if (SYS && v > want && (v >> 32) == (want >> 32)) return FTB200_ST_OK;
    if (!SYS && v == GO_ABORT) return FTB200_ST_ABORTED;
    ++spins;
    if ((spins & 15u) == 0) {
      if (ftb200::globaltimer_ns() - t0 > tp.timeout_ns) return FTB200_ST_TIMEOUT;
      if (SYS && (spins & 255u) == 0 && tp.abort_word != nullptr && *tp.abort_word != 0) return FTB200_ST_ABORTED;
      if (!SYS) __nanosleep(32);
    }
  }
}

// Cross-rank round on `slot`, executed by block 0 (threads 0..world-1, one peer each),
// then published to the other blocks through local_sync[go_idx].  Every block calls it.
// Returns false if the collective must be abandoned.
__device__ __forceinline__ bool team_round(const TeamParams& tp, int slot, int go_idx, int* sh_code) {
  const uint64_t t0 = ftb200::globaltimer_ns();
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) *sh_code = FTB200_ST_OK;
    __syncthreads();
    if (threadIdx.x < tp.world && static_cast<int>(threadIdx.x) != tp.rank) {
      const int peer = threadIdx.x;
      st_release_sys(tp.flags[peer] + slot * MAX_RANKS + tp.rank, tp.token);
      const int code = wait_equal<true>(tp.flags[tp.rank] + slot * MAX_RANKS + peer, tp.token, tp, t0);
      if (code != FTB200_ST_OK) atomicMax(sh_code, code);
    }
    __syncthreads();
    const int code = *sh_code;
    if (threadIdx.x == 0) {
      if (code != FTB200_ST_OK && tp.status != nullptr) atomicMax(tp.status, code);
      st_release_gpu(tp.local_sync + go_idx, code == FTB200_ST_OK ? tp.token : GO_ABORT);
    }
    __syncthreads();
    return code == FTB200_ST_OK;
  }
  if (threadIdx.x == 0) {
    const int code = wait_equal<false>(tp.local_sync + go_idx, tp.token, tp, t0);
    *sh_code = code;
    if (code == FTB200_ST_TIMEOUT && tp.status != nullptr) atomicMax(tp.status, code);
  }
  __syncthreads();
  return *sh_code == FTB200_ST_OK;
}

// All blocks of this launch have passed this point (arrival counter in local memory).
// Block 0 waits for the others (bounded); the others just arrive.
__device__ __forceinline__ bool grid_arrive(const TeamParams& tp, int counter_idx, int* sh_code) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();  // this block's peer stores are visible before anyone is told "done"
    int code = FTB200_ST_OK;
    uint64_t* ctr = tp.local_sync + counter_idx;
    atomicAdd(reinterpret_cast<unsigned long long*>(ctr), 1ull);
    if (blockIdx.x == 0) {
      const uint64_t t0 = ftb200::globaltimer_ns();
      uint32_t spins = 0;
      while (ld_acquire_gpu(ctr) < gridDim.x) {
        ++spins;
        if ((spins & 15u) == 0) {
          if (ftb200::globaltimer_ns() - t0 > tp.timeout_ns) { code = FTB200_ST_TIMEOUT; break; }
          if ((spins & 1023u) == 0 && tp.abort_word != nullptr && *tp.abort_word != 0) { code = FTB200_ST_ABORTED; break; }
        }
      }
      st_release_gpu(ctr, 0);  // re-arm for the next call (calls on one team are stream-ordered)
      if (code != FTB200_ST_OK) {
        if (tp.status != nullptr) atomicMax(tp.status, code);
        // release the blocks that will wait on the go-words of the rounds that follow
        st_release_gpu(tp.local_sync + 0, GO_ABORT);
        st_release_gpu(tp.local_sync + 1, GO_ABORT);
      }
    }
    *sh_code = code;
  }
  __syncthreads();
  return *sh_code == FTB200_ST_OK;
}

template <typename T>
struct Vec;  // 16-byte vectors
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float* f) { ftb200::unpack8(*reinterpret_cast<const ftb200::bf16x8*>(p), f); }
  __device__ static void store(__nv_bfloat16* p, const float* f) { *reinterpret_cast<ftb200::bf16x8*>(p) = ftb200::pack8(f); }
};
template <>
struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  __device__ static void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};


}  // namespace team
}  // namespace ftb200

// Host-side description of one rank of a team (C ABI).
struct ftb200_team_desc {
  int rank;
  int world;
  unsigned long long token;
  unsigned long long timeout_ns;
  void* flags[ftb200::team::MAX_RANKS];
  void* local_sync;
  const void* abort_word;  // device pointer of host-mapped word (may be null)
  int* status;
};

namespace ftb200 {
namespace team {
inline TeamParams to_params(const ftb200_team_desc* d) {
  TeamParams tp;
  tp.rank = d->rank;
  tp.world = d->world;
  tp.token = d->token;
  tp.timeout_ns = d->timeout_ns;
  for (int i = 0; i < MAX_RANKS; ++i) tp.flags[i] = reinterpret_cast<uint64_t*>(d->flags[i]);
  tp.local_sync = reinterpret_cast<uint64_t*>(d->local_sync);
  tp.abort_word = reinterpret_cast<const volatile int*>(d->abort_word);
  tp.status = d->status;
  return tp;
}
}  // namespace team
}  // namespace ftb200
