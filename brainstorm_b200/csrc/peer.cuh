// The all-reduce of small arrays over NVLink peer memory as a block-level device function (see peer.cu for the
// protocol): shared by the stand-alone kernel and by kernels that finish a reduction with it.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int PEER_MAX_RANKS = 16;
constexpr int PEER_MAX_FLOATS = 65536;                  // per call: 256 KiB per slot
constexpr size_t PEER_SLOT_BYTES = (size_t)PEER_MAX_FLOATS * sizeof(float);
constexpr size_t PEER_COUNTER_OFFSET = 2 * PEER_SLOT_BYTES;
constexpr size_t PEER_CALLS_OFFSET = PEER_COUNTER_OFFSET + 128;  // this rank's own call counter (the epoch)
constexpr size_t PEER_WAITED_OFFSET = PEER_CALLS_OFFSET + 8;      // nanoseconds this rank's calls have spent waiting for the others
constexpr int PEER_MAX_GROUPS = 512;                              // pieces of one call that are announced one by one
constexpr size_t PEER_GROUP_OFFSET = PEER_COUNTER_OFFSET + 256;   // [rank][group] arrival counters of those pieces
constexpr size_t PEER_WINDOW_BYTES = PEER_GROUP_OFFSET + (size_t)PEER_MAX_RANKS * PEER_MAX_GROUPS * 8;

struct PeerArgs {
  uint8_t* window[PEER_MAX_RANKS];
  int rank, world;
};

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// The exchange of the columns [c0, c0 + n) of an array, run by ALL threads of one block (any block shape with at
// least PEER_MAX_RANKS threads): dst[c] = sum (or mean) over ranks of src[c]; dst may be src.  `epoch` is the number
// of the call this belongs to (the same on every rank).  GROUPED = false: the whole array travels in one piece and
// the ranks announce it in their per-rank counters (the kernel of b200_peer_allreduce).  GROUPED = true: the array
// travels in pieces ("groups") that are announced and awaited one by one, each by the block that produced it, so a
// piece is on its way while other blocks of the kernel are still computing theirs (the column-sum kernel).
// On a wait that runs out: dst is left as it was, *error_flag is raised, and the function returns true.
template <bool GROUPED>
__device__ __forceinline__ bool peer_exchange_range(const PeerArgs& a, unsigned long long epoch, int group, const float* src,
                                                    float* dst, int c0, int n, int average, int* error_flag,
                                                    unsigned spin_limit, unsigned wait_share) {
  const int tid = (threadIdx.z * blockDim.y + threadIdx.y) * blockDim.x + threadIdx.x;
  const int nthreads = blockDim.x * blockDim.y * blockDim.z;
  __shared__ int timed_out;
  __shared__ const float* slots[PEER_MAX_RANKS];     // every rank's slot of this epoch's parity
  const int slot = (int)(epoch & 1);
  float* mine = reinterpret_cast<float*>(a.window[a.rank] + slot * PEER_SLOT_BYTES) + c0;
  src += c0;
  dst += c0;
  __syncthreads();            // the shared words above may still be in use by an earlier call of this block
  if (tid == 0) timed_out = 0;
  if (tid < a.world)
    slots[tid] = reinterpret_cast<const float*>(a.window[tid] + slot * PEER_SLOT_BYTES) + c0;
  // 128-bit accesses when the arrays allow them (the slots do whenever c0 is a multiple of 4)
  const bool vec = ((n | c0) & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
  if (vec) {
    for (int i = tid; i < (n >> 2); i += nthreads)
      reinterpret_cast<float4*>(mine)[i] = __ldcg(reinterpret_cast<const float4*>(src) + i);   // from L2: other blocks may have written src
  } else {
    for (int i = tid; i < n; i += nthreads) mine[i] = __ldcg(src + i);
  }
  __threadfence_system();     // the slot is written before the epoch is published
  __syncthreads();
  const size_t mine_at = GROUPED ? PEER_GROUP_OFFSET + ((size_t)a.rank * PEER_MAX_GROUPS + group) * 8
                                 : PEER_COUNTER_OFFSET + (size_t)a.rank * 8;
  if (tid < a.world) st_release_sys(reinterpret_cast<unsigned long long*>(a.window[tid] + mine_at), epoch);
  unsigned long long wait_begin = 0;
  if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(wait_begin));
  if (tid < a.world) {
    const size_t theirs_at = GROUPED ? PEER_GROUP_OFFSET + ((size_t)tid * PEER_MAX_GROUPS + group) * 8
                                     : PEER_COUNTER_OFFSET + (size_t)tid * 8;
    const unsigned long long* counter = reinterpret_cast<const unsigned long long*>(a.window[a.rank] + theirs_at);
    bool seen = false;
    // Ranks drift apart on the host (by seconds while a job starts up), so the default
    // bound is generous: about 20 s (2^22 polls, 4 us apart after the first thousand).
    for (unsigned it = 0; it < spin_limit && !seen; ++it) {
      seen = ld_acquire_sys(counter) >= epoch;
      if (!seen && it > 32) __nanosleep(it > 1024 ? 4000 : 200);
    }
    if (!seen) timed_out = 1;
  }
  __syncthreads();
  if (tid == 0) {     // how long the slowest rank kept this one waiting (b200_peer_wait_stats)
    unsigned long long wait_end;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(wait_end));
    atomicAdd(reinterpret_cast<unsigned long long*>(a.window[a.rank] + PEER_WAITED_OFFSET), (wait_end - wait_begin) / wait_share);
  }
  if (timed_out) {
    if (tid == 0 && error_flag) *error_flag = 1;
    return true;              // dst is left as it was; the host reports the flag
  }
  // The ranks' slots are read eight at a time: the loads of a batch are all issued before the first
  // sum needs one, so a batch costs one trip over NVLink, not one per rank.  The sums run in rank order.
  const float scale = average ? 1.0f / (float)a.world : 1.0f;
  constexpr int BATCH = 8;
  if (vec) {
    const int nv = n >> 2;
    for (int i = tid; i < nv; i += nthreads) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r0 = 0; r0 < a.world; r0 += BATCH) {
        float4 v[BATCH];
#pragma unroll
        for (int k = 0; k < BATCH; ++k)
          if (r0 + k < a.world) v[k] = __ldcv(reinterpret_cast<const float4*>(slots[r0 + k]) + i);   // not cached: written by another GPU
#pragma unroll
        for (int k = 0; k < BATCH; ++k) {
          if (r0 + k >= a.world) continue;
          if (r0 + k == 0) acc = v[k];
          else acc = make_float4(__fadd_rn(acc.x, v[k].x), __fadd_rn(acc.y, v[k].y), __fadd_rn(acc.z, v[k].z),
                                 __fadd_rn(acc.w, v[k].w));
        }
      }
      if (average) acc = make_float4(__fmul_rn(acc.x, scale), __fmul_rn(acc.y, scale), __fmul_rn(acc.z, scale),
                                     __fmul_rn(acc.w, scale));
      reinterpret_cast<float4*>(dst)[i] = acc;
    }
    return false;
  }
  for (int i = tid; i < n; i += nthreads) {
    float acc = 0.f;
    for (int r0 = 0; r0 < a.world; r0 += BATCH) {
      float v[BATCH];
#pragma unroll
      for (int k = 0; k < BATCH; ++k)
        if (r0 + k < a.world) v[k] = __ldcv(slots[r0 + k] + i);
#pragma unroll
      for (int k = 0; k < BATCH; ++k) {
        if (r0 + k >= a.world) continue;
        acc = (r0 + k == 0) ? v[k] : __fadd_rn(acc, v[k]);
      }
    }
    dst[i] = average ? __fmul_rn(acc, scale) : acc;
  }
  return false;
}

// The number of the call that is running now: this rank's call counter plus one.  The counter lives in the window,
// not in an argument, so that a call recorded into a graph takes the next number on every replay.
__device__ __forceinline__ unsigned long long peer_next_epoch(const PeerArgs& a) {
  return *reinterpret_cast<volatile unsigned long long*>(a.window[a.rank] + PEER_CALLS_OFFSET) + 1;
}
__device__ __forceinline__ void peer_close_epoch(const PeerArgs& a, unsigned long long epoch) {
  *reinterpret_cast<volatile unsigned long long*>(a.window[a.rank] + PEER_CALLS_OFFSET) = epoch;
}

// A whole array in one piece, by one block: the kernel of b200_peer_allreduce.
__device__ __forceinline__ void peer_exchange_block(const PeerArgs& a, const float* src, float* dst, int n, int average,
                                                    int* error_flag, unsigned spin_limit) {
  __shared__ unsigned long long epoch_shared;
  const int tid = (threadIdx.z * blockDim.y + threadIdx.y) * blockDim.x + threadIdx.x;
  if (tid == 0) {
    epoch_shared = peer_next_epoch(a);
    peer_close_epoch(a, epoch_shared);
  }
  __syncthreads();
  peer_exchange_range<false>(a, epoch_shared, 0, src, dst, 0, n, average, error_flag, spin_limit, 1u);
}

// Host side (peer.cu): the registered windows as kernel arguments; false when no registration is usable.
bool peer_args(PeerArgs* out);

}  // namespace b200
