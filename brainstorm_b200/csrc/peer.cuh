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
constexpr size_t PEER_WINDOW_BYTES = PEER_COUNTER_OFFSET + 256;   // counters: PEER_MAX_RANKS x 8 bytes, the call counter, padding

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

// The exchange itself, run by ALL threads of one block (any block shape with at least PEER_MAX_RANKS threads):
// dst[i] = sum (or mean) over ranks of src[i]; dst may be src.  Used by the kernel of b200_peer_allreduce and by the
// column-sum kernel, whose last block completes its sums across the ranks without a launch in between.
__device__ __forceinline__ void peer_exchange_block(const PeerArgs& a, const float* src, float* dst, int n, int average,
                                                    int* error_flag, unsigned spin_limit) {
  const int tid = (threadIdx.z * blockDim.y + threadIdx.y) * blockDim.x + threadIdx.x;
  const int nthreads = blockDim.x * blockDim.y * blockDim.z;
  __shared__ int timed_out;
  __shared__ unsigned long long epoch_shared;
  __shared__ const float* slots[PEER_MAX_RANKS];     // every rank's slot of this epoch's parity
  // The epoch is this rank's call counter.  It lives in the window, not in an argument, so
  // that a call recorded into a graph takes the next epoch on every replay.
  if (tid == 0) {
    unsigned long long* calls = reinterpret_cast<unsigned long long*>(a.window[a.rank] + PEER_CALLS_OFFSET);
    epoch_shared = *calls + 1;
    *calls = epoch_shared;
  }
  __syncthreads();
  const unsigned long long epoch = epoch_shared;
  const int slot = (int)(epoch & 1);
  float* mine = reinterpret_cast<float*>(a.window[a.rank] + slot * PEER_SLOT_BYTES);
  if (tid == 0) timed_out = 0;
  if (tid < a.world)
    slots[tid] = reinterpret_cast<const float*>(a.window[tid] + slot * PEER_SLOT_BYTES);
  // 128-bit accesses when the caller's arrays allow them (the slots always do)
  const bool vec = (n & 3) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
  if (vec) {
    for (int i = tid; i < (n >> 2); i += nthreads)
      reinterpret_cast<float4*>(mine)[i] = __ldcg(reinterpret_cast<const float4*>(src) + i);   // from L2: other blocks may have written src
  } else {
    for (int i = tid; i < n; i += nthreads) mine[i] = __ldcg(src + i);
  }
  __threadfence_system();     // the slot is written before the epoch is published
  __syncthreads();
  if (tid < a.world) {
    unsigned long long* counters = reinterpret_cast<unsigned long long*>(a.window[tid] + PEER_COUNTER_OFFSET);
    st_release_sys(counters + a.rank, epoch);
  }
  unsigned long long wait_begin = 0;
  if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(wait_begin));
  if (tid < a.world) {
    const unsigned long long* counters =
        reinterpret_cast<const unsigned long long*>(a.window[a.rank] + PEER_COUNTER_OFFSET);
    bool seen = false;
    // Ranks drift apart on the host (by seconds while a job starts up), so the default
    // bound is generous: about 20 s (2^22 polls, 4 us apart after the first thousand).
    for (unsigned it = 0; it < spin_limit && !seen; ++it) {
      seen = ld_acquire_sys(counters + tid) >= epoch;
      if (!seen && it > 32) __nanosleep(it > 1024 ? 4000 : 200);
    }
    if (!seen) timed_out = 1;
  }
  __syncthreads();
  if (tid == 0) {     // how long the slowest rank kept this one waiting (b200_peer_wait_stats)
    unsigned long long wait_end;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(wait_end));
    *reinterpret_cast<unsigned long long*>(a.window[a.rank] + PEER_WAITED_OFFSET) += wait_end - wait_begin;
  }
  if (timed_out) {
    if (tid == 0 && error_flag) *error_flag = 1;
    return;                   // dst is left as it was; the host reports the flag
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
    return;
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
}


// Host side (peer.cu): the registered windows as kernel arguments; false when no registration is usable.
bool peer_args(PeerArgs* out);

}  // namespace b200
