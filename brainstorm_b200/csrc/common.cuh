// Shared declarations of the B200 handler library: status codes, the error
// slot behind b200_last_error(), the library's current stream and a few device
// helpers.  Everything here is internal; the public C-ABI is
// include/b200_handler.h.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define B200_OK 0
#define B200_ERR_CUDA 1
#define B200_ERR_ARG 2
#define B200_ERR_DEVICE_FLAG 4
#define B200_ERR_UNSUPPORTED 5

#define B200_API extern "C" __attribute__((visibility("default")))

namespace b200 {

// ---- error slot ---------------------------------------------------------
int set_error(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define B200_CUDA(call)                                                        \
  do {                                                                         \
    cudaError_t e__ = (call);                                                  \
    if (e__ != cudaSuccess) return b200::cuda_fail(e__, #call, __FILE__, __LINE__); \
  } while (0)

// For entry points that wait for the device or move data across PCIe: these cannot
// become nodes of a recorded graph.
#define B200_NOT_WHILE_RECORDING(what)                                                        \
  do {                                                                                        \
    if (b200::state().capturing)                                                              \
      return b200::set_error(B200_ERR_UNSUPPORTED,                                            \
                             what " is not possible while a graph is being recorded "         \
                             "(between b200_graph_begin and b200_graph_end)");                \
  } while (0)

#define B200_REQUIRE(cond, ...)                                                \
  do {                                                                         \
    if (!(cond)) return b200::set_error(B200_ERR_ARG, __VA_ARGS__);            \
  } while (0)

// Checks the launch that has just been issued (asynchronous errors surface at
// the next synchronising call) and counts it (b200_launch_count).
#define B200_LAUNCH_CHECK()            \
  do {                                 \
    ++b200::state().launches;          \
    B200_CUDA(cudaGetLastError());     \
  } while (0)

// ---- per-process state ----------------------------------------------------
struct State {
  bool ready = false;
  int device = -1;
  int sm_count = 148;
  cudaStream_t stream = nullptr;      // the stream work is queued on now: streams[stream_index]
  cudaStream_t streams[2] = {nullptr, nullptr};   // [0] the library's main stream, [1] the side stream
  int stream_index = 0;
  uint64_t launches = 0;  // kernels launched by this library so far
  // tuning knobs (b200_set_tuning)
  int ew_blocks_per_sm = 32;
  int ew_threads = 1024;
  int red_blocks_per_sm = 8;   // pass-1 blocks per SM of the two-pass sums
  int axis0_peer_fused = 0;    // b200_sum_t_axis0_allreduce: 1 = the exchange runs inside the column-sum kernel, group by group
                               // (measured slower than the all-reduce kernel behind it, which is the default)
  int axis0_fold = 1;          // column sums: the last pass-1 block of a column group does pass 2 (0: a launch of its own)
  int gemm_path = 0;  // 0 = auto, 1 = force SIMT, 2 = force tensor-core
  int gemm_bn = 0;    // 0 = auto, else forced tile width (32/64/128/256)
  int use_pdl = 1;    // programmatic dependent launch inside the LSTM time loops
  int gemm_pair = 0;   // 256-wide GEMM tiles on pairs of SMs (tcgen05 cta_group::2)
  int gemm_chunk_kb = 0;     // k-blocks accumulated in tensor memory before a drain (0 = default)
  int sm_share = 1;   // split-K plans for sm_count / sm_share SMs (two streams sharing the GPU)
  bool pdl_now = false;  // set while a time loop is issuing its kernels
  // graph recording (b200_graph_begin .. b200_graph_end)
  bool capturing = false;
  uint64_t* replay_epoch = nullptr;  // device word, advanced before every graph replay
  int live_graphs = 0;               // recorded graphs that have not been destroyed yet
  // bounded device waits on another rank (peer all-reduce): polls before the kernel gives up
  uint32_t peer_spin_limit = 1u << 22;
};
State& state();
int require_ready();
// Releases a library-owned work buffer that recorded graphs may have baked in: freed at
// once (stream-ordered) when no recorded graph is alive, else when the last one is destroyed.
void retire_work_buffer(void* p);

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Programmatic dependent launch: a kernel calls pdl_launch_dependents() to let the
// next kernel of the stream begin its prologue early, and pdl_wait() before it
// touches anything the previous kernel wrote or still reads.  Both are no-ops for
// kernels launched the ordinary way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with the "programmatic stream serialization" attribute when `pdl` is set.
template <class... KArgs, class... Args>
static inline cudaError_t launch_maybe_pdl(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- device helpers -------------------------------------------------------
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

// Sum over a thread block in a fixed order (lane tree, then warp 0 over the warp
// partials): the same inputs always give the same bits.  `smem` holds >= 32
// floats.  The result is valid in every thread.
__device__ __forceinline__ float block_sum(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? smem[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? smem[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

}  // namespace b200
