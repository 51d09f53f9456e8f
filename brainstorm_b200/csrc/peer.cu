// All-reduce of small arrays over NVLink peer memory, one kernel per call.
//
// The exchanges on the handler path that sit next to a reduction are small: the sums
// over the batch axis that sum_t(axis=0) completes across the batch shards (BatchNorm
// statistics, the op suite's axis-0 sum) are a few thousand floats.  A library
// collective costs tens of microseconds of launch and protocol for them.  Here every
// rank (one process per GPU) owns a "window" of device memory that all other ranks of
// the node have mapped (cudaIpc): two data slots and one arrival counter per rank.  One
// CTA per call
//   0. takes the next epoch from this rank's call counter (device memory, so a recorded
//      call advances it on every replay),
//   1. copies the local values into this rank's slot of the current epoch's parity,
//   2. publishes the epoch to every rank's counter array (system-scope release store
//      over NVLink),
//   3. waits until all ranks have published this epoch (bounded spin on local memory),
//   4. adds the slots of all ranks in rank order -- the same order on every rank, so all
//      replicas get the same bits -- and writes the result.
// Two slots suffice: a rank can only be one epoch ahead of the slowest one, because its
// next wait needs everybody's next publication, which follows their reads of this epoch.
// Plain peer loads and stores only; no multimem, no NCCL.  The wait is bounded (about
// 20 seconds by default; b200_set_tuning key 8 sets the number of polls); on a timeout the
// kernel leaves dst untouched, raises the library's device error flag and returns.  The
// next synchronising call reports the flag and switches the peer path off
// (b200_peer_enabled() == 0): epochs and slots of the ranks are no longer in step, so
// callers go back to their library collective until b200_peer_setup is called again.
//
// Kernels of different ranks wait for one another, so every rank must run on its own
// GPU (one process per GPU, as everywhere in this library).
#include <string.h>

#include "common.cuh"
#include "peer.cuh"

namespace b200 {

int* device_error_flag();   // gemm_tc.cu: mapped host word reported at the next synchronisation

struct PeerState {
  int rank = -1, world = 0;
  bool disabled = false;                  // set when a wait ran out (see peer_disable)
  uint8_t* window[PEER_MAX_RANKS] = {};   // [rank] = own window, others = mapped peers
} g_peer;

__global__ void __launch_bounds__(1024)
peer_allreduce_kernel(PeerArgs a, const float* src, float* dst, int n, int average,   // dst may be src
                      int* error_flag, unsigned spin_limit) {
  peer_exchange_block(a, src, dst, n, average, error_flag, spin_limit);
}

bool peer_args(PeerArgs* out) {
  if (g_peer.world <= 0 || g_peer.disabled) return false;
  for (int r = 0; r < PEER_MAX_RANKS; ++r) out->window[r] = g_peer.window[r];
  out->rank = g_peer.rank;
  out->world = g_peer.world;
  return true;
}

// Called by the synchronising entry points when they find the device error flag raised:
// a peer all-reduce may have given up, after which the ranks' epochs disagree.
void peer_disable() {
  if (g_peer.world > 0) g_peer.disabled = true;
}

}  // namespace b200

using namespace b200;

// Size of the window every rank allocates (b200_peer_window_alloc) and exports.
B200_API uint64_t b200_peer_window_bytes(void) { return PEER_WINDOW_BYTES; }
B200_API int b200_peer_max_floats(void) { return PEER_MAX_FLOATS; }

// The window of this rank: plain cudaMalloc memory (stream-ordered pool memory cannot
// be exported), zeroed.  `handle` receives the 64 bytes other processes open.
B200_API int b200_peer_window_alloc(uint64_t* ptr, void* handle) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(ptr != nullptr && handle != nullptr, "NULL argument");
  void* p = nullptr;
  B200_CUDA(cudaMalloc(&p, PEER_WINDOW_BYTES));
  B200_CUDA(cudaMemset(p, 0, PEER_WINDOW_BYTES));
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "cudaIpcGetMemHandle", __FILE__, __LINE__);
  }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle, &h, sizeof(h));
  *ptr = (uint64_t)(uintptr_t)p;
  return B200_OK;
}

// Maps the window another process of this node exported.
B200_API int b200_peer_window_open(const void* handle, uint64_t* ptr) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(ptr != nullptr && handle != nullptr, "NULL argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  B200_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = (uint64_t)(uintptr_t)p;
  return B200_OK;
}

// Gives back a window that never reached b200_peer_setup (a rank whose set-up failed half
// way): `own` != 0 frees a window of b200_peer_window_alloc, else unmaps one of
// b200_peer_window_open.
B200_API int b200_peer_window_release(uint64_t ptr, int own) {
  if (ptr == 0) return B200_OK;
  if (own) B200_CUDA(cudaFree((void*)(uintptr_t)ptr));
  else B200_CUDA(cudaIpcCloseMemHandle((void*)(uintptr_t)ptr));
  return B200_OK;
}

// windows[r] for r in [0, world): this rank's own window at [rank], the mapped ones elsewhere.
// Starts the epochs at zero and clears this rank's arrival counters, so windows that were
// used before can be registered again.  The host must put a barrier over all ranks between
// this call and the first b200_peer_allreduce (no rank may publish an epoch into a counter
// array that is still to be cleared).
B200_API int b200_peer_setup(int rank, int world, const uint64_t* windows) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(world >= 1 && world <= PEER_MAX_RANKS && rank >= 0 && rank < world && windows != nullptr,
               "bad rank / world (at most %d ranks)", PEER_MAX_RANKS);
  B200_REQUIRE(windows[rank] != 0, "this rank's own window is NULL");
  B200_CUDA(cudaStreamSynchronize(state().stream));   // calls on an earlier registration have finished
  B200_CUDA(cudaMemset((uint8_t*)(uintptr_t)windows[rank] + PEER_COUNTER_OFFSET, 0,
                       PEER_WINDOW_BYTES - PEER_COUNTER_OFFSET));
  g_peer.rank = rank;
  g_peer.world = world;
  g_peer.disabled = false;
  for (int r = 0; r < world; ++r) g_peer.window[r] = (uint8_t*)(uintptr_t)windows[r];
  return B200_OK;
}

// Calls made since b200_peer_setup and the time they spent between publishing their epoch and seeing
// everybody else's (the other ranks' lateness plus one trip over NVLink).  Synchronises.
B200_API int b200_peer_wait_stats(uint64_t* calls, uint64_t* waited_ns) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(g_peer.world > 0 && calls != nullptr && waited_ns != nullptr, "no peer registration or NULL argument");
  B200_CUDA(cudaStreamSynchronize(state().stream));
  unsigned long long both[2] = {0, 0};
  B200_CUDA(cudaMemcpy(both, g_peer.window[g_peer.rank] + PEER_CALLS_OFFSET, sizeof(both), cudaMemcpyDeviceToHost));
  *calls = both[0];
  *waited_ns = both[1];
  return B200_OK;
}

// 1 while b200_peer_allreduce may be used: after b200_peer_setup and until a wait ran out.
B200_API int b200_peer_enabled(void) { return g_peer.world > 0 && !g_peer.disabled; }

// Unmaps the peers' windows and frees this rank's.  All ranks must have finished their
// last b200_peer_allreduce (synchronise, then a host barrier) before any rank calls this.
B200_API int b200_peer_teardown(void) {
  if (g_peer.world == 0) return B200_OK;
  for (int r = 0; r < g_peer.world; ++r) {
    if (!g_peer.window[r]) continue;
    if (r == g_peer.rank) cudaFree(g_peer.window[r]);
    else cudaIpcCloseMemHandle(g_peer.window[r]);
    g_peer.window[r] = nullptr;
  }
  cudaGetLastError();   // a window that could not be unmapped must not fail the next launch check
  g_peer.world = 0;
  g_peer.rank = -1;
  g_peer.disabled = false;
  return B200_OK;
}

// dst[i] = sum over ranks of src[i] (or the mean), n <= b200_peer_max_floats().  Every rank
// calls it in the same order with the same n; dst may be src.  Queued on the library's
// current stream like any other kernel; a rank that never arrives makes the others give up
// after the poll limit (about 20 seconds by default), leave dst as it was and raise the
// device error flag: the next synchronising call returns the error and the peer path is
// off until the next b200_peer_setup.
B200_API int b200_peer_allreduce(const float* src, float* dst, int n, int average) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(g_peer.world > 0, "b200_peer_setup has not been called");
  B200_REQUIRE(!g_peer.disabled, "the peer all-reduce is switched off: an earlier call gave up waiting for a rank; "
                                 "register the windows again with b200_peer_setup");
  B200_REQUIRE(n >= 0 && n <= PEER_MAX_FLOATS, "at most %d floats per call", PEER_MAX_FLOATS);
  if (n == 0) return B200_OK;
  B200_REQUIRE(src != nullptr && dst != nullptr, "NULL operand");
  PeerArgs a;
  for (int r = 0; r < PEER_MAX_RANKS; ++r) a.window[r] = g_peer.window[r];
  a.rank = g_peer.rank;
  a.world = g_peer.world;
  int threads = (n + 31) / 32 * 32;          // at least one warp (the ranks' counters are handled by threads 0..world-1)
  if (threads > 1024) threads = 1024;
  peer_allreduce_kernel<<<1, threads, 0, state().stream>>>(a, src, dst, n, average, device_error_flag(),
                                                           state().peer_spin_limit);
  B200_LAUNCH_CHECK();
  return B200_OK;
}
