// The gradient / batch-statistics all-reduce behind the C-ABI: NCCL over NVLink.
//
// A data-parallel run of the handler path (one process per GPU, the batch axis sharded)
// needs exactly one kind of exchange: a sum or an average of a device array over the
// ranks -- the flat gradient vector after a backward pass, and the results of
// sum_t(axis=0) over the batch axis.  These entry points give a host that binds this
// library without any Python framework that exchange:
//   * rank 0 asks for an id (b200_comm_unique_id), the host hands its 128 bytes to the
//     other ranks by whatever means it has, every rank calls b200_comm_init;
//   * b200_comm_allreduce queues an in-place all-reduce on the library's current stream,
//     in program order with the kernels around it;
//   * b200_comm_allreduce_async queues it on a second stream behind the work queued so
//     far, so that kernels queued afterwards run beside it (the gradients of one layer
//     travel while the layers before it are still in their backward pass);
//     b200_comm_join makes later work wait for all of those.
// All of it can be part of a recorded graph (b200_graph_begin .. b200_graph_end).
//
// NCCL is not linked: it is looked up at run time (the copy a framework in the same
// process has already loaded, else libnccl.so.2 from the loader's path, else the file
// named by B200_NCCL_LIB).  Without it b200_comm_init fails with a message and
// everything else in the library works as before.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace b200 {
namespace {

// The few declarations of NCCL's public C interface that are used here (stable across 2.x).
struct NcclId { char bytes[128]; };
typedef void* NcclComm;
constexpr int kNcclFloat32 = 7, kNcclSum = 0, kNcclAvg = 4;
typedef int (*GetUniqueIdFn)(NcclId*);
typedef int (*CommInitRankFn)(NcclComm*, int, NcclId, int);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
typedef int (*CommDestroyFn)(NcclComm);
typedef const char* (*GetErrorStringFn)(int);

struct CommState {
  void* dl = nullptr;
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  AllReduceFn all_reduce = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  GetErrorStringFn error_string = nullptr;
  NcclComm comm = nullptr;
  int rank = -1, world = 0;
  cudaStream_t side = nullptr;      // carries the asynchronous all-reduces
  cudaEvent_t fork = nullptr, join = nullptr;
  bool pending = false;             // asynchronous all-reduces queued since the last join
} g_comm;

int load_nccl() {
  if (g_comm.all_reduce) return B200_OK;
  const char* names[3] = {getenv("B200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  void* dl = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);   // already in the process?
  for (int i = 0; i < 3 && !dl; ++i)
    if (names[i] && names[i][0]) dl = dlopen(names[i], RTLD_NOW | RTLD_LOCAL);
  if (!dl)
    return set_error(B200_ERR_UNSUPPORTED, "NCCL is not available (libnccl.so.2 not found; set B200_NCCL_LIB): %s",
                     dlerror());
  g_comm.get_unique_id = (GetUniqueIdFn)dlsym(dl, "ncclGetUniqueId");
  g_comm.comm_init_rank = (CommInitRankFn)dlsym(dl, "ncclCommInitRank");
  g_comm.comm_destroy = (CommDestroyFn)dlsym(dl, "ncclCommDestroy");
  g_comm.error_string = (GetErrorStringFn)dlsym(dl, "ncclGetErrorString");
  AllReduceFn ar = (AllReduceFn)dlsym(dl, "ncclAllReduce");
  if (!g_comm.get_unique_id || !g_comm.comm_init_rank || !g_comm.comm_destroy || !ar)
    return set_error(B200_ERR_UNSUPPORTED, "the NCCL library that was found lacks a symbol this library needs");
  g_comm.dl = dl;
  g_comm.all_reduce = ar;
  return B200_OK;
}

int nccl_fail(int rc, const char* what) {
  return set_error(B200_ERR_CUDA, "NCCL error %d (%s) in %s", rc,
                   g_comm.error_string ? g_comm.error_string(rc) : "?", what);
}

}  // namespace
}  // namespace b200

using namespace b200;

// Fills id[0..128) with a fresh communicator id (call on one rank, hand to all).
B200_API int b200_comm_unique_id(void* id) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(id != nullptr, "id is NULL");
  if (int rc = load_nccl()) return rc;
  NcclId nid;
  if (int rc = g_comm.get_unique_id(&nid)) return nccl_fail(rc, "ncclGetUniqueId");
  memcpy(id, &nid, sizeof(nid));
  return B200_OK;
}

// Collective over all ranks: joins the communicator `id` names as rank `rank` of `world`
// on the GPU this process is bound to.
B200_API int b200_comm_init(int rank, int world, const void* id) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(id != nullptr && world >= 1 && rank >= 0 && rank < world, "bad rank / world / id");
  B200_REQUIRE(g_comm.comm == nullptr, "a communicator exists already (b200_comm_destroy first)");
  if (int rc = load_nccl()) return rc;
  NcclId nid;
  memcpy(&nid, id, sizeof(nid));
  if (int rc = g_comm.comm_init_rank(&g_comm.comm, world, nid, rank)) {
    g_comm.comm = nullptr;
    return nccl_fail(rc, "ncclCommInitRank");
  }
  if (!g_comm.side) {
    B200_CUDA(cudaStreamCreateWithFlags(&g_comm.side, cudaStreamNonBlocking));
    B200_CUDA(cudaEventCreateWithFlags(&g_comm.fork, cudaEventDisableTiming));
    B200_CUDA(cudaEventCreateWithFlags(&g_comm.join, cudaEventDisableTiming));
  }
  g_comm.rank = rank;
  g_comm.world = world;
  g_comm.pending = false;
  return B200_OK;
}

// Number of ranks of the communicator (0: none).
B200_API int b200_comm_world(void) { return g_comm.comm ? g_comm.world : 0; }

// data[i] = sum over ranks of data[i] (average != 0: the mean), in place, queued on the
// library's current stream.  Every rank makes the same calls in the same order.
B200_API int b200_comm_allreduce(float* data, int64_t count, int average) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(g_comm.comm != nullptr, "b200_comm_init has not been called");
  B200_REQUIRE(count >= 0, "negative count");
  if (count == 0) return B200_OK;
  B200_REQUIRE(data != nullptr, "NULL operand");
  if (int rc = g_comm.all_reduce(data, data, (size_t)count, kNcclFloat32, average ? kNcclAvg : kNcclSum, g_comm.comm,
                                 state().stream))
    return nccl_fail(rc, "ncclAllReduce");
  return B200_OK;
}

// The same all-reduce on the communication stream: it starts when everything queued on
// the current stream so far has finished, and what is queued afterwards does not wait
// for it until b200_comm_join.
B200_API int b200_comm_allreduce_async(float* data, int64_t count, int average) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(g_comm.comm != nullptr, "b200_comm_init has not been called");
  B200_REQUIRE(count >= 0, "negative count");
  if (count == 0) return B200_OK;
  B200_REQUIRE(data != nullptr, "NULL operand");
  B200_CUDA(cudaEventRecord(g_comm.fork, state().stream));
  B200_CUDA(cudaStreamWaitEvent(g_comm.side, g_comm.fork, 0));
  if (int rc = g_comm.all_reduce(data, data, (size_t)count, kNcclFloat32, average ? kNcclAvg : kNcclSum, g_comm.comm,
                                 g_comm.side))
    return nccl_fail(rc, "ncclAllReduce");
  g_comm.pending = true;
  return B200_OK;
}

// Work queued on the current stream after this call sees the results of every
// b200_comm_allreduce_async issued before it.
B200_API int b200_comm_join(void) {
  if (int rc = require_ready()) return rc;
  if (!g_comm.pending) return B200_OK;
  B200_CUDA(cudaEventRecord(g_comm.join, g_comm.side));
  B200_CUDA(cudaStreamWaitEvent(state().stream, g_comm.join, 0));
  g_comm.pending = false;
  return B200_OK;
}

// Collective: leaves the communicator.  Work queued before must have finished on every
// rank (synchronise, then a host barrier).
B200_API int b200_comm_destroy(void) {
  if (!g_comm.comm) return B200_OK;
  NcclComm c = g_comm.comm;
  g_comm.comm = nullptr;
  g_comm.world = 0;
  g_comm.rank = -1;
  g_comm.pending = false;
  if (int rc = g_comm.comm_destroy(c)) return nccl_fail(rc, "ncclCommDestroy");
  return B200_OK;
}
