// Lifecycle, memory and transfer entry points of the B200 handler library.
// Device memory comes from the CUDA stream-ordered pool (cudaMallocAsync) with an
// unlimited release threshold, so the short-lived temporaries that layers
// allocate on every pass are recycled without touching the driver.
#include <stdarg.h>
#include <string.h>

#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace b200 {

int gemm_tc_check_flag();  // gemm_tc.cu: reports a barrier timeout of a tensor-core kernel
int static_scratch_setup();  // reduce.cu: resolves the built-in scratch array of b200_sum_t_static

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
  const char* base = strrchr(file, '/');
  return set_error(B200_ERR_CUDA, "CUDA error %d (%s) in %s at %s:%d", (int)e,
                   cudaGetErrorString(e), what, base ? base + 1 : file, line);
}

State& state() {
  static State s;
  return s;
}

int require_ready() {
  if (!state().ready)
    return set_error(B200_ERR_ARG, "b200_init() has not been called in this process");
  return B200_OK;
}

}  // namespace b200

using namespace b200;

namespace {
struct RecordedGraph {
  cudaGraphExec_t exec = nullptr;
  uint64_t kernels = 0;            // kernel launches recorded (for b200_launch_count)
  std::vector<void*> owned;        // arrays released by the host that replays still use
  std::vector<void*> made;         // arrays allocated during the recording
};
struct Recording {
  cudaStream_t side_stream = nullptr;
  std::vector<void*> deferred;     // released by the host during the recording
  std::vector<void*> made;         // allocated during the recording
  uint64_t launches_at_begin = 0;
} g_rec;
// Arrays that were allocated while a graph was being recorded have their addresses baked
// into it.  The host may keep or drop them as it likes; when it drops one while the graph
// is alive, the memory stays allocated until the graph is destroyed.
std::unordered_map<void*, RecordedGraph*> g_made_by;
// Work buffers of the library (split-K partials) that were replaced while a recorded
// graph was alive: a replay may still write to them, so they stay allocated until the
// last graph is gone.
std::vector<void*> g_retired;
}  // namespace

namespace b200 {
void retire_work_buffer(void* p) {
  if (!p) return;
  if (state().live_graphs > 0) g_retired.push_back(p);
  else cudaFreeAsync(p, state().stream);
}
}  // namespace b200

B200_API const char* b200_last_error(void) { return g_err; }

B200_API int b200_device_count(int* count) {
  B200_REQUIRE(count != nullptr, "count is NULL");
  *count = 0;
  B200_CUDA(cudaGetDeviceCount(count));
  return B200_OK;
}

B200_API int b200_init(int device) {
  State& s = state();
  if (s.ready && s.device == device) return B200_OK;
  B200_REQUIRE(!s.ready, "library already initialised on device %d", s.device);
  int n = 0;
  B200_CUDA(cudaGetDeviceCount(&n));
  B200_REQUIRE(device >= 0 && device < n, "device %d out of range (%d visible)", device, n);
  B200_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  B200_CUDA(cudaGetDeviceProperties(&prop, device));
  B200_REQUIRE(prop.major == 10,
               "device %d is sm_%d%d; this library holds sm_100a code only", device,
               prop.major, prop.minor);
  s.sm_count = prop.multiProcessorCount;
  B200_CUDA(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
  s.streams[0] = s.stream;
  s.stream_index = 0;
  cudaMemPool_t pool;
  B200_CUDA(cudaDeviceGetDefaultMemPool(&pool, device));
  uint64_t keep = UINT64_MAX;
  B200_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
  s.device = device;
  if (int rc = static_scratch_setup()) return rc;
  s.ready = true;
  return B200_OK;
}

B200_API int b200_device_info(int* device, int* sm_count, uint64_t* free_bytes,
                              uint64_t* total_bytes) {
  if (int rc = require_ready()) return rc;
  size_t f = 0, t = 0;
  B200_CUDA(cudaMemGetInfo(&f, &t));
  if (device) *device = state().device;
  if (sm_count) *sm_count = state().sm_count;
  if (free_bytes) *free_bytes = f;
  if (total_bytes) *total_bytes = t;
  return B200_OK;
}

B200_API int b200_set_tuning(int key, int value) {
  State& s = state();
  switch (key) {
    case 0: B200_REQUIRE(value >= 1 && value <= 64, "blocks per SM out of range"); s.ew_blocks_per_sm = value; break;
    case 1: B200_REQUIRE(value >= 64 && value <= 1024 && value % 32 == 0, "threads per block out of range"); s.ew_threads = value; break;
    case 2: B200_REQUIRE(value >= 0 && value <= 2, "gemm path must be 0, 1 or 2"); s.gemm_path = value; break;
    case 3: s.gemm_bn = value; break;
    case 5: s.use_pdl = value ? 1 : 0; break;
    case 7: s.gemm_pair = value ? 1 : 0; break;
    case 6: B200_REQUIRE(value >= 1 && value <= 8, "SM share divisor out of range"); s.sm_share = value; break;
    case 10: B200_REQUIRE(value >= 1 && value <= 27, "reduction blocks per SM out of range"); s.red_blocks_per_sm = value; break;
    case 11: B200_REQUIRE(value == 0 || value == 1, "axis-0 fold is 0 or 1"); s.axis0_fold = value; break;
    case 12: B200_REQUIRE(value == 0 || value == 1, "in-kernel exchange is 0 or 1"); s.axis0_peer_fused = value; break;
    case 9: B200_REQUIRE(value == 0 || value == 1 || value == 2 || value == 4 || value == 8, "chunk must be 0, 1, 2, 4 or 8 k-blocks");
            s.gemm_chunk_kb = value; break;
    case 8: B200_REQUIRE(value >= 0 && value <= 30, "spin limit exponent out of range (0 = default)");
            s.peer_spin_limit = value ? (1u << value) : (1u << 22); break;
    default: return set_error(B200_ERR_ARG, "unknown tuning key %d", key);
  }
  return B200_OK;
}

B200_API uint64_t b200_launch_count(void) { return state().launches; }

B200_API uint64_t b200_stream(void) { return (uint64_t)(uintptr_t)state().streams[0]; }

// ---- a second compute stream ---------------------------------------------------------
// Work of two layers that does not depend on each other timestep by timestep (a stack
// of LSTM layers: layer l+1 at time t needs layer l only up to time t) can run side by
// side.  b200_use_stream(1) makes every following call of this library queue its work
// on the side stream, b200_use_stream(0) returns to the main stream.  Ordering
// between the two is explicit: b200_mark records a marker on the current stream,
// b200_wait_mark makes the current stream wait for one.  Allocations are
// stream-ordered: memory that the side stream touches before it has waited for the
// main stream must be allocated while the side stream is current.
B200_API int b200_use_stream(int index) {
  if (int rc = require_ready()) return rc;
  State& s = state();
  B200_REQUIRE(index == 0 || index == 1, "stream index must be 0 or 1");
  if (!s.streams[index]) B200_CUDA(cudaStreamCreateWithFlags(&s.streams[index], cudaStreamNonBlocking));
  s.stream_index = index;
  s.stream = s.streams[index];
  return B200_OK;
}

B200_API int b200_mark_create(uint64_t* mark) {
  B200_REQUIRE(mark != nullptr, "mark is NULL");
  cudaEvent_t e;
  B200_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  *mark = (uint64_t)(uintptr_t)e;
  return B200_OK;
}
B200_API int b200_mark(uint64_t mark) {
  if (int rc = require_ready()) return rc;
  B200_CUDA(cudaEventRecord((cudaEvent_t)(uintptr_t)mark, state().stream));
  return B200_OK;
}
B200_API int b200_wait_mark(uint64_t mark) {
  if (int rc = require_ready()) return rc;
  B200_CUDA(cudaStreamWaitEvent(state().stream, (cudaEvent_t)(uintptr_t)mark, 0));
  return B200_OK;
}
B200_API int b200_mark_destroy(uint64_t mark) {
  if (mark) B200_CUDA(cudaEventDestroy((cudaEvent_t)(uintptr_t)mark));
  return B200_OK;
}

B200_API int b200_malloc(uint64_t* ptr, uint64_t bytes, int zero) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(ptr != nullptr, "ptr is NULL");
  void* p = nullptr;
  // Zero-byte arrays are routine (buffers are first created for a 0x0 batch);
  // give them a real, distinct address.
  size_t n = bytes ? (size_t)bytes : 16;
  if (state().capturing) {
    // An allocation on the recording stream would belong to the graph.  The array has
    // to exist outside it as well (the caller may keep it), so it is made on a side
    // stream, for real and at once; only the zero fill is recorded.
    B200_CUDA(cudaMallocAsync(&p, n, g_rec.side_stream));
    B200_CUDA(cudaStreamSynchronize(g_rec.side_stream));
    g_rec.made.push_back(p);
  } else {
    B200_CUDA(cudaMallocAsync(&p, n, state().stream));
  }
  if (zero) B200_CUDA(cudaMemsetAsync(p, 0, n, state().stream));
  *ptr = (uint64_t)(uintptr_t)p;
  return B200_OK;
}

B200_API int b200_free(uint64_t ptr) {
  if (!state().ready || ptr == 0) return B200_OK;
  if (state().capturing) {
    // the recorded kernels keep using this address on every replay: the memory
    // stays allocated for as long as the graph exists
    g_rec.deferred.push_back((void*)(uintptr_t)ptr);
    return B200_OK;
  }
  if (!g_made_by.empty()) {
    auto it = g_made_by.find((void*)(uintptr_t)ptr);
    if (it != g_made_by.end()) {   // replays of that graph still use the address
      it->second->owned.push_back(it->first);
      g_made_by.erase(it);
      return B200_OK;
    }
  }
  B200_CUDA(cudaFreeAsync((void*)(uintptr_t)ptr, state().stream));
  return B200_OK;
}

// ---- recorded graphs -------------------------------------------------------------------
// b200_graph_begin() puts the library stream into capture mode: every kernel, fill
// and device-to-device copy issued through this library until b200_graph_end() is
// recorded instead of executed.  The result replays with one call
// (b200_graph_launch), which removes the per-kernel launch cost of steps made of
// many small kernels.  All addresses and scalar arguments are frozen into the graph.
// Random masks are the exception: the RNG kernels add a device-side replay counter
// to their Philox counter, so every replay draws fresh numbers.
__global__ void advance_epoch_kernel(uint64_t* epoch) { *epoch += 1; }

B200_API int b200_graph_begin(void) {
  if (int rc = require_ready()) return rc;
  State& s = state();
  B200_REQUIRE(!s.capturing, "a graph is already being recorded");
  B200_REQUIRE(s.stream_index == 0, "a recording starts on the main stream");
  if (!g_rec.side_stream) B200_CUDA(cudaStreamCreateWithFlags(&g_rec.side_stream, cudaStreamNonBlocking));
  if (!s.replay_epoch) {
    B200_CUDA(cudaMalloc((void**)&s.replay_epoch, sizeof(uint64_t)));
    B200_CUDA(cudaMemsetAsync(s.replay_epoch, 0, sizeof(uint64_t), s.stream));
  }
  // work queued so far must not be overtaken by allocations made on the side stream
  B200_CUDA(cudaStreamSynchronize(s.stream));
  if (int rc = gemm_tc_check_flag()) return rc;
  g_rec.deferred.clear();
  g_rec.made.clear();
  g_rec.launches_at_begin = s.launches;
  B200_CUDA(cudaStreamBeginCapture(s.stream, cudaStreamCaptureModeRelaxed));
  s.capturing = true;
  return B200_OK;
}

static void release_all(std::vector<void*>& ptrs) {
  for (void* p : ptrs) cudaFreeAsync(p, state().stream);
  ptrs.clear();
}

// Ends the recording.  With graph == NULL the recording is discarded.
B200_API int b200_graph_end(uint64_t* graph) {
  State& s = state();
  B200_REQUIRE(s.capturing, "no graph is being recorded");
  s.capturing = false;
  cudaGraph_t g = nullptr;
  const cudaError_t e = cudaStreamEndCapture(s.stream, &g);
  const uint64_t recorded = s.launches - g_rec.launches_at_begin;
  s.launches = g_rec.launches_at_begin;   // recorded kernels have not run
  if (e != cudaSuccess || g == nullptr || graph == nullptr) {
    if (g) cudaGraphDestroy(g);
    release_all(g_rec.deferred);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return cuda_fail(e, "cudaStreamEndCapture", __FILE__, __LINE__);
    }
    if (graph == nullptr) return B200_OK;
    return set_error(B200_ERR_CUDA, "the recording produced no graph");
  }
  cudaGraphExec_t exec = nullptr;
  const cudaError_t ei = cudaGraphInstantiate(&exec, g, 0);
  cudaGraphDestroy(g);
  if (ei != cudaSuccess) {
    release_all(g_rec.deferred);
    return cuda_fail(ei, "cudaGraphInstantiate", __FILE__, __LINE__);
  }
  RecordedGraph* r = new RecordedGraph;
  r->exec = exec;
  r->kernels = recorded;
  r->owned.swap(g_rec.deferred);
  r->made.swap(g_rec.made);
  for (void* p : r->made) g_made_by[p] = r;
  for (void* p : r->owned) g_made_by.erase(p);    // made and released inside the recording
  ++s.live_graphs;
  *graph = (uint64_t)(uintptr_t)r;
  return B200_OK;
}

B200_API int b200_graph_launch(uint64_t graph) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(graph != 0, "graph is NULL");
  B200_NOT_WHILE_RECORDING("replaying a graph");
  State& s = state();
  RecordedGraph* r = (RecordedGraph*)(uintptr_t)graph;
  advance_epoch_kernel<<<1, 1, 0, s.stream>>>(s.replay_epoch);
  B200_LAUNCH_CHECK();
  B200_CUDA(cudaGraphLaunch(r->exec, s.stream));
  s.launches += r->kernels;
  return B200_OK;
}

B200_API int b200_graph_kernel_count(uint64_t graph, uint64_t* kernels) {
  B200_REQUIRE(graph != 0 && kernels != nullptr, "NULL argument");
  *kernels = ((RecordedGraph*)(uintptr_t)graph)->kernels;
  return B200_OK;
}

B200_API int b200_graph_destroy(uint64_t graph) {
  if (graph == 0) return B200_OK;
  RecordedGraph* r = (RecordedGraph*)(uintptr_t)graph;
  for (void* p : r->made) {
    auto it = g_made_by.find(p);
    if (it != g_made_by.end() && it->second == r) g_made_by.erase(it);
  }
  if (state().ready) {
    // replays still queued use the memory: the frees are ordered after them
    cudaGraphExecDestroy(r->exec);
    release_all(r->owned);
    if (--state().live_graphs <= 0) {
      state().live_graphs = 0;
      release_all(g_retired);
    }
  }
  delete r;
  return B200_OK;
}

B200_API int b200_host_alloc(void** ptr, uint64_t bytes) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(ptr != nullptr, "ptr is NULL");
  B200_CUDA(cudaHostAlloc(ptr, bytes ? (size_t)bytes : 16, cudaHostAllocDefault));
  return B200_OK;
}

B200_API int b200_host_free(void* ptr) {
  if (ptr) B200_CUDA(cudaFreeHost(ptr));
  return B200_OK;
}

// Host -> device.  The copy is ordered on the library stream; with pageable
// source memory the runtime stages it before returning, with pinned memory the
// caller must keep the source untouched until b200_sync().
B200_API int b200_memcpy_h2d(uint64_t dst, const void* src, uint64_t bytes) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("a host-to-device copy");
  if (bytes == 0) return B200_OK;
  B200_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, src, (size_t)bytes, cudaMemcpyHostToDevice,
                            state().stream));
  return B200_OK;
}

// Device -> host; returns after the data has arrived (synchronises the stream).
B200_API int b200_memcpy_d2h(void* dst, uint64_t src, uint64_t bytes) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("a device-to-host copy");
  if (bytes) {
    B200_CUDA(cudaMemcpyAsync(dst, (const void*)(uintptr_t)src, (size_t)bytes,
                              cudaMemcpyDeviceToHost, state().stream));
  }
  B200_CUDA(cudaStreamSynchronize(state().stream));
  return gemm_tc_check_flag();
}

// Device -> page-locked host memory without waiting: the copy is queued on the library
// stream behind the kernels that produce the data; the host reads `dst` after an event
// recorded behind the copy has been reached (b200_event_record + b200_event_wait).
B200_API int b200_memcpy_d2h_async(void* dst, uint64_t src, uint64_t bytes) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("a device-to-host copy");
  if (bytes)
    B200_CUDA(cudaMemcpyAsync(dst, (const void*)(uintptr_t)src, (size_t)bytes, cudaMemcpyDeviceToHost, state().stream));
  return B200_OK;
}

// Row-pitched transfers for strided views: `rows` rows of `row_bytes` bytes.
B200_API int b200_memcpy2d_h2d(uint64_t dst, uint64_t dst_pitch, const void* src,
                               uint64_t src_pitch, uint64_t row_bytes, uint64_t rows) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("a host-to-device copy");
  if (rows == 0 || row_bytes == 0) return B200_OK;
  B200_CUDA(cudaMemcpy2DAsync((void*)(uintptr_t)dst, dst_pitch, src, src_pitch, row_bytes, rows,
                              cudaMemcpyHostToDevice, state().stream));
  return B200_OK;
}

B200_API int b200_memcpy2d_d2h(void* dst, uint64_t dst_pitch, uint64_t src, uint64_t src_pitch,
                               uint64_t row_bytes, uint64_t rows) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("a device-to-host copy");
  if (rows && row_bytes) {
    B200_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, (const void*)(uintptr_t)src, src_pitch, row_bytes,
                                rows, cudaMemcpyDeviceToHost, state().stream));
  }
  B200_CUDA(cudaStreamSynchronize(state().stream));
  return gemm_tc_check_flag();
}

// ---- uploads that overlap with compute ---------------------------------------------
// A second stream carries host->device copies so that the next batch can be uploaded
// while kernels of the current one run.  b200_upload_async orders the copy after
// `after_event` (an event of b200_event_record, 0 for none: the caller names the last
// kernels that read the destination); b200_upload_join makes everything queued on the
// compute stream afterwards wait for the uploads issued so far.
static cudaStream_t g_copy_stream = nullptr;
static cudaEvent_t g_copy_done = nullptr;

B200_API int b200_upload_async(uint64_t dst, const void* src, uint64_t bytes, uint64_t after_event) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("an upload");
  if (!g_copy_stream) {
    B200_CUDA(cudaStreamCreateWithFlags(&g_copy_stream, cudaStreamNonBlocking));
    B200_CUDA(cudaEventCreateWithFlags(&g_copy_done, cudaEventDisableTiming));
  }
  if (after_event) B200_CUDA(cudaStreamWaitEvent(g_copy_stream, (cudaEvent_t)(uintptr_t)after_event, 0));
  if (bytes)
    B200_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, src, (size_t)bytes, cudaMemcpyHostToDevice, g_copy_stream));
  return B200_OK;
}

// The same for a row-pitched destination (a strided view): `rows` rows of `row_bytes` bytes.
B200_API int b200_upload2d_async(uint64_t dst, uint64_t dst_pitch, const void* src, uint64_t src_pitch,
                                 uint64_t row_bytes, uint64_t rows, uint64_t after_event) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("an upload");
  if (int rc = b200_upload_async(0, nullptr, 0, after_event)) return rc;   // stream set-up and ordering
  if (rows && row_bytes)
    B200_CUDA(cudaMemcpy2DAsync((void*)(uintptr_t)dst, dst_pitch, src, src_pitch, row_bytes, rows,
                                cudaMemcpyHostToDevice, g_copy_stream));
  return B200_OK;
}

B200_API int b200_upload_join(void) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("joining the upload stream");
  if (!g_copy_stream) return B200_OK;
  B200_CUDA(cudaEventRecord(g_copy_done, g_copy_stream));
  B200_CUDA(cudaStreamWaitEvent(state().stream, g_copy_done, 0));
  return B200_OK;
}

B200_API int b200_sync(void) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("waiting for the device");
  B200_CUDA(cudaStreamSynchronize(state().stream));
  return gemm_tc_check_flag();
}

// ---- timing helpers for the benchmark (events on the library stream) --------
B200_API int b200_event_create(uint64_t* ev) {
  B200_REQUIRE(ev != nullptr, "ev is NULL");
  cudaEvent_t e;
  B200_CUDA(cudaEventCreate(&e));
  *ev = (uint64_t)(uintptr_t)e;
  return B200_OK;
}
B200_API int b200_event_record(uint64_t ev) {
  if (int rc = require_ready()) return rc;
  B200_NOT_WHILE_RECORDING("recording an event");
  B200_CUDA(cudaEventRecord((cudaEvent_t)(uintptr_t)ev, state().stream));
  return B200_OK;
}
// Blocks the host until the event has been reached (nothing else is waited for).
B200_API int b200_event_wait(uint64_t ev) {
  B200_REQUIRE(ev != 0, "ev is NULL");
  B200_CUDA(cudaEventSynchronize((cudaEvent_t)(uintptr_t)ev));
  return gemm_tc_check_flag();
}
B200_API int b200_event_elapsed_ms(uint64_t start, uint64_t stop, float* ms) {
  B200_REQUIRE(ms != nullptr, "ms is NULL");
  B200_CUDA(cudaEventSynchronize((cudaEvent_t)(uintptr_t)stop));
  B200_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)(uintptr_t)start, (cudaEvent_t)(uintptr_t)stop));
  return B200_OK;
}
B200_API int b200_event_destroy(uint64_t ev) {
  if (ev) B200_CUDA(cudaEventDestroy((cudaEvent_t)(uintptr_t)ev));
  return B200_OK;
}
