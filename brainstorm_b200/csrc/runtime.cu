// Lifecycle, memory and transfer entry points of the B200 handler library.
// Device memory comes from the CUDA stream-ordered pool (cudaMallocAsync) with an
// unlimited release threshold, so the short-lived temporaries that layers
// allocate on every pass are recycled without touching the driver.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace b200 {

int gemm_tc_check_flag();  // gemm_tc.cu: reports a barrier timeout of a tensor-core kernel

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
  cudaMemPool_t pool;
  B200_CUDA(cudaDeviceGetDefaultMemPool(&pool, device));
  uint64_t keep = UINT64_MAX;
  B200_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
  s.device = device;
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
    default: return set_error(B200_ERR_ARG, "unknown tuning key %d", key);
  }
  return B200_OK;
}

B200_API uint64_t b200_launch_count(void) { return state().launches; }

B200_API uint64_t b200_stream(void) { return (uint64_t)(uintptr_t)state().stream; }

B200_API int b200_malloc(uint64_t* ptr, uint64_t bytes, int zero) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(ptr != nullptr, "ptr is NULL");
  void* p = nullptr;
  // Zero-byte arrays are routine (buffers are first created for a 0x0 batch);
  // give them a real, distinct address.
  size_t n = bytes ? (size_t)bytes : 16;
  B200_CUDA(cudaMallocAsync(&p, n, state().stream));
  if (zero) B200_CUDA(cudaMemsetAsync(p, 0, n, state().stream));
  *ptr = (uint64_t)(uintptr_t)p;
  return B200_OK;
}

B200_API int b200_free(uint64_t ptr) {
  if (!state().ready || ptr == 0) return B200_OK;
  B200_CUDA(cudaFreeAsync((void*)(uintptr_t)ptr, state().stream));
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
  if (bytes == 0) return B200_OK;
  B200_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, src, (size_t)bytes, cudaMemcpyHostToDevice,
                            state().stream));
  return B200_OK;
}

// Device -> host; returns after the data has arrived (synchronises the stream).
B200_API int b200_memcpy_d2h(void* dst, uint64_t src, uint64_t bytes) {
  if (int rc = require_ready()) return rc;
  if (bytes) {
    B200_CUDA(cudaMemcpyAsync(dst, (const void*)(uintptr_t)src, (size_t)bytes,
                              cudaMemcpyDeviceToHost, state().stream));
  }
  B200_CUDA(cudaStreamSynchronize(state().stream));
  return gemm_tc_check_flag();
}

// Row-pitched transfers for strided views: `rows` rows of `row_bytes` bytes.
B200_API int b200_memcpy2d_h2d(uint64_t dst, uint64_t dst_pitch, const void* src,
                               uint64_t src_pitch, uint64_t row_bytes, uint64_t rows) {
  if (int rc = require_ready()) return rc;
  if (rows == 0 || row_bytes == 0) return B200_OK;
  B200_CUDA(cudaMemcpy2DAsync((void*)(uintptr_t)dst, dst_pitch, src, src_pitch, row_bytes, rows,
                              cudaMemcpyHostToDevice, state().stream));
  return B200_OK;
}

B200_API int b200_memcpy2d_d2h(void* dst, uint64_t dst_pitch, uint64_t src, uint64_t src_pitch,
                               uint64_t row_bytes, uint64_t rows) {
  if (int rc = require_ready()) return rc;
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
  if (!g_copy_stream) {
    B200_CUDA(cudaStreamCreateWithFlags(&g_copy_stream, cudaStreamNonBlocking));
    B200_CUDA(cudaEventCreateWithFlags(&g_copy_done, cudaEventDisableTiming));
  }
  if (after_event) B200_CUDA(cudaStreamWaitEvent(g_copy_stream, (cudaEvent_t)(uintptr_t)after_event, 0));
  if (bytes)
    B200_CUDA(cudaMemcpyAsync((void*)(uintptr_t)dst, src, (size_t)bytes, cudaMemcpyHostToDevice, g_copy_stream));
  return B200_OK;
}

B200_API int b200_upload_join(void) {
  if (int rc = require_ready()) return rc;
  if (!g_copy_stream) return B200_OK;
  B200_CUDA(cudaEventRecord(g_copy_done, g_copy_stream));
  B200_CUDA(cudaStreamWaitEvent(state().stream, g_copy_done, 0));
  return B200_OK;
}

B200_API int b200_sync(void) {
  if (int rc = require_ready()) return rc;
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
  B200_CUDA(cudaEventRecord((cudaEvent_t)(uintptr_t)ev, state().stream));
  return B200_OK;
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
