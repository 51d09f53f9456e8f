/* C-ABI of libb200handler.so: the B200 (sm_100a) backend of the brainstorm
 * Handler API.
 *
 * The reference has no FFI on this path: its backends are Python classes that
 * implement `Handler` (brainstorm/handlers/base_handler.py:13).  Each entry point
 * below is what a binding of one Handler method binds; the comment names the
 * abstract method it serves (base_handler.py:LINE) and the CPU implementation it
 * must agree with (numpy_handler.py:LINE).
 *
 * Conventions
 *  - Every function returns 0 on success, non-zero otherwise; b200_last_error()
 *    then describes the failure.  Nothing traps on the device.
 *  - One process drives one GPU, from one host thread at a time: the library keeps
 *    per-process state (current stream, recording state, work buffers) without locks,
 *    like the reference's handlers (one handler object per network).
 *  - Pointers are device addresses of fp32 data unless stated otherwise.  Work is
 *    queued on the library's stream in program order; only the functions marked
 *    "synchronises" wait for it.
 *  - Elementwise operands are row-pitched 2-D views: `rows` rows of `cols`
 *    contiguous elements, row r of operand x starting at x + r*ldx.  A contiguous
 *    array of n elements is passed as rows=1, cols=n.  An output may be the same
 *    array as an input (in-place forms).  Zero-size extents are valid no-ops.
 */
#ifndef B200_HANDLER_H
#define B200_HANDLER_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- lifecycle / errors ------------------------------------------------- */
const char* b200_last_error(void);
int b200_device_count(int* count);
/* Binds the process to one GPU (one process per GPU), creates the stream and
 * configures the stream-ordered memory pool.  Fails on anything but sm_100. */
int b200_init(int device);
int b200_device_info(int* device, int* sm_count, uint64_t* free_bytes, uint64_t* total_bytes);
/* key 0: elementwise blocks per SM; 1: elementwise threads per block;
 * 2: GEMM path (0 auto, 1 CUDA cores, 2 tensor cores only); 3: forced GEMM tile width;
 * 5: programmatic dependent launch inside the LSTM time loops (default 1);
 * 6: split-K plans for 1/value of the SMs (default 1; 2 while two streams share the GPU);
 * 7: 256-wide GEMM tiles on pairs of SMs (tcgen05 cta_group::2; default 0: measured slower
 *    than the single-SM tiles so far);
 * 8: the bounded wait of the peer all-reduce gives up after 2^value polls (0 = the default,
 *    2^22 polls, about 20 seconds);
 * 9: k-blocks of 32 that the tensor-core GEMM accumulates in tensor memory between two
 *    drains into fp32 registers (1, 2, 4 or 8; 0 = the default, 2): shorter chunks lose
 *    less to the tensor core's truncating accumulation and cost a little throughput;
 * 10: pass-1 blocks per SM of the two-pass sums (default 8; changes what
 *    b200_sum_t_scratch_floats returns);
 * 11: column sums (axis 0) run their second pass inside the first kernel: the block that
 *    finishes a column group last adds the group's partial sums, in the same fixed order
 *    (default 1; 0 = a second launch; same bits either way);
 * 12: b200_sum_t_axis0_allreduce runs its exchange inside the column-sum kernel, group by
 *    group (1), or as the all-reduce kernel behind it (0, the default: measured faster);
 *    same bits either way. */
int b200_set_tuning(int key, int value);
uint64_t b200_stream(void);                            /* the main stream (a cudaStream_t) */
/* A second compute stream, for work that may run beside the main stream's (a stack of
 * LSTM layers: the reference walks layer by layer, brainstorm/structure/network.py:429-430,
 * but layer l+1 at time t needs layer l only up to time t).  b200_use_stream(1) makes
 * every following call queue on the side stream, b200_use_stream(0) returns to the
 * main stream.  Ordering between the streams is explicit: b200_mark records a marker
 * on the current stream, b200_wait_mark makes the current stream wait for one.  Memory
 * that the side stream touches before it has waited for the main stream must have been
 * allocated while the side stream was current (allocations are stream-ordered).  The
 * reference has no counterpart. */
int b200_use_stream(int index);
int b200_mark_create(uint64_t* mark);
int b200_mark(uint64_t mark);
int b200_wait_mark(uint64_t mark);
int b200_mark_destroy(uint64_t mark);
/* Number of kernels this library has launched in this process so far. */
uint64_t b200_launch_count(void);
int b200_sync(void);                                   /* synchronises */

/* ---- memory: Handler.allocate/zeros/ones (base_handler.py:80,102,91;
 *      numpy_handler.py:36-43: allocate is zero-filled) --------------------- */
int b200_malloc(uint64_t* ptr, uint64_t bytes, int zero);
int b200_free(uint64_t ptr);
int b200_host_alloc(void** ptr, uint64_t bytes);       /* pinned staging memory */
int b200_host_free(void* ptr);

/* ---- transfers: set_from_numpy / create_from_numpy (base_handler.py:197,145;
 *      numpy_handler.py:64,54) and get_numpy_copy (base_handler.py:186;
 *      numpy_handler.py:60) ------------------------------------------------- */
int b200_memcpy_h2d(uint64_t dst, const void* src, uint64_t bytes);
int b200_memcpy_d2h(void* dst, uint64_t src, uint64_t bytes);             /* synchronises */
/* The same without waiting, into page-locked memory: for the per-update read of the loss
 * (Network.get_loss_values, brainstorm/structure/network.py:466), which a caller may take
 * one step late; read dst after an event recorded behind the copy (b200_event_wait). */
int b200_memcpy_d2h_async(void* dst, uint64_t src, uint64_t bytes);
int b200_memcpy2d_h2d(uint64_t dst, uint64_t dst_pitch, const void* src, uint64_t src_pitch,
                      uint64_t row_bytes, uint64_t rows);
int b200_memcpy2d_d2h(void* dst, uint64_t dst_pitch, uint64_t src, uint64_t src_pitch,
                      uint64_t row_bytes, uint64_t rows);                 /* synchronises */

/* Uploads on a second stream, so that the next batch's host->device copy overlaps the
 * current batch's kernels (the input side of Network.provide_external_data,
 * brainstorm/structure/network.py:399-403).  The copy starts after `after_event` (an
 * event recorded with b200_event_record; 0 = at once); b200_upload_join makes work
 * queued on the compute stream afterwards wait for all uploads issued so far.  The
 * host source must be page-locked and stay untouched until then. */
int b200_upload_async(uint64_t dst, const void* src, uint64_t bytes, uint64_t after_event);
int b200_upload2d_async(uint64_t dst, uint64_t dst_pitch, const void* src, uint64_t src_pitch,
                        uint64_t row_bytes, uint64_t rows, uint64_t after_event);   /* row-pitched destination */
int b200_upload_join(void);

/* ---- recorded steps: one replay call instead of one launch per kernel -------
 * The caller side of the path, a training step (TrainingStepper.run,
 * brainstorm/training/steppers.py:61-70,103-121), is a fixed sequence of handler
 * calls on fixed buffers.  Between b200_graph_begin and b200_graph_end every kernel,
 * fill and device-to-device copy of this library is recorded into a CUDA graph
 * instead of executed; b200_graph_launch replays the whole sequence.  Addresses and
 * scalar arguments are frozen in the recording; random masks are not: every replay
 * draws from a new Philox stream.  While recording, calls that wait for the device
 * or cross PCIe (transfers, uploads, b200_sync, events) fail with an error and
 * record nothing; arrays allocated are real allocations; arrays released while
 * recording, and arrays that were allocated while recording and are released later,
 * stay allocated until b200_graph_destroy (replays keep using their addresses), and so
 * do the library's own work buffers.  b200_graph_end(NULL) discards the recording.
 * The reference has no counterpart (its GPU backend launches kernel by kernel). */
int b200_graph_begin(void);                                               /* synchronises */
int b200_graph_end(uint64_t* graph);
int b200_graph_launch(uint64_t graph);
int b200_graph_kernel_count(uint64_t graph, uint64_t* kernels);
int b200_graph_destroy(uint64_t graph);

/* ---- all-reduce of small arrays over NVLink peer memory ---------------------
 * For the exchanges that sit next to a reduction on this path: the sums over the batch
 * axis that sum_t(axis=0) completes across batch shards (BatchNorm statistics,
 * brainstorm/layers/batch_normalization_layer.py:63,117; a few thousand floats).  Every
 * rank (one process per GPU of one node) allocates a window, exports its handle, opens
 * the other ranks' handles (exchanged by the host) and registers all of them; one
 * single-CTA kernel per call then publishes the values, waits (bounded, about 20 seconds;
 * b200_set_tuning key 8) for all ranks and adds the ranks' values in rank order, so every
 * rank gets the same bits.  Plain peer loads and stores.  Up to 16 ranks, up to
 * b200_peer_max_floats() floats per call; every rank makes the same calls in the same
 * order.  A wait that runs out leaves dst untouched and raises the device error flag: the
 * next synchronising call fails, and b200_peer_enabled() is 0 until the windows are
 * registered again (the ranks' call counters no longer agree).  b200_peer_setup clears this
 * rank's arrival counters: put a host barrier over all ranks between it and the first
 * b200_peer_allreduce.  b200_peer_window_release gives back a window that never reached
 * b200_peer_setup (own != 0: allocated here; 0: opened from a handle).
 * b200_peer_wait_stats reports the calls made since b200_peer_setup and the nanoseconds
 * they spent between publishing their values and seeing every other rank's (how late
 * the slowest rank was, plus one trip over NVLink); it synchronises.  The reference has
 * no counterpart (it has no multi-GPU code). */
uint64_t b200_peer_window_bytes(void);
int b200_peer_max_floats(void);
int b200_peer_window_alloc(uint64_t* ptr, void* handle /* 64 bytes */);
int b200_peer_window_open(const void* handle /* 64 bytes */, uint64_t* ptr);
int b200_peer_window_release(uint64_t ptr, int own);
int b200_peer_setup(int rank, int world, const uint64_t* windows);
int b200_peer_enabled(void);
int b200_peer_allreduce(const float* src, float* dst, int n, int average);
int b200_peer_wait_stats(uint64_t* calls, uint64_t* waited_ns);
/* b200_sum_t(axis 0) and b200_peer_allreduce of its result in one call.  By default the
 * all-reduce kernel is queued behind the column-sum kernel.  With b200_set_tuning(12, 1)
 * it is ONE kernel: the block of the column-sum kernel that finishes a group of 128
 * columns sends that group through the exchange at once, while other groups are still
 * being summed (same slots, bounded wait and error reporting as b200_peer_allreduce;
 * after a wait that ran out, out holds the local sums); on two B200s that form measured
 * 200 us against 191 us for the two kernels on a (65536, 4096) array.  out[c] = sum (average != 0: mean) over the ranks of the local column
 * sums, the same bits on every rank and the same bits as the two calls.  cols <=
 * b200_peer_max_floats(); scratch as for b200_sum_t(axis 0); every rank makes the call.
 * Serves sum_t(axis=0) of batch-sharded data (BatchNorm statistics,
 * batch_normalization_layer.py:63,83,121,133). */
int b200_sum_t_axis0_allreduce(const float* a, int64_t rows, int64_t cols, int64_t ld, float* out, float* scratch, int64_t scratch_floats, int average);
int b200_peer_teardown(void);

/* ---- all-reduce of device arrays over NCCL -----------------------------------
 * The one exchange a batch-sharded run of the handler path needs: the flat gradient
 * vector after Network.backward_pass, before the stepper reads it
 * (brainstorm/training/steppers.py:61-69), and the sums over the batch axis that
 * BatchNorm takes (brainstorm/layers/batch_normalization_layer.py:63-86,117-151).  One
 * process per GPU.  Rank 0 asks for an id, the host hands its 128 bytes to every rank,
 * every rank calls b200_comm_init (collective).  b200_comm_allreduce queues an in-place
 * sum (average != 0: mean) on the library's current stream; b200_comm_allreduce_async
 * queues it on a communication stream behind the work queued so far, so that kernels
 * queued afterwards run beside it, until b200_comm_join.  All three can be recorded into
 * a graph.  NCCL is looked up at run time (the copy already in the process, else
 * libnccl.so.2, else the file named by B200_NCCL_LIB); without it b200_comm_init fails
 * and the rest of the library is unaffected.  The reference has no counterpart (it has
 * no multi-GPU code). */
int b200_comm_unique_id(void* id /* 128 bytes */);
int b200_comm_init(int rank, int world, const void* id /* 128 bytes */);
int b200_comm_world(void);
int b200_comm_allreduce(float* data, int64_t count, int average);
int b200_comm_allreduce_async(float* data, int64_t count, int average);
int b200_comm_join(void);
int b200_comm_destroy(void);

/* ---- CUDA-event timing on the library stream (benchmark support) --------- */
int b200_event_create(uint64_t* ev);
int b200_event_record(uint64_t ev);
int b200_event_wait(uint64_t ev);                                         /* waits for this event only */
int b200_event_elapsed_ms(uint64_t start, uint64_t stop, float* ms);      /* synchronises */
int b200_event_destroy(uint64_t ev);

/* ---- copy / fill: base_handler.py:115 (copy_to(src, dest)), :157 (fill);
 *      numpy_handler.py:47,57 ----------------------------------------------- */
int b200_copy_to(const float* src, float* dest, int64_t rows, int64_t cols, int64_t lds, int64_t ldd);
int b200_fill(float* mem, float val, int64_t rows, int64_t cols, int64_t ld);

/* ---- tensor (.) tensor: add_tt :284, subtract_tt :752, mult_tt :683,
 *      divide_tt :480, modulo_tt :606, mult_add_tt :635 (out += a*b, product and
 *      sum rounded separately); numpy_handler.py:86,264,245,190,227,233 ------- */
int b200_add_tt(const float* a, const float* b, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldb, int64_t ldo);
int b200_subtract_tt(const float* a, const float* b, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldb, int64_t ldo);
int b200_mult_tt(const float* a, const float* b, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldb, int64_t ldo);
int b200_divide_tt(const float* a, const float* b, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldb, int64_t ldo);
int b200_modulo_tt(const float* a, const float* b, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldb, int64_t ldo);
int b200_mult_add_tt(const float* a, const float* b, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldb, int64_t ldo);

/* ---- scalar (.) tensor: add_st :271, mult_st :670, mult_add_st :622
 *      (out += s*t); numpy_handler.py:83,242,230 ---------------------------- */
int b200_add_st(float s, const float* t, float* out, int64_t rows, int64_t cols, int64_t ldt, int64_t ldo);
int b200_mult_st(float s, const float* t, float* out, int64_t rows, int64_t cols, int64_t ldt, int64_t ldo);
int b200_mult_add_st(float s, const float* t, float* out, int64_t rows, int64_t cols, int64_t ldt, int64_t ldo);

/* ---- matrix (.) broadcast vector: add_mv :252, subtract_mv :736, mult_mv :649,
 *      divide_mv :461; mult_add_mv is defined by the backends only
 *      (numpy_handler.py:239, out += m*v); numpy_handler.py:80,261,236,187.
 *      v_is_col == 0: v holds `cols` values (a (1, cols) row vector);
 *      v_is_col == 1: v holds `rows` values (a (rows, 1) column vector).
 *      broadcast_t :351 / numpy_handler.py:103 copies v along the other axis. */
int b200_add_mv(const float* m, const float* v, float* out, int64_t rows, int64_t cols, int64_t ldm, int64_t ldo, int v_is_col);
int b200_subtract_mv(const float* m, const float* v, float* out, int64_t rows, int64_t cols, int64_t ldm, int64_t ldo, int v_is_col);
int b200_mult_mv(const float* m, const float* v, float* out, int64_t rows, int64_t cols, int64_t ldm, int64_t ldo, int v_is_col);
int b200_divide_mv(const float* m, const float* v, float* out, int64_t rows, int64_t cols, int64_t ldm, int64_t ldo, int v_is_col);
int b200_mult_add_mv(const float* m, const float* v, float* out, int64_t rows, int64_t cols, int64_t ldm, int64_t ldo, int v_is_col);
int b200_broadcast_t(const float* v, float* out, int64_t rows, int64_t cols, int64_t ldo, int v_is_col);

/* ---- unary: abs_t :222, sign_t :697, sqrt_t :724, log_t :545, clip_t :374;
 *      numpy_handler.py:74,248,258,207,107 ---------------------------------- */
int b200_abs_t(const float* a, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldo);
int b200_sign_t(const float* a, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldo);
int b200_sqrt_t(const float* a, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldo);
int b200_log_t(const float* a, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldo);
int b200_clip_t(const float* a, float a_min, float a_max, float* out, int64_t rows, int64_t cols, int64_t lda, int64_t ldo);

/* ---- activations: sigmoid :815, tanh :854, rel :786, el :882 and their
 *      derivatives :827,:867,:799,:903 (dx = dy * f'(y); the x argument of the
 *      Handler methods is unused by every backend and is not passed);
 *      numpy_handler.py:277-309 --------------------------------------------- */
int b200_sigmoid(const float* x, float* y, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy);
int b200_tanh(const float* x, float* y, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy);
int b200_rel(const float* x, float* y, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy);
int b200_el(const float* x, float* y, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy);
int b200_sigmoid_deriv(const float* y, const float* dy, float* dx, int64_t rows, int64_t cols, int64_t ldy, int64_t lddy, int64_t lddx);
int b200_tanh_deriv(const float* y, const float* dy, float* dx, int64_t rows, int64_t cols, int64_t ldy, int64_t lddy, int64_t lddx);
int b200_rel_deriv(const float* y, const float* dy, float* dx, int64_t rows, int64_t cols, int64_t ldy, int64_t lddy, int64_t lddx);
int b200_el_deriv(const float* y, const float* dy, float* dx, int64_t rows, int64_t cols, int64_t ldy, int64_t lddy, int64_t lddx);

/* ---- predicated: copy_to_if :129, fill_if :168, add_into_if :234;
 *      numpy_handler.py:173,196,77 (cond != 0 selects) ---------------------- */
int b200_copy_to_if(const float* src, float* dest, const float* cond, int64_t rows, int64_t cols, int64_t lds, int64_t ldd, int64_t ldc);
int b200_fill_if(float* mem, float val, const float* cond, int64_t rows, int64_t cols, int64_t ldm, int64_t ldc);
int b200_add_into_if(const float* a, float* out, const float* cond, int64_t rows, int64_t cols, int64_t lda, int64_t ldo, int64_t ldc);

/* ---- last-axis concat / split-accumulate: merge_tt :560, split_add_tt :712;
 *      numpy_handler.py:221,251 (contiguous operands) ------------------------ */
int b200_merge_tt(const float* a, const float* b, float* out, int64_t rows, int64_t na, int64_t nb);
int b200_split_add_tt(const float* x, float* out_a, float* out_b, int64_t rows, int64_t na, int64_t nb);

/* ---- labels (bit-exact): binarize_v :330, index_m_by_v :522;
 *      numpy_handler.py:99,202.  Labels are fp32 values holding integers and are
 *      truncated like astype(int32).  v has one label per row at v + r*ldv.
 *      index_m_by_v skips rows whose label is outside [0, cols) and sets
 *      *bad_label_flag (device int, may be NULL) instead of reading out of
 *      bounds. -------------------------------------------------------------- */
int b200_binarize_v(const float* v, int64_t ldv, float* out, int64_t rows, int64_t cols, int64_t ldo);
int b200_index_m_by_v(const float* m, int64_t ldm, const float* v, int64_t ldv, float* out, int64_t ldo, int64_t rows, int64_t cols, int* bad_label_flag);

/* ---- reductions: sum_t :767 / numpy_handler.py:268; softmax_m :843 /
 *      numpy_handler.py:292; is_fully_finite :210 / numpy_handler.py:69.
 *      axis 0: out[c] = sum_r a[r,c]; axis 1: out[r] = sum_c a[r,c]; axis -1:
 *      out[0] = sum of everything.  Sums are deterministic two-pass trees; the
 *      caller provides the scratch for the partials (size from
 *      b200_sum_t_scratch_floats, which depends on the extents and on the number of
 *      SMs of the GPU the process was bound to, never on the pointers). ------- */
int64_t b200_sum_t_scratch_floats(int64_t rows, int64_t cols, int64_t ld, int axis);
int b200_sum_t(const float* a, int64_t rows, int64_t cols, int64_t ld, int axis, float* out, float* scratch, int64_t scratch_floats);
/* No counterpart in the reference.  sum_t for hosts that may not allocate device
 * memory while running (their own pool already owns the GPU, or they must never
 * enter the CUDA allocator): the partial sums go to a 1 MiB array built into the
 * library instead of caller scratch; the call allocates nothing.  Same result as
 * b200_sum_t.  Extents that need more than b200_sum_t_static_max_scratch_floats()
 * are rejected.  b200_init resolves the array's device address, once per device.
 * Calls share the array; calls that overlap on the GPU race. */
int64_t b200_sum_t_static_max_scratch_floats(void);
int b200_sum_t_static(const float* a, int64_t rows, int64_t cols, int64_t ld, int axis, float* out);
int b200_softmax_m(const float* m, float* out, int64_t rows, int64_t cols, int64_t ldm, int64_t ldo);
/* ORs 1 into *flag (device int, zeroed by the caller) if any element is Inf/NaN. */
int b200_nonfinite_flag(const float* a, int64_t rows, int64_t cols, int64_t ld, int* flag);

/* ---- GEMM: dot_mm :444, dot_add_mm :427; numpy_handler.py:181,176.
 *      out (M x N, row pitch ldo) = or += op(a) . op(b), op(a) is M x K and
 *      op(b) is K x N; with transa the array a is K x M (pitch lda), with transb
 *      the array b is N x K (pitch ldb).  out must not overlap a or b. -------- */
int b200_dot_mm(const float* a, const float* b, float* out, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldo, int transa, int transb);
int b200_dot_add_mm(const float* a, const float* b, float* out, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldo, int transa, int transb);

/* ---- fused LSTM sequence passes: the per-timestep body of
 *      LstmLayerImpl.forward_pass (brainstorm/layers/lstm_layer.py:115-145) and
 *      LstmLayerImpl.backward_pass (:171-205).  Per timestep: one stacked recurrent
 *      GEMM on the tensor cores + one gate kernel; the loop over time runs inside
 *      the library.  Buffers are the layer's own (T+1, B, H) arrays (context slot
 *      at index T); gate order is z, i, f, o as in the parameter vector (:39-55).
 *      act: 0 sigmoid, 1 tanh, 2 rel, 3 el, 4 linear.  xproj (T*B, 4H) holds the
 *      input projections; y_work (T+1, B, H), dg_work (T+1, B, 4H) and r_work
 *      (B, 4H) are 16-byte aligned work arrays of the caller. ------------------ */
int b200_lstm_forward(const float* xproj, const float* r_stack, const float* bias, const float* peep,
                      float* za, float* zb, float* ia, float* ib, float* fa, float* fb, float* oa, float* ob,
                      float* ca, float* cb, float* y, float* y_work, float* r_work, int T, int B, int H, int act);
int b200_lstm_backward(const float* deltas, const float* r_stack, const float* peep,
                       const float* zb, const float* ib, const float* fb, const float* ob, const float* ca, const float* cb,
                       float* dza, float* dzb, float* dia, float* dib, float* dfa, float* dfb, float* doa, float* dob,
                       float* dca, float* dcb, float* dg_work, float* r_work, int T, int B, int H, int act);
/* The same passes over a piece of the sequence: forward timesteps t0 .. t1-1, backward
 * t1-1 down to t0 (pieces in that order).  For callers that run a stack of LSTM layers
 * side by side (see b200_use_stream): layer l+1 can start a piece as soon as layer l
 * has finished it. */
int b200_lstm_forward_steps(const float* xproj, const float* r_stack, const float* bias, const float* peep,
                            float* za, float* zb, float* ia, float* ib, float* fa, float* fb, float* oa, float* ob,
                            float* ca, float* cb, float* y, float* y_work, float* r_work, int T, int B, int H, int act,
                            int t0, int t1);
int b200_lstm_backward_steps(const float* deltas, const float* r_stack, const float* peep,
                             const float* zb, const float* ib, const float* fb, const float* ob, const float* ca, const float* cb,
                             float* dza, float* dzb, float* dia, float* dib, float* dfa, float* dfb, float* doa, float* dob,
                             float* dca, float* dcb, float* dg_work, float* r_work, int T, int B, int H, int act,
                             int t0, int t1);

/* ---- convolution and pooling (NHWC): conv2d_forward_batch :411, conv2d_backward_batch :392,
 *      maxpool2d_* :590/:572, avgpool2d_* :314/:297; numpy_handler.py:149,110,216,210,94,89 with
 *      the loops of brainstorm/handlers/_cpuop.pyx.  Convolution is im2col over all images
 *      + the GEMM above (col is (N*oh*ow, kh*kw*C), channel fastest); col2im ADDS the
 *      columns back into in_deltas.  Pooling mode 0 = max (argmax holds the float index
 *      (y*W + x)*C + c inside the image, -1 for an empty window, as _cpuop.pyx:27 does),
 *      mode 1 = average over the non-padding pixels; the backward forms ADD into
 *      in_deltas.  Gather-form kernels, no atomics. ----------------------------------- */
int b200_im2col(const float* inputs, float* col, int N, int H, int W, int C, int kh, int kw, int pad, int sy, int sx, int oh, int ow);
int b200_col2im_add(const float* col, float* in_deltas, int N, int H, int W, int C, int kh, int kw, int pad, int sy, int sx, int oh, int ow);
int b200_pool2d_forward(int mode, const float* inputs, float* outputs, float* argmax, int N, int H, int W, int C, int kh, int kw, int pad, int sy, int sx, int oh, int ow);
int b200_pool2d_backward(int mode, const float* out_deltas, const float* argmax, float* in_deltas, int N, int H, int W, int C, int kh, int kw, int pad, int sy, int sx, int oh, int ow);

/* ---- fused layer arithmetic.  The reference has no such calls: its layers spell this
 *      arithmetic as chains of Handler calls (brainstorm/layers/highway_layer.py:39-71,
 *      batch_normalization_layer.py:54-152, fully_connected_layer.py:51-62), one trip
 *      through memory per call.  Each entry below does the work of the cited chain in one
 *      pass, rounding every product, sum and quotient separately in the chain's order, so
 *      the results are the bits the chain gives on this library.  Contiguous operands,
 *      16-byte aligned, element counts and column counts multiples of 4 (anything else
 *      is rejected; the host side then runs the reference's chain).
 *      highway_forward: y = T*(H - x) + x.  highway_backward: dx += (1 - T)*dy,
 *      dH += T*dy, dT += (H - x)*dy.
 *      bn_mean: mu_b = s*sum, running = decay*running + one_minus_decay*mu_b (:63-73).
 *      bn_center_sqsum: centered = x + mu (row vector), sq_sum = column sums of
 *      centered^2 (:76-86).  bn_sigma: sigma_b = sqrt(inv_m*sq_sum + eps) and the same
 *      running update (:87-96).  bn_normalize: x_hat = centered / sigma, out =
 *      x_hat*gamma + beta (:100-104).  bn_backward_sums: sums[0:cols] = column sums of
 *      dout*x_hat, sums[cols:2 cols] = column sums of dout (:121-133).
 *      bn_backward_vectors: dgamma += sums[0:cols], dbeta += sums[cols:], vec = [inv_m *
 *      sums[0:cols], inv_m*sums[cols:], gamma / sigma_b] (3 cols floats, :123-146).
 *      bn_backward_deltas: in_deltas += ((dout - x_hat*vec0) - vec1)*vec2 (:126-151).
 *      The column sums use the partial-sum layout of b200_sum_t(axis 0) on a contiguous
 *      array; scratch of b200_bn_scratch_floats(rows, cols) floats from the caller.
 *      bias_act: out = f(out + bias) in place, row pitch ld; act 0 sigmoid, 1 tanh,
 *      2 rel, 3 el, 4 linear (fully_connected_layer.py:61-62). --------------------- */
int b200_highway_forward(const float* x, const float* H, const float* T, float* y, int64_t n);
int b200_highway_backward(const float* x, const float* H, const float* T, const float* dy, float* dx, float* dH, float* dT, int64_t n);
int64_t b200_bn_scratch_floats(int64_t rows, int64_t cols);
int b200_bn_mean(const float* sum, float s, float decay, float one_minus_decay, float* mu_b, float* running, int64_t cols);
int b200_bn_center_sqsum(const float* x, const float* mu, float* centered, float* sq_sum, int64_t rows, int64_t cols, float* scratch, int64_t scratch_floats);
int b200_bn_sigma(const float* sq_sum, float inv_m, float eps, float decay, float one_minus_decay, float* sigma_b, float* running, int64_t cols);
int b200_bn_normalize(const float* centered, const float* sigma, const float* gamma, const float* beta, float* x_hat, float* out, int64_t rows, int64_t cols);
int b200_bn_backward_sums(const float* dout, const float* x_hat, float* sums, int64_t rows, int64_t cols, float* scratch, int64_t scratch_floats);
int b200_bn_backward_vectors(const float* sums, float inv_m, const float* gamma, const float* sigma_b, float* dgamma, float* dbeta, float* vec, int64_t cols);
int b200_bn_backward_deltas(const float* dout, const float* x_hat, const float* vec, float* in_deltas, int64_t rows, int64_t cols);
int b200_bias_act(float* out, const float* bias, int64_t rows, int64_t cols, int64_t ld, int act);

/* ---- random: generate_probability_mask :507, fill_gaussian :494;
 *      numpy_handler.py:199,193.  Device-side Philox4x32-10 streams addressed by
 *      (seed, offset); the host-RNG parity mode of the Python handler does not
 *      use these. ----------------------------------------------------------- */
int b200_generate_probability_mask(float* mask, int64_t n, float probability, uint64_t seed, uint64_t offset);
int b200_fill_gaussian(float mean, float std, float* out, int64_t n, uint64_t seed, uint64_t offset);

#ifdef __cplusplus
}
#endif
#endif /* B200_HANDLER_H */
