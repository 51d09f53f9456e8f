// Reductions of the B200 handler: sum_t over axis 0 / 1 / all, row softmax and the
// finite check.  All HBM-bandwidth bound (every input byte is read once).
//
// Sums are deterministic two-pass trees: pass 1 writes one partial per block (or
// per row-chunk and column) into caller-provided scratch in a fixed order, pass 2
// adds the partials in a fixed order.  No floating-point atomics anywhere, so the
// same input always gives the same bits.
#include "common.cuh"
#include "peer.cuh"

namespace b200 {

constexpr int RED_THREADS = 256;
constexpr int RED_MAX_PARTIALS = 4096;  // upper bound of pass-1 blocks / row chunks

// ---- sum over everything ------------------------------------------------------------
// Block b sums elements [b*chunk, min(n, (b+1)*chunk)); chunk is a multiple of 4.
template <bool VEC>
__global__ void __launch_bounds__(RED_THREADS)
sum_all_pass1(const float* a, int64_t n, int64_t chunk, float* partial) {
  __shared__ float smem[32];
  const int64_t lo = (int64_t)blockIdx.x * chunk;
  int64_t hi = lo + chunk;
  if (hi > n) hi = n;
  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
  if (VEC) {
    const int64_t nv = (hi - lo) >> 2;
    const float4* p = reinterpret_cast<const float4*>(a + lo);
    int64_t i = threadIdx.x;
    for (; i + 3 * RED_THREADS < nv; i += 4 * RED_THREADS) {
      const float4 v0 = __ldcs(p + i), v1 = __ldcs(p + i + RED_THREADS),
                   v2 = __ldcs(p + i + 2 * RED_THREADS), v3 = __ldcs(p + i + 3 * RED_THREADS);
      acc0 += (v0.x + v0.y) + (v0.z + v0.w);
      acc1 += (v1.x + v1.y) + (v1.z + v1.w);
      acc2 += (v2.x + v2.y) + (v2.z + v2.w);
      acc3 += (v3.x + v3.y) + (v3.z + v3.w);
    }
    for (; i < nv; i += RED_THREADS) {
      const float4 v0 = __ldcs(p + i);
      acc0 += (v0.x + v0.y) + (v0.z + v0.w);
    }
    for (int64_t j = lo + (nv << 2) + threadIdx.x; j < hi; j += RED_THREADS) acc1 += a[j];
  } else {
    int64_t i = lo + threadIdx.x;
    for (; i + 3 * RED_THREADS < hi; i += 4 * RED_THREADS) {
      acc0 += a[i];
      acc1 += a[i + RED_THREADS];
      acc2 += a[i + 2 * RED_THREADS];
      acc3 += a[i + 3 * RED_THREADS];
    }
    for (; i < hi; i += RED_THREADS) acc0 += a[i];
  }
  const float s = block_sum((acc0 + acc1) + (acc2 + acc3), smem);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// out[0] = sum of partial[0..count) in a fixed order (one block).
__global__ void __launch_bounds__(RED_THREADS)
sum_all_pass2(const float* partial, int count, float* out) {
  __shared__ float smem[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < count; i += RED_THREADS) acc += partial[i];
  const float s = block_sum(acc, smem);
  if (threadIdx.x == 0) out[0] = s;
}

// ---- sum over axis 0 (column sums) ----------------------------------------------------
// Pass 2 without a second launch.  Every block of a column group (blockIdx.x) takes a ticket
// after its partial sums are visible; the block that draws the last ticket adds the group's
// partials in the fixed order of sum_axis0_pass2 (so the bits do not depend on which block
// that is) and hands the ticket counter back at zero.  The counters belong to the library,
// one set per library stream: calls on one stream are ordered, and the two streams never
// share a set.
constexpr int AXIS0_TICKET_SLOTS = 4096;     // column groups per call that can use the folded form
__device__ unsigned g_axis0_tickets[2][AXIS0_TICKET_SLOTS + 1];   // the last one of a set counts finished column groups

// Called by all 256 threads of a 32 x 8 block after they have stored their partials (or, with a
// single chunk of rows, their sums).  `width` columns from `col0` belong to this block.
// peer_mode 1 / 2: each group's sums are then completed across the ranks (sum / mean) by the
// block that finished the group -- the all-reduce over peer memory of peer.cuh, run inside this
// kernel, group by group, instead of as a launch behind it.
__device__ __forceinline__ void axis0_fold_pass2(unsigned* tickets, const float* partial, const float* partial2, float* out,
                                                 float* out2, int64_t cols, int64_t col0, int width,
                                                 const PeerArgs& peer, int peer_mode, int* error_flag, unsigned spin_limit) {
  __shared__ int is_last;
  const int t = threadIdx.y * 32 + threadIdx.x;
  const int chunks = (int)gridDim.y;
  if (chunks > 1) {
    __threadfence();
    __syncthreads();
    if (t == 0) {
      const unsigned drawn = atomicAdd(&tickets[blockIdx.x], 1u);
      is_last = drawn == gridDim.y - 1;
      if (is_last) tickets[blockIdx.x] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int j = t; j < width * (partial2 ? 2 : 1); j += 256) {
      const float* p = j < width ? partial : partial2;
      float* o = j < width ? out : out2;
      const int64_t c = col0 + (j < width ? j : j - width);
      if (c >= cols) continue;
      float s0 = 0.f, s1 = 0.f;
      int k = 0;
      for (; k + 1 < chunks; k += 2) {
        s0 += __ldcg(p + (int64_t)k * cols + c);
        s1 += __ldcg(p + (int64_t)(k + 1) * cols + c);
      }
      if (k < chunks) s0 += __ldcg(p + (int64_t)k * cols + c);
      o[c] = s0 + s1;
    }
  }
  if (peer_mode == 0) return;
  // This group's sums are final on this rank: complete them across the ranks now, while other
  // groups of the kernel are still being summed.
  __shared__ unsigned long long epoch;
  __threadfence();
  __syncthreads();
  if (t == 0) epoch = peer_next_epoch(peer);
  __syncthreads();
  const int n = (int)(cols - col0 < width ? cols - col0 : width);
  peer_exchange_range<true>(peer, epoch, (int)blockIdx.x, out, out, (int)col0, n, peer_mode == 2, error_flag, spin_limit,
                            gridDim.x);
  // one ticket per finished group; the block that draws the last one closes the call's number
  __threadfence();
  __syncthreads();
  if (t == 0) {
    const unsigned drawn = atomicAdd(&tickets[AXIS0_TICKET_SLOTS], 1u);
    if (drawn == gridDim.x - 1) {
      tickets[AXIS0_TICKET_SLOTS] = 0;
      peer_close_epoch(peer, epoch);
    }
  }
}

// Block = 32 x 8 threads.  VEC: a thread owns 4 adjacent columns (block covers
// 128 columns), else 1 column (block covers 32).  blockIdx.y selects a chunk of
// rows; the block's result goes to dst[blockIdx.y * cols + c].
template <bool VEC>
__global__ void __launch_bounds__(256)
sum_axis0_pass1(const float* a, int64_t rows, int64_t cols, int64_t ld, int64_t rows_per_chunk,
                float* dst, float* out, unsigned* tickets, PeerArgs peer, int peer_mode, int* error_flag,
                unsigned spin_limit) {
  constexpr int W = VEC ? 4 : 1;
  __shared__ float smem[8][32 * W + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t c = ((int64_t)blockIdx.x * 32 + tx) * W;
  const int64_t r_lo = (int64_t)blockIdx.y * rows_per_chunk;
  int64_t r_hi = r_lo + rows_per_chunk;
  if (r_hi > rows) r_hi = rows;
  constexpr int U = 8;   // rows in flight per thread
  float acc[U][W];
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int w = 0; w < W; ++w) acc[u][w] = 0.f;
  if (c < cols) {
    int64_t r = r_lo + ty;
    for (; r + 8 * (U - 1) < r_hi; r += 8 * U) {
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float* p = a + (r + 8 * u) * ld + c;
        if (VEC) v[u] = __ldcs(reinterpret_cast<const float4*>(p));
        else v[u] = make_float4(__ldcs(p), 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        acc[u][0] += v[u].x;
        if (VEC) { acc[u][1 % W] += v[u].y; acc[u][2 % W] += v[u].z; acc[u][3 % W] += v[u].w; }
      }
    }
    for (; r < r_hi; r += 8) {
      const float* p = a + r * ld + c;
      if (VEC) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(p));
        acc[0][0] += v.x; acc[0][1 % W] += v.y; acc[0][2 % W] += v.z; acc[0][3 % W] += v.w;
      } else {
        acc[0][0] += __ldcs(p);
      }
    }
  }
#pragma unroll
  for (int w = 0; w < W; ++w)
    smem[ty][tx * W + w] = ((acc[0][w] + acc[1][w]) + (acc[2][w] + acc[3][w])) +
                           ((acc[4][w] + acc[5][w]) + (acc[6][w] + acc[7][w]));
  __syncthreads();
  // 32*W columns, summed over the 8 row lanes in a fixed order
  for (int j = ty * 32 + tx; j < 32 * W; j += 256) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += smem[k][j];
    const int64_t cc = (int64_t)blockIdx.x * 32 * W + j;
    if (cc < cols) dst[(int64_t)blockIdx.y * cols + cc] = s;
  }
  if (tickets)
    axis0_fold_pass2(tickets, dst, nullptr, out, nullptr, cols, (int64_t)blockIdx.x * 32 * W, 32 * W, peer, peer_mode,
                     error_flag, spin_limit);
}

// ---- column sums with the producing elementwise step folded in (BatchNorm) -------------
// The BatchNorm layer (brainstorm/layers/batch_normalization_layer.py) takes every one of its
// batch statistics as "an elementwise op into a temporary, then sum_t(axis=0)".  These two
// pass-1 kernels do the elementwise step while they read, with exactly the row walk and the
// order of additions of sum_axis0_pass1<true>, so the sums have the same bits as the two-call
// form; pass 2 is sum_axis0_pass2.  128-bit accesses: cols and ld multiples of 4, 16-byte
// aligned bases.
//   MODE 0 (forward, :67-86): c = x + mu[col] is written to `centered`; sums of c * c.
//   MODE 1 (backward, :121-136): sums of dout * x_hat (to dst) and of dout (to dst2).
template <int MODE>
__global__ void __launch_bounds__(256)
bn_colsum_pass1(const float* a, const float* b, const float* vec, float* centered, int64_t rows, int64_t cols,
                int64_t rows_per_chunk, float* dst, float* dst2, float* out, unsigned* tickets) {
  __shared__ float smem[8][32 * 4 + 1];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t c = ((int64_t)blockIdx.x * 32 + tx) * 4;
  const int64_t r_lo = (int64_t)blockIdx.y * rows_per_chunk;
  int64_t r_hi = r_lo + rows_per_chunk;
  if (r_hi > rows) r_hi = rows;
  constexpr int U = 8;
  constexpr int SETS = MODE == 1 ? 2 : 1;
  float acc[SETS][U][4];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int w = 0; w < 4; ++w) acc[s][u][w] = 0.f;
  if (c < cols) {
    float4 mu = make_float4(0.f, 0.f, 0.f, 0.f);
    if (MODE == 0) mu = *reinterpret_cast<const float4*>(vec + c);
    auto take = [&](int u, float4 va, float4 vb, int64_t r) {
      if (MODE == 0) {
        const float4 cv = make_float4(__fadd_rn(va.x, mu.x), __fadd_rn(va.y, mu.y), __fadd_rn(va.z, mu.z),
                                      __fadd_rn(va.w, mu.w));
        *reinterpret_cast<float4*>(centered + r * cols + c) = cv;
        acc[0][u][0] += __fmul_rn(cv.x, cv.x); acc[0][u][1] += __fmul_rn(cv.y, cv.y);
        acc[0][u][2] += __fmul_rn(cv.z, cv.z); acc[0][u][3] += __fmul_rn(cv.w, cv.w);
      } else {
        acc[0][u][0] += __fmul_rn(va.x, vb.x); acc[0][u][1] += __fmul_rn(va.y, vb.y);
        acc[0][u][2] += __fmul_rn(va.z, vb.z); acc[0][u][3] += __fmul_rn(va.w, vb.w);
        acc[SETS - 1][u][0] += va.x; acc[SETS - 1][u][1] += va.y; acc[SETS - 1][u][2] += va.z; acc[SETS - 1][u][3] += va.w;
      }
    };
    int64_t r = r_lo + ty;
    for (; r + 8 * (U - 1) < r_hi; r += 8 * U) {
      float4 va[U], vb[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        va[u] = *reinterpret_cast<const float4*>(a + (r + 8 * u) * cols + c);
        if (MODE == 1) vb[u] = *reinterpret_cast<const float4*>(b + (r + 8 * u) * cols + c);
        else vb[u] = va[u];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) take(u, va[u], vb[u], r + 8 * u);
    }
    for (; r < r_hi; r += 8) {
      const float4 va = *reinterpret_cast<const float4*>(a + r * cols + c);
      const float4 vb = MODE == 1 ? *reinterpret_cast<const float4*>(b + r * cols + c) : va;
      take(0, va, vb, r);
    }
  }
#pragma unroll
  for (int s = 0; s < SETS; ++s) {
#pragma unroll
    for (int w = 0; w < 4; ++w)
      smem[ty][tx * 4 + w] = ((acc[s][0][w] + acc[s][1][w]) + (acc[s][2][w] + acc[s][3][w])) +
                             ((acc[s][4][w] + acc[s][5][w]) + (acc[s][6][w] + acc[s][7][w]));
    __syncthreads();
    float* part = s == 0 ? dst : dst2;
    for (int j = ty * 32 + tx; j < 32 * 4; j += 256) {
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) t += smem[k][j];
      const int64_t cc = (int64_t)blockIdx.x * 32 * 4 + j;
      if (cc < cols) part[(int64_t)blockIdx.y * cols + cc] = t;
    }
    __syncthreads();
  }
  if (tickets)
    axis0_fold_pass2(tickets, dst, MODE == 1 ? dst2 : nullptr, out, MODE == 1 ? out + cols : nullptr, cols,
                     (int64_t)blockIdx.x * 128, 128, PeerArgs{}, 0, nullptr, 0);
}

// out[c] = sum over chunks of partial[chunk * cols + c], fixed order
__global__ void __launch_bounds__(256)
sum_axis0_pass2(const float* partial, int chunks, int64_t cols, float* out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s0 = 0.f, s1 = 0.f;
  int k = 0;
  for (; k + 1 < chunks; k += 2) {
    s0 += partial[(int64_t)k * cols + c];
    s1 += partial[(int64_t)(k + 1) * cols + c];
  }
  if (k < chunks) s0 += partial[(int64_t)k * cols + c];
  out[c] = s0 + s1;
}

// ---- sum over axis 1 (row sums): one warp per row --------------------------------------
template <bool VEC>
__global__ void __launch_bounds__(256)
sum_axis1_kernel(const float* a, int64_t rows, int64_t cols, int64_t ld, float* out) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* p = a + row * ld;
  float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
  if (VEC) {
    const int64_t nv = cols >> 2;
    const float4* q = reinterpret_cast<const float4*>(p);
    int64_t i = lane;
    for (; i + 96 < nv; i += 128) {
      const float4 v0 = __ldcs(q + i), v1 = __ldcs(q + i + 32), v2 = __ldcs(q + i + 64),
                   v3 = __ldcs(q + i + 96);
      acc0 += (v0.x + v0.y) + (v0.z + v0.w);
      acc1 += (v1.x + v1.y) + (v1.z + v1.w);
      acc2 += (v2.x + v2.y) + (v2.z + v2.w);
      acc3 += (v3.x + v3.y) + (v3.z + v3.w);
    }
    for (; i < nv; i += 32) {
      const float4 v0 = __ldcs(q + i);
      acc0 += (v0.x + v0.y) + (v0.z + v0.w);
    }
  } else {
    int64_t i = lane;
    for (; i + 96 < cols; i += 128) {
      acc0 += p[i]; acc1 += p[i + 32]; acc2 += p[i + 64]; acc3 += p[i + 96];
    }
    for (; i < cols; i += 32) acc0 += p[i];
  }
  const float s = warp_sum((acc0 + acc1) + (acc2 + acc3));
  if (lane == 0) out[row] = s;
}

// ---- softmax over rows ------------------------------------------------------------------
// The row lives in registers between the three phases (max, exp+sum, divide), so
// the matrix is read once and written once.  G threads cooperate on a row
// (G = 32: one warp per row; G = 256: one block per row); each holds VPT values.
template <int G, int VPT, bool VEC>
__global__ void __launch_bounds__(256)
softmax_rows_kernel(const float* m, float* out, int64_t rows, int cols, int64_t ldm, int64_t ldo) {
  __shared__ float smem[32];
  constexpr int ROWS_PER_BLOCK = 256 / G;
  const int g = threadIdx.x % G;
  int64_t row = (int64_t)blockIdx.x * ROWS_PER_BLOCK + threadIdx.x / G;
  const bool active = row < rows;
  if (!active) {
    if (G == 32) return;  // warps are independent
    row = rows - 1;       // G == 256: whole block shares a row, never reached
  }
  const float* p = m + row * ldm;
  float x[VPT];
  float mx = -INFINITY;
  if (VEC) {
#pragma unroll
    for (int k = 0; k < VPT / 4; ++k) {
      const int c = (g + k * G) * 4;
      float4 v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      if (c < cols) v = *reinterpret_cast<const float4*>(p + c);
      x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
      mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
    }
  } else {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int c = g + k * G;
      x[k] = (c < cols) ? p[c] : -INFINITY;
      mx = fmaxf(mx, x[k]);
    }
  }
  mx = (G == 32) ? warp_max(mx) : block_max(mx, smem);
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    x[k] = expf(x[k] - mx);  // padding: exp(-inf) = 0
    sum += x[k];
  }
  sum = (G == 32) ? warp_sum(sum) : block_sum(sum, smem);
  float* o = out + row * ldo;
  if (VEC) {
#pragma unroll
    for (int k = 0; k < VPT / 4; ++k) {
      const int c = (g + k * G) * 4;
      if (c < cols)
        *reinterpret_cast<float4*>(o + c) =
            make_float4(__fdiv_rn(x[4 * k], sum), __fdiv_rn(x[4 * k + 1], sum),
                        __fdiv_rn(x[4 * k + 2], sum), __fdiv_rn(x[4 * k + 3], sum));
    }
  } else {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int c = g + k * G;
      if (c < cols) o[c] = __fdiv_rn(x[k], sum);
    }
  }
}

// Rows too long for registers: one block per row, three passes over the row
// (which stays in L2 between them).
__global__ void __launch_bounds__(256)
softmax_long_rows_kernel(const float* m, float* out, int64_t cols, int64_t ldm, int64_t ldo) {
  __shared__ float smem[32];
  const float* p = m + (int64_t)blockIdx.x * ldm;
  float* o = out + (int64_t)blockIdx.x * ldo;
  float mx = -INFINITY;
  for (int64_t c = threadIdx.x; c < cols; c += 256) mx = fmaxf(mx, p[c]);
  mx = block_max(mx, smem);
  float sum = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += 256) sum += expf(p[c] - mx);
  sum = block_sum(sum, smem);
  for (int64_t c = threadIdx.x; c < cols; c += 256) o[c] = __fdiv_rn(expf(p[c] - mx), sum);
}

// ---- finite check --------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
nonfinite_kernel(const float* a, int64_t rows, int64_t cols, int64_t ld, int* flag) {
  const int64_t n = rows * cols;
  int bad = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    const float v = a[r * ld + c];
    bad |= !isfinite(v);
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(flag, 1);
}

// Pass-1 grids are oversubscribed on purpose: `red_blocks_per_sm` (8) blocks per SM although
// only three of the 128-bit column-sum blocks (80 registers) are resident at a time.  Short
// blocks handed out dynamically even out what the memory system gives each SM; a grid of
// exactly one resident wave was measured slower (column sums 6.20 -> 5.97 TB/s, sum over
// everything 6.45 -> 6.31), because every SM then waits for the slowest block.
unsigned* axis0_tickets(int64_t groups);

static int axis0_plan(int64_t rows, int64_t cols, bool vec, int64_t* rows_per_chunk) {
  const State& s = state();
  const int64_t gx = ceil_div(cols, vec ? 128 : 32);
  int64_t chunks = ceil_div((int64_t)s.sm_count * s.red_blocks_per_sm, gx);
  const int64_t max_chunks = ceil_div(rows, 64);  // at least 64 rows per chunk
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks > RED_MAX_PARTIALS) chunks = RED_MAX_PARTIALS;
  if (chunks < 1) chunks = 1;
  *rows_per_chunk = ceil_div(rows, chunks);
  return (int)ceil_div(rows, *rows_per_chunk);
}

static int all_plan(int64_t n, int64_t* chunk) {
  const State& s = state();
  int64_t blocks = ceil_div(n, (int64_t)RED_THREADS * 16);
  const int64_t cap = (int64_t)s.sm_count * s.red_blocks_per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks > RED_MAX_PARTIALS) blocks = RED_MAX_PARTIALS;
  if (blocks < 1) blocks = 1;
  int64_t c = ceil_div(n, blocks);
  c = (c + 3) & ~(int64_t)3;
  *chunk = c;
  return (int)ceil_div(n, c);
}

}  // namespace b200

using namespace b200;

// Scratch floats that b200_sum_t needs for these extents (0: none).
B200_API int64_t b200_sum_t_scratch_floats(int64_t rows, int64_t cols, int64_t ld, int axis) {
  if (rows <= 0 || cols <= 0) return 0;
  if (axis == 1) return 0;
  if (axis == 0) {
    const bool vec = (cols % 4 == 0) && (ld % 4 == 0);
    int64_t rpc;
    const int chunks = axis0_plan(rows, cols, vec, &rpc);
    return chunks > 1 ? (int64_t)chunks * cols : 0;
  }
  // all: non-contiguous input goes through row sums first
  if (rows > 1 && ld != cols) return rows + RED_MAX_PARTIALS;
  return RED_MAX_PARTIALS;
}

static int sum_all_contiguous(const float* a, int64_t n, float* out, float* scratch) {
  const State& s = state();
  int64_t chunk;
  const int blocks = all_plan(n, &chunk);
  float* dst = blocks > 1 ? scratch : out;
  if (aligned16(a))
    sum_all_pass1<true><<<blocks, RED_THREADS, 0, s.stream>>>(a, n, chunk, dst);
  else
    sum_all_pass1<false><<<blocks, RED_THREADS, 0, s.stream>>>(a, n, chunk, dst);
  B200_LAUNCH_CHECK();
  if (blocks > 1) {
    sum_all_pass2<<<1, RED_THREADS, 0, s.stream>>>(scratch, blocks, out);
    B200_LAUNCH_CHECK();
  }
  return B200_OK;
}

namespace b200 { int* device_error_flag(); }   // gemm_tc.cu: the mapped word that bounded device waits raise
B200_API int b200_peer_allreduce(const float* src, float* dst, int n, int average);   // peer.cu
B200_API int b200_peer_enabled(void);

// Column sums.  peer_mode 1 / 2 also completes them across the ranks (sum / mean) over peer memory: inside the
// kernel when the ticket counters can serve this launch, else by the all-reduce kernel behind it.
static int sum_axis0(const float* a, int64_t rows, int64_t cols, int64_t ld, float* out, float* scratch, int peer_mode) {
  const State& s = state();
  const bool vec = (cols % 4 == 0) && (ld % 4 == 0) && aligned16(a);
  // the plan must not depend on the pointer: recompute with the layout-only rule
  const bool vec_layout = (cols % 4 == 0) && (ld % 4 == 0);
  int64_t rpc;
  const int chunks = axis0_plan(rows, cols, vec_layout, &rpc);
  float* dst = chunks > 1 ? scratch : out;
  const int64_t groups = ceil_div(cols, vec ? 128 : 32);
  unsigned* tickets = (chunks > 1 || peer_mode) ? axis0_tickets(groups) : nullptr;
  PeerArgs peer{};
  const bool fused = peer_mode != 0 && s.axis0_peer_fused && tickets != nullptr && groups <= PEER_MAX_GROUPS && peer_args(&peer);
  const int mode = fused ? peer_mode : 0;
  unsigned* use = (chunks > 1 || fused) ? tickets : nullptr;
  dim3 grid((unsigned)groups, chunks);
  if (vec)
    sum_axis0_pass1<true><<<grid, dim3(32, 8), 0, s.stream>>>(a, rows, cols, ld, rpc, dst, out, use, peer, mode,
                                                              device_error_flag(), s.peer_spin_limit);
  else
    sum_axis0_pass1<false><<<grid, dim3(32, 8), 0, s.stream>>>(a, rows, cols, ld, rpc, dst, out, use, peer, mode,
                                                               device_error_flag(), s.peer_spin_limit);
  B200_LAUNCH_CHECK();
  if (chunks > 1 && !use) {
    sum_axis0_pass2<<<(unsigned)ceil_div(cols, 256), 256, 0, s.stream>>>(scratch, chunks, cols, out);
    B200_LAUNCH_CHECK();
  }
  if (peer_mode != 0 && !fused) return b200_peer_allreduce(out, out, (int)cols, peer_mode == 2);
  return B200_OK;
}

// axis: 0 -> out[c] = sum_r a[r, c]; 1 -> out[r] = sum_c a[r, c]; -1 -> out[0] = sum of all.
B200_API int b200_sum_t(const float* a, int64_t rows, int64_t cols, int64_t ld, int axis, float* out,
                        float* scratch, int64_t scratch_floats) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(rows >= 0 && cols >= 0 && out != nullptr, "bad extent or NULL out");
  B200_REQUIRE(axis == 0 || axis == 1 || axis == -1, "axis must be 0, 1 or -1 (all)");
  const State& s = state();
  if (rows * cols == 0) {  // empty sum = 0 for every output element
    const int64_t nout = axis == 0 ? cols : (axis == 1 ? rows : 1);
    if (nout) B200_CUDA(cudaMemsetAsync(out, 0, nout * sizeof(float), s.stream));
    return B200_OK;
  }
  B200_REQUIRE(a != nullptr && ld >= cols, "bad operand");
  const int64_t need = b200_sum_t_scratch_floats(rows, cols, ld, axis);
  B200_REQUIRE(need == 0 || (scratch != nullptr && scratch_floats >= need),
               "sum_t needs %lld floats of scratch, got %lld", (long long)need,
               (long long)scratch_floats);
  if (axis == 0) return sum_axis0(a, rows, cols, ld, out, scratch, 0);
  if (axis == 1) {
    const bool vec = (cols % 4 == 0) && (ld % 4 == 0) && aligned16(a);
    const unsigned grid = (unsigned)ceil_div(rows, 8);
    if (vec) sum_axis1_kernel<true><<<grid, 256, 0, s.stream>>>(a, rows, cols, ld, out);
    else sum_axis1_kernel<false><<<grid, 256, 0, s.stream>>>(a, rows, cols, ld, out);
    B200_LAUNCH_CHECK();
    return B200_OK;
  }
  if (rows == 1 || ld == cols) return sum_all_contiguous(a, rows * cols, out, scratch);
  // pitched: row sums into scratch[0..rows), then the flat sum of those
  float* rowsum = scratch + RED_MAX_PARTIALS;
  sum_axis1_kernel<false><<<(unsigned)ceil_div(rows, 8), 256, 0, s.stream>>>(a, rows, cols, ld, rowsum);
  B200_LAUNCH_CHECK();
  return sum_all_contiguous(rowsum, rows, out, scratch);
}

// b200_sum_t(axis 0) completed across the ranks of the peer registration (b200_peer_setup): out[c] = sum (average != 0:
// mean) over ranks of the local column sums, the same bits on every rank.  By default the all-reduce kernel is queued
// behind the column-sum kernel; with tuning key 12 set it is one kernel: the block that finishes a group of 128
// columns sends that group through the exchange of b200_peer_allreduce at once (same slots, same bounded wait, same
// error reporting; after a wait that ran out `out` holds the local sums), while the other groups are still being
// summed.  (Measured on two GPUs, (65536, 4096): 200 us in one kernel, 191 us as two; the sum alone 177 us.)  cols <= b200_peer_max_floats(); every rank makes the call.
B200_API int b200_sum_t_axis0_allreduce(const float* a, int64_t rows, int64_t cols, int64_t ld, float* out, float* scratch,
                                        int64_t scratch_floats, int average) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(rows >= 0 && cols >= 0 && out != nullptr, "bad extent or NULL out");
  B200_REQUIRE(cols <= PEER_MAX_FLOATS, "at most %d columns", PEER_MAX_FLOATS);
  B200_REQUIRE(b200_peer_enabled(), "no usable peer registration (b200_peer_setup)");
  if (cols == 0) return B200_OK;
  if (rows == 0) {
    B200_CUDA(cudaMemsetAsync(out, 0, cols * sizeof(float), state().stream));
    return b200_peer_allreduce(out, out, (int)cols, average);
  }
  B200_REQUIRE(a != nullptr && ld >= cols, "bad operand");
  const int64_t need = b200_sum_t_scratch_floats(rows, cols, ld, 0);
  B200_REQUIRE(need == 0 || (scratch != nullptr && scratch_floats >= need), "sum_t needs %lld floats of scratch, got %lld",
               (long long)need, (long long)scratch_floats);
  return sum_axis0(a, rows, cols, ld, out, scratch, average ? 2 : 1);
}

B200_API int b200_softmax_m(const float* m, float* out, int64_t rows, int64_t cols, int64_t ldm,
                            int64_t ldo) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(rows >= 0 && cols >= 0, "negative extent");
  if (rows * cols == 0) return B200_OK;
  B200_REQUIRE(m && out && ldm >= cols && ldo >= cols, "bad operand");
  const State& s = state();
  const bool vec = (cols % 4 == 0) && (ldm % 4 == 0) && (ldo % 4 == 0) && aligned16(m) && aligned16(out);
  const int c = (int)cols;
#define SOFTMAX_CASE(G, VPT)                                                                   \
  do {                                                                                         \
    const unsigned grid = (unsigned)ceil_div(rows, 256 / G);                                   \
    if (vec && VPT >= 4)                                                                       \
      softmax_rows_kernel<G, (VPT >= 4 ? VPT : 4), true><<<grid, 256, 0, s.stream>>>(m, out, rows, c, ldm, ldo); \
    else                                                                                       \
      softmax_rows_kernel<G, VPT, false><<<grid, 256, 0, s.stream>>>(m, out, rows, c, ldm, ldo); \
  } while (0)
  if (cols <= 32) SOFTMAX_CASE(32, 1);
  else if (cols <= 128) SOFTMAX_CASE(32, 4);
  else if (cols <= 256) SOFTMAX_CASE(32, 8);
  else if (cols <= 512) SOFTMAX_CASE(32, 16);
  else if (cols <= 1024) SOFTMAX_CASE(32, 32);
  else if (cols <= 2048) SOFTMAX_CASE(256, 8);
  else if (cols <= 4096) SOFTMAX_CASE(256, 16);
  else if (cols <= 8192) SOFTMAX_CASE(256, 32);
  else {
    B200_REQUIRE(rows < ((int64_t)1 << 31), "too many rows");
    softmax_long_rows_kernel<<<(unsigned)rows, 256, 0, s.stream>>>(m, out, cols, ldm, ldo);
  }
#undef SOFTMAX_CASE
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// *flag (device int, caller-zeroed) is set to 1 if any element is Inf or NaN.
B200_API int b200_nonfinite_flag(const float* a, int64_t rows, int64_t cols, int64_t ld, int* flag) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(flag != nullptr, "flag is NULL");
  if (rows * cols <= 0) return B200_OK;
  const State& s = state();
  int64_t blocks = ceil_div(rows * cols, 256 * 8);
  if (blocks > (int64_t)s.sm_count * 8) blocks = (int64_t)s.sm_count * 8;
  nonfinite_kernel<<<(unsigned)blocks, 256, 0, s.stream>>>(a, rows, cols, ld, flag);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// ---- BatchNorm statistics in one pass over the data --------------------------------------
// Scratch floats the two entry points below need (contiguous (rows, cols) operands).
B200_API int64_t b200_bn_scratch_floats(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  int64_t rpc;
  const int chunks = axis0_plan(rows, cols, true, &rpc);
  return 2 * (int64_t)chunks * cols;
}

static int bn_operands_ok(const void* p0, const void* p1, const void* p2, int64_t rows, int64_t cols) {
  B200_REQUIRE(rows > 0 && cols > 0 && cols % 4 == 0, "the fused BatchNorm kernels need a multiple of 4 columns");
  B200_REQUIRE(aligned16(p0) && aligned16(p1) && aligned16(p2), "the fused BatchNorm kernels need 16-byte aligned operands");
  return B200_OK;
}

// centered[r, c] = x[r, c] + mu[c];  sq_sum[c] = sum_r centered[r, c]^2  (batch_normalization_layer.py:76-86:
// add_mv, mult_tt, sum_t in one pass; same bits as the three calls).
B200_API int b200_bn_center_sqsum(const float* x, const float* mu, float* centered, float* sq_sum, int64_t rows,
                                  int64_t cols, float* scratch, int64_t scratch_floats) {
  if (int rc = require_ready()) return rc;
  if (int rc = bn_operands_ok(x, mu, centered, rows, cols)) return rc;
  const State& s = state();
  int64_t rpc;
  const int chunks = axis0_plan(rows, cols, true, &rpc);
  B200_REQUIRE(chunks == 1 || (scratch && scratch_floats >= (int64_t)chunks * cols), "scratch too small");
  float* dst = chunks > 1 ? scratch : sq_sum;
  dim3 grid((unsigned)ceil_div(cols, 128), chunks);
  unsigned* tickets = chunks > 1 ? axis0_tickets(grid.x) : nullptr;
  bn_colsum_pass1<0><<<grid, dim3(32, 8), 0, s.stream>>>(x, nullptr, mu, centered, rows, cols, rpc, dst, nullptr, sq_sum, tickets);
  B200_LAUNCH_CHECK();
  if (chunks > 1 && !tickets) {
    sum_axis0_pass2<<<(unsigned)ceil_div(cols, 256), 256, 0, s.stream>>>(scratch, chunks, cols, sq_sum);
    B200_LAUNCH_CHECK();
  }
  return B200_OK;
}

// sums[c] = sum_r dout[r, c] * x_hat[r, c];  sums[cols + c] = sum_r dout[r, c]  (:121-133: mult_tt + sum_t and
// sum_t in one pass over both arrays; same bits as the three calls).
B200_API int b200_bn_backward_sums(const float* dout, const float* x_hat, float* sums, int64_t rows, int64_t cols,
                                   float* scratch, int64_t scratch_floats) {
  if (int rc = require_ready()) return rc;
  if (int rc = bn_operands_ok(dout, x_hat, sums, rows, cols)) return rc;
  const State& s = state();
  int64_t rpc;
  const int chunks = axis0_plan(rows, cols, true, &rpc);
  B200_REQUIRE(chunks == 1 || (scratch && scratch_floats >= 2 * (int64_t)chunks * cols), "scratch too small");
  float* d0 = chunks > 1 ? scratch : sums;
  float* d1 = chunks > 1 ? scratch + (int64_t)chunks * cols : sums + cols;
  dim3 grid((unsigned)ceil_div(cols, 128), chunks);
  unsigned* tickets = chunks > 1 ? axis0_tickets(grid.x) : nullptr;
  bn_colsum_pass1<1><<<grid, dim3(32, 8), 0, s.stream>>>(dout, x_hat, nullptr, nullptr, rows, cols, rpc, d0, d1, sums, tickets);
  B200_LAUNCH_CHECK();
  if (chunks > 1 && !tickets) {
    sum_axis0_pass2<<<(unsigned)ceil_div(cols, 256), 256, 0, s.stream>>>(d0, chunks, cols, sums);
    B200_LAUNCH_CHECK();
    sum_axis0_pass2<<<(unsigned)ceil_div(cols, 256), 256, 0, s.stream>>>(d1, chunks, cols, sums + cols);
    B200_LAUNCH_CHECK();
  }
  return B200_OK;
}

// ---- sum_t without any allocation ------------------------------------------------------
// Some hosts of this library may not allocate device memory once they are running:
// a serving process whose own memory pool has already taken the whole GPU, or a
// control loop that must never enter the CUDA allocator because an allocation can
// fail or stall the device at an arbitrary moment.  For them the partial sums of
// the two-pass tree live in a fixed array inside the library image instead of in
// caller-provided scratch.  Every GPU that loads the library carries the array
// (1 MiB) until the process exits.
#define B200_STATIC_SCRATCH_FLOATS (256 * 1024)
static __device__ __align__(256) float g_static_sum_scratch[B200_STATIC_SCRATCH_FLOATS];

namespace b200 {
// In host code the symbol above is only a stand-in, not a device address.  The real
// address is looked up once per device, with that device current, when b200_init binds
// the process to its GPU; b200_sum_t_static only reads it here afterwards.
static float* g_static_scratch_ptr[64] = {nullptr};
static unsigned* g_axis0_tickets_ptr[64] = {nullptr};    // the ticket counters of the folded second pass, same rule

int static_scratch_setup() {
  int dev = -1;
  B200_CUDA(cudaGetDevice(&dev));
  B200_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  if (g_static_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    B200_CUDA(cudaGetSymbolAddress((void**)&p, g_static_sum_scratch));
    B200_REQUIRE(p != nullptr, "cudaGetSymbolAddress returned a NULL address");
    g_static_scratch_ptr[dev] = p;
  }
  if (g_axis0_tickets_ptr[dev] == nullptr) {
    unsigned* t = nullptr;
    B200_CUDA(cudaGetSymbolAddress((void**)&t, g_axis0_tickets));
    B200_REQUIRE(t != nullptr, "cudaGetSymbolAddress returned a NULL address");
    g_axis0_tickets_ptr[dev] = t;
  }
  return B200_OK;
}

// The ticket counters for a column-sum launch of `groups` column groups on the current stream,
// or NULL when the second pass has to be a launch of its own (more groups than counters, the
// folded form switched off, or no address yet).
unsigned* axis0_tickets(int64_t groups) {
  const State& s = state();
  if (!s.axis0_fold || groups > AXIS0_TICKET_SLOTS || s.device < 0 || s.device >= 64) return nullptr;
  unsigned* base = g_axis0_tickets_ptr[s.device];
  return base ? base + (s.stream_index ? AXIS0_TICKET_SLOTS + 1 : 0) : nullptr;
}
}  // namespace b200

B200_API int64_t b200_sum_t_static_max_scratch_floats(void) { return B200_STATIC_SCRATCH_FLOATS; }

// Same result as b200_sum_t (same kernels, same order of additions), but the
// partial sums go to the library's built-in array: the call allocates nothing.
// Extents whose partials need more than the array holds are rejected.  All calls
// share the one array, which keeps the previous call's partials: nothing in it has
// to start at zero (pass 1 writes every partial that pass 2 reads), but two such
// calls that overlap on the GPU (different streams or processes' threads) race on it.
B200_API int b200_sum_t_static(const float* a, int64_t rows, int64_t cols, int64_t ld, int axis,
                               float* out) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(axis == 0 || axis == 1 || axis == -1, "axis must be 0, 1 or -1 (all)");
  const int64_t need = b200_sum_t_scratch_floats(rows, cols, ld, axis);
  B200_REQUIRE(need <= B200_STATIC_SCRATCH_FLOATS,
               "sum_t over (%lld, %lld) axis %d needs %lld floats of scratch; the built-in array "
               "holds %lld: use b200_sum_t with caller-provided scratch",
               (long long)rows, (long long)cols, axis, (long long)need,
               (long long)B200_STATIC_SCRATCH_FLOATS);
  float* scratch = g_static_scratch_ptr[state().device];
  B200_REQUIRE(scratch != nullptr, "the built-in scratch array has no address on device %d", state().device);
  return b200_sum_t(a, rows, cols, ld, axis, out, scratch, B200_STATIC_SCRATCH_FLOATS);
}
