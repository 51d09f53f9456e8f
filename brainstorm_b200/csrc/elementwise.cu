// Elementwise, scalar-broadcast, vector-broadcast and label kernels of the B200
// handler.  All of them are HBM-bandwidth bound: the work is to keep enough
// 128-bit loads in flight per SM and to touch every byte exactly once.
//
// One generic kernel family serves every op.  An op is a functor with NIN input
// streams; an input stream may be the output array itself (accumulating and
// in-place forms), so nothing is declared __restrict__ and every thread reads
// all of its inputs before it writes.  Accumulating ops round the product and
// the sum separately (__fmul_rn/__fadd_rn) like the CPU backend does.
#include "common.cuh"

namespace b200 {

struct Params {
  float p0, p1;
};

// ---- functors -----------------------------------------------------------------
// LAUNCH: 0 = 1024 threads x 32 blocks per SM (the default), 1 = 512 x 32, 2 = 1024 x 16.
// Measured at 1 GiB per operand: the functors that spend many instructions per element
// (expf, a correctly rounded square root or logarithm) gain 3-4 % from 512-thread blocks
// (three resident blocks of ~40 registers instead of one of 1024 threads), tanh and the
// sigmoid 1 % from the smaller grid; everything else is fastest at the default.
#define B200_FUNCTOR_L(NAME, NIN_, LAUNCH_, EXPR)                              \
  struct NAME {                                                                \
    static constexpr int NIN = NIN_;                                           \
    static constexpr int LAUNCH = LAUNCH_;                                     \
    __device__ __forceinline__ static float apply(float a, float b, float c,   \
                                                  const Params& p) {           \
      (void)a; (void)b; (void)c; (void)p;                                      \
      return EXPR;                                                             \
    }                                                                          \
  };
#define B200_FUNCTOR(NAME, NIN_, EXPR)                                         \
  struct NAME {                                                                \
    static constexpr int NIN = NIN_;                                           \
    static constexpr int LAUNCH = 0;                                           \
    __device__ __forceinline__ static float apply(float a, float b, float c,   \
                                                  const Params& p) {           \
      (void)a; (void)b; (void)c; (void)p;                                      \
      return EXPR;                                                             \
    }                                                                          \
  };

__device__ __forceinline__ float sigmoid_f(float x) {
  // sign-split stable form: 1/(1+exp(-x)) for x >= 0, exp(x)/(1+exp(x)) for x < 0
  // A refined hardware reciprocal instead of an IEEE division: r = 1/(1+e) is the
  // x >= 0 result to under 1 ulp; e*r differs from e/(1+e) by at most 1 ulp more.
  const float e = expf(-fabsf(x));
  const float d = 1.0f + e;                       // in (1, 2]: no special cases
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  r = fmaf(fmaf(-d, r, 1.0f), r, r);              // one Newton step: below 1 ulp
  return (x >= 0.0f) ? r : __fmul_rn(e, r);
}
__device__ __forceinline__ float sign_f(float x) {
  return (x > 0.0f) ? 1.0f : ((x < 0.0f) ? -1.0f : x);  // sign(+-0) = +-0, NaN stays NaN
}
__device__ __forceinline__ float el_f(float x) {
  // x*(x>=0) + (exp(x)-1)*(x<0), evaluated like the CPU backend (no expm1)
  return (x >= 0.0f) ? x : __fsub_rn(expf(x), 1.0f);
}
__device__ __forceinline__ float el_deriv_f(float y, float dy) {
  return (y >= 0.0f) ? dy : __fmul_rn(dy, __fadd_rn(y, 1.0f));
}

B200_FUNCTOR(FAdd, 2, __fadd_rn(a, b))
B200_FUNCTOR(FSub, 2, __fsub_rn(a, b))
B200_FUNCTOR(FMul, 2, __fmul_rn(a, b))
B200_FUNCTOR(FDiv, 2, __fdiv_rn(a, b))
B200_FUNCTOR(FMod, 2, fmodf(a, b))
B200_FUNCTOR(FMulAdd, 3, __fadd_rn(c, __fmul_rn(a, b)))            // c is `out`
B200_FUNCTOR(FAddS, 1, __fadd_rn(a, p.p0))
B200_FUNCTOR(FMulS, 1, __fmul_rn(p.p0, a))
B200_FUNCTOR(FMulAddS, 2, __fadd_rn(b, __fmul_rn(p.p0, a)))        // b is `out`
B200_FUNCTOR(FFill, 0, p.p0)
B200_FUNCTOR(FCopy, 1, a)
B200_FUNCTOR(FAbs, 1, fabsf(a))
B200_FUNCTOR(FSign, 1, sign_f(a))
B200_FUNCTOR_L(FSqrt, 1, 1, __fsqrt_rn(a))
B200_FUNCTOR_L(FLog, 1, 1, logf(a))
B200_FUNCTOR(FClip, 1, (a != a) ? a : fminf(fmaxf(a, p.p0), p.p1))
B200_FUNCTOR_L(FSigmoid, 1, 2, sigmoid_f(a))
B200_FUNCTOR_L(FTanh, 1, 2, tanhf(a))
B200_FUNCTOR(FRel, 1, (a > 0.0f) ? a : __fmul_rn(a, 0.0f))          // -0.0 / NaN like x*(x>0)
B200_FUNCTOR_L(FEl, 1, 1, el_f(a))
// derivative forms: a = y, b = dy
B200_FUNCTOR(FSigmoidD, 2, __fmul_rn(__fmul_rn(b, a), __fsub_rn(1.0f, a)))
B200_FUNCTOR(FTanhD, 2, __fmul_rn(b, __fsub_rn(1.0f, __fmul_rn(a, a))))
B200_FUNCTOR(FRelD, 2, (a > 0.0f) ? b : __fmul_rn(b, 0.0f))
B200_FUNCTOR(FElD, 2, el_deriv_f(a, b))
// predicated forms: b = cond
B200_FUNCTOR(FCopyIf, 3, (b != 0.0f) ? a : c)                        // a = src, c = dest
B200_FUNCTOR(FFillIf, 2, (a != 0.0f) ? p.p0 : b)                     // a = cond, b = mem
B200_FUNCTOR(FAddIf, 3, (b != 0.0f) ? __fadd_rn(c, a) : c)           // a = a, c = out

// ---- memory access helpers ------------------------------------------------------
template <bool STREAM>
__device__ __forceinline__ float4 ld4(const float* p) {
  if (STREAM) return __ldcs(reinterpret_cast<const float4*>(p));
  return *reinterpret_cast<const float4*>(p);
}
template <bool STREAM>
__device__ __forceinline__ void st4(float* p, float4 v) {
  if (STREAM) __stcs(reinterpret_cast<float4*>(p), v);
  else *reinterpret_cast<float4*>(p) = v;
}
template <bool STREAM>
__device__ __forceinline__ float ld1(const float* p) {
  if (STREAM) return __ldcs(p);
  return *p;
}
template <bool STREAM>
__device__ __forceinline__ void st1(float* p, float v) {
  if (STREAM) __stcs(p, v);
  else *p = v;
}

template <class F>
__device__ __forceinline__ float4 apply4(float4 a, float4 b, float4 c, const Params& p) {
  float4 r;
  r.x = F::apply(a.x, b.x, c.x, p);
  r.y = F::apply(a.y, b.y, c.y, p);
  r.z = F::apply(a.z, b.z, c.z, p);
  r.w = F::apply(a.w, b.w, c.w, p);
  return r;
}

// ---- flat kernels (contiguous operands) -----------------------------------------
// Vector form.  All pointers have the same offset from a 16-byte boundary; the
// host passes them already advanced by `head` elements (0..3), which block 0
// handles with scalar accesses together with the `tail` (< 4) at the end.
constexpr int EW_UNROLL = 4;

template <class F, bool STREAM>
__global__ void __launch_bounds__(1024)
ew_flat_vec(const float* i0, const float* i1, const float* i2, float* out, int64_t nvec, int head,
            int tail, Params p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < nvec;
       base += stride * EW_UNROLL) {
    float4 a[EW_UNROLL], b[EW_UNROLL], c[EW_UNROLL];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + u * stride;
      a[u] = z; b[u] = z; c[u] = z;
      if (i < nvec) {
        if (F::NIN > 0) a[u] = ld4<STREAM>(i0 + 4 * i);
        if (F::NIN > 1) b[u] = ld4<STREAM>(i1 + 4 * i);
        if (F::NIN > 2) c[u] = ld4<STREAM>(i2 + 4 * i);
      }
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + u * stride;
      if (i < nvec) st4<STREAM>(out + 4 * i, apply4<F>(a[u], b[u], c[u], p));
    }
  }
  if (blockIdx.x == 0) {
    const int t = threadIdx.x;
    int64_t j = -1;
    if (t < head) j = (int64_t)t - head;                         // before the body
    else if (t >= 32 && t < 32 + tail) j = 4 * nvec + (t - 32);  // after the body
    if (t < head || (t >= 32 && t < 32 + tail)) {
      const float a = (F::NIN > 0) ? i0[j] : 0.f;
      const float b = (F::NIN > 1) ? i1[j] : 0.f;
      const float c = (F::NIN > 2) ? i2[j] : 0.f;
      out[j] = F::apply(a, b, c, p);
    }
  }
}

// Scalar form for operands whose offsets from a 16-byte boundary differ.
template <class F, bool STREAM>
__global__ void __launch_bounds__(1024)
ew_flat_scalar(const float* i0, const float* i1, const float* i2, float* out, int64_t n, Params p) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < n;
       base += stride * EW_UNROLL) {
    float a[EW_UNROLL], b[EW_UNROLL], c[EW_UNROLL];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + u * stride;
      a[u] = 0.f; b[u] = 0.f; c[u] = 0.f;
      if (i < n) {
        if (F::NIN > 0) a[u] = ld1<STREAM>(i0 + i);
        if (F::NIN > 1) b[u] = ld1<STREAM>(i1 + i);
        if (F::NIN > 2) c[u] = ld1<STREAM>(i2 + i);
      }
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + u * stride;
      if (i < n) st1<STREAM>(out + i, F::apply(a[u], b[u], c[u], p));
    }
  }
}

// Row-pitched form (strided views): element (r, c) of stream k is at r*ld_k + c.
template <class F>
__global__ void __launch_bounds__(1024)
ew_pitched(const float* i0, const float* i1, const float* i2, float* out, int64_t rows,
           int64_t cols, int64_t ld0, int64_t ld1_, int64_t ld2, int64_t ldo, Params p) {
  const int64_t n = rows * cols;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t r = i / cols, c = i - r * cols;
    const float a = (F::NIN > 0) ? i0[r * ld0 + c] : 0.f;
    const float b = (F::NIN > 1) ? i1[r * ld1_ + c] : 0.f;
    const float cc = (F::NIN > 2) ? i2[r * ld2 + c] : 0.f;
    out[r * ldo + c] = F::apply(a, b, cc, p);
  }
}

static inline int ew_grid(int64_t work_items, int threads, int blocks_per_sm = 0) {
  const State& s = state();
  int64_t need = ceil_div(work_items, (int64_t)threads * EW_UNROLL);
  int64_t cap = (int64_t)s.sm_count * (blocks_per_sm ? blocks_per_sm : s.ew_blocks_per_sm);
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

// Bytes beyond which operands cannot stay in L2 between kernels: use streaming
// (evict-first) accesses so that they do not displace what is reused.
constexpr int64_t STREAM_MIN_ELEMS = (int64_t)8 << 20;  // 32 MiB per operand

template <class F>
static int launch_ew(const float* i0, const float* i1, const float* i2, float* out, int64_t rows,
                     int64_t cols, int64_t ld0, int64_t ld1_, int64_t ld2, int64_t ldo, Params p) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(rows >= 0 && cols >= 0, "negative extent");
  const int64_t n = rows * cols;
  if (n == 0) return B200_OK;
  B200_REQUIRE(out != nullptr && (F::NIN < 1 || i0) && (F::NIN < 2 || i1) && (F::NIN < 3 || i2),
               "NULL operand");
  const State& s = state();
  const bool contiguous = rows == 1 || ((F::NIN < 1 || ld0 == cols) && (F::NIN < 2 || ld1_ == cols) &&
                                        (F::NIN < 3 || ld2 == cols) && ldo == cols);
  // the functor's own launch shape applies while the tuning knobs are at their defaults
  const bool tuned = s.ew_threads != 1024 || s.ew_blocks_per_sm != 32;
  const int threads = (!tuned && F::LAUNCH == 1) ? 512 : s.ew_threads;
  const int bps = (!tuned && F::LAUNCH == 2) ? 16 : 0;
  if (!contiguous) {
    ew_pitched<F><<<ew_grid(n, threads), threads, 0, s.stream>>>(i0, i1, i2, out, rows, cols, ld0,
                                                                 ld1_, ld2, ldo, p);
    B200_LAUNCH_CHECK();
    return B200_OK;
  }
  auto mis = [](const void* q) { return (int)((reinterpret_cast<uintptr_t>(q) >> 2) & 3); };
  const int mo = mis(out);
  const bool same = (F::NIN < 1 || mis(i0) == mo) && (F::NIN < 2 || mis(i1) == mo) &&
                    (F::NIN < 3 || mis(i2) == mo);
  const bool stream = n >= STREAM_MIN_ELEMS;
  if (same && n >= 8) {
    const int head = (4 - mo) & 3;
    const int64_t nvec = (n - head) / 4;
    const int tail = (int)((n - head) - 4 * nvec);
    const float* q0 = i0 ? i0 + head : nullptr;
    const float* q1 = i1 ? i1 + head : nullptr;
    const float* q2 = i2 ? i2 + head : nullptr;
    const int grid = ew_grid(nvec, threads, bps);
    if (stream)
      ew_flat_vec<F, true><<<grid, threads, 0, s.stream>>>(q0, q1, q2, out + head, nvec, head, tail, p);
    else
      ew_flat_vec<F, false><<<grid, threads, 0, s.stream>>>(q0, q1, q2, out + head, nvec, head, tail, p);
  } else {
    const int grid = ew_grid(n, threads);
    if (stream)
      ew_flat_scalar<F, true><<<grid, threads, 0, s.stream>>>(i0, i1, i2, out, n, p);
    else
      ew_flat_scalar<F, false><<<grid, threads, 0, s.stream>>>(i0, i1, i2, out, n, p);
  }
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// ---- matrix (.) broadcast vector --------------------------------------------------
// out[r, c] = f(m[r, c], v[c])   (v_is_col == 0: v is a row vector of `cols`)
// out[r, c] = f(m[r, c], v[r])   (v_is_col == 1: v is a column vector of `rows`)
// ACC forms also read out.  Vector form: a thread owns one float4 column group
// and walks down the rows, so a row vector is loaded once per thread.
template <class F, bool COL, bool STREAM>
__global__ void __launch_bounds__(1024)
mv_vec(const float* m, const float* v, float* out, int64_t rows, int cols4, int64_t ldm, int64_t ldo,
       Params p) {
  // blockDim = (column groups, row lanes); a thread keeps its column group and
  // walks down the rows, four rows in flight.
  const int c4 = blockIdx.x * blockDim.x + threadIdx.x;
  if (c4 >= cols4) return;
  float4 vr = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!COL) vr = *reinterpret_cast<const float4*>(v + 4 * (int64_t)c4);
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  const int64_t rstride = (int64_t)gridDim.y * blockDim.y;
  for (int64_t r0 = (int64_t)blockIdx.y * blockDim.y + threadIdx.y; r0 < rows; r0 += rstride * EW_UNROLL) {
    float4 a[EW_UNROLL], c[EW_UNROLL];
    float vc[EW_UNROLL];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t r = r0 + u * rstride;
      a[u] = z; c[u] = z; vc[u] = 0.f;
      if (r < rows) {
        a[u] = ld4<STREAM>(m + r * ldm + 4 * (int64_t)c4);
        if (F::NIN > 2) c[u] = ld4<STREAM>(out + r * ldo + 4 * (int64_t)c4);
        if (COL) vc[u] = v[r];
      }
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t r = r0 + u * rstride;
      if (r < rows) {
        const float4 b = COL ? make_float4(vc[u], vc[u], vc[u], vc[u]) : vr;
        st4<STREAM>(out + r * ldo + 4 * (int64_t)c4, apply4<F>(a[u], b, c[u], p));
      }
    }
  }
}

// Scalar form of the same walk for operands that are not 16-byte aligned (views at
// odd element offsets of a flat buffer): a thread owns ONE column, consecutive
// threads consecutive columns (coalesced), four rows in flight, no index division.
template <class F, bool COL>
__global__ void __launch_bounds__(1024)
mv_scalar(const float* m, const float* v, float* out, int64_t rows, int64_t cols, int64_t ldm,
          int64_t ldo, Params p) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const float vr = COL ? 0.f : v[c];
  const int64_t rstride = (int64_t)gridDim.y * blockDim.y;
  for (int64_t r0 = (int64_t)blockIdx.y * blockDim.y + threadIdx.y; r0 < rows; r0 += rstride * EW_UNROLL) {
    float a[EW_UNROLL], cc[EW_UNROLL], vc[EW_UNROLL];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t r = r0 + u * rstride;
      a[u] = 0.f; cc[u] = 0.f; vc[u] = 0.f;
      if (r < rows) {
        a[u] = m[r * ldm + c];
        if (F::NIN > 2) cc[u] = out[r * ldo + c];
        if (COL) vc[u] = v[r];
      }
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t r = r0 + u * rstride;
      if (r < rows) out[r * ldo + c] = F::apply(a[u], COL ? vc[u] : vr, cc[u], p);
    }
  }
}

template <class F>
static int launch_mv(const float* m, const float* v, float* out, int64_t rows, int64_t cols,
                     int64_t ldm, int64_t ldo, int v_is_col) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(rows >= 0 && cols >= 0, "negative extent");
  if (rows * cols == 0) return B200_OK;
  B200_REQUIRE(m && v && out, "NULL operand");
  B200_REQUIRE(ldm >= cols && ldo >= cols, "leading dimension smaller than the row length");
  const State& s = state();
  Params p{0.f, 0.f};
  const bool vec = (cols % 4 == 0) && cols >= 128 && aligned16(m) && aligned16(out) &&
                   (ldm % 4 == 0) && (ldo % 4 == 0) && (v_is_col || aligned16(v)) &&
                   cols < ((int64_t)1 << 31);
  if (vec) {
    const int cols4 = (int)(cols / 4);
    const int tx = cols4 >= 256 ? 256 : (cols4 >= 128 ? 128 : (cols4 >= 64 ? 64 : 32));
    int ty = s.ew_threads / tx;
    if (ty < 1) ty = 1;
    while (ty > 1 && (int64_t)ty * EW_UNROLL > rows) ty >>= 1;
    const dim3 threads(tx, ty);
    const int gx = (int)ceil_div(cols4, tx);
    int64_t gy = ceil_div((int64_t)s.sm_count * s.ew_blocks_per_sm, gx);
    const int64_t gy_max = ceil_div(rows, (int64_t)ty * EW_UNROLL);
    if (gy > gy_max) gy = gy_max;
    if (gy > 65535) gy = 65535;
    if (gy < 1) gy = 1;
    dim3 grid(gx, (unsigned)gy);
    const bool stream = rows * cols >= STREAM_MIN_ELEMS;
    if (v_is_col) {
      if (stream) mv_vec<F, true, true><<<grid, threads, 0, s.stream>>>(m, v, out, rows, cols4, ldm, ldo, p);
      else mv_vec<F, true, false><<<grid, threads, 0, s.stream>>>(m, v, out, rows, cols4, ldm, ldo, p);
    } else {
      if (stream) mv_vec<F, false, true><<<grid, threads, 0, s.stream>>>(m, v, out, rows, cols4, ldm, ldo, p);
      else mv_vec<F, false, false><<<grid, threads, 0, s.stream>>>(m, v, out, rows, cols4, ldm, ldo, p);
    }
  } else {
    const int tx = cols >= 256 ? 256 : (cols >= 128 ? 128 : (cols >= 64 ? 64 : 32));
    int ty = s.ew_threads / tx;
    if (ty < 1) ty = 1;
    while (ty > 1 && (int64_t)ty * EW_UNROLL > rows) ty >>= 1;
    const int64_t gx = ceil_div(cols, tx);
    B200_REQUIRE(gx < ((int64_t)1 << 31), "too many columns");
    int64_t gy = ceil_div((int64_t)s.sm_count * s.ew_blocks_per_sm, gx);
    const int64_t gy_max = ceil_div(rows, (int64_t)ty * EW_UNROLL);
    if (gy > gy_max) gy = gy_max;
    if (gy > 65535) gy = 65535;
    if (gy < 1) gy = 1;
    const dim3 grid((unsigned)gx, (unsigned)gy), threads(tx, ty);
    if (v_is_col) mv_scalar<F, true><<<grid, threads, 0, s.stream>>>(m, v, out, rows, cols, ldm, ldo, p);
    else mv_scalar<F, false><<<grid, threads, 0, s.stream>>>(m, v, out, rows, cols, ldm, ldo, p);
  }
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// out[r, c] = f(out[r, c] + bias[c]) in place: the tail of FullyConnectedLayerImpl.forward_pass
// (brainstorm/layers/fully_connected_layer.py:61-62: add_mv, then the in-place activation) as one
// kernel.  Same walk as mv_vec; the sum is rounded before the activation is applied, as there.
template <class F>
__global__ void __launch_bounds__(1024)
bias_act_vec(float* out, const float* bias, int64_t rows, int cols4, int64_t ld, Params p) {
  const int c4 = blockIdx.x * blockDim.x + threadIdx.x;
  if (c4 >= cols4) return;
  const float4 b = *reinterpret_cast<const float4*>(bias + 4 * (int64_t)c4);
  const int64_t rstride = (int64_t)gridDim.y * blockDim.y;
  for (int64_t r0 = (int64_t)blockIdx.y * blockDim.y + threadIdx.y; r0 < rows; r0 += rstride * EW_UNROLL) {
    float4 a[EW_UNROLL];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t r = r0 + u * rstride;
      a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < rows) a[u] = *reinterpret_cast<const float4*>(out + r * ld + 4 * (int64_t)c4);
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t r = r0 + u * rstride;
      if (r >= rows) continue;
      float4 v;
      v.x = F::apply(__fadd_rn(a[u].x, b.x), 0.f, 0.f, p);
      v.y = F::apply(__fadd_rn(a[u].y, b.y), 0.f, 0.f, p);
      v.z = F::apply(__fadd_rn(a[u].z, b.z), 0.f, 0.f, p);
      v.w = F::apply(__fadd_rn(a[u].w, b.w), 0.f, 0.f, p);
      *reinterpret_cast<float4*>(out + r * ld + 4 * (int64_t)c4) = v;
    }
  }
}

// The same for rows without a pitch: the flat walk of ew_flat_vec, the bias vector read through L1.
template <class F, bool STREAM>
__global__ void __launch_bounds__(1024)
bias_act_flat(float* out, const float* bias, int64_t nvec, int cols4, Params p) {
  const bool narrow = nvec < ((int64_t)1 << 31);      // 64-bit division only when it has to be
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; base < nvec; base += stride * EW_UNROLL) {
    float4 a[EW_UNROLL];
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + u * stride;
      a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < nvec) a[u] = ld4<STREAM>(out + 4 * i);
    }
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u) {
      const int64_t i = base + u * stride;
      if (i >= nvec) continue;
      const float4 b = *reinterpret_cast<const float4*>(bias + 4 * (narrow ? (int64_t)((unsigned)i % (unsigned)cols4) : i % cols4));
      float4 v;
      v.x = F::apply(__fadd_rn(a[u].x, b.x), 0.f, 0.f, p);
      v.y = F::apply(__fadd_rn(a[u].y, b.y), 0.f, 0.f, p);
      v.z = F::apply(__fadd_rn(a[u].z, b.z), 0.f, 0.f, p);
      v.w = F::apply(__fadd_rn(a[u].w, b.w), 0.f, 0.f, p);
      st4<STREAM>(out + 4 * i, v);
    }
  }
}

template <class F>
static int launch_bias_act(float* out, const float* bias, int64_t rows, int64_t cols, int64_t ld) {
  const State& s = state();
  const int cols4 = (int)(cols / 4);
  if (ld == cols) {
    const bool tuned = s.ew_threads != 1024 || s.ew_blocks_per_sm != 32;
    const int threads = (!tuned && F::LAUNCH == 1) ? 512 : s.ew_threads;
    const int bps = (!tuned && F::LAUNCH == 2) ? 16 : 0;
    const int64_t nvec = rows * cols4;
    if (nvec * 4 >= STREAM_MIN_ELEMS)
      bias_act_flat<F, true><<<ew_grid(nvec, threads, bps), threads, 0, s.stream>>>(out, bias, nvec, cols4, Params{0.f, 0.f});
    else
      bias_act_flat<F, false><<<ew_grid(nvec, threads, bps), threads, 0, s.stream>>>(out, bias, nvec, cols4, Params{0.f, 0.f});
    B200_LAUNCH_CHECK();
    return B200_OK;
  }
  const int tx = cols4 >= 256 ? 256 : (cols4 >= 128 ? 128 : (cols4 >= 64 ? 64 : 32));
  int ty = s.ew_threads / tx;
  if (ty < 1) ty = 1;
  while (ty > 1 && (int64_t)ty * EW_UNROLL > rows) ty >>= 1;
  const int gx = (int)ceil_div(cols4, tx);
  int64_t gy = ceil_div((int64_t)s.sm_count * s.ew_blocks_per_sm, gx);
  const int64_t gy_max = ceil_div(rows, (int64_t)ty * EW_UNROLL);
  if (gy > gy_max) gy = gy_max;
  if (gy > 65535) gy = 65535;
  if (gy < 1) gy = 1;
  bias_act_vec<F><<<dim3(gx, (unsigned)gy), dim3(tx, ty), 0, s.stream>>>(out, bias, rows, cols4, ld, Params{0.f, 0.f});
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// ---- labels ---------------------------------------------------------------------
// out[r, c] = (c == int(v[r])) ? 1 : 0 ; every element of out is written once.
// A thread owns one float4 column group (or one column) and walks down the rows
// eight at a time: the eight labels are fetched first (broadcast loads), then the
// eight stores are issued back to back, so no store waits on a label.
constexpr int BIN_ROWS = 8;
template <bool VEC, bool STREAM>
__global__ void __launch_bounds__(256)
binarize_kernel(const float* v, int64_t ldv, float* out, int64_t rows, int64_t cols, int64_t ldo) {
  const int64_t per_row = VEC ? (cols >> 2) : cols;
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= per_row) return;
  const int c = (int)(VEC ? (g << 2) : g);
  const int64_t rstride = (int64_t)gridDim.y * BIN_ROWS;
  for (int64_t r0 = (int64_t)blockIdx.y * BIN_ROWS; r0 < rows; r0 += rstride) {
    int lab[BIN_ROWS];
#pragma unroll
    for (int u = 0; u < BIN_ROWS; ++u) lab[u] = (r0 + u < rows) ? (int)v[(r0 + u) * ldv] : -1;
#pragma unroll
    for (int u = 0; u < BIN_ROWS; ++u) {
      if (r0 + u >= rows) break;
      float* o = out + (r0 + u) * ldo + c;
      if (VEC)
        st4<STREAM>(o, make_float4(lab[u] == c ? 1.f : 0.f, lab[u] == c + 1 ? 1.f : 0.f,
                                   lab[u] == c + 2 ? 1.f : 0.f, lab[u] == c + 3 ? 1.f : 0.f));
      else
        st1<STREAM>(o, lab[u] == c ? 1.f : 0.f);
    }
  }
}

// out[r] = m[r, int(v[r])]; labels outside [0, cols) set the error flag and
// leave out[r] untouched instead of reading out of bounds.
__global__ void __launch_bounds__(256)
index_rows_kernel(const float* m, int64_t ldm, const float* v, int64_t ldv, float* out, int64_t ldo,
                  int64_t rows, int64_t cols, int* bad) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int lab = (int)v[r * ldv];
  if (lab < 0 || lab >= cols) {
    if (bad) atomicExch(bad, 1);
    return;
  }
  out[r * ldo] = m[r * ldm + lab];
}

// last-axis concat / split-accumulate (Merge layer): 2-D views of `rows` rows
__global__ void __launch_bounds__(256)
merge_kernel(const float* a, const float* b, float* out, int64_t rows, int64_t na, int64_t nb) {
  const int64_t n = rows * (na + nb);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / (na + nb), c = i - r * (na + nb);
    out[i] = (c < na) ? a[r * na + c] : b[r * nb + (c - na)];
  }
}
__global__ void __launch_bounds__(256)
split_add_kernel(const float* x, float* oa, float* ob, int64_t rows, int64_t na, int64_t nb) {
  const int64_t n = rows * (na + nb);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / (na + nb), c = i - r * (na + nb);
    if (c < na) oa[r * na + c] = __fadd_rn(oa[r * na + c], x[i]);
    else ob[r * nb + (c - na)] = __fadd_rn(ob[r * nb + (c - na)], x[i]);
  }
}

}  // namespace b200

using namespace b200;

// ---- C-ABI ------------------------------------------------------------------------
#define B200_TT(NAME, F)                                                                        \
  B200_API int NAME(const float* a, const float* b, float* out, int64_t rows, int64_t cols,     \
                    int64_t lda, int64_t ldb, int64_t ldo) {                                    \
    return launch_ew<F>(a, b, nullptr, out, rows, cols, lda, ldb, 0, ldo, Params{0.f, 0.f});   \
  }
B200_TT(b200_add_tt, FAdd)
B200_TT(b200_subtract_tt, FSub)
B200_TT(b200_mult_tt, FMul)
B200_TT(b200_divide_tt, FDiv)
B200_TT(b200_modulo_tt, FMod)

B200_API int b200_mult_add_tt(const float* a, const float* b, float* out, int64_t rows, int64_t cols,
                              int64_t lda, int64_t ldb, int64_t ldo) {
  return launch_ew<FMulAdd>(a, b, out, out, rows, cols, lda, ldb, ldo, ldo, Params{0.f, 0.f});
}

#define B200_ST(NAME, F)                                                                        \
  B200_API int NAME(float s, const float* t, float* out, int64_t rows, int64_t cols, int64_t ldt, \
                    int64_t ldo) {                                                              \
    return launch_ew<F>(t, nullptr, nullptr, out, rows, cols, ldt, 0, 0, ldo, Params{s, 0.f});  \
  }
B200_ST(b200_add_st, FAddS)
B200_ST(b200_mult_st, FMulS)

B200_API int b200_mult_add_st(float s, const float* t, float* out, int64_t rows, int64_t cols,
                              int64_t ldt, int64_t ldo) {
  return launch_ew<FMulAddS>(t, out, nullptr, out, rows, cols, ldt, ldo, 0, ldo, Params{s, 0.f});
}

#define B200_UNARY(NAME, F)                                                                     \
  B200_API int NAME(const float* a, float* out, int64_t rows, int64_t cols, int64_t lda,        \
                    int64_t ldo) {                                                              \
    return launch_ew<F>(a, nullptr, nullptr, out, rows, cols, lda, 0, 0, ldo, Params{0.f, 0.f}); \
  }
B200_UNARY(b200_copy_to, FCopy)
B200_UNARY(b200_abs_t, FAbs)
B200_UNARY(b200_sign_t, FSign)
B200_UNARY(b200_sqrt_t, FSqrt)
B200_UNARY(b200_log_t, FLog)
B200_UNARY(b200_sigmoid, FSigmoid)
B200_UNARY(b200_tanh, FTanh)
B200_UNARY(b200_rel, FRel)
B200_UNARY(b200_el, FEl)

B200_API int b200_clip_t(const float* a, float a_min, float a_max, float* out, int64_t rows,
                         int64_t cols, int64_t lda, int64_t ldo) {
  return launch_ew<FClip>(a, nullptr, nullptr, out, rows, cols, lda, 0, 0, ldo, Params{a_min, a_max});
}

B200_API int b200_fill(float* mem, float val, int64_t rows, int64_t cols, int64_t ld) {
  return launch_ew<FFill>(nullptr, nullptr, nullptr, mem, rows, cols, 0, 0, 0, ld, Params{val, 0.f});
}

#define B200_DERIV(NAME, F)                                                                     \
  B200_API int NAME(const float* y, const float* dy, float* dx, int64_t rows, int64_t cols,     \
                    int64_t ldy, int64_t lddy, int64_t lddx) {                                  \
    return launch_ew<F>(y, dy, nullptr, dx, rows, cols, ldy, lddy, 0, lddx, Params{0.f, 0.f}); \
  }
B200_DERIV(b200_sigmoid_deriv, FSigmoidD)
B200_DERIV(b200_tanh_deriv, FTanhD)
B200_DERIV(b200_rel_deriv, FRelD)
B200_DERIV(b200_el_deriv, FElD)

B200_API int b200_copy_to_if(const float* src, float* dest, const float* cond, int64_t rows,
                             int64_t cols, int64_t lds, int64_t ldd, int64_t ldc) {
  return launch_ew<FCopyIf>(src, cond, dest, dest, rows, cols, lds, ldc, ldd, ldd, Params{0.f, 0.f});
}
B200_API int b200_fill_if(float* mem, float val, const float* cond, int64_t rows, int64_t cols,
                          int64_t ldm, int64_t ldc) {
  return launch_ew<FFillIf>(cond, mem, nullptr, mem, rows, cols, ldc, ldm, 0, ldm, Params{val, 0.f});
}
B200_API int b200_add_into_if(const float* a, float* out, const float* cond, int64_t rows,
                              int64_t cols, int64_t lda, int64_t ldo, int64_t ldc) {
  return launch_ew<FAddIf>(a, cond, out, out, rows, cols, lda, ldc, ldo, ldo, Params{0.f, 0.f});
}

#define B200_MV(NAME, F)                                                                        \
  B200_API int NAME(const float* m, const float* v, float* out, int64_t rows, int64_t cols,     \
                    int64_t ldm, int64_t ldo, int v_is_col) {                                   \
    return launch_mv<F>(m, v, out, rows, cols, ldm, ldo, v_is_col);                             \
  }
B200_MV(b200_add_mv, FAdd)
B200_MV(b200_subtract_mv, FSub)
B200_MV(b200_mult_mv, FMul)
B200_MV(b200_divide_mv, FDiv)
B200_MV(b200_mult_add_mv, FMulAdd)

// broadcast_t is out[r, c] = v[c] or v[r]: the "second operand" functor of the
// broadcast kernels with the matrix stream ignored.
namespace b200 {
struct FSecond {
  static constexpr int NIN = 2;
  __device__ __forceinline__ static float apply(float, float b, float, const Params&) { return b; }
};
}  // namespace b200
B200_API int b200_broadcast_t(const float* v, float* out, int64_t rows, int64_t cols, int64_t ldo,
                              int v_is_col) {
  return launch_mv<FSecond>(out, v, out, rows, cols, ldo, ldo, v_is_col);
}

B200_API int b200_binarize_v(const float* v, int64_t ldv, float* out, int64_t rows, int64_t cols,
                             int64_t ldo) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(rows >= 0 && cols >= 0, "negative extent");
  if (rows * cols == 0) return B200_OK;
  B200_REQUIRE(v && out && ldo >= cols && ldv >= 1, "bad operand");
  const State& s = state();
  const bool vec = (cols % 4 == 0) && aligned16(out) && (ldo % 4 == 0);
  const bool stream = rows * cols >= STREAM_MIN_ELEMS;
  const int64_t per_row = vec ? cols / 4 : cols;
  const int threads = per_row >= 256 ? 256 : (per_row >= 128 ? 128 : (per_row >= 64 ? 64 : 32));
  const int64_t gx = ceil_div(per_row, threads);
  B200_REQUIRE(gx < ((int64_t)1 << 31), "too many columns");
  int64_t gy = ceil_div((int64_t)s.sm_count * s.ew_blocks_per_sm * 256 / threads, gx);
  const int64_t gy_max = ceil_div(rows, BIN_ROWS);
  if (gy > gy_max) gy = gy_max;
  if (gy > 65535) gy = 65535;
  if (gy < 1) gy = 1;
  const dim3 grid((unsigned)gx, (unsigned)gy);
  if (vec) {
    if (stream) binarize_kernel<true, true><<<grid, threads, 0, s.stream>>>(v, ldv, out, rows, cols, ldo);
    else binarize_kernel<true, false><<<grid, threads, 0, s.stream>>>(v, ldv, out, rows, cols, ldo);
  } else {
    if (stream) binarize_kernel<false, true><<<grid, threads, 0, s.stream>>>(v, ldv, out, rows, cols, ldo);
    else binarize_kernel<false, false><<<grid, threads, 0, s.stream>>>(v, ldv, out, rows, cols, ldo);
  }
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_index_m_by_v(const float* m, int64_t ldm, const float* v, int64_t ldv, float* out,
                               int64_t ldo, int64_t rows, int64_t cols, int* bad_label_flag) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(rows >= 0 && cols >= 0, "negative extent");
  if (rows == 0) return B200_OK;
  B200_REQUIRE(m && v && out && cols > 0, "bad operand");
  index_rows_kernel<<<(unsigned)ceil_div(rows, 256), 256, 0, state().stream>>>(
      m, ldm, v, ldv, out, ldo, rows, cols, bad_label_flag);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_merge_tt(const float* a, const float* b, float* out, int64_t rows, int64_t na,
                           int64_t nb) {
  if (int rc = require_ready()) return rc;
  if (rows * (na + nb) <= 0) return B200_OK;
  merge_kernel<<<ew_grid(rows * (na + nb) * EW_UNROLL, 256), 256, 0, state().stream>>>(a, b, out, rows, na, nb);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_split_add_tt(const float* x, float* out_a, float* out_b, int64_t rows, int64_t na,
                               int64_t nb) {
  if (int rc = require_ready()) return rc;
  if (rows * (na + nb) <= 0) return B200_OK;
  split_add_kernel<<<ew_grid(rows * (na + nb) * EW_UNROLL, 256), 256, 0, state().stream>>>(x, out_a, out_b, rows, na, nb);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// act: 0 sigmoid, 1 tanh, 2 rel, 3 el, 4 linear (bias only).  cols and ld multiples of 4, 16-byte aligned operands.
B200_API int b200_bias_act(float* out, const float* bias, int64_t rows, int64_t cols, int64_t ld, int act) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(rows >= 0 && cols >= 0 && act >= 0 && act <= 4, "bad extent or activation code");
  if (rows * cols == 0) return B200_OK;
  B200_REQUIRE(out && bias && cols % 4 == 0 && ld % 4 == 0 && ld >= cols && aligned16(out) && aligned16(bias) &&
               cols < ((int64_t)1 << 31), "bias_act needs 16-byte aligned operands and a multiple of 4 columns");
  switch (act) {
    case 0: return launch_bias_act<FSigmoid>(out, bias, rows, cols, ld);
    case 1: return launch_bias_act<FTanh>(out, bias, rows, cols, ld);
    case 2: return launch_bias_act<FRel>(out, bias, rows, cols, ld);
    case 3: return launch_bias_act<FEl>(out, bias, rows, cols, ld);
    default: return launch_bias_act<FCopy>(out, bias, rows, cols, ld);
  }
}
