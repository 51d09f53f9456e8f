// Fused forms of three layers' elementwise work, for networks that run on the B200 handler.
//
// The reference's Highway and BatchNorm layers (brainstorm/layers/highway_layer.py,
// batch_normalization_layer.py) spell their arithmetic as chains of handler calls, one
// kernel and one trip through memory per call: ten array streams for the Highway forward
// pass where four suffice, eighteen for the BatchNorm backward pass where six do.  The
// kernels here compute the same values in the same rounding order (products and sums
// rounded separately, exactly the sequence of the handler calls they replace), so a
// network gives the same bits with or without them.  All operands are contiguous arrays
// of n elements (or (rows, cols)), 16-byte aligned, n and cols multiples of 4; the host
// side falls back to the reference's layer code for anything else.
#include "common.cuh"

namespace b200 {

constexpr int FL_THREADS = 512;
constexpr int FL_UNROLL = 2;

static inline int fl_grid(int64_t nvec) {
  const State& s = state();
  int64_t need = ceil_div(nvec, (int64_t)FL_THREADS * FL_UNROLL);
  const int64_t cap = (int64_t)s.sm_count * 16;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

#define FL_EACH4(r, EXPR_X, EXPR_Y, EXPR_Z, EXPR_W) \
  r = make_float4(EXPR_X, EXPR_Y, EXPR_Z, EXPR_W)

// y = T * (H - x) + x   (highway_layer.py:47-50: subtract_tt, mult_tt, add_tt)
__global__ void __launch_bounds__(FL_THREADS)
highway_fwd_kernel(const float4* x, const float4* H, const float4* T, float4* y, int64_t nvec) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const float4 a = x[i], h = H[i], t = T[i];
    float4 r;
    FL_EACH4(r, __fadd_rn(__fmul_rn(t.x, __fsub_rn(h.x, a.x)), a.x), __fadd_rn(__fmul_rn(t.y, __fsub_rn(h.y, a.y)), a.y),
             __fadd_rn(__fmul_rn(t.z, __fsub_rn(h.z, a.z)), a.z), __fadd_rn(__fmul_rn(t.w, __fsub_rn(h.w, a.w)), a.w));
    y[i] = r;
  }
}

// dx += (1 - T) * dy;  dH += T * dy;  dT += (H - x) * dy   (highway_layer.py:64-71)
__global__ void __launch_bounds__(FL_THREADS)
highway_bwd_kernel(const float4* x, const float4* H, const float4* T, const float4* dy, float4* dx, float4* dH,
                   float4* dT, int64_t nvec) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const float4 a = x[i], h = H[i], t = T[i], d = dy[i];
    float4 gx = dx[i], gh = dH[i], gt = dT[i];
#define HW_B(c)                                                        \
    gx.c = __fadd_rn(gx.c, __fmul_rn(__fsub_rn(1.0f, t.c), d.c));      \
    gh.c = __fadd_rn(gh.c, __fmul_rn(t.c, d.c));                       \
    gt.c = __fadd_rn(gt.c, __fmul_rn(__fsub_rn(h.c, a.c), d.c));
    HW_B(x) HW_B(y) HW_B(z) HW_B(w)
#undef HW_B
    dx[i] = gx; dH[i] = gh; dT[i] = gt;
  }
}

// x_hat = centered / sigma[col];  out = x_hat * gamma[col] + beta[col]   (batch_normalization_layer.py:100-104)
__global__ void __launch_bounds__(FL_THREADS)
bn_normalize_kernel(const float4* centered, const float4* sigma, const float4* gamma, const float4* beta, float4* x_hat,
                    float4* out, int64_t nvec, int cols4) {
  const bool narrow = nvec < ((int64_t)1 << 31);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const int c = narrow ? (int)((unsigned)i % (unsigned)cols4) : (int)(i % cols4);   // 64-bit division only when it has to be
    const float4 v = centered[i], s = sigma[c], g = gamma[c], b = beta[c];
    float4 xh, o;
    FL_EACH4(xh, __fdiv_rn(v.x, s.x), __fdiv_rn(v.y, s.y), __fdiv_rn(v.z, s.z), __fdiv_rn(v.w, s.w));
    FL_EACH4(o, __fadd_rn(__fmul_rn(xh.x, g.x), b.x), __fadd_rn(__fmul_rn(xh.y, g.y), b.y),
             __fadd_rn(__fmul_rn(xh.z, g.z), b.z), __fadd_rn(__fmul_rn(xh.w, g.w), b.w));
    x_hat[i] = xh;
    out[i] = o;
  }
}

// in_deltas += ((dout - x_hat * g[col]) - b[col]) * coeff[col]   (batch_normalization_layer.py:126-151:
// mult_mv, subtract_tt, subtract_mv, mult_mv, add_tt), g = dgamma / m, b = dbeta / m, coeff = gamma / sigma_b
__global__ void __launch_bounds__(FL_THREADS)
bn_deltas_kernel(const float4* dout, const float4* x_hat, const float4* g, const float4* b, const float4* coeff,
                 float4* in_deltas, int64_t nvec, int cols4) {
  const bool narrow = nvec < ((int64_t)1 << 31);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const int c = narrow ? (int)((unsigned)i % (unsigned)cols4) : (int)(i % cols4);   // 64-bit division only when it has to be
    const float4 d = dout[i], xh = x_hat[i], gg = g[c], bb = b[c], cf = coeff[c];
    float4 acc = in_deltas[i];
#define BN_D(k) acc.k = __fadd_rn(__fmul_rn(__fsub_rn(__fsub_rn(d.k, __fmul_rn(xh.k, gg.k)), bb.k), cf.k), acc.k);
    BN_D(x) BN_D(y) BN_D(z) BN_D(w)
#undef BN_D
    in_deltas[i] = acc;
  }
}

// The per-feature vector arithmetic between the passes, one launch each.
// forward, mean (:63-73): mu_b = s * sum (s = -1/m); running = decay * running + (1 - decay) * mu_b
__global__ void bn_mean_kernel(const float* sum, float s, float decay, float one_minus_decay, float* mu_b, float* running,
                               int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const float m = __fmul_rn(s, sum[c]);
  mu_b[c] = m;
  running[c] = __fadd_rn(__fmul_rn(decay, running[c]), __fmul_rn(one_minus_decay, m));
}
// forward, deviation (:83-96): sigma_b = sqrt(inv_m * sq_sum + eps); running = decay * running + (1 - decay) * sigma_b
__global__ void bn_sigma_kernel(const float* sq_sum, float inv_m, float eps, float decay, float one_minus_decay,
                                float* sigma_b, float* running, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const float sg = __fsqrt_rn(__fadd_rn(__fmul_rn(inv_m, sq_sum[c]), eps));
  sigma_b[c] = sg;
  running[c] = __fadd_rn(__fmul_rn(decay, running[c]), __fmul_rn(one_minus_decay, sg));
}
// backward (:123-146): dgamma += sums[c]; dbeta += sums[cols + c]; g = inv_m * sums[c]; b = inv_m * sums[cols + c];
// coeff = gamma / sigma_b.  vec holds g, b, coeff back to back (3 * cols floats).
__global__ void bn_backward_vectors_kernel(const float* sums, float inv_m, const float* gamma, const float* sigma_b,
                                           float* dgamma, float* dbeta, float* vec, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const float sg = sums[c], sb = sums[cols + c];
  dgamma[c] = __fadd_rn(sg, dgamma[c]);
  dbeta[c] = __fadd_rn(sb, dbeta[c]);
  vec[c] = __fmul_rn(inv_m, sg);
  vec[cols + c] = __fmul_rn(inv_m, sb);
  vec[2 * cols + c] = __fdiv_rn(gamma[c], sigma_b[c]);
}

static int fl_check(int64_t n, std::initializer_list<const void*> ptrs) {
  B200_REQUIRE(n >= 0 && n % 4 == 0, "the fused layer kernels need a multiple of 4 elements");
  for (const void* p : ptrs) B200_REQUIRE(p != nullptr && aligned16(p), "the fused layer kernels need 16-byte aligned operands");
  return B200_OK;
}

}  // namespace b200

using namespace b200;

B200_API int b200_highway_forward(const float* x, const float* H, const float* T, float* y, int64_t n) {
  if (int rc = require_ready()) return rc;
  if (n == 0) return B200_OK;
  if (int rc = fl_check(n, {x, H, T, y})) return rc;
  highway_fwd_kernel<<<fl_grid(n / 4), FL_THREADS, 0, state().stream>>>((const float4*)x, (const float4*)H, (const float4*)T,
                                                                      (float4*)y, n / 4);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_highway_backward(const float* x, const float* H, const float* T, const float* dy, float* dx, float* dH,
                                   float* dT, int64_t n) {
  if (int rc = require_ready()) return rc;
  if (n == 0) return B200_OK;
  if (int rc = fl_check(n, {x, H, T, dy, dx, dH, dT})) return rc;
  highway_bwd_kernel<<<fl_grid(n / 4), FL_THREADS, 0, state().stream>>>((const float4*)x, (const float4*)H, (const float4*)T,
                                                                      (const float4*)dy, (float4*)dx, (float4*)dH,
                                                                      (float4*)dT, n / 4);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_bn_mean(const float* sum, float s, float decay, float one_minus_decay, float* mu_b, float* running,
                          int64_t cols) {
  if (int rc = require_ready()) return rc;
  if (cols <= 0) return B200_OK;
  B200_REQUIRE(sum && mu_b && running, "NULL operand");
  bn_mean_kernel<<<(unsigned)ceil_div(cols, 256), 256, 0, state().stream>>>(sum, s, decay, one_minus_decay, mu_b, running, (int)cols);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_bn_sigma(const float* sq_sum, float inv_m, float eps, float decay, float one_minus_decay, float* sigma_b,
                           float* running, int64_t cols) {
  if (int rc = require_ready()) return rc;
  if (cols <= 0) return B200_OK;
  B200_REQUIRE(sq_sum && sigma_b && running, "NULL operand");
  bn_sigma_kernel<<<(unsigned)ceil_div(cols, 256), 256, 0, state().stream>>>(sq_sum, inv_m, eps, decay, one_minus_decay, sigma_b,
                                                                          running, (int)cols);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_bn_normalize(const float* centered, const float* sigma, const float* gamma, const float* beta, float* x_hat,
                               float* out, int64_t rows, int64_t cols) {
  if (int rc = require_ready()) return rc;
  if (rows * cols == 0) return B200_OK;
  B200_REQUIRE(cols % 4 == 0, "the fused layer kernels need a multiple of 4 columns");
  if (int rc = fl_check(rows * cols, {centered, sigma, gamma, beta, x_hat, out})) return rc;
  bn_normalize_kernel<<<fl_grid(rows * cols / 4), FL_THREADS, 0, state().stream>>>(
      (const float4*)centered, (const float4*)sigma, (const float4*)gamma, (const float4*)beta, (float4*)x_hat, (float4*)out,
      rows * cols / 4, (int)(cols / 4));
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_bn_backward_vectors(const float* sums, float inv_m, const float* gamma, const float* sigma_b, float* dgamma,
                                      float* dbeta, float* vec, int64_t cols) {
  if (int rc = require_ready()) return rc;
  if (cols <= 0) return B200_OK;
  B200_REQUIRE(sums && gamma && sigma_b && dgamma && dbeta && vec, "NULL operand");
  bn_backward_vectors_kernel<<<(unsigned)ceil_div(cols, 256), 256, 0, state().stream>>>(sums, inv_m, gamma, sigma_b, dgamma, dbeta,
                                                                                     vec, (int)cols);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_bn_backward_deltas(const float* dout, const float* x_hat, const float* vec, float* in_deltas, int64_t rows,
                                     int64_t cols) {
  if (int rc = require_ready()) return rc;
  if (rows * cols == 0) return B200_OK;
  B200_REQUIRE(cols % 4 == 0, "the fused layer kernels need a multiple of 4 columns");
  if (int rc = fl_check(rows * cols, {dout, x_hat, vec, in_deltas})) return rc;
  bn_deltas_kernel<<<fl_grid(rows * cols / 4), FL_THREADS, 0, state().stream>>>(
      (const float4*)dout, (const float4*)x_hat, (const float4*)vec, (const float4*)(vec + cols), (const float4*)(vec + 2 * cols),
      (float4*)in_deltas, rows * cols / 4, (int)(cols / 4));
  B200_LAUNCH_CHECK();
  return B200_OK;
}
