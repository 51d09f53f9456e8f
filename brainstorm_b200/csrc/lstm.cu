// Fused LSTM sequence passes for the B200 handler.
//
// The reference's LSTM layer (brainstorm/layers/lstm_layer.py) issues, per
// timestep, 4 recurrent GEMMs and 15 (forward, :117-145) / 16 (backward, :173-205)
// elementwise handler calls on (batch, hidden) arrays.  Here one timestep is ONE
// stacked recurrent GEMM on the tensor cores ([Rz;Ri;Rf;Ro] is one contiguous
// (4H, H) matrix in the parameter vector) followed by ONE gate kernel that also
// finishes the GEMM's split-K sum, and the loop over time runs inside the library,
// so a whole sequence pass is a single call from the host.
//
// The gate kernels reproduce the reference's arithmetic order exactly
// (pre-activation = ((input projection + recurrent projection) + peephole) + bias,
// products rounded before they are added), write every internal buffer the
// reference layer writes, and are HBM/latency bound: forward reads 9 and writes 12
// floats per (batch, hidden) element, backward reads 15 and writes 14.
#include "common.cuh"

namespace b200 {

int gemm_tc_partials(int transa, int transb, int64_t M, int64_t N, int64_t K, const float* a, int64_t lda,
                     const float* b, int64_t ldb, float* c, int64_t ldc, const float** ptr, int* splits,
                     int64_t* split_stride, int64_t* ld);

// Marks the kernels issued while it is alive as a programmatic-dependent-launch chain.
struct PdlScope {
  explicit PdlScope(bool on) { state().pdl_now = on; }
  ~PdlScope() { state().pdl_now = false; }
};

enum { ACT_SIGMOID = 0, ACT_TANH = 1, ACT_REL = 2, ACT_EL = 3, ACT_LINEAR = 4 };

__device__ __forceinline__ float sigmoid_dev(float x) {
  const float e = expf(-fabsf(x));
  const float d = 1.0f + e;
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  r = fmaf(fmaf(-d, r, 1.0f), r, r);
  return (x >= 0.0f) ? r : __fmul_rn(e, r);
}
__device__ __forceinline__ float act_fwd(int act, float x) {
  switch (act) {
    case ACT_SIGMOID: return sigmoid_dev(x);
    case ACT_TANH: return tanhf(x);
    case ACT_REL: return (x > 0.0f) ? x : __fmul_rn(x, 0.0f);
    case ACT_EL: return (x >= 0.0f) ? x : __fsub_rn(expf(x), 1.0f);
    default: return x;
  }
}
// dx = dy * f'(y), with the reference's rounding order
__device__ __forceinline__ float act_bwd(int act, float y, float dy) {
  switch (act) {
    case ACT_SIGMOID: return __fmul_rn(__fmul_rn(dy, y), __fsub_rn(1.0f, y));
    case ACT_TANH: return __fmul_rn(dy, __fsub_rn(1.0f, __fmul_rn(y, y)));
    case ACT_REL: return (y > 0.0f) ? dy : __fmul_rn(dy, 0.0f);
    case ACT_EL: return (y >= 0.0f) ? dy : __fmul_rn(dy, __fadd_rn(y, 1.0f));
    default: return dy;
  }
}
__device__ __forceinline__ float sigmoid_bwd(float y, float dy) {
  return __fmul_rn(__fmul_rn(dy, y), __fsub_rn(1.0f, y));
}
__device__ __forceinline__ float madd(float acc, float a, float b) {  // acc + round(a*b)
  return __fadd_rn(acc, __fmul_rn(a, b));
}

struct LstmFwdStep {
  const float* xproj;   // (B, 4H) input projections of this step, gate order z,i,f,o
  const float* rpart;   // recurrent projections: `splits` partial (B, 4H) matrices
  int splits;
  int64_t split_stride, rld;
  const float* bias;    // 4H: bz,bi,bf,bo
  const float* peep;    // 3H: pi,pf,po
  const float* ca_prev; // (B, H)
  float *za, *zb, *ia, *ib, *fa, *fb, *oa, *ob, *ca, *cb, *y;  // (B, H) slices of this step
  float* y_work;        // aligned copy of y for the next step's GEMM
  int B, H, act;
};

__global__ void __launch_bounds__(256) lstm_gate_fwd_kernel(LstmFwdStep p) {
  pdl_launch_dependents();
  pdl_wait();   // the recurrent GEMM of this step must have finished
  const int64_t n = (int64_t)p.B * p.H;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int b = (int)(i / p.H), h = (int)(i - (int64_t)b * p.H);
  // issue every independent load before the first use
  const float* xp = p.xproj + (int64_t)b * 4 * p.H + h;
  const float x0 = xp[0], x1 = xp[p.H], x2 = xp[2 * p.H], x3 = xp[3 * p.H];
  const float cprev = p.ca_prev[i];
  const float bz = p.bias[h], bi = p.bias[p.H + h], bf = p.bias[2 * p.H + h], bo = p.bias[3 * p.H + h];
  const float wpi = p.peep[h], wpf = p.peep[p.H + h], wpo = p.peep[2 * p.H + h];
  float r[4] = {0.f, 0.f, 0.f, 0.f};
  const float* q0 = p.rpart + (int64_t)b * p.rld + h;
  int s = 0;
  for (; s + 4 <= p.splits; s += 4) {   // four splits in flight (the usual count is 4)
    float v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int g = 0; g < 4; ++g) v[u][g] = q0[(int64_t)(s + u) * p.split_stride + g * p.H];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int g = 0; g < 4; ++g) r[g] = (s + u == 0) ? v[u][g] : __fadd_rn(r[g], v[u][g]);
  }
  for (; s < p.splits; ++s) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const float v = q0[(int64_t)s * p.split_stride + g * p.H];
      r[g] = (s == 0) ? v : __fadd_rn(r[g], v);
    }
  }
  // block input (lstm_layer.py:117-119)
  const float za = __fadd_rn(__fadd_rn(x0, r[0]), bz);
  const float zb = act_fwd(p.act, za);
  // input gate (:122-125)
  const float ia = __fadd_rn(madd(__fadd_rn(x1, r[1]), cprev, wpi), bi);
  const float ib = sigmoid_dev(ia);
  // forget gate (:128-131)
  const float fa = __fadd_rn(madd(__fadd_rn(x2, r[2]), cprev, wpf), bf);
  const float fb = sigmoid_dev(fa);
  // cell (:134-135)
  const float ca = madd(__fmul_rn(ib, zb), fb, cprev);
  // output gate (:138-141)
  const float oa = __fadd_rn(madd(__fadd_rn(x3, r[3]), ca, wpo), bo);
  const float ob = sigmoid_dev(oa);
  // block output (:144-145)
  const float cb = act_fwd(p.act, ca);
  const float y = __fmul_rn(ob, cb);
  p.za[i] = za; p.zb[i] = zb; p.ia[i] = ia; p.ib[i] = ib; p.fa[i] = fa; p.fb[i] = fb;
  p.oa[i] = oa; p.ob[i] = ob; p.ca[i] = ca; p.cb[i] = cb; p.y[i] = y; p.y_work[i] = y;
}

struct LstmBwdStep {
  const float* deltas;  // (B, H) output deltas of this step
  const float* rpart;   // recurrent delta projections (B, H): `splits` partials, or NULL
  int splits;
  int64_t split_stride, rld;
  const float* peep;    // 3H
  const float *zb, *ib, *fb, *ob, *cb, *ca_prev;     // forward values of this step
  const float *dia_n, *dfa_n, *dca_n, *fb_n;         // step t+1
  float *dza, *dzb, *dia, *dib, *dfa, *dfb, *doa, *dob, *dca, *dcb;  // (B, H) slices of this step
  float* dg_work;       // (B, 4H) aligned stacked copy of dZa,dIa,dFa,dOa
  int B, H, act;
};

__global__ void __launch_bounds__(256) lstm_gate_bwd_kernel(LstmBwdStep p) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n = (int64_t)p.B * p.H;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int b = (int)(i / p.H), h = (int)(i - (int64_t)b * p.H);
  // issue every independent load before the first use
  const float d0 = p.deltas[i];
  const float dia_n = p.dia_n[i], dfa_n = p.dfa_n[i], dca_n = p.dca_n[i], fb_n = p.fb_n[i];
  const float ob = p.ob[i], cb = p.cb[i], fb = p.fb[i], zb = p.zb[i], ib = p.ib[i], ca_prev = p.ca_prev[i];
  // dy = output deltas + recurrent deltas (lstm_layer.py:173-177)
  float dy = d0;
  if (p.rpart) {
    const float* q0 = p.rpart + (int64_t)b * p.rld + h;
    float r = 0.f;
    int s = 0;
    for (; s + 8 <= p.splits; s += 8) {   // eight partials in flight
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = q0[(int64_t)(s + u) * p.split_stride];
#pragma unroll
      for (int u = 0; u < 8; ++u) r = (s + u == 0) ? v[u] : __fadd_rn(r, v[u]);
    }
    for (; s < p.splits; ++s) {
      const float v = q0[(int64_t)s * p.split_stride];
      r = (s == 0) ? v : __fadd_rn(r, v);
    }
    dy = __fadd_rn(dy, r);
  }
  const float pi = p.peep[h], pf = p.peep[p.H + h], po = p.peep[2 * p.H + h];
  float dca = 0.0f;                                   // :168 (dCa starts at zero)
  dca = madd(dca, dia_n, pi);                         // :180
  dca = madd(dca, dfa_n, pf);                         // :181
  const float dob = __fmul_rn(dy, cb);                // :184
  const float doa = sigmoid_bwd(ob, dob);             // :185
  dca = madd(dca, doa, po);                           // :187
  float dcb = __fmul_rn(dy, ob);                      // :190
  dcb = act_bwd(p.act, cb, dcb);                      // :191
  dca = __fadd_rn(dca, dcb);                          // :192
  dca = madd(dca, dca_n, fb_n);                       // :193
  const float dfb = __fmul_rn(dca, ca_prev);          // :196
  const float dfa = sigmoid_bwd(fb, dfb);             // :197
  const float dib = __fmul_rn(dca, zb);               // :200
  const float dia = sigmoid_bwd(ib, dib);             // :201
  const float dzb = __fmul_rn(dca, ib);               // :204
  const float dza = act_bwd(p.act, zb, dzb);          // :205
  p.dob[i] = dob; p.doa[i] = doa; p.dcb[i] = dcb; p.dca[i] = dca; p.dfb[i] = dfb; p.dfa[i] = dfa;
  p.dib[i] = dib; p.dia[i] = dia; p.dzb[i] = dzb; p.dza[i] = dza;
  float* g = p.dg_work + (int64_t)b * 4 * p.H + h;
  g[0] = dza; g[p.H] = dia; g[2 * p.H] = dfa; g[3 * p.H] = doa;
}

}  // namespace b200

using namespace b200;

// Forward pass over a whole sequence.  All eleven forward buffers are (T+1, B, H)
// with the context slot at index T (so step t-1 of t = 0 is slot T), as the reference
// lays them out (lstm_layer.py:35-67).  xproj is (T*B, 4H) and already holds the
// input projections x.[Wz;Wi;Wf;Wo]^T; r_stack is [Rz;Ri;Rf;Ro] (4H, H); y_work is a
// 16-byte aligned (T+1, B, H) array whose slot T the caller has loaded with y[T].
//
// b200_lstm_forward_steps runs timesteps [t0, t1) only: a caller that overlaps this
// layer with the layer that produces its input walks the sequence in pieces.
B200_API int b200_lstm_forward_steps(const float* xproj, const float* r_stack, const float* bias,
                                     const float* peep, float* za, float* zb, float* ia, float* ib, float* fa,
                                     float* fb, float* oa, float* ob, float* ca, float* cb, float* y,
                                     float* y_work, float* r_work, int T, int B, int H, int act, int t0,
                                     int t1) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(T >= 0 && B > 0 && H > 0 && act >= 0 && act <= 4, "bad extents or activation code");
  B200_REQUIRE(0 <= t0 && t0 <= t1 && t1 <= T, "timestep range [%d, %d) outside [0, %d)", t0, t1, T);
  const State& s = state();
  const int64_t bh = (int64_t)B * H;
  const unsigned grid = (unsigned)ceil_div(bh, 256);
  PdlScope pdl_scope(s.use_pdl != 0);
  for (int t = t0; t < t1; ++t) {
    const int tp = (t + T) % (T + 1);  // t - 1, wrapping to the context slot
    LstmFwdStep p;
    if (int rc = gemm_tc_partials(0, 1, B, 4 * (int64_t)H, H, y_work + tp * bh, H, r_stack, H, r_work,
                                  4 * (int64_t)H, &p.rpart, &p.splits, &p.split_stride, &p.rld))
      return rc;
    p.xproj = xproj + (int64_t)t * B * 4 * H;
    p.bias = bias; p.peep = peep;
    p.ca_prev = ca + tp * bh;
    p.za = za + t * bh; p.zb = zb + t * bh; p.ia = ia + t * bh; p.ib = ib + t * bh;
    p.fa = fa + t * bh; p.fb = fb + t * bh; p.oa = oa + t * bh; p.ob = ob + t * bh;
    p.ca = ca + t * bh; p.cb = cb + t * bh; p.y = y + t * bh; p.y_work = y_work + t * bh;
    p.B = B; p.H = H; p.act = act;
    B200_CUDA(launch_maybe_pdl(s.pdl_now, lstm_gate_fwd_kernel, dim3(grid), dim3(256), 0, s.stream, p));
    B200_LAUNCH_CHECK();
  }
  return B200_OK;
}

B200_API int b200_lstm_forward(const float* xproj, const float* r_stack, const float* bias,
                               const float* peep, float* za, float* zb, float* ia, float* ib, float* fa,
                               float* fb, float* oa, float* ob, float* ca, float* cb, float* y,
                               float* y_work, float* r_work, int T, int B, int H, int act) {
  return b200_lstm_forward_steps(xproj, r_stack, bias, peep, za, zb, ia, ib, fa, fb, oa, ob, ca, cb, y, y_work,
                                 r_work, T, B, H, act, 0, T);
}

// Backward pass over a whole sequence (lstm_layer.py:171-205).  deltas is the
// (T+1, B, H) output-delta buffer; the ten backward buffers are (T+1, B, H) with zeros
// in slot T; dg_work is a 16-byte aligned (T+1, B, 4H) array whose slot T is zero: on
// return slots 0..T-1 hold [dZa, dIa, dFa, dOa] side by side for the weight-gradient
// and input-delta GEMMs that follow.  b200_lstm_backward_steps walks timesteps
// t1-1 down to t0 only (the pieces must be run from the end of the sequence backwards).
B200_API int b200_lstm_backward_steps(const float* deltas, const float* r_stack, const float* peep,
                                      const float* zb, const float* ib, const float* fb, const float* ob,
                                      const float* ca, const float* cb, float* dza, float* dzb, float* dia,
                                      float* dib, float* dfa, float* dfb, float* doa, float* dob, float* dca,
                                      float* dcb, float* dg_work, float* r_work, int T, int B, int H, int act,
                                      int t0, int t1) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(T >= 0 && B > 0 && H > 0 && act >= 0 && act <= 4, "bad extents or activation code");
  B200_REQUIRE(0 <= t0 && t0 <= t1 && t1 <= T, "timestep range [%d, %d) outside [0, %d)", t0, t1, T);
  const State& s = state();
  const int64_t bh = (int64_t)B * H;
  const unsigned grid = (unsigned)ceil_div(bh, 256);
  PdlScope pdl_scope(s.use_pdl != 0);
  for (int t = t1 - 1; t >= t0; --t) {
    const int tp = (t + T) % (T + 1), tn = t + 1;
    LstmBwdStep p;
    p.rpart = nullptr; p.splits = 0; p.split_stride = 0; p.rld = 0;
    if (t < T - 1) {  // dG[t+1] (B, 4H) . [Rz;Ri;Rf;Ro] (4H, H); slot T is all zero, so skip it
      if (int rc = gemm_tc_partials(0, 0, B, H, 4 * (int64_t)H, dg_work + (int64_t)tn * 4 * bh, 4 * (int64_t)H,
                                    r_stack, H, r_work, H, &p.rpart, &p.splits, &p.split_stride, &p.rld))
        return rc;
    }
    p.deltas = deltas + t * bh; p.peep = peep;
    p.zb = zb + t * bh; p.ib = ib + t * bh; p.fb = fb + t * bh; p.ob = ob + t * bh; p.cb = cb + t * bh;
    p.ca_prev = ca + tp * bh;
    p.dia_n = dia + tn * bh; p.dfa_n = dfa + tn * bh; p.dca_n = dca + tn * bh; p.fb_n = fb + tn * bh;
    p.dza = dza + t * bh; p.dzb = dzb + t * bh; p.dia = dia + t * bh; p.dib = dib + t * bh;
    p.dfa = dfa + t * bh; p.dfb = dfb + t * bh; p.doa = doa + t * bh; p.dob = dob + t * bh;
    p.dca = dca + t * bh; p.dcb = dcb + t * bh;
    p.dg_work = dg_work + (int64_t)t * 4 * bh;
    p.B = B; p.H = H; p.act = act;
    B200_CUDA(launch_maybe_pdl(s.pdl_now, lstm_gate_bwd_kernel, dim3(grid), dim3(256), 0, s.stream, p));
    B200_LAUNCH_CHECK();
  }
  return B200_OK;
}

B200_API int b200_lstm_backward(const float* deltas, const float* r_stack, const float* peep,
                                const float* zb, const float* ib, const float* fb, const float* ob,
                                const float* ca, const float* cb, float* dza, float* dzb, float* dia,
                                float* dib, float* dfa, float* dfb, float* doa, float* dob, float* dca,
                                float* dcb, float* dg_work, float* r_work, int T, int B, int H, int act) {
  return b200_lstm_backward_steps(deltas, r_stack, peep, zb, ib, fb, ob, ca, cb, dza, dzb, dia, dib, dfa, dfb, doa,
                                  dob, dca, dcb, dg_work, r_work, T, B, H, act, 0, T);
}
