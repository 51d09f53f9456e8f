// Convolution support (im2col / col2im around the tensor-core GEMM) and 2-D
// pooling for the B200 handler, NHWC layout as in the reference.  All kernels are
// gather-form: one thread owns one OUTPUT element of the kernel and sums its
// contributions in a fixed order, so overlapping windows need no atomics and the
// results are deterministic.  HBM / L2 bound, channel index fastest (coalesced).
#include "common.cuh"

namespace b200 {

struct Geo {
  int N, H, W, C;      // images, NHWC
  int kh, kw, pad, sy, sx;
  int oh, ow;          // output positions per image
};

// Every kernel comes in four forms: index arithmetic in 32 bits when the largest index fits
// (always, for the networks this serves; 64-bit divisions cost more than the memory access
// they address), and V = 4 channels per thread with 128-bit accesses when the channel count
// is a multiple of 4 and the arrays are 16-byte aligned.
template <int V>
__device__ __forceinline__ void load_v(const float* p, float (&r)[V]) {
  if (V == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    r[0] = t.x; r[1 % V] = t.y; r[2 % V] = t.z; r[3 % V] = t.w;
  } else {
    r[0] = *p;
  }
}
template <int V>
__device__ __forceinline__ void store_v(float* p, const float (&r)[V]) {
  if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r[0], r[1 % V], r[2 % V], r[3 % V]);
  else *p = r[0];
}

// col[(n, oy, ox), (ky, kx, c)] = in[n, oy*sy - pad + ky, ox*sx - pad + kx, c] or 0
template <typename I, int V>
__global__ void __launch_bounds__(256) im2col_kernel(const float* __restrict__ in, float* __restrict__ col, Geo g) {
  const I CV = g.C / V;
  const I KV = (I)g.kh * g.kw * CV;
  const I total = (I)g.N * g.oh * g.ow * KV;
  for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (I)gridDim.x * blockDim.x) {
    const I row = i / KV;
    I k = i - row * KV;
    const int c = (int)(k % CV); k /= CV;
    const int kx = (int)(k % g.kw), ky = (int)(k / g.kw);
    const int ox = (int)(row % g.ow);
    const I t = row / g.ow;
    const int oy = (int)(t % g.oh), n = (int)(t / g.oh);
    const int y = oy * g.sy - g.pad + ky, x = ox * g.sx - g.pad + kx;
    float v[V];
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = 0.f;
    if (y >= 0 && y < g.H && x >= 0 && x < g.W) load_v<V>(in + ((((I)n * g.H + y) * g.W + x) * CV + c) * V, v);
    store_v<V>(col + i * V, v);
  }
}

// The same for channel counts that rule out 128-bit accesses (an RGB input layer): one thread per
// (output position, kernel row) copies the kw * C floats of that kernel row, which are contiguous
// in the image and in the patch matrix, so the index arithmetic is paid once per kernel row
// instead of once per float, and a warp still writes one contiguous stretch of the matrix.
template <typename I>
__global__ void __launch_bounds__(256) im2col_rows_kernel(const float* __restrict__ in, float* __restrict__ col, Geo g) {
  const int run = g.kw * g.C;
  const I total = (I)g.N * g.oh * g.ow * g.kh;
  for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (I)gridDim.x * blockDim.x) {
    const I row = i / g.kh;
    const int ky = (int)(i - row * g.kh);
    const int ox = (int)(row % g.ow);
    const I t = row / g.ow;
    const int oy = (int)(t % g.oh), n = (int)(t / g.oh);
    const int y = oy * g.sy - g.pad + ky, x0 = ox * g.sx - g.pad;
    float* dst = col + i * run;
    if (y < 0 || y >= g.H) {
      for (int j = 0; j < run; ++j) dst[j] = 0.f;
      continue;
    }
    const float* src = in + (((I)n * g.H + y) * g.W + x0) * g.C;      // x0 may be negative: guarded below
    for (int kx = 0; kx < g.kw; ++kx) {
      const bool inside = x0 + kx >= 0 && x0 + kx < g.W;
      for (int c = 0; c < g.C; ++c) dst[kx * g.C + c] = inside ? src[kx * g.C + c] : 0.f;
    }
  }
}

// in_deltas[n, y, x, c] += sum over the windows (oy, ox, ky, kx) that cover (y, x)
template <typename I, int V>
__global__ void __launch_bounds__(256) col2im_add_kernel(const float* __restrict__ col, float* in_deltas, Geo g) {
  const I CV = g.C / V;
  const I KV = (I)g.kh * g.kw * CV;
  const I total = (I)g.N * g.H * g.W * CV;
  for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (I)gridDim.x * blockDim.x) {
    const int c = (int)(i % CV);
    I t = i / CV;
    const int x = (int)(t % g.W); t /= g.W;
    const int y = (int)(t % g.H), n = (int)(t / g.H);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int ky = 0; ky < g.kh; ++ky) {
      const int yy = y + g.pad - ky;
      if (yy < 0 || yy % g.sy) continue;
      const int oy = yy / g.sy;
      if (oy >= g.oh) continue;
      for (int kx = 0; kx < g.kw; ++kx) {
        const int xx = x + g.pad - kx;
        if (xx < 0 || xx % g.sx) continue;
        const int ox = xx / g.sx;
        if (ox >= g.ow) continue;
        float v[V];
        load_v<V>(col + ((((I)n * g.oh + oy) * g.ow + ox) * KV + ((I)ky * g.kw + kx) * CV + c) * V, v);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += v[j];
      }
    }
    float d[V];
    load_v<V>(in_deltas + i * V, d);
#pragma unroll
    for (int j = 0; j < V; ++j) d[j] = __fadd_rn(d[j], acc[j]);
    store_v<V>(in_deltas + i * V, d);
  }
}

// mode 0: max pooling (writes argmax as a float index (y*W + x)*C + c, -1 and output 0 for
// an empty window); mode 1: average over the non-padding pixels of the window
template <typename I, int V>
__global__ void __launch_bounds__(256) pool_fwd_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                       float* __restrict__ argmax, Geo g, int mode) {
  const I CV = g.C / V;
  const I total = (I)g.N * g.oh * g.ow * CV;
  for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (I)gridDim.x * blockDim.x) {
    const int c = (int)(i % CV) * V;
    I t = i / CV;
    const int ox = (int)(t % g.ow); t /= g.ow;
    const int oy = (int)(t % g.oh), n = (int)(t / g.oh);
    const int y0 = max(oy * g.sy - g.pad, 0), y1 = min(oy * g.sy - g.pad + g.kh, g.H);
    const int x0 = max(ox * g.sx - g.pad, 0), x1 = min(ox * g.sx - g.pad + g.kw, g.W);
    const float* img = in + (I)n * g.H * g.W * g.C;
    float res[V];
    if (mode == 0) {
      float best[V], am[V];
      int idx[V];
#pragma unroll
      for (int j = 0; j < V; ++j) { best[j] = -3.402823466e+38f; idx[j] = -1; }
      for (int y = y0; y < y1; ++y)
        for (int x = x0; x < x1; ++x) {
          float v[V];
          const int at = (y * g.W + x) * g.C + c;
          load_v<V>(img + at, v);
#pragma unroll
          for (int j = 0; j < V; ++j)
            if (v[j] > best[j]) { best[j] = v[j]; idx[j] = at + j; }
        }
#pragma unroll
      for (int j = 0; j < V; ++j) { res[j] = idx[j] < 0 ? 0.f : best[j]; am[j] = (float)idx[j]; }
      store_v<V>(argmax + i * V, am);
    } else {
      float s[V];
#pragma unroll
      for (int j = 0; j < V; ++j) s[j] = 0.f;
      for (int y = y0; y < y1; ++y)
        for (int x = x0; x < x1; ++x) {
          float v[V];
          load_v<V>(img + (y * g.W + x) * g.C + c, v);
#pragma unroll
          for (int j = 0; j < V; ++j) s[j] += v[j];
        }
      const int cnt = max((y1 - y0) * (x1 - x0), 1);
#pragma unroll
      for (int j = 0; j < V; ++j) res[j] = __fdiv_rn(s[j], (float)cnt);
    }
    store_v<V>(out + i * V, res);
  }
}

// in_deltas[n, y, x, c] += contributions of every output window covering (y, x):
// max pooling: out_deltas where argmax points at this element; average pooling:
// out_deltas / (non-padding window size)
template <typename I, int V>
__global__ void __launch_bounds__(256) pool_bwd_kernel(const float* __restrict__ out_deltas,
                                                       const float* __restrict__ argmax, float* in_deltas,
                                                       Geo g, int mode) {
  const I CV = g.C / V;
  const I total = (I)g.N * g.H * g.W * CV;
  for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (I)gridDim.x * blockDim.x) {
    const int c = (int)(i % CV) * V;
    I t = i / CV;
    const int x = (int)(t % g.W); t /= g.W;
    const int y = (int)(t % g.H), n = (int)(t / g.H);
    const int me = (y * g.W + x) * g.C + c;
    // windows covering (y, x): oy*sy - pad <= y < oy*sy - pad + kh, likewise for x
    const int ny = y + g.pad - g.kh + 1, nx = x + g.pad - g.kw + 1;
    const int oy_lo = ny > 0 ? (ny + g.sy - 1) / g.sy : 0, oy_hi = min(g.oh - 1, (y + g.pad) / g.sy);
    const int ox_lo = nx > 0 ? (nx + g.sx - 1) / g.sx : 0, ox_hi = min(g.ow - 1, (x + g.pad) / g.sx);
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int oy = oy_lo; oy <= oy_hi; ++oy) {
      const int wy = oy * g.sy - g.pad;
      for (int ox = ox_lo; ox <= ox_hi; ++ox) {
        const int wx = ox * g.sx - g.pad;
        const I o = (((I)n * g.oh + oy) * g.ow + ox) * g.C + c;
        float od[V];
        load_v<V>(out_deltas + o, od);
        if (mode == 0) {
          float am[V];
          load_v<V>(argmax + o, am);
#pragma unroll
          for (int j = 0; j < V; ++j)
            if ((int)am[j] == me + j) acc[j] += od[j];
        } else {
          const int cnt = (min(wy + g.kh, g.H) - max(wy, 0)) * (min(wx + g.kw, g.W) - max(wx, 0));
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += __fdiv_rn(od[j], (float)cnt);
        }
      }
    }
    float d[V];
    load_v<V>(in_deltas + i * V, d);
#pragma unroll
    for (int j = 0; j < V; ++j) d[j] = __fadd_rn(d[j], acc[j]);
    store_v<V>(in_deltas + i * V, d);
  }
}

static int check_geo(const Geo& g) {
  B200_REQUIRE(g.N >= 0 && g.H > 0 && g.W > 0 && g.C > 0 && g.kh > 0 && g.kw > 0 && g.sy > 0 && g.sx > 0 &&
                   g.pad >= 0 && g.oh >= 0 && g.ow >= 0,
               "bad convolution / pooling geometry");
  B200_REQUIRE((int64_t)g.H * g.W * g.C < ((int64_t)1 << 24),
               "image too large for float-encoded argmax indices");
  return B200_OK;
}
// Picks the form of a kernel template K<index type, channels per thread>: `largest` is the largest element
// index any of its arrays sees, `vec` says whether 4 channels per thread are possible.
#define CONV_POOL_LAUNCH(KERNEL, work, largest, vec, ...)                                                  \
  do {                                                                                                   \
    const bool narrow_ = (largest) < ((int64_t)1 << 31) - ((int64_t)state().sm_count * 32 * 256);        \
    const unsigned grid_ = grid_for((vec) ? (work) / 4 : (work));                                        \
    if (narrow_ && (vec)) KERNEL<int, 4><<<grid_, 256, 0, state().stream>>>(__VA_ARGS__);                 \
    else if (narrow_) KERNEL<int, 1><<<grid_, 256, 0, state().stream>>>(__VA_ARGS__);                     \
    else if (vec) KERNEL<int64_t, 4><<<grid_, 256, 0, state().stream>>>(__VA_ARGS__);                     \
    else KERNEL<int64_t, 1><<<grid_, 256, 0, state().stream>>>(__VA_ARGS__);                              \
  } while (0)

static unsigned grid_for(int64_t total);
static inline bool vec4_ok(int C, const void* a, const void* b, const void* c = nullptr) {
  return C % 4 == 0 && aligned16(a) && aligned16(b) && (c == nullptr || aligned16(c));
}

static unsigned grid_for(int64_t total) {
  int64_t b = ceil_div(total, 256);
  const int64_t cap = (int64_t)state().sm_count * 32;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace b200

using namespace b200;

B200_API int b200_im2col(const float* inputs, float* col, int N, int H, int W, int C, int kh, int kw,
                         int pad, int sy, int sx, int oh, int ow) {
  if (int rc = require_ready()) return rc;
  Geo g{N, H, W, C, kh, kw, pad, sy, sx, oh, ow};
  if (int rc = check_geo(g)) return rc;
  const int64_t total = (int64_t)N * oh * ow * kh * kw * C;
  if (total == 0) return B200_OK;
  if (!vec4_ok(C, inputs, col)) {
    const int64_t work = (int64_t)N * oh * ow * kh;
    if (total + (int64_t)N * H * W * C < ((int64_t)1 << 31) - ((int64_t)state().sm_count * 32 * 256))
      im2col_rows_kernel<int><<<grid_for(work), 256, 0, state().stream>>>(inputs, col, g);
    else
      im2col_rows_kernel<int64_t><<<grid_for(work), 256, 0, state().stream>>>(inputs, col, g);
    B200_LAUNCH_CHECK();
    return B200_OK;
  }
  CONV_POOL_LAUNCH(im2col_kernel, total, total + (int64_t)N * H * W * C, true, inputs, col, g);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_col2im_add(const float* col, float* in_deltas, int N, int H, int W, int C, int kh, int kw,
                             int pad, int sy, int sx, int oh, int ow) {
  if (int rc = require_ready()) return rc;
  Geo g{N, H, W, C, kh, kw, pad, sy, sx, oh, ow};
  if (int rc = check_geo(g)) return rc;
  const int64_t total = (int64_t)N * H * W * C;
  if (total == 0) return B200_OK;
  CONV_POOL_LAUNCH(col2im_add_kernel, total, total + (int64_t)N * oh * ow * kh * kw * C, vec4_ok(C, col, in_deltas), col, in_deltas, g);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_pool2d_forward(int mode, const float* inputs, float* outputs, float* argmax, int N, int H,
                                 int W, int C, int kh, int kw, int pad, int sy, int sx, int oh, int ow) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(mode == 0 || mode == 1, "mode must be 0 (max) or 1 (average)");
  B200_REQUIRE(mode == 1 || argmax != nullptr, "max pooling needs an argmax array");
  Geo g{N, H, W, C, kh, kw, pad, sy, sx, oh, ow};
  if (int rc = check_geo(g)) return rc;
  const int64_t total = (int64_t)N * oh * ow * C;
  if (total == 0) return B200_OK;
  CONV_POOL_LAUNCH(pool_fwd_kernel, total, (int64_t)N * H * W * C + total, vec4_ok(C, inputs, outputs, argmax), inputs, outputs,
                   argmax, g, mode);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

B200_API int b200_pool2d_backward(int mode, const float* out_deltas, const float* argmax, float* in_deltas,
                                  int N, int H, int W, int C, int kh, int kw, int pad, int sy, int sx,
                                  int oh, int ow) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(mode == 0 || mode == 1, "mode must be 0 (max) or 1 (average)");
  B200_REQUIRE(mode == 1 || argmax != nullptr, "max pooling needs an argmax array");
  Geo g{N, H, W, C, kh, kw, pad, sy, sx, oh, ow};
  if (int rc = check_geo(g)) return rc;
  const int64_t total = (int64_t)N * H * W * C;
  if (total == 0) return B200_OK;
  CONV_POOL_LAUNCH(pool_bwd_kernel, total, total + (int64_t)N * oh * ow * C, vec4_ok(C, out_deltas, in_deltas, argmax), out_deltas,
                   argmax, in_deltas, g, mode);
  B200_LAUNCH_CHECK();
  return B200_OK;
}
