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

// col[(n, oy, ox), (ky, kx, c)] = in[n, oy*sy - pad + ky, ox*sx - pad + kx, c] or 0
__global__ void __launch_bounds__(256) im2col_kernel(const float* __restrict__ in, float* __restrict__ col, Geo g) {
  const int64_t K = (int64_t)g.kh * g.kw * g.C;
  const int64_t total = (int64_t)g.N * g.oh * g.ow * K;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / K;
    int64_t k = i - row * K;
    const int c = (int)(k % g.C); k /= g.C;
    const int kx = (int)(k % g.kw), ky = (int)(k / g.kw);
    const int ox = (int)(row % g.ow);
    const int64_t t = row / g.ow;
    const int oy = (int)(t % g.oh), n = (int)(t / g.oh);
    const int y = oy * g.sy - g.pad + ky, x = ox * g.sx - g.pad + kx;
    col[i] = (y >= 0 && y < g.H && x >= 0 && x < g.W)
                 ? in[(((int64_t)n * g.H + y) * g.W + x) * g.C + c] : 0.f;
  }
}

// in_deltas[n, y, x, c] += sum over the windows (oy, ox, ky, kx) that cover (y, x)
__global__ void __launch_bounds__(256) col2im_add_kernel(const float* __restrict__ col, float* in_deltas, Geo g) {
  const int64_t K = (int64_t)g.kh * g.kw * g.C;
  const int64_t total = (int64_t)g.N * g.H * g.W * g.C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % g.C);
    int64_t t = i / g.C;
    const int x = (int)(t % g.W); t /= g.W;
    const int y = (int)(t % g.H), n = (int)(t / g.H);
    float acc = 0.f;
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
        acc += col[(((int64_t)n * g.oh + oy) * g.ow + ox) * K + ((int64_t)ky * g.kw + kx) * g.C + c];
      }
    }
    in_deltas[i] = __fadd_rn(in_deltas[i], acc);
  }
}

// mode 0: max pooling (writes argmax as a float index (y*W + x)*C + c, -1 and output 0 for
// an empty window); mode 1: average over the non-padding pixels of the window
__global__ void __launch_bounds__(256) pool_fwd_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                       float* __restrict__ argmax, Geo g, int mode) {
  const int64_t total = (int64_t)g.N * g.oh * g.ow * g.C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % g.C);
    int64_t t = i / g.C;
    const int ox = (int)(t % g.ow); t /= g.ow;
    const int oy = (int)(t % g.oh), n = (int)(t / g.oh);
    const int y0 = max(oy * g.sy - g.pad, 0), y1 = min(oy * g.sy - g.pad + g.kh, g.H);
    const int x0 = max(ox * g.sx - g.pad, 0), x1 = min(ox * g.sx - g.pad + g.kw, g.W);
    const float* img = in + (int64_t)n * g.H * g.W * g.C;
    if (mode == 0) {
      float best = -3.402823466e+38f;
      int idx = -1;
      for (int y = y0; y < y1; ++y)
        for (int x = x0; x < x1; ++x) {
          const float v = img[((int64_t)y * g.W + x) * g.C + c];
          if (v > best) { best = v; idx = (y * g.W + x) * g.C + c; }
        }
      out[i] = idx < 0 ? 0.f : best;
      argmax[i] = (float)idx;
    } else {
      float s = 0.f;
      for (int y = y0; y < y1; ++y)
        for (int x = x0; x < x1; ++x) s += img[((int64_t)y * g.W + x) * g.C + c];
      const int cnt = max((y1 - y0) * (x1 - x0), 1);
      out[i] = __fdiv_rn(s, (float)cnt);
    }
  }
}

// in_deltas[n, y, x, c] += contributions of every output window covering (y, x):
// max pooling: out_deltas where argmax points at this element; average pooling:
// out_deltas / (non-padding window size)
__global__ void __launch_bounds__(256) pool_bwd_kernel(const float* __restrict__ out_deltas,
                                                       const float* __restrict__ argmax, float* in_deltas,
                                                       Geo g, int mode) {
  const int64_t total = (int64_t)g.N * g.H * g.W * g.C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % g.C);
    int64_t t = i / g.C;
    const int x = (int)(t % g.W); t /= g.W;
    const int y = (int)(t % g.H), n = (int)(t / g.H);
    const int me = (y * g.W + x) * g.C + c;
    // windows covering (y, x): oy*sy - pad <= y < oy*sy - pad + kh, likewise for x
    const int ny = y + g.pad - g.kh + 1, nx = x + g.pad - g.kw + 1;
    const int oy_lo = ny > 0 ? (ny + g.sy - 1) / g.sy : 0, oy_hi = min(g.oh - 1, (y + g.pad) / g.sy);
    const int ox_lo = nx > 0 ? (nx + g.sx - 1) / g.sx : 0, ox_hi = min(g.ow - 1, (x + g.pad) / g.sx);
    float acc = 0.f;
    for (int oy = oy_lo; oy <= oy_hi; ++oy) {
      const int wy = oy * g.sy - g.pad;
      for (int ox = ox_lo; ox <= ox_hi; ++ox) {
        const int wx = ox * g.sx - g.pad;
        const int64_t o = (((int64_t)n * g.oh + oy) * g.ow + ox) * g.C + c;
        if (mode == 0) {
          if ((int)argmax[o] == me) acc += out_deltas[o];
        } else {
          const int cnt = (min(wy + g.kh, g.H) - max(wy, 0)) * (min(wx + g.kw, g.W) - max(wx, 0));
          acc += __fdiv_rn(out_deltas[o], (float)cnt);
        }
      }
    }
    in_deltas[i] = __fadd_rn(in_deltas[i], acc);
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
  im2col_kernel<<<grid_for(total), 256, 0, state().stream>>>(inputs, col, g);
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
  col2im_add_kernel<<<grid_for(total), 256, 0, state().stream>>>(col, in_deltas, g);
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
  pool_fwd_kernel<<<grid_for(total), 256, 0, state().stream>>>(inputs, outputs, argmax, g, mode);
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
  pool_bwd_kernel<<<grid_for(total), 256, 0, state().stream>>>(out_deltas, argmax, in_deltas, g, mode);
  B200_LAUNCH_CHECK();
  return B200_OK;
}
