// Counter-based random numbers for the handler: Philox4x32-10 (Salmon et al.,
// "Parallel random numbers: as easy as 1, 2, 3", SC'11) keyed by a 64-bit seed
// and indexed by (call offset, element group), so a mask is reproducible from
// (seed, offset) alone and needs no generator state in memory.  HBM-write bound.
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

__device__ __forceinline__ float u01(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }

// mode 0: out = (u < p0) ? 1 : 0   mode 1: out = p0 + p1 * normal
__global__ void __launch_bounds__(256)
rng_kernel(float* out, int64_t n, float p0, float p1, uint64_t seed, uint64_t offset, int mode,
           const uint64_t* __restrict__ replay_epoch) {
  // Inside a recorded graph the arguments are frozen; the replay counter (upper half of
  // the call offset, which counts calls and stays far below 2^32) makes every replay a new stream.
  if (replay_epoch) offset += *replay_epoch << 32;
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  const int64_t groups = (n + 3) >> 2;
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups;
       g += (int64_t)gridDim.x * blockDim.x) {
    const uint4 r = philox4x32_10(
        make_uint4((uint32_t)g, (uint32_t)((uint64_t)g >> 32), (uint32_t)offset, (uint32_t)(offset >> 32)), key);
    float v[4];
    if (mode == 0) {
      v[0] = u01(r.x) < p0 ? 1.f : 0.f;
      v[1] = u01(r.y) < p0 ? 1.f : 0.f;
      v[2] = u01(r.z) < p0 ? 1.f : 0.f;
      v[3] = u01(r.w) < p0 ? 1.f : 0.f;
    } else {
      // Box-Muller on (0, 1] x [0, 1)
      const float a0 = sqrtf(-2.0f * logf(1.0f - u01(r.x))), a1 = sqrtf(-2.0f * logf(1.0f - u01(r.z)));
      float s0, c0, s1, c1;
      sincospif(2.0f * u01(r.y), &s0, &c0);
      sincospif(2.0f * u01(r.w), &s1, &c1);
      v[0] = p0 + p1 * a0 * c0; v[1] = p0 + p1 * a0 * s0;
      v[2] = p0 + p1 * a1 * c1; v[3] = p0 + p1 * a1 * s1;
    }
    const int64_t base = g << 2;
    if (base + 3 < n && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
      *reinterpret_cast<float4*>(out + base) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      for (int k = 0; k < 4 && base + k < n; ++k) out[base + k] = v[k];
    }
  }
}

static int launch_rng(float* out, int64_t n, float p0, float p1, uint64_t seed, uint64_t offset, int mode) {
  if (int rc = require_ready()) return rc;
  if (n <= 0) return B200_OK;
  B200_REQUIRE(out != nullptr, "NULL operand");
  const State& s = state();
  int64_t blocks = ceil_div(ceil_div(n, 4), 256);
  if (blocks > (int64_t)s.sm_count * 8) blocks = (int64_t)s.sm_count * 8;
  rng_kernel<<<(unsigned)blocks, 256, 0, s.stream>>>(out, n, p0, p1, seed, offset, mode,
                                                     s.capturing ? s.replay_epoch : nullptr);
  B200_LAUNCH_CHECK();
  return B200_OK;
}
}  // namespace b200

using namespace b200;

B200_API int b200_generate_probability_mask(float* mask, int64_t n, float probability, uint64_t seed,
                                            uint64_t offset) {
  return launch_rng(mask, n, probability, 0.f, seed, offset, 0);
}

B200_API int b200_fill_gaussian(float mean, float std, float* out, int64_t n, uint64_t seed,
                                uint64_t offset) {
  return launch_rng(out, n, mean, std, seed, offset, 1);
}
