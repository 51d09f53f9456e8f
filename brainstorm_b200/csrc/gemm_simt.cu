// Plain fp32 FMA GEMM on the CUDA cores: out (+)= op(a) . op(b) for any transpose
// combination, any leading dimensions and any alignment.  It is the exact-fp32
// companion of the tensor-core kernel: used for operands that the tensor-core
// path cannot take (tiny or oddly shaped problems) and as the in-library
// cross-check of that kernel.
#include "common.cuh"

namespace b200 {

constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 16;

// A(m, k) = a[m * sam + k * sak];  B(k, n) = b[k * sbk + n * sbn]
template <bool A_KFAST, bool B_NFAST>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const float* a, const float* b, float* c, int M, int N, int K, int64_t sam,
                 int64_t sak, int64_t sbk, int64_t sbn, int64_t ldc, int accumulate) {
  __shared__ float As[SG_BK][SG_BM + 4];
  __shared__ float Bs[SG_BK][SG_BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += SG_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;  // 0..1023
      int mm, kk;
      if (A_KFAST) { kk = idx & 15; mm = idx >> 4; } else { mm = idx & 63; kk = idx >> 6; }
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? a[gm * sam + gk * sak] : 0.f;
      int nn, kb;
      if (B_NFAST) { nn = idx & 63; kb = idx >> 6; } else { kb = idx & 15; nn = idx >> 4; }
      const int gn = n0 + nn, gkb = k0 + kb;
      Bs[kb][nn] = (gn < N && gkb < K) ? b[gkb * sbk + gn * sbn] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SG_BK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float* p = c + (int64_t)gm * ldc + gn;
      *p = accumulate ? __fadd_rn(*p, acc[i][j]) : acc[i][j];
    }
  }
}

int gemm_simt(int transa, int transb, int64_t M, int64_t N, int64_t K, const float* a, int64_t lda,
              const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate) {
  const State& s = state();
  dim3 grid((unsigned)ceil_div(N, SG_BN), (unsigned)ceil_div(M, SG_BM));
  const int64_t sam = transa ? 1 : lda, sak = transa ? lda : 1;
  const int64_t sbk = transb ? 1 : ldb, sbn = transb ? ldb : 1;
  const int m = (int)M, n = (int)N, k = (int)K;
  if (!transa && !transb)
    gemm_simt_kernel<true, true><<<grid, 256, 0, s.stream>>>(a, b, c, m, n, k, sam, sak, sbk, sbn, ldc, accumulate);
  else if (!transa && transb)
    gemm_simt_kernel<true, false><<<grid, 256, 0, s.stream>>>(a, b, c, m, n, k, sam, sak, sbk, sbn, ldc, accumulate);
  else if (transa && !transb)
    gemm_simt_kernel<false, true><<<grid, 256, 0, s.stream>>>(a, b, c, m, n, k, sam, sak, sbk, sbn, ldc, accumulate);
  else
    gemm_simt_kernel<false, false><<<grid, 256, 0, s.stream>>>(a, b, c, m, n, k, sam, sak, sbk, sbn, ldc, accumulate);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

}  // namespace b200
