// dot_mm / dot_add_mm entry points: argument checks and the choice between the
// tensor-core kernel (tcgen05, TMA-fed, 3xTF32 split) and the CUDA-core kernel.
#include "common.cuh"

namespace b200 {
int gemm_simt(int transa, int transb, int64_t M, int64_t N, int64_t K, const float* a, int64_t lda,
              const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate);
// Returns B200_ERR_UNSUPPORTED (without launching) when the operands do not meet
// the tensor-core kernel's layout rules.
int gemm_tc(int transa, int transb, int64_t M, int64_t N, int64_t K, const float* a, int64_t lda,
            const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate);

static int gemm_dispatch(const float* a, const float* b, float* out, int64_t M, int64_t N, int64_t K,
                         int64_t lda, int64_t ldb, int64_t ldo, int transa, int transb,
                         int accumulate) {
  if (int rc = require_ready()) return rc;
  B200_REQUIRE(M >= 0 && N >= 0 && K >= 0, "negative extent");
  if (M * N == 0) return B200_OK;
  B200_REQUIRE(out != nullptr && ldo >= N, "bad output operand");
  if (K == 0) {  // empty contraction: a zero matrix
    if (!accumulate)
      B200_CUDA(cudaMemset2DAsync(out, ldo * sizeof(float), 0, N * sizeof(float), M, state().stream));
    return B200_OK;
  }
  B200_REQUIRE(a != nullptr && b != nullptr, "NULL operand");
  B200_REQUIRE(lda >= (transa ? M : K) && ldb >= (transb ? K : N), "leading dimension too small");
  B200_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "extent exceeds 2^31");
  const int path = state().gemm_path;
  if (path != 1) {
    const int rc = gemm_tc(transa, transb, M, N, K, a, lda, b, ldb, out, ldo, accumulate);
    if (rc != B200_ERR_UNSUPPORTED) return rc;
    B200_REQUIRE(path != 2, "tensor-core GEMM forced but operands are not eligible: %s",
                 "see b200_last_error of the probe");
  }
  return gemm_simt(transa, transb, M, N, K, a, lda, b, ldb, out, ldo, accumulate);
}
}  // namespace b200

using namespace b200;

B200_API int b200_dot_mm(const float* a, const float* b, float* out, int64_t M, int64_t N, int64_t K,
                         int64_t lda, int64_t ldb, int64_t ldo, int transa, int transb) {
  return gemm_dispatch(a, b, out, M, N, K, lda, ldb, ldo, transa, transb, 0);
}

B200_API int b200_dot_add_mm(const float* a, const float* b, float* out, int64_t M, int64_t N,
                             int64_t K, int64_t lda, int64_t ldb, int64_t ldo, int transa,
                             int transb) {
  return gemm_dispatch(a, b, out, M, N, K, lda, ldb, ldo, transa, transb, 1);
}
