// Placeholder until the tcgen05 kernel lands: reports "unsupported" so that the
// dispatcher uses the CUDA-core kernel.
#include "common.cuh"
namespace b200 {
int gemm_tc(int, int, int64_t, int64_t, int64_t, const float*, int64_t, const float*, int64_t, float*,
            int64_t, int) {
  return B200_ERR_UNSUPPORTED;
}
}  // namespace b200
