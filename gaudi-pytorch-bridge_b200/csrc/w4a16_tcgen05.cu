// W4A16 GEMM (placeholder until the fused kernel lands in this file).
#include "common.cuh"

namespace b200q {
int w4a16_gemm_impl(const void*, int64_t, const int32_t*, const void*, const int32_t*, int, int, int64_t, int64_t,
                    int64_t, int64_t, void*, int, int64_t, cudaStream_t) {
  return B200Q_ERR_UNSUPPORTED;
}
}  // namespace b200q
