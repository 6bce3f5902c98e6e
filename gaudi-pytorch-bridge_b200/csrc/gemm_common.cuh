// Argument block and epilogue shared by the GEMM kernels.
#pragma once

#include "common.cuh"

namespace b200q {

struct GemmParams {
  const void* A;
  const void* B;
  int a_dtype, b_dtype, trans_a, trans_b;
  int64_t M, N, K, lda, ldb;
  int64_t batch, a_batch_stride, b_batch_stride, out_batch_stride;
  void* out;
  int out_dtype;
  int64_t ldo;
  const float* a_scale;
  float a_scale_host;
  int a_scale_mode;
  const float* b_scale;
  float b_scale_host;
  int b_scale_mode;
  const void* bias;
  int bias_dtype, bias_mode;
  int64_t bias_ld, bias_batch_stride;
  const void* D;
  int d_dtype;
  int64_t ldd, d_batch_stride;
};

__device__ __forceinline__ float bcast_scale(const float* dev, float host, int mode, int64_t m, int64_t n, int64_t N) {
  switch (mode) {
    case B200Q_BCAST_SCALAR_HOST: return host;
    case B200Q_BCAST_SCALAR_DEV: return __ldg(dev);
    case B200Q_BCAST_PER_COL: return __ldg(dev + n);
    case B200Q_BCAST_PER_ROW: return __ldg(dev + m);
    case B200Q_BCAST_FULL: return __ldg(dev + m * N + n);
    default: return 1.f;
  }
}

__device__ __forceinline__ float ld_out_typed(const void* base, int dtype, int64_t idx) {
  return dtype == B200Q_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx])
                             : static_cast<const float*>(base)[idx];
}

// out = ((acc * sa) * sb) + bias + D, rounded once to the output dtype.
__device__ __forceinline__ float epilogue_value(const GemmParams& p, int64_t b, int64_t m, int64_t n, float acc) {
  float v = acc;
  if (p.a_scale_mode != B200Q_BCAST_NONE) v *= bcast_scale(p.a_scale, p.a_scale_host, p.a_scale_mode, m, n, p.N);
  if (p.b_scale_mode != B200Q_BCAST_NONE) v *= bcast_scale(p.b_scale, p.b_scale_host, p.b_scale_mode, m, n, p.N);
  if (p.bias_mode != B200Q_BCAST_NONE) {
    int64_t idx = p.bias_mode == B200Q_BCAST_PER_COL   ? n
                  : p.bias_mode == B200Q_BCAST_PER_ROW ? m
                  : p.bias_mode == B200Q_BCAST_FULL    ? b * p.bias_batch_stride + m * p.bias_ld + n
                                                       : 0;
    v += ld_out_typed(p.bias, p.bias_dtype, idx);
  }
  if (p.D) v += ld_out_typed(p.D, p.d_dtype, b * p.d_batch_stride + m * p.ldd + n);
  return v;
}

__device__ __forceinline__ void epilogue_store_one(const GemmParams& p, int64_t b, int64_t m, int64_t n, float acc) {
  float v = epilogue_value(p, b, m, n, acc);
  int64_t idx = b * p.out_batch_stride + m * p.ldo + n;
  if (p.out_dtype == B200Q_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(v);
  else static_cast<float*>(p.out)[idx] = v;
}

int gemm_generic_launch(const GemmParams& p, cudaStream_t st);
int gemm_tcgen05_launch(const GemmParams& p, cudaStream_t st);  // returns B200Q_ERR_UNSUPPORTED if not eligible

}  // namespace b200q
