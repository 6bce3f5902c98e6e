// Generic CUDA-core FP8 GEMM: the path for operand layouts, ranks and sizes that the
// tcgen05 kernel does not take (MN-major operands, K not a multiple of 16, unaligned
// bases, tiny problems).  Correct for every argument combination of b200q_fp8_gemm;
// shared-memory tiled, fp32 accumulation, same epilogue order as the fast path.
#include "common.cuh"
#include "gemm_common.cuh"

namespace b200q {

constexpr int GT = 32;   // output tile edge
constexpr int GK = 32;   // k step

__device__ __forceinline__ float ld_fp8(const uint8_t* p, int fmt) {
  return fmt == B200Q_E4M3 ? fp8_to_float<B200Q_E4M3>(*p) : fp8_to_float<B200Q_E5M2>(*p);
}

__global__ void __launch_bounds__(256) gemm_generic_kernel(GemmParams p) {
  __shared__ float sA[GK][GT + 1];  // [k][m]
  __shared__ float sB[GK][GT + 1];  // [k][n]
  const int64_t b = blockIdx.z;
  const uint8_t* A = static_cast<const uint8_t*>(p.A) + b * p.a_batch_stride;
  const uint8_t* B = static_cast<const uint8_t*>(p.B) + b * p.b_batch_stride;
  const int64_t m0 = (int64_t)blockIdx.y * GT, n0 = (int64_t)blockIdx.x * GT;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (int64_t k0 = 0; k0 < p.K; k0 += GK) {
    for (int i = threadIdx.x; i < GT * GK; i += 256) {
      // A tile: walk the contiguous dimension of the stored matrix with consecutive threads
      int mi = p.trans_a ? (i % GT) : (i / GK), ki = p.trans_a ? (i / GT) : (i % GK);
      int64_t m = m0 + mi, k = k0 + ki;
      float v = 0.f;
      if (m < p.M && k < p.K) v = ld_fp8(A + (p.trans_a ? k * p.lda + m : m * p.lda + k), p.a_dtype);
      sA[ki][mi] = v;
      int ni = p.trans_b ? (i / GK) : (i % GT), kj = p.trans_b ? (i % GK) : (i / GT);
      int64_t n = n0 + ni, kk = k0 + kj;
      float w = 0.f;
      if (n < p.N && kk < p.K) w = ld_fp8(B + (p.trans_b ? n * p.ldb + kk : kk * p.ldb + n), p.b_dtype);
      sB[kj][ni] = w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a0 = sA[k][ty], a1 = sA[k][ty + 16], b0 = sB[k][tx], b1 = sB[k][tx + 16];
      acc[0][0] = fmaf(a0, b0, acc[0][0]); acc[0][1] = fmaf(a0, b1, acc[0][1]);
      acc[1][0] = fmaf(a1, b0, acc[1][0]); acc[1][1] = fmaf(a1, b1, acc[1][1]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      int64_t m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
      if (m < p.M && n < p.N) epilogue_store_one(p, b, m, n, acc[i][j]);
    }
}

int gemm_generic_launch(const GemmParams& p, cudaStream_t st) {
  if (p.swiglu) return B200Q_ERR_UNSUPPORTED;  // the fused SwiGLU epilogue exists in the CTA-pair kernel only
  if (p.M == 0 || p.N == 0 || p.batch == 0) return B200Q_OK;
  dim3 grid((unsigned)((p.N + GT - 1) / GT), (unsigned)((p.M + GT - 1) / GT), (unsigned)p.batch);
  if (grid.y > 65535u || grid.z > 65535u) return B200Q_ERR_TOO_LARGE;
  gemm_generic_kernel<<<grid, 256, 0, st>>>(p);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // namespace b200q
