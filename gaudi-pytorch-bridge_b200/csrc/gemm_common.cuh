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
  // fused output cast: 0 = none, else B200Q_E4M3 / B200Q_E5M2: the result is rounded to out_dtype
  // (as the unfused GEMM would store it), multiplied by the output scale in out_dtype and
  // rounded to fp8 -- the composition cast_to_fp8_v2(fp8_gemm_v2(...), scale) bit for bit
  int out8_dtype;
  const float* out8_scale;  // device scalar, or null: out8_scale_host
  float out8_scale_host;
  // fused SwiGLU (needs out8_dtype = E4M3): B holds gate and up weights interleaved in blocks of
  // 128 rows (rows [256 b, 256 b + 128) gate, the next 128 up, both of hidden units
  // [128 b, 128 b + 128)); `out` receives e4m3 [M][N / 2]:
  //   cast(bf16(silu(gate) * up), out8 scale)  with gate / up rounded to out_dtype first,
  // the bytes of fp8_gemm_v2 followed by the SwiGLU + cast kernel
  int swiglu;
  // Routed output (route_count > 0; bf16 results of the CTA-pair kernel only): block
  // i = m / route_rows of the token rows goes to buffer route_out[i] -- which may be memory of
  // another GPU mapped into this process -- at row route_row_offset + m % route_rows.  The
  // row-parallel projection of a tensor-parallel layer uses it to deliver each partial-sum block
  // straight to the rank that reduces it.
  void* route_out[8];
  int route_count;
  int64_t route_rows, route_row_offset;
  float* out8_amax;  // fused output cast only: max |fp8 value written| (atomic max on the bit pattern), or null
  int b_static;      // B is not written by work still in flight: it may be read before the preceding kernel completes
};

// value in out_dtype -> fp8 byte of the fused output cast
__device__ __forceinline__ uint32_t out8_byte(const GemmParams& p, float v, float s) {
  float t, y;
  if (p.out_dtype == B200Q_BF16) {
    t = round_to_bf16(v);
    y = round_to_bf16(t * round_to_bf16(s));
  } else {
    t = v;
    y = t * s;
  }
  uint32_t b = p.out8_dtype == B200Q_E4M3 ? (cvt_fp8x2<B200Q_E4M3>(y, 0.f) & 0xFFu) : (cvt_fp8x2<B200Q_E5M2>(y, 0.f) & 0xFFu);
  if (y != y) b = 0x7Fu;
  return b;
}
__device__ __forceinline__ float out8_scale_value(const GemmParams& p) {
  return p.out8_scale ? __ldg(p.out8_scale) : p.out8_scale_host;
}

// magnitude code (fp8 byte without its sign) -> the running maximum of |out|; codes order like the
// magnitudes they stand for, and the all-ones code is NaN (e4m3) or NaN / above inf (e5m2)
__device__ __forceinline__ void out8_amax_update(const GemmParams& p, uint32_t code) {
  const float mag = p.out8_dtype == B200Q_E4M3 ? fp8_to_float<B200Q_E4M3>(code) : fp8_to_float<B200Q_E5M2>(code);
  atomicMax(reinterpret_cast<unsigned int*>(p.out8_amax), __float_as_uint(mag));
}

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

// out = ((acc * sa) * sb) + bias + D, rounded once to the output dtype; the fetch of an
// element's operands (epi_load) is separate from their application (epi_apply).
struct EpiOperands {
  float sa, sb, bias, d;
};

__device__ __forceinline__ EpiOperands epi_load(const GemmParams& p, int64_t b, int64_t m, int64_t n) {
  EpiOperands o;
  o.sa = p.a_scale_mode != B200Q_BCAST_NONE ? bcast_scale(p.a_scale, p.a_scale_host, p.a_scale_mode, m, n, p.N) : 1.f;
  o.sb = p.b_scale_mode != B200Q_BCAST_NONE ? bcast_scale(p.b_scale, p.b_scale_host, p.b_scale_mode, m, n, p.N) : 1.f;
  o.bias = 0.f;
  if (p.bias_mode != B200Q_BCAST_NONE) {
    int64_t idx = p.bias_mode == B200Q_BCAST_PER_COL   ? n
                  : p.bias_mode == B200Q_BCAST_PER_ROW ? m
                  : p.bias_mode == B200Q_BCAST_FULL    ? b * p.bias_batch_stride + m * p.bias_ld + n
                                                       : 0;
    o.bias = ld_out_typed(p.bias, p.bias_dtype, idx);
  }
  o.d = p.D ? ld_out_typed(p.D, p.d_dtype, b * p.d_batch_stride + m * p.ldd + n) : 0.f;
  return o;
}

__device__ __forceinline__ float epi_apply(const GemmParams& p, float acc, const EpiOperands& o) {
  float v = acc;
  if (p.a_scale_mode != B200Q_BCAST_NONE) v *= o.sa;
  if (p.b_scale_mode != B200Q_BCAST_NONE) v *= o.sb;
  if (p.bias_mode != B200Q_BCAST_NONE) v += o.bias;
  if (p.D) v += o.d;
  return v;
}

__device__ __forceinline__ float epilogue_value(const GemmParams& p, int64_t b, int64_t m, int64_t n, float acc) {
  return epi_apply(p, acc, epi_load(p, b, m, n));
}

// v = the value before the rounding to the output dtype; s8 = out8_scale_value(p) (read by the caller:
// once per thread, not once per element)
__device__ __forceinline__ void epilogue_store_value(const GemmParams& p, int64_t b, int64_t m, int64_t n, float v, float s8) {
  int64_t idx = b * p.out_batch_stride + m * p.ldo + n;
  if (p.out8_dtype) {
    const uint32_t byte = out8_byte(p, v, s8);
    static_cast<uint8_t*>(p.out)[idx] = (uint8_t)byte;
    if (p.out8_amax) out8_amax_update(p, byte & 0x7Fu);
    return;
  }
  if (p.out_dtype == B200Q_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(v);
  else static_cast<float*>(p.out)[idx] = v;
}

__device__ __forceinline__ void epilogue_store_one(const GemmParams& p, int64_t b, int64_t m, int64_t n, float acc) {
  epilogue_store_value(p, b, m, n, epilogue_value(p, b, m, n, acc), p.out8_dtype ? out8_scale_value(p) : 1.f);
}

int gemm_generic_launch(const GemmParams& p, cudaStream_t st);
int gemm_tcgen05_launch(const GemmParams& p, cudaStream_t st);  // returns B200Q_ERR_UNSUPPORTED if not eligible

}  // namespace b200q
