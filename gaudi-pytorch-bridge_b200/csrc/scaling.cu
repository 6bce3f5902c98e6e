// FP8 scale management around the casts: amax of a tensor without casting it, the scale that
// an amax implies, and the amax-history step of delayed scaling.  All three keep their state on
// the device (no host read of the amax), so a "current scaling" cast is three launches on one
// stream: amax -> scale -> cast with a device scalar scale.
//
// Follows the host-side composition the reference builds from ATen ops for its FP8 optimizer
// state (habana_kernels/lazy_optimizer_kernels.cpp:113-126, CastMomentToFp8WithScale):
//   amax  = max(abs(x));  exp = floor(log2(fp8_max / amax));  sf = 2^exp
//   scale = where(amax > 0, sf, scale)
//   cast_to_fp8_v2(x, scale, stochastic_rounding=true, is_amax=false, dtype, scale_shape={1})
#include "common.cuh"

namespace b200q {

// ---------------------------------------------------------------------------- amax only
// 2 (bf16) or 4 (fp32) bytes read per element, nothing written but one word: HBM-bound.
template <typename InT>
__global__ void __launch_bounds__(256, 8) amax_kernel(const InT* __restrict__ in, int64_t n, float* amax) {
  pdl_release();
  constexpr int kPer16 = 16 / sizeof(InT);  // elements per 16-byte load
  const int64_t nvec = n / kPer16;
  const uint4* v = reinterpret_cast<const uint4*>(in);
  uint32_t bits = 0;   // fp32: |x| bit pattern;  bf16: two running maxima packed as bf16x2
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  auto fold = [&](const uint4& w) {
    if (sizeof(InT) == 2) {
      // unsigned 16-bit maxima of the two halves: for non-negative bf16 patterns the integer
      // order is the value order and NaN patterns (> 0x7F80) win, as torch.max propagates NaN
      const uint32_t a = __vmaxu2(w.x & 0x7FFF7FFFu, w.y & 0x7FFF7FFFu), b = __vmaxu2(w.z & 0x7FFF7FFFu, w.w & 0x7FFF7FFFu);
      bits = __vmaxu2(bits, __vmaxu2(a, b));
    } else {
      bits = max(bits, max(max(w.x & 0x7FFFFFFFu, w.y & 0x7FFFFFFFu), max(w.z & 0x7FFFFFFFu, w.w & 0x7FFFFFFFu)));
    }
  };
  // four independent 16-byte loads in flight per thread, 2048 threads per SM
#pragma unroll 1
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    const uint4 w0 = __ldcs(v + i), w1 = __ldcs(v + i + stride), w2 = __ldcs(v + i + 2 * stride), w3 = __ldcs(v + i + 3 * stride);
    fold(w0); fold(w1); fold(w2); fold(w3);
  }
  for (; i < nvec; i += stride) fold(__ldcs(v + i));
  uint32_t fbits = sizeof(InT) == 2 ? max(bits << 16, bits & 0xFFFF0000u) : bits;
  // ragged tail (fewer than 16 bytes): first threads of block 0
  if (blockIdx.x == 0) {
    const int64_t t = nvec * kPer16 + threadIdx.x;
    if (t < n) {
      const float x = sizeof(InT) == 2 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(in)[t])
                                       : reinterpret_cast<const float*>(in)[t];
      fbits = max(fbits, __float_as_uint(x) & 0x7FFFFFFFu);
    }
  }
  block_amax_to_global(fbits, amax);
}

int amax_impl(const void* in, int in_dtype, int64_t n, float* amax, cudaStream_t st) {
  if (!amax || n < 0 || (n > 0 && !in)) return B200Q_ERR_BAD_ARGUMENT;
  if (in_dtype != B200Q_BF16 && in_dtype != B200Q_F32) return B200Q_ERR_BAD_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(in) & 15) return B200Q_ERR_UNSUPPORTED;
  if (int rc = clear_amax(amax, st)) return rc;
  if (n == 0) return B200Q_OK;
  const int64_t nvec = n / (in_dtype == B200Q_BF16 ? 8 : 4);
  int64_t blocks = (nvec + 256 * 4 - 1) / (256 * 4);
  if (blocks < 1) blocks = 1;
  if (blocks > kNumSMs * 16) blocks = kNumSMs * 16;  // two rounds of 8 resident blocks per SM
  // (the pass starts under the clearing kernel and waits for it only before its atomicMax)
  const dim3 grid((unsigned)blocks), block(256);
  if (in_dtype == B200Q_BF16) {
    if (launch_overlapped(amax_kernel<__nv_bfloat16>, grid, block, 0, st, static_cast<const __nv_bfloat16*>(in), n, amax) != cudaSuccess) {
      (void)cudaGetLastError();
      amax_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16*>(in), n, amax);
    }
  } else {
    if (launch_overlapped(amax_kernel<float>, grid, block, 0, st, static_cast<const float*>(in), n, amax) != cudaSuccess) {
      (void)cudaGetLastError();
      amax_kernel<float><<<grid, block, 0, st>>>(static_cast<const float*>(in), n, amax);
    }
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// ---------------------------------------------------------------------------- amax -> scale
// One thread.  q = fp8_max / amax in fp32.
//   pow2:   scale = 2^floor(log2(q)), the exponent taken from q's bit pattern (exact; a log2
//           evaluated in floating point can round up to the next integer when q is within an
//           ulp below a power of two)
//   else:   scale = q / 2^margin
// amax == 0 (or NaN) keeps the previous scale, as the reference's where(amax > 0, sf, scale).
__global__ void scale_from_amax_kernel(const float* amax, float* scale, float* scale_inv, float fp8_max, int pow2,
                                       int margin) {
  const float a = *amax;
  if (!(a > 0.f)) {
    if (scale_inv) *scale_inv = 1.f / *scale;
    return;
  }
  const float q = fp8_max / a;
  float s;
  if (pow2) {
    if (isinf(q)) {
      s = q;
    } else {
      int e;
      (void)frexpf(q, &e);     // q = m * 2^e, m in [0.5, 1)
      s = ldexpf(1.f, e - 1);  // 2^floor(log2 q); flushes to 0 / inf outside the fp32 range like pow(2, exp)
    }
  } else {
    s = ldexpf(q, -margin);
  }
  *scale = s;
  if (scale_inv) *scale_inv = 1.f / s;
}

int scale_from_amax_impl(const float* amax, float* scale, float* scale_inv, float fp8_max, int pow2, int margin,
                         cudaStream_t st) {
  if (!amax || !scale || !(fp8_max > 0.f)) return B200Q_ERR_BAD_ARGUMENT;
  scale_from_amax_kernel<<<1, 1, 0, st>>>(amax, scale, scale_inv, fp8_max, pow2, margin);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// ---------------------------------------------------------------------------- delayed scaling
// history[len] is a ring of past amax values.  One step: store the new amax at slot `pos`,
// reduce the ring (max, or the newest entry), derive the scale as above.  One warp.
__global__ void amax_history_kernel(float* history, int len, int pos, const float* new_amax, int use_max, float* scale,
                                    float* scale_inv, float fp8_max, int pow2, int margin) {
  const int lane = threadIdx.x;
  if (lane == 0) history[pos] = *new_amax;
  __syncwarp();
  uint32_t m = 0;
  if (use_max) {
    for (int i = lane; i < len; i += 32) m = max(m, __float_as_uint(history[i]) & 0x7FFFFFFFu);
    m = warp_max_u32(m);
  } else {
    m = __float_as_uint(history[pos]) & 0x7FFFFFFFu;
  }
  if (lane != 0) return;
  const float a = __uint_as_float(m);
  if (!(a > 0.f)) {
    if (scale_inv) *scale_inv = 1.f / *scale;
    return;
  }
  const float q = fp8_max / a;
  float s;
  if (pow2) {
    if (isinf(q)) {
      s = q;
    } else {
      int e;
      (void)frexpf(q, &e);
      s = ldexpf(1.f, e - 1);
    }
  } else {
    s = ldexpf(q, -margin);
  }
  *scale = s;
  if (scale_inv) *scale_inv = 1.f / s;
}

int amax_history_impl(float* history, int len, int pos, const float* new_amax, int use_max, float* scale,
                      float* scale_inv, float fp8_max, int pow2, int margin, cudaStream_t st) {
  if (!history || !new_amax || !scale || len < 1 || pos < 0 || pos >= len || !(fp8_max > 0.f)) return B200Q_ERR_BAD_ARGUMENT;
  amax_history_kernel<<<1, 32, 0, st>>>(history, len, pos, new_amax, use_max, scale, scale_inv, fp8_max, pow2, margin);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // namespace b200q
