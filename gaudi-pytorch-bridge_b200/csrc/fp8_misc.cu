// The smaller FP8 operators of the reference that sit beside the casts and the GEMM:
//   softmax_fp8          hpu_ops/backend/softmax_fp8_gen.cpp:65-160  (scaled softmax, bf16 or e4m3 out)
//   sum_fp8              hpu_ops/backend/fp8_ops_gen.cpp:20-49       (sum over fp8 input, fp32 accumulate)
//   in_place_interleave_ hpu_ops/backend/fp8_ops.cpp:498-545         (row j <- row j / 4, in place)
// All three are bandwidth-bound; none allocates.
#include <cstdlib>

#include "common.cuh"
#include "fp8_misc.cuh"

#include <atomic>

namespace b200q {

// ---------------------------------------------------------------------------- softmax_fp8
// x = in * inv_attn_heads * input_scale + fused_add   (fp32; a factor that is absent is 1 / 0)
// y = softmax(x) over the last dimension, rounded to bf16
// out = y (bf16)                       without scales
//     = e4m3(bf16(y * output_scale))   with scales (RNE, saturating)
// One warp per row; the row is read twice (online max / sum of exponentials, then the write
// pass), the second time from L1 / L2.
__device__ __forceinline__ float ld_softmax_in(const SoftmaxParams& p, int64_t i) {
  if (p.in_dtype == B200Q_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p.in)[i]);
  const __nv_fp8_storage_t b = static_cast<const __nv_fp8_storage_t*>(p.in)[i];
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}

__global__ void __launch_bounds__(256) softmax_fp8_kernel(const SoftmaxParams p) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  float pre = p.pre_scale;
  if (p.inv_attn_heads) pre *= __ldg(p.inv_attn_heads);
  if (p.input_scale) pre *= __ldg(p.input_scale);
  const __nv_bfloat16* fa = nullptr;
  if (p.fused_add) {
    int64_t r = row, off = 0;
    for (int d = p.nd - 1; d >= 0; --d) {
      off += (r % p.size[d]) * p.fa_stride[d];
      r /= p.size[d];
    }
    fa = p.fused_add + off;
  }
  const int64_t base = row * p.cols;
  // pass 1: running maximum and sum of exp(x - max)
  float m = -INFINITY, s = 0.f;
  for (int64_t c = lane; c < p.cols; c += 32) {
    float x = ld_softmax_in(p, base + c) * pre;
    if (fa) x += __bfloat162float(fa[c]);
    if (x > m) {
      s = s * expf(m - x) + 1.f;
      m = x;
    } else {
      s += expf(x - m);
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xFFFFFFFFu, m, o), s2 = __shfl_xor_sync(0xFFFFFFFFu, s, o);
    const float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * expf(m2 - mm));
    m = mm;
  }
  const float inv = 1.f / s;
  const float so = p.output_scale ? __ldg(p.output_scale) : p.output_scale_host;
  // pass 2
  for (int64_t c = lane; c < p.cols; c += 32) {
    float x = ld_softmax_in(p, base + c) * pre;
    if (fa) x += __bfloat162float(fa[c]);
    const float y = round_to_bf16(expf(x - m) * inv);
    if (p.out_fp8) {
      const float z = round_to_bf16(y * so);
      uint32_t b = cvt_fp8x2<B200Q_E4M3>(z, 0.f) & 0xFFu;
      if (z != z) b = 0x7Fu;
      static_cast<uint8_t*>(p.out)[base + c] = (uint8_t)b;
    } else {
      static_cast<__nv_bfloat16*>(p.out)[base + c] = __float2bfloat16_rn(y);
    }
  }
}

// bf16 rows of up to 32 * 8 * NV elements whose length is a multiple of 8: the row is read once,
// with 16-byte loads, and stays in registers for the three passes max / sum / write.  The
// kernel is bound by instruction issue and by the special-function unit, not by HBM, unless
// every pass is lean, so:
//   * without a fused addend the maximum is taken on the packed bf16 pairs (one instruction
//     per two values; a negative input scale flips the sign bits first, x = (-raw) * (-scale));
//   * every exponential is computed once (ex2.approx on x * log2(e) - max, 2 ulp) and kept as
//     fp32 in the registers that held the packed input;
//   * NaN is a property of the whole row (a NaN or +inf input, or a row of -inf, makes the sum
//     NaN), so it is tested once per row, not per value;
//   * an output scale that is a power of two commutes with the rounding to bf16, which saves
//     the second rounding.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// WPR = warps per row (1, 2 or 4: rows of up to 4096, 8192, 16384 elements): each warp holds one
// contiguous part of the row; maximum and sum are exchanged through shared memory with a barrier
// of the row's warps only.
// IN8: the input is e4m3 (exactly representable in bf16: converted to packed bf16 pairs as it is read).
template <int NV, bool FA, int WPR, bool IN8>
__global__ void __launch_bounds__(128) softmax_bf16_rowreg_kernel(const SoftmaxParams p) {
  pdl_enter();
  __shared__ float xch[2][4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = ((int64_t)blockIdx.x * 4 + warp) / WPR;
  const int part = warp % WPR;
  if (row >= p.rows) return;  // (the warps of a row leave together)
  const int64_t part_cols = p.cols / WPR, col0 = part * part_cols;
  auto row_reduce = [&](float v, int which, bool is_max) {  // over the row's warps, after the warp's own reduction
    if (WPR == 1) return v;
    if (lane == 0) xch[which][warp] = v;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + warp / WPR), "r"(32 * WPR) : "memory");
    const int w0 = warp - part;
    float r = xch[which][w0];
#pragma unroll
    for (int i = 1; i < WPR; ++i) r = is_max ? fmaxf(r, xch[which][w0 + i]) : r + xch[which][w0 + i];
    return r;
  };
  float pre = p.pre_scale;
  if (p.inv_attn_heads) pre *= __ldg(p.inv_attn_heads);
  if (p.input_scale) pre *= __ldg(p.input_scale);
  constexpr float kLog2e = 1.4426950408889634f;
  pre *= kLog2e;
  const int nvec = (int)(part_cols >> 3);
  uint32_t w[NV][4];
  if constexpr (IN8) {
    const uint2* src = reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(p.in) + row * p.cols + col0);
    uint2 raw[NV];  // all loads first, so that they are in flight together
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      raw[i] = v < nvec ? __ldcs(src + v) : make_uint2(0xF8F8F8F8u, 0xF8F8F8F8u);  // (e4m3 has no infinity: patched below)
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const uint32_t b[2] = {raw[i].x, raw[i].y};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(b[k >> 1] >> (16 * (k & 1))), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
        w[i][k] = pack_bf16x2(f.x, f.y);
      }
      if (lane + 32 * i >= nvec) w[i][0] = w[i][1] = w[i][2] = w[i][3] = 0xFF80FF80u;  // -inf beyond the row
    }
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.in) + row * p.cols + col0);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      const uint4 t = v < nvec ? __ldcs(src + v) : make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);  // -inf
      w[i][0] = t.x, w[i][1] = t.y, w[i][2] = t.z, w[i][3] = t.w;
    }
  }
  float e[NV][8];  // x after pass 1 (with a fused addend only), the exponentials after pass 2
  float m;
  if constexpr (FA) {
    int64_t r = row, off = 0;
    for (int d = p.nd - 1; d >= 0; --d) {
      off += (r % p.size[d]) * p.fa_stride[d];
      r /= p.size[d];
    }
    const uint4* fa = reinterpret_cast<const uint4*>(p.fused_add + off + col0);
    m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        const uint4 f = __ldg(fa + v);
        const uint32_t fs[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          e[i][2 * k] = fmaf(__uint_as_float(fs[k] << 16), kLog2e, __uint_as_float(w[i][k] << 16) * pre);
          e[i][2 * k + 1] = fmaf(__uint_as_float(fs[k] & 0xFFFF0000u), kLog2e, __uint_as_float(w[i][k] & 0xFFFF0000u) * pre);
          m = fmaxf(m, fmaxf(e[i][2 * k], e[i][2 * k + 1]));
        }
      }
    }
  } else {
    if (pre < 0.f) {
      pre = -pre;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if (lane + 32 * i < nvec) {
#pragma unroll
          for (int k = 0; k < 4; ++k) w[i][k] ^= 0x80008000u;
        }
      }
    }
    uint32_t pm = 0xFF80FF80u;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k) pm = max_bf16x2(pm, w[i][k]);
    }
    m = fmaxf(__uint_as_float(pm << 16), __uint_as_float(pm & 0xFFFF0000u)) * pre;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  m = row_reduce(m, 0, true);
  float s = 0.f;
  const float neg_m = -m;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (lane + 32 * i < nvec) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if constexpr (FA) {
          e[i][2 * k] = ex2_approx(e[i][2 * k] + neg_m);
          e[i][2 * k + 1] = ex2_approx(e[i][2 * k + 1] + neg_m);
        } else {
          e[i][2 * k] = ex2_approx(fmaf(__uint_as_float(w[i][k] << 16), pre, neg_m));
          e[i][2 * k + 1] = ex2_approx(fmaf(__uint_as_float(w[i][k] & 0xFFFF0000u), pre, neg_m));
        }
        s += e[i][2 * k] + e[i][2 * k + 1];
      }
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
  s = row_reduce(s, 1, false);
  float inv = 1.f / s;
  const float so = p.output_scale ? __ldg(p.output_scale) : p.output_scale_host;
  uint2* out8 = reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.out) + row * p.cols + col0);
  uint4* out16 = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + row * p.cols + col0);
  if (inv != inv) {  // the whole row is NaN
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        if (p.out_fp8) __stcs(out8 + v, make_uint2(0x7F7F7F7Fu, 0x7F7F7F7Fu));
        else __stcs(out16 + v, make_uint4(0x7FFF7FFFu, 0x7FFF7FFFu, 0x7FFF7FFFu, 0x7FFF7FFFu));
      }
    }
    return;
  }
  if (!p.out_fp8) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec)
        __stcs(out16 + v, make_uint4(pack_bf16x2(e[i][0] * inv, e[i][1] * inv), pack_bf16x2(e[i][2] * inv, e[i][3] * inv),
                                     pack_bf16x2(e[i][4] * inv, e[i][5] * inv), pack_bf16x2(e[i][6] * inv, e[i][7] * inv)));
    }
    return;
  }
  // e4m3(bf16(bf16(e * inv) * so)).  so = 2^k (normal, finite): bf16(e * inv) * so == bf16(e * (inv * so))
  // wherever the e4m3 result is not 0 on both sides, so one rounding is enough.
  const uint32_t so_bits = __float_as_uint(so);
  const uint32_t so_exp = (so_bits >> 23) & 0xFFu;
  const bool pow2 = (so_bits & 0x807FFFFFu) == 0 && so_exp > 32 && so_exp < 222;
  if (pow2) inv *= so;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    uint32_t o2[2];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t zb = pack_bf16x2(e[i][2 * k] * inv, e[i][2 * k + 1] * inv);
      if (!pow2) zb = pack_bf16x2(__uint_as_float(zb << 16) * so, __uint_as_float(zb & 0xFFFF0000u) * so);
      const uint32_t b = cvt_fp8x2<B200Q_E4M3>(__uint_as_float(zb << 16), __uint_as_float(zb & 0xFFFF0000u)) & 0xFFFFu;
      if (k & 1) o2[k >> 1] |= b << 16;
      else o2[k >> 1] = b;
    }
    if (v < nvec) __stcs(out8 + v, make_uint2(o2[0], o2[1]));
  }
}

template <int NV, int WPR>
static int launch_softmax_rowreg(const SoftmaxParams& p, cudaStream_t st) {
  const int rows_per_block = 4 / WPR;
  const int64_t blocks = (p.rows + rows_per_block - 1) / rows_per_block;
  if (blocks > 0x7FFFFFFF) return B200Q_ERR_TOO_LARGE;
  auto kern = p.in_dtype == B200Q_BF16
                  ? (p.fused_add ? softmax_bf16_rowreg_kernel<NV, true, WPR, false> : softmax_bf16_rowreg_kernel<NV, false, WPR, false>)
                  : (p.fused_add ? softmax_bf16_rowreg_kernel<NV, true, WPR, true> : softmax_bf16_rowreg_kernel<NV, false, WPR, true>);
  if (launch_overlapped(kern, dim3((unsigned)blocks), dim3(128), 0, st, p) != cudaSuccess) {  // (it calls pdl_enter())
    (void)cudaGetLastError();
    kern<<<(int)blocks, 128, 0, st>>>(p);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int softmax_fp8_impl(const SoftmaxParams& p, cudaStream_t st) {
  if (p.rows == 0 || p.cols == 0) return B200Q_OK;
  // fast path: bf16 rows that fit a warp's registers, 16-byte aligned everywhere
  bool fa_ok = true;
  if (p.fused_add) {
    fa_ok = (reinterpret_cast<uintptr_t>(p.fused_add) & 15) == 0;
    for (int d = 0; d < p.nd; ++d) fa_ok = fa_ok && (p.fa_stride[d] % 8) == 0;
  }
  const bool aligned = ((reinterpret_cast<uintptr_t>(p.in) | reinterpret_cast<uintptr_t>(p.out)) & 15) == 0;
  const bool in_ok = p.in_dtype == B200Q_BF16 || p.in_dtype == B200Q_E4M3;
  // Rows of more than 2048 elements are split over four warps: a quarter of the registers per
  // thread, three to four times the warps per SM, so that loads, arithmetic and stores of different
  // rows overlap (4096 columns: 43.4 -> 38.4 us from bf16, 93.5 -> 41.2 us from e4m3; rows of up to
  // 2048 elements are faster with one warp each).
  static const bool one_warp = std::getenv("B200Q_SOFTMAX_ONE_WARP") != nullptr;  // comparison switch
  if (!one_warp && in_ok && fa_ok && aligned && (p.cols % 32) == 0 && p.cols > 2048 && p.cols <= 4 * 32 * 8 * 16) {
    const int64_t per_lane = (p.cols / 32 + 31) / 32;
    if (per_lane <= 4) return launch_softmax_rowreg<4, 4>(p, st);
    if (per_lane <= 8) return launch_softmax_rowreg<8, 4>(p, st);
    return launch_softmax_rowreg<16, 4>(p, st);
  }
  if (in_ok && (p.cols % 8) == 0 && p.cols <= 32 * 8 * 16 && fa_ok && aligned) {
    const int64_t per_lane = (p.cols / 8 + 31) / 32;
    if (per_lane <= 1) return launch_softmax_rowreg<1, 1>(p, st);
    if (per_lane <= 2) return launch_softmax_rowreg<2, 1>(p, st);
    if (per_lane <= 4) return launch_softmax_rowreg<4, 1>(p, st);
    if (per_lane <= 8) return launch_softmax_rowreg<8, 1>(p, st);
    return launch_softmax_rowreg<16, 1>(p, st);
  }
  // longer rows: two or four warps per row, each with a contiguous part in its registers
  if (in_ok && fa_ok && aligned) {
    if ((p.cols % 16) == 0 && p.cols <= 2 * 32 * 8 * 16) return launch_softmax_rowreg<16, 2>(p, st);
    if ((p.cols % 32) == 0 && p.cols <= 4 * 32 * 8 * 16) return launch_softmax_rowreg<16, 4>(p, st);
  }
  const int warps = 8;
  const int64_t blocks = (p.rows + warps - 1) / warps;
  if (blocks > 0x7FFFFFFF) return B200Q_ERR_TOO_LARGE;
  if (launch_overlapped(softmax_fp8_kernel, dim3((unsigned)blocks), dim3(warps * 32), 0, st, p) != cudaSuccess) {
    (void)cudaGetLastError();
    softmax_fp8_kernel<<<(int)blocks, warps * 32, 0, st>>>(p);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// ---------------------------------------------------------------------------- sum_fp8
// in viewed as [outer][reduce][inner] (contiguous), fp32 accumulation in a fixed order:
// chunk c of the reduce range is summed sequentially by one thread (inner > 1) or by one block
// with a fixed tree (inner == 1); the chunk sums are then added in chunk order (16 chunks or
// more: eight interleaved partial orders, then those in order).  Same result on every run.
template <int FMT>
__device__ __forceinline__ float fp8_to_float(uint8_t b) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, Fp8Fmt<FMT>::kInterp)));
}

template <int FMT>
__global__ void __launch_bounds__(256) sum_fp8_strided_kernel(const uint8_t* __restrict__ in, float* __restrict__ partial,
                                                              int64_t outer, int64_t reduce, int64_t inner, int chunks) {
  pdl_enter();
  const int64_t n_out = outer * inner;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_out) return;
  const int chunk = blockIdx.y;
  const int64_t per = (reduce + chunks - 1) / chunks;
  const int64_t r0 = chunk * per, r1 = min(reduce, r0 + per);
  const int64_t o = idx / inner, i = idx % inner;
  const uint8_t* src = in + (o * reduce) * inner + i;
  float acc = 0.f;
  for (int64_t r = r0; r < r1; ++r) acc += fp8_to_float<FMT>(src[r * inner]);
  partial[(int64_t)chunk * n_out + idx] = acc;
}

// inner a multiple of 16, 16-byte aligned rows: a thread owns 16 neighbouring inner positions, reads
// them with one 16-byte load per reduce row (eight rows in flight) and keeps 16 fp32 sums.
template <int FMT>
__global__ void __launch_bounds__(256) sum_fp8_strided16_kernel(const uint8_t* __restrict__ in, float* __restrict__ partial,
                                                                int64_t outer, int64_t reduce, int64_t inner, int chunks) {
  pdl_enter();
  const int64_t inner16 = inner >> 4;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // (o, 16-group)
  if (idx >= outer * inner16) return;
  const int chunk = blockIdx.y;
  const int64_t per = (reduce + chunks - 1) / chunks;
  const int64_t r0 = chunk * per, r1 = min(reduce, r0 + per);
  const int64_t o = idx / inner16, i0 = (idx - o * inner16) << 4;
  const uint4* src = reinterpret_cast<const uint4*>(in + (o * reduce) * inner + i0);
  const int64_t stride = inner >> 4;  // in 16-byte units
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  auto add = [&](const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[k] >> (16 * h)), Fp8Fmt<FMT>::kInterp);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
        acc[4 * k + 2 * h] += f.x;
        acc[4 * k + 2 * h + 1] += f.y;
      }
    }
  };
  int64_t r = r0;
  for (; r + 8 <= r1; r += 8) {  // rows in order: the sums do not depend on the unrolling
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __ldcs(src + (r + j) * stride);
#pragma unroll
    for (int j = 0; j < 8; ++j) add(v[j]);
  }
  for (; r < r1; ++r) add(__ldcs(src + r * stride));
  float* dst = partial + (int64_t)chunk * (outer * inner) + o * inner + i0;
#pragma unroll
  for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
}

template <int FMT>
__global__ void __launch_bounds__(256) sum_fp8_rows_kernel(const uint8_t* __restrict__ in, float* __restrict__ partial,
                                                           int64_t outer, int64_t reduce, int chunks) {
  pdl_enter();
  // grid (outer, chunks): one block sums one chunk of one row
  const int64_t row = blockIdx.x;
  const int chunk = blockIdx.y;
  const int64_t per = (reduce + chunks - 1) / chunks;
  const int64_t r0 = (int64_t)chunk * per, r1 = min(reduce, r0 + per);
  const int64_t len = r1 > r0 ? r1 - r0 : 0;
  const uint8_t* s = in + row * reduce + r0;
  float acc = 0.f;
  // bytes up to the first 16-byte boundary, 16-byte vectors, bytes after the last vector
  int64_t head = (16 - (int64_t)(reinterpret_cast<uintptr_t>(s) & 15)) & 15;
  if (head > len) head = len;
  if ((int64_t)threadIdx.x < head) acc += fp8_to_float<FMT>(s[threadIdx.x]);
  const int64_t nvec = (len - head) / 16;
  const uint4* v = reinterpret_cast<const uint4*>(s + head);
  float a4[4] = {0.f, 0.f, 0.f, 0.f};  // one chain per 32-bit word of the vector (fixed order all the same)
  auto add = [&](const uint4& w) {
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(ws[k] >> (16 * h)), Fp8Fmt<FMT>::kInterp);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
        a4[k] += f.x;
        a4[k] += f.y;
      }
    }
  };
  int64_t i = threadIdx.x;
  for (; i + 3 * (int64_t)blockDim.x < nvec; i += 4 * (int64_t)blockDim.x) {  // four loads in flight, added in index order
    const uint4 w0 = __ldcs(v + i), w1 = __ldcs(v + i + blockDim.x), w2 = __ldcs(v + i + 2 * (int64_t)blockDim.x),
                w3 = __ldcs(v + i + 3 * (int64_t)blockDim.x);
    add(w0); add(w1); add(w2); add(w3);
  }
  for (; i < nvec; i += blockDim.x) add(__ldcs(v + i));
  acc += (a4[0] + a4[1]) + (a4[2] + a4[3]);
  const int64_t tail0 = head + nvec * 16;
  if (threadIdx.x < 16 && tail0 + (int64_t)threadIdx.x < len) acc += fp8_to_float<FMT>(s[tail0 + threadIdx.x]);
  // fixed order: a butterfly inside each warp (no barrier), then the warp sums in warp order
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float sm[8];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = sm[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) t += sm[w];
    partial[(int64_t)chunk * outer + row] = t;
  }
}

template <int FMT>
__global__ void __launch_bounds__(256) sum_fp8_finish_kernel(const float* __restrict__ partial, void* out, int out_dtype,
                                                             int64_t n_out, int chunks) {
  pdl_enter();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_out) return;
  float acc = 0.f;
  for (int c = 0; c < chunks; ++c) acc += partial[(int64_t)c * n_out + idx];
  if (out_dtype == B200Q_F32) {
    static_cast<float*>(out)[idx] = acc;
  } else if (out_dtype == B200Q_BF16) {
    static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(acc);
  } else {
    uint32_t b = out_dtype == B200Q_E4M3 ? (cvt_fp8x2<B200Q_E4M3>(acc, 0.f) & 0xFFu) : (cvt_fp8x2<B200Q_E5M2>(acc, 0.f) & 0xFFu);
    if (acc != acc) b = 0x7Fu;
    static_cast<uint8_t*>(out)[idx] = (uint8_t)b;
  }
}

// Many chunks: a block of 32 outputs x 8 chunk lanes; lane y adds chunks y, y + 8, ... in order
// (coalesced 128-byte loads, four in flight), the 8 lane sums are then added in lane order.
__global__ void __launch_bounds__(256) sum_fp8_finish_wide_kernel(const float* __restrict__ partial, void* out, int out_dtype,
                                                                  int64_t n_out, int chunks) {
  pdl_enter();
  __shared__ float sm[8][33];
  const int x = threadIdx.x & 31, y = threadIdx.x >> 5;
  const int64_t idx = (int64_t)blockIdx.x * 32 + x;
  float acc = 0.f;
  if (idx < n_out) {
    int c = y;
    for (; c + 24 < chunks; c += 32) {
      const float p0 = partial[(int64_t)c * n_out + idx], p1 = partial[(int64_t)(c + 8) * n_out + idx],
                  p2 = partial[(int64_t)(c + 16) * n_out + idx], p3 = partial[(int64_t)(c + 24) * n_out + idx];
      acc += p0; acc += p1; acc += p2; acc += p3;
    }
    for (; c < chunks; c += 8) acc += partial[(int64_t)c * n_out + idx];
  }
  sm[y][x] = acc;
  __syncthreads();
  if (y != 0 || idx >= n_out) return;
#pragma unroll
  for (int j = 1; j < 8; ++j) acc += sm[j][x];
  if (out_dtype == B200Q_F32) {
    static_cast<float*>(out)[idx] = acc;
  } else if (out_dtype == B200Q_BF16) {
    static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(acc);
  } else {
    uint32_t b = out_dtype == B200Q_E4M3 ? (cvt_fp8x2<B200Q_E4M3>(acc, 0.f) & 0xFFu) : (cvt_fp8x2<B200Q_E5M2>(acc, 0.f) & 0xFFu);
    if (acc != acc) b = 0x7Fu;
    static_cast<uint8_t*>(out)[idx] = (uint8_t)b;
  }
}

int sum_fp8_chunks(int64_t outer, int64_t reduce, int64_t inner) {
  // enough chunks to occupy the device when there are few outputs, each at least 4096 elements
  const int64_t n_out = outer * inner;
  int64_t want = (int64_t)kNumSMs * 8 * 256 / (n_out > 0 ? n_out : 1);
  if (inner == 1) want = (int64_t)kNumSMs * 4 / (outer > 0 ? outer : 1);
  int64_t cap = reduce / 4096;
  if (inner > 1 && (inner % 16) == 0) {  // 16 positions per thread: fewer threads per chunk, shorter chunks
    want = (int64_t)kNumSMs * 8 * 256 / (n_out / 16 > 0 ? n_out / 16 : 1);
    cap = reduce / 64;
  }
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  if (want > 1024) want = 1024;
  return (int)want;
}

size_t sum_fp8_workspace_bytes_impl(int64_t outer, int64_t reduce, int64_t inner) {
  return (size_t)sum_fp8_chunks(outer, reduce, inner) * (size_t)(outer * inner) * sizeof(float);
}

int sum_fp8_impl(const void* in, int in_dtype, void* out, int out_dtype, int64_t outer, int64_t reduce, int64_t inner,
                 void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (outer < 0 || reduce < 0 || inner < 0) return B200Q_ERR_BAD_ARGUMENT;
  if (in_dtype != B200Q_E4M3 && in_dtype != B200Q_E5M2) return B200Q_ERR_BAD_ARGUMENT;
  const int64_t n_out = outer * inner;
  if (n_out == 0) return B200Q_OK;
  if (!out || (reduce > 0 && !in)) return B200Q_ERR_BAD_ARGUMENT;
  const int chunks = sum_fp8_chunks(outer, reduce, inner);
  if (!workspace || workspace_bytes < (size_t)chunks * n_out * sizeof(float)) return B200Q_ERR_BAD_ARGUMENT;
  // one chunk and fp32 output: the chunk sums are the result, written where it belongs
  const bool direct = chunks == 1 && out_dtype == B200Q_F32;
  float* partial = direct ? static_cast<float*>(out) : static_cast<float*>(workspace);
  const uint8_t* src = static_cast<const uint8_t*>(in);
  const int fin_blocks = (int)((n_out + 255) / 256);
  if (inner == 1) {
    if (outer > 0x7FFFFFFF) return B200Q_ERR_TOO_LARGE;
    dim3 grid((unsigned)outer, (unsigned)chunks);
    // threads per block: about four 16-byte vectors each (a short row in a big block is all tree and no sum)
    const int64_t vecs = (reduce + chunks - 1) / chunks / 16;
    int threads = 32;
    while (threads < 256 && threads * 4 < vecs) threads *= 2;
    if (in_dtype == B200Q_E4M3) launch_dependent(sum_fp8_rows_kernel<B200Q_E4M3>, grid, dim3(threads), 0, st, src, partial, outer, reduce, chunks);
    else launch_dependent(sum_fp8_rows_kernel<B200Q_E5M2>, grid, dim3(threads), 0, st, src, partial, outer, reduce, chunks);
  } else if ((inner % 16) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
    dim3 grid((unsigned)((n_out / 16 + 255) / 256), (unsigned)chunks);
    if (in_dtype == B200Q_E4M3) launch_dependent(sum_fp8_strided16_kernel<B200Q_E4M3>, grid, dim3(256), 0, st, src, partial, outer, reduce, inner, chunks);
    else launch_dependent(sum_fp8_strided16_kernel<B200Q_E5M2>, grid, dim3(256), 0, st, src, partial, outer, reduce, inner, chunks);
  } else {
    dim3 grid((unsigned)((n_out + 255) / 256), (unsigned)chunks);
    if (in_dtype == B200Q_E4M3) launch_dependent(sum_fp8_strided_kernel<B200Q_E4M3>, grid, dim3(256), 0, st, src, partial, outer, reduce, inner, chunks);
    else launch_dependent(sum_fp8_strided_kernel<B200Q_E5M2>, grid, dim3(256), 0, st, src, partial, outer, reduce, inner, chunks);
  }
  B200Q_LAUNCH_CHECK();
  if (direct) return B200Q_OK;
  if (chunks >= 16) launch_dependent(sum_fp8_finish_wide_kernel, dim3((unsigned)((n_out + 31) / 32)), dim3(256), 0, st, (const float*)partial, out, out_dtype, n_out, chunks);
  else launch_dependent(sum_fp8_finish_kernel<0>, dim3((unsigned)fin_blocks), dim3(256), 0, st, (const float*)partial, out, out_dtype, n_out, chunks);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// ---------------------------------------------------------------------------- in_place_interleave_
// rows[j] <- rows[j / 4] for j in [0, n_rows), in place.  A row is a destination and, for j <
// n_rows / 4, also a source; destinations [lo, hi) with lo > (hi - 1) / 4 have all their sources
// below lo, so the rows are rewritten in phases from the top: [n/4, n), then [n/16, n/4), ...
//
// A phase is laid out by SOURCE row: a thread reads kIlvPieces pieces of source row s once and
// writes them to the (up to four) destinations 4s .. 4s + 3 that lie inside the phase, all loads
// issued before the first store.  Long rows are split over blockIdx.x; rows shorter than a block
// share one (tpr threads per row, a power of two).
constexpr int kIlvPieces = 4;

template <typename T>
__global__ void __launch_bounds__(256) interleave_phase_kernel(uint8_t* base, int64_t row_bytes, int64_t lo, int64_t hi,
                                                               int64_t s_first, int64_t s_end, int tpr) {
  pdl_enter();
  const int rows_per_block = 256 / tpr;
  const int64_t s = s_first + (int64_t)blockIdx.y * rows_per_block + threadIdx.x / tpr;
  if (s >= s_end) return;
  const int64_t n = row_bytes / (int64_t)sizeof(T);
  const T* src = reinterpret_cast<const T*>(base + s * row_bytes);
  const int64_t d0 = 4 * s > lo ? 4 * s : lo, d1 = 4 * s + 4 < hi ? 4 * s + 4 : hi;
  const int lane = threadIdx.x % tpr;
  for (int64_t i0 = (int64_t)blockIdx.x * tpr * kIlvPieces + lane; i0 < n; i0 += (int64_t)gridDim.x * tpr * kIlvPieces) {
    T v[kIlvPieces];
#pragma unroll
    for (int k = 0; k < kIlvPieces; ++k)
      if (i0 + (int64_t)k * tpr < n) v[k] = src[i0 + (int64_t)k * tpr];
    for (int64_t d = d0; d < d1; ++d) {
      if (d == s) continue;  // (row 0 is its own source)
      T* dst = reinterpret_cast<T*>(base + d * row_bytes);
#pragma unroll
      for (int k = 0; k < kIlvPieces; ++k)
        if (i0 + (int64_t)k * tpr < n) dst[i0 + (int64_t)k * tpr] = v[k];
    }
  }
}

int in_place_interleave_impl(void* data, int64_t n_rows, int64_t row_bytes, cudaStream_t st) {
  if (n_rows < 0 || row_bytes < 0 || (n_rows % 4) != 0) return B200Q_ERR_BAD_ARGUMENT;
  if (n_rows == 0 || row_bytes == 0) return B200Q_OK;
  if (!data) return B200Q_ERR_BAD_ARGUMENT;
  const bool wide = (row_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(data) & 15) == 0;
  const int64_t n = wide ? row_bytes / 16 : row_bytes;  // pieces per row
  int tpr = 256;
  while (tpr > 1 && tpr / 2 * kIlvPieces >= n) tpr /= 2;
  const int rows_per_block = 256 / tpr;
  int64_t bx = (n + (int64_t)tpr * kIlvPieces - 1) / ((int64_t)tpr * kIlvPieces);
  if (bx > 4096) bx = 4096;
  int64_t hi = n_rows;
  while (hi > 1) {
    const int64_t lo = (hi - 1) / 4 + 1;
    const int64_t s_end = (hi - 1) / 4 + 1;
    int64_t s = lo / 4;
    while (s < s_end) {  // grid.y is limited to 65535
      int64_t by = (s_end - s + rows_per_block - 1) / rows_per_block;
      if (by > 65535) by = 65535;
      const dim3 grid((unsigned)bx, (unsigned)by);
      if (wide) launch_dependent(interleave_phase_kernel<uint4>, grid, dim3(256), 0, st, static_cast<uint8_t*>(data), row_bytes, lo, hi, s, s_end, tpr);
      else launch_dependent(interleave_phase_kernel<uint8_t>, grid, dim3(256), 0, st, static_cast<uint8_t*>(data), row_bytes, lo, hi, s, s_end, tpr);
      B200Q_LAUNCH_CHECK();
      s += by * rows_per_block;
    }
    hi = lo;
  }
  return B200Q_OK;
}

// ---------------------------------------------------------------------------- im2col for conv2d_fp8
// One-byte elements.  out[(n, ho, wo)][k], k = (c, i, j) over the channels [c0, c0 + cg) and the
// kernel window, zero where the window leaves the image and for k in [cg * kh * kw, ld_out):
// the K-major left operand of the GEMM that computes the convolution (K padded to ld_out).
//
// A block builds the rows of one output line (n, ho) for a chunk of channels.  It first copies
// the input patch it needs -- chunk channels x kh image rows, each padded with zero bytes on both
// sides (the left pad rounded up to 4 so that the copy runs in 32-bit words), rows outside the
// image as zeros, plus one row of zeros for the K padding -- into shared memory, and a table
// k -> patch offset of (c, i, j); the gather itself then has no bounds test and no division: a
// warp takes one output pixel at a time, its lanes consecutive 4-byte words of k (a 128-byte
// store per warp), each byte one shared-memory load at table[k] + wo * sw.
struct Im2colParams {
  const uint8_t* in;
  uint8_t* out;
  int64_t N, C, H, W, Ho, Wo;
  int kh, kw, sh, sw, ph, pw, dh, dw;
  int64_t c0, cg, ld_out;
  int chunk;     // channels per block (a multiple of 4 when there is more than one chunk)
  int chunks;    // blocks per output line
  int lp;        // zero bytes in front of an image row in the patch: pw rounded up to 4
  int pitch;     // bytes of a patch row: lp + W + pw rounded up to 4
  int patch_al;  // bytes reserved for the patch and the row of zeros, a multiple of 16
};

__global__ void __launch_bounds__(256) im2col_u8_kernel(const Im2colParams p) {
  extern __shared__ __align__(16) uint8_t im2col_smem[];
  uint8_t* patch = im2col_smem;
  uint32_t* table = reinterpret_cast<uint32_t*>(im2col_smem + p.patch_al);
  const int64_t line = blockIdx.x / p.chunks;  // (n, ho)
  const int ch = (int)(blockIdx.x % p.chunks);
  const int64_t n = line / p.Ho, ho = line % p.Ho;
  const int cc0 = ch * p.chunk;  // first channel of the chunk, relative to c0
  const int cn = (int)(p.cg - cc0 < p.chunk ? p.cg - cc0 : p.chunk);
  const int win = p.kh * p.kw;
  const int64_t K = p.cg * win;
  const int k_begin = cc0 * win;  // a multiple of 4 (chunk % 4 == 0 unless there is one chunk)
  const int k_real = (cc0 + cn) * win;                            // end of the real k of this chunk
  const int k_end = ch == p.chunks - 1 ? (int)p.ld_out : k_real;  // the last chunk also writes the padding
  const int zero_at = cn * p.kh * p.pitch;                         // a row of zeros
  // patch: [c][i][lp + x], 16 threads per row, 32-bit words
  const int wpr = p.pitch >> 2;
  const bool words_ok = (p.W & 3) == 0 && (reinterpret_cast<uintptr_t>(p.in) & 3) == 0;
  for (int r = threadIdx.x >> 4; r <= cn * p.kh; r += 16) {  // (the row cn * kh is the row of zeros)
    const int c = r / p.kh, i = r - c * p.kh;
    const int64_t y = ho * p.sh - p.ph + (int64_t)i * p.dh;
    const bool inside = r < cn * p.kh && y >= 0 && y < p.H;
    const uint8_t* src = p.in + ((n * p.C + p.c0 + cc0 + (inside ? c : 0)) * p.H + (inside ? y : 0)) * p.W;
    uint32_t* dst = reinterpret_cast<uint32_t*>(patch + r * p.pitch);
    for (int c4 = threadIdx.x & 15; c4 < wpr; c4 += 16) {
      const int x0 = 4 * c4 - p.lp;  // image column of the word's first byte
      uint32_t word = 0;
      if (inside) {
        if (words_ok && x0 >= 0 && x0 + 4 <= p.W) {
          word = __ldg(reinterpret_cast<const uint32_t*>(src + x0));
        } else {
#pragma unroll
          for (int b = 0; b < 4; ++b)
            if (x0 + b >= 0 && x0 + b < p.W) word |= (uint32_t)__ldg(src + x0 + b) << (8 * b);
        }
      }
      dst[c4] = word;
    }
  }
  for (int k = k_begin + threadIdx.x; k < k_end; k += 256) {
    uint32_t off = (uint32_t)zero_at;
    if (k < k_real && k < K) {
      const int kl = k - k_begin;
      const int c = kl / win, rem = kl - c * win;
      const int i = rem / p.kw, j = rem - i * p.kw;
      off = (uint32_t)((c * p.kh + i) * p.pitch + (p.lp - p.pw) + j * p.dw);
    }
    table[k - k_begin] = off;
  }
  __syncthreads();
  const int words = (k_end - k_begin) >> 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* out_line = p.out + (line * p.Wo) * p.ld_out + k_begin;
  for (int wo = warp; wo < p.Wo; wo += 8) {
    const uint8_t* base = patch + wo * p.sw;  // (an offset into the row of zeros stays inside it: wo * sw < pitch)
    uint32_t* dst = reinterpret_cast<uint32_t*>(out_line + (int64_t)wo * p.ld_out);
    for (int w = lane; w < words; w += 32) {
      const uint4 t = *reinterpret_cast<const uint4*>(table + 4 * w);
      const uint32_t b0 = base[t.x], b1 = base[t.y], b2 = base[t.z], b3 = base[t.w];
      __stcs(dst + w, __byte_perm(b0 | (b1 << 8), b2 | (b3 << 8), 0x5410));
    }
  }
}

// Fallback for images whose rows do not fit the patch kernel's shared memory (a row of 4 channels x kh
// lines beyond 96 KB): one 4-byte output word per thread, every byte located by division.
__global__ void __launch_bounds__(256) im2col_u8_wide_kernel(const Im2colParams p) {
  const int64_t words_per_row = p.ld_out >> 2;
  const int64_t total = p.N * p.Ho * p.Wo * words_per_row;
  const int64_t K = p.cg * p.kh * p.kw;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = t / words_per_row;
    const int64_t k0 = (t % words_per_row) * 4;
    const int64_t wo = row % p.Wo, ho = (row / p.Wo) % p.Ho, n = row / (p.Wo * p.Ho);
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int64_t k = k0 + b;
      if (k < K) {
        const int64_t j = k % p.kw, i = (k / p.kw) % p.kh, c = p.c0 + k / (p.kw * p.kh);
        const int64_t y = ho * p.sh - p.ph + i * p.dh, x = wo * p.sw - p.pw + j * p.dw;
        if (y >= 0 && y < p.H && x >= 0 && x < p.W) word |= (uint32_t)p.in[((n * p.C + c) * p.H + y) * p.W + x] << (8 * b);
      }
    }
    reinterpret_cast<uint32_t*>(p.out)[t] = word;
  }
}

static int im2col_wide_launch(const Im2colParams& p, cudaStream_t st) {
  const int64_t total = p.N * p.Ho * p.Wo * (p.ld_out >> 2);
  int64_t blocks = (total + 255) / 256;
  if (blocks > kNumSMs * 32) blocks = kNumSMs * 32;
  im2col_u8_wide_kernel<<<(int)blocks, 256, 0, st>>>(p);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int im2col_u8_impl(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W, int kh, int kw, int sh, int sw,
                   int ph, int pw, int dh, int dw, int64_t c0, int64_t cg, int64_t ld_out, cudaStream_t st) {
  if (N < 0 || C < 0 || H < 0 || W < 0 || kh < 1 || kw < 1 || sh < 1 || sw < 1 || ph < 0 || pw < 0 || dh < 1 || dw < 1 ||
      c0 < 0 || cg < 0 || c0 + cg > C || (ld_out & 15) || ld_out < cg * kh * kw)
    return B200Q_ERR_BAD_ARGUMENT;
  Im2colParams p;
  p.in = static_cast<const uint8_t*>(in); p.out = static_cast<uint8_t*>(out);
  p.N = N; p.C = C; p.H = H; p.W = W;
  p.Ho = (H + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
  p.Wo = (W + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
  p.kh = kh; p.kw = kw; p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw; p.dh = dh; p.dw = dw;
  p.c0 = c0; p.cg = cg; p.ld_out = ld_out;
  if (p.Ho <= 0 || p.Wo <= 0 || N == 0) return B200Q_OK;
  if (!in || !out) return B200Q_ERR_BAD_ARGUMENT;
  p.chunk = p.chunks = p.lp = p.pitch = p.patch_al = 0;
  if (W + 2 * (int64_t)pw > (1 << 20) || N * p.Ho > (1ll << 30)) return im2col_wide_launch(p, st);
  p.lp = (pw + 3) & ~3;
  // patch row pitch: an ODD number of 32-bit words, so that the rows (c, i) that the lanes of a warp
  // gather from at one column fall into different banks (a pitch of 64 bytes put every second row
  // on the same banks: 110 M conflicts on the benchmark's case against 9 M)
  p.pitch = (int)((((p.lp + W + pw + 3) >> 2) | 1) << 2);
  // channels per block: patch (chunk * kh rows + the row of zeros) + table (4 bytes per k, + the K
  // padding) within about 40 KB, so that five blocks share an SM and the grid has several times
  // as many blocks as the machine holds at once (the last wave costs little); equal chunks
  const int64_t pad_k = ld_out - cg * kh * kw;
  const int64_t per_channel = (int64_t)kh * p.pitch + 4ll * kh * kw;
  int64_t room = 40 * 1024 - 4 * pad_k - p.pitch - 64;
  if (room < 4 * per_channel) room = 96 * 1024 - 4 * pad_k - p.pitch - 64;  // wide images: one block per SM or two
  int64_t chunk = cg > 0 ? cg : 1;
  if (chunk * per_channel > room) {
    const int64_t most = (room / per_channel) & ~3ll;
    if (most < 4) return im2col_wide_launch(p, st);  // the image rows of 4 channels do not fit
    const int64_t parts = (cg + most - 1) / most;
    chunk = ((cg + parts - 1) / parts + 3) & ~3ll;
  }
  p.chunk = (int)chunk;
  p.chunks = (int)((cg + chunk - 1) / chunk);
  if (p.chunks < 1) p.chunks = 1;
  if (N * p.Ho * p.chunks > 0x7FFFFFFFll) return im2col_wide_launch(p, st);
  p.patch_al = (int)(((chunk * kh + 1) * p.pitch + 15) & ~15ll);
  const int64_t table_k = chunk * kh * kw + (ld_out - cg * kh * kw);
  const int smem = p.patch_al + (int)(4 * ((table_k + 3) & ~3ll));
  static std::atomic<int> configured[kMaxDevices];
  const int dev = current_device_index();
  if (dev < 0) return B200Q_ERR_CUDA;
  if (!configured[dev].load(std::memory_order_acquire)) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(im2col_u8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    configured[dev].store(1, std::memory_order_release);
  }
  im2col_u8_kernel<<<(int)(N * p.Ho * p.chunks), 256, smem, st>>>(p);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// ---------------------------------------------------------------------------- channels-last path of conv2d_fp8
// One-byte elements.  out[n][hw][c] = in[n][c][hw]: a block moves a tile of 64 channels x 64
// pixels.  A thread loads four channels x four pixels as four 32-bit words (a warp reads 64
// contiguous bytes of two channel rows per instruction), transposes the 4 x 4 bytes in registers
// with eight byte permutes, and parks the four words -- four channels of one pixel each -- in a
// shared-memory tile [pixel][channel]; the tile is then written out with a warp storing the 64
// contiguous bytes of two pixels per instruction.
constexpr int kTrTile = 64;
constexpr int kTrPitch = kTrTile + 4;  // bytes; 17 words: the transposed writes spread over 16 banks

__global__ void __launch_bounds__(256) nchw_to_nhwc_u8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t C,
                                                              int64_t HW, int wide) {
  pdl_enter();
  __shared__ __align__(16) uint8_t tile[kTrTile * kTrPitch];
  const int64_t n = blockIdx.z, c0 = (int64_t)blockIdx.y * kTrTile, p0 = (int64_t)blockIdx.x * kTrTile;
  const uint8_t* src = in + n * C * HW;
  uint8_t* dst = out + n * HW * C;
  const int t = threadIdx.x, cb = t >> 4, pb = t & 15;
  uint32_t r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t c = c0 + 4 * cb + i, p = p0 + 4 * pb;
    r[i] = 0u;
    if (c < C) {
      if (wide && p + 3 < HW) {
        r[i] = __ldcs(reinterpret_cast<const uint32_t*>(src + c * HW + p));
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (p + k < HW) r[i] |= (uint32_t)src[c * HW + p + k] << (8 * k);
      }
    }
  }
  const uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[0], r[1], 0x7362);
  const uint32_t t2 = __byte_perm(r[2], r[3], 0x5140), t3 = __byte_perm(r[2], r[3], 0x7362);
  const uint32_t o[4] = {__byte_perm(t0, t2, 0x5410), __byte_perm(t0, t2, 0x7632), __byte_perm(t1, t3, 0x5410),
                         __byte_perm(t1, t3, 0x7632)};
#pragma unroll
  for (int k = 0; k < 4; ++k) *reinterpret_cast<uint32_t*>(tile + (4 * pb + k) * kTrPitch + 4 * cb) = o[k];
  __syncthreads();
  // (C is a multiple of 4: a word of four channels is inside the tensor or outside it as a whole)
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int pl = 16 * k + (t >> 4), c4 = 4 * (t & 15);
    const int64_t p = p0 + pl, c = c0 + c4;
    if (p < HW && c < C)
      *reinterpret_cast<uint32_t*>(dst + p * C + c) = *reinterpret_cast<const uint32_t*>(tile + pl * kTrPitch + c4);
  }
}

int nchw_to_nhwc_u8_impl(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W, cudaStream_t st) {
  if (N < 0 || C < 0 || H < 0 || W < 0 || (C % 4) != 0) return B200Q_ERR_BAD_ARGUMENT;
  const int64_t HW = H * W;
  if (N == 0 || C == 0 || HW == 0) return B200Q_OK;
  if (!in || !out || (reinterpret_cast<uintptr_t>(out) & 3)) return B200Q_ERR_BAD_ARGUMENT;
  const int64_t bx = (HW + kTrTile - 1) / kTrTile, by = (C + kTrTile - 1) / kTrTile;
  if (bx > 0x7FFFFFFF || by > 65535 || N > 65535) return B200Q_ERR_TOO_LARGE;
  const int wide = (HW % 4) == 0 && (reinterpret_cast<uintptr_t>(in) & 3) == 0;
  launch_dependent(nchw_to_nhwc_u8_kernel, dim3((unsigned)bx, (unsigned)by, (unsigned)N), dim3(256), 0, st,
                   static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), C, HW, wide);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// im2col from the channels-last copy: out[(n, ho, wo)][k], k = (i, j, c - c0): every window
// position is cg contiguous bytes of one input pixel, so the matrix is built from 16-byte copies.
// A thread owns one 16-byte column piece (i, j, 16 channels) -- its window offset is computed once
// -- and walks kIm2Rows consecutive output rows, four loads in flight.
constexpr int kIm2Rows = 16;

struct Im2colNhwcParams {
  const uint8_t* in;
  uint8_t* out;
  int64_t C, H, W, Ho, Wo, rows, ld_out;
  int kh, kw, sh, sw, ph, pw, dh, dw;
  int64_t c0;
  int cg16, pieces, pieces_ld;  // 16-byte pieces per channel group, per window row (kh kw cg / 16), per output row
};

__global__ void __launch_bounds__(256) im2col_nhwc_u8_kernel(const Im2colNhwcParams p) {
  pdl_enter();
  const int64_t row0 = (int64_t)blockIdx.x * kIm2Rows;
  const int nrows = (int)(p.rows - row0 < kIm2Rows ? p.rows - row0 : kIm2Rows);
  // (n, ho, wo) of the block's first row
  const int64_t hw = p.Ho * p.Wo;
  const int64_t n0 = row0 / hw;
  const int ho0 = (int)((row0 - n0 * hw) / p.Wo), wo0 = (int)(row0 - n0 * hw - (int64_t)ho0 * p.Wo);
  for (int kp = threadIdx.x; kp < p.pieces_ld; kp += blockDim.x) {
    const bool pad = kp >= p.pieces;  // columns beyond kh kw cg: zeros
    const int ij = kp / p.cg16, c16 = kp - ij * p.cg16;
    const int i = ij / p.kw, j = ij - i * p.kw;
    const int dh_off = i * p.dh - p.ph, dw_off = j * p.dw - p.pw;
    // the walk over the rows keeps (h, w) of the window position and the byte offset of that input
    // pixel, stepping all three: no multiplication per row
    const int64_t w_step = (int64_t)p.sw * p.C;                                   // wo + 1
    const int64_t line_step = ((int64_t)p.sh * p.W - p.Wo * p.sw) * p.C;          // wo = Wo - 1 -> 0, ho + 1
    const int64_t image_step = ((int64_t)p.H - p.Ho * p.sh) * p.W * p.C;          // ho = Ho - 1 -> 0, n + 1
    int h = ho0 * p.sh + dh_off, w = wo0 * p.sw + dw_off;
    const uint8_t* src = p.in + p.c0 + 16 * (int64_t)c16 + ((n0 * p.H + h) * p.W + w) * p.C;
    uint8_t* dst = p.out + row0 * p.ld_out + 16 * (int64_t)kp;
    int ho = ho0, wo = wo0;
    for (int r = 0; r < nrows; r += 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        if (r + u < nrows) {
          if (!pad && (unsigned)h < (unsigned)p.H && (unsigned)w < (unsigned)p.W) v[u] = __ldg(reinterpret_cast<const uint4*>(src));
          w += p.sw;
          src += w_step;
          if (++wo == p.Wo) {
            wo = 0;
            w = dw_off;
            h += p.sh;
            src += line_step;
            if (++ho == p.Ho) {
              ho = 0;
              h = dh_off;
              src += image_step;
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (r + u < nrows) __stcs(reinterpret_cast<uint4*>(dst + (int64_t)(r + u) * p.ld_out), v[u]);
    }
  }
}

int im2col_nhwc_u8_impl(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W, int kh, int kw, int sh, int sw,
                        int ph, int pw, int dh, int dw, int64_t c0, int64_t cg, int64_t ld_out, cudaStream_t st) {
  if (N < 0 || C <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0 || dh <= 0 || dw <= 0 ||
      c0 < 0 || cg <= 0 || c0 + cg > C)
    return B200Q_ERR_BAD_ARGUMENT;
  if ((C % 16) || (c0 % 16) || (cg % 16) || (ld_out % 16) || ld_out < cg * kh * kw) return B200Q_ERR_BAD_ARGUMENT;
  const int64_t Ho = (H + 2 * ph - (int64_t)dh * (kh - 1) - 1) / sh + 1, Wo = (W + 2 * pw - (int64_t)dw * (kw - 1) - 1) / sw + 1;
  if (Ho <= 0 || Wo <= 0) return B200Q_ERR_BAD_ARGUMENT;
  if (N == 0) return B200Q_OK;
  if (!in || !out || ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15)) return B200Q_ERR_BAD_ARGUMENT;
  if (cg * kh * kw / 16 > 0x7FFFFFFF || ld_out / 16 > 0x7FFFFFFF) return B200Q_ERR_TOO_LARGE;
  Im2colNhwcParams p;
  p.in = static_cast<const uint8_t*>(in); p.out = static_cast<uint8_t*>(out);
  p.C = C; p.H = H; p.W = W; p.Ho = Ho; p.Wo = Wo; p.rows = N * Ho * Wo; p.ld_out = ld_out;
  p.kh = kh; p.kw = kw; p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw; p.dh = dh; p.dw = dw;
  p.c0 = c0; p.cg16 = (int)(cg / 16); p.pieces = (int)(cg * kh * kw / 16); p.pieces_ld = (int)(ld_out / 16);
  const int64_t blocks = (p.rows + kIm2Rows - 1) / kIm2Rows;
  if (blocks > 0x7FFFFFFF) return B200Q_ERR_TOO_LARGE;
  int threads = 32;
  while (threads < 256 && threads < p.pieces_ld) threads += 32;
  launch_dependent(im2col_nhwc_u8_kernel, dim3((unsigned)blocks), dim3(threads), 0, st, p);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // namespace b200q
