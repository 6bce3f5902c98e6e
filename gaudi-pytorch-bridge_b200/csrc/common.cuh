// Shared device/host helpers for the b200q kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "b200q.h"

namespace b200q {

constexpr int kNumSMs = 148;  // B200

// ---- host-side bookkeeping (abi.cu owns the storage) ----
extern std::atomic<uint64_t> g_launches;
int record_cuda_error(cudaError_t e, const char* where);
inline void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

#define B200Q_CUDA_OK(expr)                                                   \
  do {                                                                        \
    cudaError_t e__ = (expr);                                                 \
    if (e__ != cudaSuccess) return ::b200q::record_cuda_error(e__, #expr);    \
  } while (0)

#define B200Q_LAUNCH_CHECK()                                                  \
  do {                                                                        \
    ::b200q::count_launch();                                                  \
    cudaError_t e__ = cudaGetLastError();                                     \
    if (e__ != cudaSuccess) return ::b200q::record_cuda_error(e__, "launch"); \
  } while (0)

// Programmatic dependent launch.  A kernel launched with launch_overlapped() may be set up and
// start running before the kernel in front of it in the stream has finished; it must call
// pdl_enter() before its first access to global memory (the call returns once that kernel
// and its writes are complete), and everything before the call -- block scheduling, barrier and
// tensor-memory set-up, descriptor prefetch -- overlaps the predecessor's tail.  pdl_enter() also
// lets the successor be set up early in the same way.  Both parts are no-ops in an ordinary
// launch.  Between two kernels of 10-30 us this takes 1.5-2.5 us of launch gap away.
#ifdef __CUDACC__
// Lets the kernel behind this one in the stream be set up now, without waiting for anything
// itself: for a kernel that is launched behind a kernel which has already waited (the amax
// clearing kernel) and waits on its own only before it publishes (block_amax_to_global).
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// launch_overlapped() with the ordinary launch as its fallback (for a driver that refuses the
// attribute); the kernel calls pdl_enter() before its first access to global memory.
template <typename... KArgs, typename... Args>
inline void launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  if (launch_overlapped(kernel, grid, block, smem, st, args...) == cudaSuccess) return;
  (void)cudaGetLastError();
  kernel<<<grid, block, smem, st>>>(static_cast<KArgs>(args)...);
}
#endif

// Clears an amax word with a one-thread kernel behind which the kernel that accumulates into it
// (through block_amax_to_global, which waits for the clearing kernel before its atomicMax) can be
// launched with launch_overlapped().  Defined beside the casts.
int clear_amax(float* amax, cudaStream_t st);

// Per-device one-time setup helper: `slot` is a static array of kMaxDevices ints owned by the
// caller (0 = not yet done on that device).  Returns the current device index or -1.
constexpr int kMaxDevices = 64;
inline int current_device_index() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// Device status word of the current device: 0 = fine; kernels with bounded waits write a
// code here.  Returns null if its address cannot be obtained.
int* device_status_ptr();

// ---- small device helpers ----
__device__ __forceinline__ float bf16_bits_to_float(uint32_t b16) { return __uint_as_float(b16 << 16); }

__device__ __forceinline__ float round_to_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

template <int FMT>
struct Fp8Fmt;
template <>
struct Fp8Fmt<B200Q_E4M3> {
  static constexpr float kMax = 448.f;
  static constexpr int kMant = 3;
  static constexpr int kEmin = 127 - 6;  // biased fp32 exponent of the smallest normal
  static constexpr float kQuantum = 0.001953125f;  // 2^-9
  static constexpr __nv_fp8_interpretation_t kInterp = __NV_E4M3;
};
template <>
struct Fp8Fmt<B200Q_E5M2> {
  static constexpr float kMax = 57344.f;
  static constexpr int kMant = 2;
  static constexpr int kEmin = 127 - 14;
  static constexpr float kQuantum = 1.52587890625e-05f;  // 2^-16
  static constexpr __nv_fp8_interpretation_t kInterp = __NV_E5M2;
};

// Two floats -> two fp8 bytes (a in the low byte), round half to even, saturating.
template <int FMT>
__device__ __forceinline__ uint32_t cvt_fp8x2(float a, float b) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, Fp8Fmt<FMT>::kInterp);
}

template <int FMT>
__device__ __forceinline__ float fp8_to_float(uint32_t byte) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, Fp8Fmt<FMT>::kInterp);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

template <int FMT>
__device__ __forceinline__ float clampf(float v) {
  // fminf/fmaxf drop NaN; NaN bytes are patched by the caller from the unclamped value.
  return fminf(fmaxf(v, -Fp8Fmt<FMT>::kMax), Fp8Fmt<FMT>::kMax);
}

// silu(g) * u: silu in fp32, product rounded once to bf16 (the dtype the unfused graph would
// hold).  Shared by the stand-alone SwiGLU + cast kernel and the fused GEMM epilogue, which
// must produce the same bytes.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  float s = g / (1.f + expf(-g));
  return round_to_bf16(s * u);
}

// Philox4x32-10; counter = (block lo, block hi, offset lo, offset hi), key = seed.
__device__ __forceinline__ uint4 philox4x32_10(uint64_t block, uint64_t seed, uint64_t offset) {
  uint32_t c0 = (uint32_t)block, c1 = (uint32_t)(block >> 32);
  uint32_t c2 = (uint32_t)offset, c3 = (uint32_t)(offset >> 32);
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// Stochastic rounding of the fp32 product v to a float that the fp8 format represents exactly
// (NaN passes through; the caller writes the NaN byte).  r holds RB random bits (8 when v is a
// bf16 value, 16 otherwise).  With d = 23 - mantissa bits and g = d - 16:
//   a = min(|v|, max); below the smallest normal the value is first lifted by that amount so
//   that the dropped bits sit at the same place (u = a + 2^Emin, an fp32 addition);
//   r_d = (r >> (8 - g)) << 16 for RB == 8 in the normal range (the top g bits are all that a
//   bf16 value can need), otherwise (r << (d - RB)) + (1 << (d - RB - 1));
//   bits(u) += r_d, low d bits cleared, the lift removed, clamped to max, sign restored.
template <int FMT, int RB>
__device__ __forceinline__ float sr_round(float v, uint32_t r) {
  constexpr int d = 23 - Fp8Fmt<FMT>::kMant;
  constexpr int g = d - 16;
  const float min_normal = __uint_as_float((uint32_t)Fp8Fmt<FMT>::kEmin << 23);
  const uint32_t sign = __float_as_uint(v) & 0x80000000u;
  if (v != v) return v;
  const float a = fminf(fabsf(v), Fp8Fmt<FMT>::kMax);
  const bool sub = a < min_normal;
  const float u = sub ? a + min_normal : a;
  uint32_t r_d = (r << (d - RB)) + (1u << (d - RB - 1));
  if (RB == 8 && !sub) r_d = (r >> (8 - g)) << 16;
  const uint32_t b = (__float_as_uint(u) + r_d) & ~((1u << d) - 1u);
  float res = __uint_as_float(b);
  if (sub) res -= min_normal;
  res = fminf(res, Fp8Fmt<FMT>::kMax);
  return __uint_as_float(__float_as_uint(res) | sign);
}

// The RB random bits of global element index gi (see philox4x32_10): block gi / (128 / RB),
// consecutive bytes (RB = 8) or halves (RB = 16) of the block's four words.
template <int RB>
__device__ __forceinline__ uint32_t sr_random_bits(uint64_t gi, uint64_t seed, uint64_t offset) {
  constexpr int per = 128 / RB, per_word = 32 / RB;
  const uint4 r = philox4x32_10(gi / per, seed, offset);
  const int e = (int)(gi % per);
  const int w = e / per_word;
  const uint32_t word = w == 0 ? r.x : w == 1 ? r.y : w == 2 ? r.z : r.w;
  return (word >> ((e % per_word) * RB)) & ((1u << RB) - 1u);
}

__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// Block-wide max of a non-negative float's bit pattern, then one atomicMax per block.
// Works on bit patterns so that NaN (pattern above +inf) wins and is propagated.
__device__ __forceinline__ void block_amax_to_global(uint32_t local_bits, float* amax) {
  __shared__ uint32_t s_warp[32];
  uint32_t w = warp_max_u32(local_bits);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) s_warp[wid] = w;
  __syncthreads();
  if (wid == 0) {
    int nw = (blockDim.x + 31) >> 5;
    uint32_t v = lane < nw ? s_warp[lane] : 0u;
    v = warp_max_u32(v);
    if (lane == 0 && v != 0u) {
      // (a kernel launched with programmatic stream serialization behind the kernel that clears
      // `amax` must not touch it before that kernel is complete; a no-op in an ordinary launch)
      asm volatile("griddepcontrol.wait;" ::: "memory");
      atomicMax(reinterpret_cast<unsigned int*>(amax), v);
    }
  }
}

}  // namespace b200q
