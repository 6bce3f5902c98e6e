// dequant_int4: packed 4-bit weights -> bf16 / fp32, (nibble - zero_point) * scale.
//
// HBM-bound: 0.5 B read and 2 B (bf16) written per weight.  One thread expands one
// packed word per step; a warp reads 128 contiguous bytes and writes 512 (bf16)
// contiguous bytes with 128-bit stores.  Scales and packed zero points of a group
// are re-read by every row of the group and stay in L1/L2.
#include "common.cuh"

namespace b200q {

struct DequantParams {
  const int32_t* packed;
  const void* scale;
  const void* zp;
  void* out;
  int64_t rows, cols_packed, scale_rows, group_rows;
  int zp_kind, is_signed;
  int64_t col_blocks;  // blocks along the columns; the 1-D grid is col_blocks * row_blocks
};

template <bool SIGNED>
__device__ __forceinline__ int nib(uint32_t w, int i) {
  int v = (int)((w >> (4 * i)) & 0xFu);
  if (SIGNED) v = (v ^ 8) - 8;
  return v;
}

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) { return round_to_bf16(v); }

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* f, bool vec);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* f, bool vec) {
  if (vec) {
    float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = p[i];
  }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f, bool vec) {
  if (vec) {
    uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(p[i]);
  }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float* f, bool vec);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float* f, bool vec) {
  if (vec) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(f[0], f[1], f[2], f[3]));
    __stcs(reinterpret_cast<float4*>(p) + 1, make_float4(f[4], f[5], f[6], f[7]));
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = f[i];
  }
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* f, bool vec) {
  if (vec) {
    __stcs(reinterpret_cast<uint4*>(p), make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                                    pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7])));
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = __float2bfloat16_rn(f[i]);
  }
}

// (q - zp) * scale for the 8 values of one word; every float step is rounded in T.
template <typename T, bool SIGNED>
__device__ __forceinline__ void expand_word(uint32_t w, const float* s, int zp_kind, uint32_t zw, const float* zf,
                                            float* o) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int q = nib<SIGNED>(w, i);
    float d;
    if (zp_kind == B200Q_ZP_PACKED) d = (float)(q - nib<SIGNED>(zw, i));
    else if (zp_kind == B200Q_ZP_FLOAT) d = round_to<T>((float)q - zf[i]);
    else d = (float)q;
    o[i] = d * s[i];  // the store rounds to T
  }
}


// ---- packed bf16x2 expansion (bf16 output, packed or no zero point) --------------------------
// A nibble q OR-ed into the mantissa of the bf16 constant 128.0 (0x4300) is exactly 128 + q, so
// two nibbles become a bf16x2 with one shift and one logic op, (128+q) - (128+z) is exact, and
// the product with the bf16 scale is a single bf16x2 multiply with one rounding: the same value
// as (q - z) converted to bf16 and multiplied by the scale in bf16.
// Pair i of a word holds nibbles i and i+4 (low / high half).
template <bool SIGNED>
__device__ __forceinline__ uint32_t nib_pair(uint32_t w, int i) {
  // signed: (q ^ 8) is q + 8 for the two's-complement nibble, and 0x4308 is 128 + 8
  return SIGNED ? (((w >> (4 * i)) & 0x000F000Fu) ^ 0x43084308u) : (((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u);
}
__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Scales / zero references of one group, re-paired to (i, i+4) order once per group.
struct GroupBf2 {
  uint32_t sp[4];  // {s_i, s_{i+4}}
  uint32_t zr[4];  // {128 + z_i, 128 + z_{i+4}} (or the plain offset when there is no zero point)
};

template <bool SIGNED>
__device__ __forceinline__ void load_group_bf2(GroupBf2& g, const __nv_bfloat16* scale8, bool has_zp, uint32_t zw) {
  uint4 s = __ldg(reinterpret_cast<const uint4*>(scale8));  // s0..s7 in natural order
  g.sp[0] = __byte_perm(s.x, s.z, 0x5410);  // {s0, s4}
  g.sp[1] = __byte_perm(s.x, s.z, 0x7632);  // {s1, s5}
  g.sp[2] = __byte_perm(s.y, s.w, 0x5410);  // {s2, s6}
  g.sp[3] = __byte_perm(s.y, s.w, 0x7632);  // {s3, s7}
#pragma unroll
  for (int i = 0; i < 4; ++i) g.zr[i] = has_zp ? nib_pair<SIGNED>(zw, i) : (SIGNED ? 0x43084308u : 0x43004300u);
}

template <bool SIGNED>
__device__ __forceinline__ uint4 expand_word_bf2(uint32_t w, const GroupBf2& g) {
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = bf2_mul(bf2_sub(nib_pair<SIGNED>(w, i), g.zr[i]), g.sp[i]);  // {o_i, o_{i+4}}
  return make_uint4(__byte_perm(o[0], o[1], 0x5410), __byte_perm(o[2], o[3], 0x5410),   // o0 o1 | o2 o3
                    __byte_perm(o[0], o[1], 0x7632), __byte_perm(o[2], o[3], 0x7632));  // o4 o5 | o6 o7
}

constexpr int kFastRows = 16;

// bf16 output, operator layout, 16-byte aligned everything: one thread expands one packed word
// of each of kFastRows consecutive rows (all loads issued before the first use).
template <bool SIGNED>
__global__ void __launch_bounds__(256) dequant_rowpacked_bf16_kernel(DequantParams p) {
  pdl_enter();
  const int64_t bx = blockIdx.x % p.col_blocks, by = blockIdx.x / p.col_blocks;
  const int64_t cp = bx * blockDim.x + threadIdx.x;
  if (cp >= p.cols_packed) return;
  const int64_t cols = p.cols_packed * 8;
  const __nv_bfloat16* scale = static_cast<const __nv_bfloat16*>(p.scale);
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
  const int64_t r0 = by * kFastRows;
  uint32_t w[kFastRows];
#pragma unroll
  for (int j = 0; j < kFastRows; ++j) {
    int64_t r = r0 + j;
    w[j] = r < p.rows ? (uint32_t)__ldcs(p.packed + r * p.cols_packed + cp) : 0u;
  }
  // group index of the first row by one division, then by counting (a 64-bit division per row
  // would cost more than the expansion itself)
  int64_t sr = r0 / p.group_rows;
  int64_t left = (sr + 1) * p.group_rows - r0;  // rows of this block that still belong to group sr
  bool fresh = true;
  GroupBf2 g;
  __nv_bfloat16* orow = out + r0 * cols + cp * 8;
#pragma unroll
  for (int j = 0; j < kFastRows; ++j) {
    if (r0 + j >= p.rows) break;
    if (left == 0) {
      ++sr;
      left = p.group_rows;
      fresh = true;
    }
    if (fresh) {
      uint32_t zw = 0;
      if (p.zp_kind == B200Q_ZP_PACKED) zw = (uint32_t)__ldg(static_cast<const int32_t*>(p.zp) + sr * p.cols_packed + cp);
      load_group_bf2<SIGNED>(g, scale + sr * cols + cp * 8, p.zp_kind == B200Q_ZP_PACKED, zw);
      fresh = false;
    }
    --left;
    __stcs(reinterpret_cast<uint4*>(orow), expand_word_bf2<SIGNED>(w[j], g));
    orow += cols;
  }
}

constexpr int kRowsPerBlock = 8;

// Operator layout: packed [rows][cols_packed] -> out [rows][8*cols_packed].
template <typename T, bool SIGNED>
__global__ void __launch_bounds__(256) dequant_rowpacked_kernel(DequantParams p) {
  pdl_enter();
  const int64_t bx = blockIdx.x % p.col_blocks, by = blockIdx.x / p.col_blocks;
  const int64_t cp = bx * blockDim.x + threadIdx.x;
  if (cp >= p.cols_packed) return;
  const int64_t cols = p.cols_packed * 8;
  const T* scale = static_cast<const T*>(p.scale);
  T* out = static_cast<T*>(p.out);
  const bool vec = (cols * sizeof(T)) % 16 == 0 &&
                   ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scale) |
                     (p.zp_kind == B200Q_ZP_FLOAT ? reinterpret_cast<uintptr_t>(p.zp) : 0)) & 15) == 0;
  const int64_t r0 = by * kRowsPerBlock;
  uint32_t w[kRowsPerBlock];
#pragma unroll
  for (int j = 0; j < kRowsPerBlock; ++j) {
    int64_t r = r0 + j;
    w[j] = r < p.rows ? (uint32_t)__ldcs(p.packed + r * p.cols_packed + cp) : 0u;
  }
  int64_t last_sr = -1;
  float s[8], zf[8];
  uint32_t zw = 0;
#pragma unroll
  for (int j = 0; j < kRowsPerBlock; ++j) {
    int64_t r = r0 + j;
    if (r >= p.rows) break;
    int64_t sr = r / p.group_rows;
    if (sr != last_sr) {
      load8<T>(scale + sr * cols + cp * 8, s, vec);
      if (p.zp_kind == B200Q_ZP_PACKED) zw = (uint32_t)__ldg(static_cast<const int32_t*>(p.zp) + sr * p.cols_packed + cp);
      else if (p.zp_kind == B200Q_ZP_FLOAT) load8<T>(static_cast<const T*>(p.zp) + sr * cols + cp * 8, zf, vec);
      last_sr = sr;
    }
    float o[8];
    expand_word<T, SIGNED>(w[j], s, p.zp_kind, zw, zf, o);
    store8<T>(out + r * cols + cp * 8, o, vec);
  }
}

// AutoGPTQ layout: packed [rows/8][cols]; nibble i of word (pr, c) is W[8*pr+i][c].
// One thread takes 8 consecutive words of a packed row -> an 8x8 block of the output.
template <typename T, bool SIGNED>
__global__ void __launch_bounds__(256) dequant_kpacked_kernel(DequantParams p) {
  pdl_enter();
  const int64_t cols = p.cols_packed;  // carries the number of columns in this layout
  const int64_t c8 = (blockIdx.x % p.col_blocks) * blockDim.x + threadIdx.x;  // block of 8 columns
  const int64_t pr = blockIdx.x / p.col_blocks;
  if (c8 * 8 >= cols) return;
  const T* scale = static_cast<const T*>(p.scale);
  T* out = static_cast<T*>(p.out);
  const bool vec = (cols * sizeof(T)) % 16 == 0 &&
                   ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scale) |
                     reinterpret_cast<uintptr_t>(p.packed)) & 15) == 0 && cols % 8 == 0;
  const int64_t c = c8 * 8;
  uint32_t w[8];
  const int32_t* src = p.packed + pr * cols + c;
  if (vec && (cols % 4) == 0) {
    uint4 a = __ldcs(reinterpret_cast<const uint4*>(src)), b = __ldcs(reinterpret_cast<const uint4*>(src) + 1);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = (uint32_t)src[i];
  }
  const int64_t sr = (pr * 8) / p.group_rows;
  float s[8];
  load8<T>(scale + sr * cols + c, s, vec);
  uint32_t zw = 0;
  if (p.zp_kind == B200Q_ZP_PACKED) zw = (uint32_t)__ldg(static_cast<const int32_t*>(p.zp) + sr * (cols / 8) + c8);
#pragma unroll
  for (int i = 0; i < 8; ++i) {  // output row 8*pr + i
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int q = nib<SIGNED>(w[j], i);
      int z = p.zp_kind == B200Q_ZP_PACKED ? nib<SIGNED>(zw, j) : 0;
      o[j] = (float)(q - z) * s[j];
    }
    store8<T>(out + (pr * 8 + i) * cols + c, o, vec);
  }
}

// every dequantisation kernel calls pdl_enter() first: it may be launched under its predecessor's tail
template <typename Kernel, typename Params>
static void launch_or_fallback(Kernel kernel, dim3 grid, cudaStream_t st, const Params& p) {
  if (launch_overlapped(kernel, grid, dim3(256), 0, st, p) == cudaSuccess) return;
  (void)cudaGetLastError();
  kernel<<<grid, 256, 0, st>>>(p);
}

int dequant_int4_impl(const int32_t* packed, const void* scale, const void* zp, int zp_kind, int is_signed,
                      int out_dtype, void* out, int64_t rows, int64_t cols_packed, int64_t scale_rows, int k_packed,
                      cudaStream_t st) {
  if (rows == 0 || cols_packed == 0) return B200Q_OK;
  if (scale_rows <= 0 || rows % scale_rows) return B200Q_ERR_BAD_ARGUMENT;
  DequantParams p;
  p.packed = packed; p.scale = scale; p.zp = zp; p.out = out; p.rows = rows; p.cols_packed = cols_packed;
  p.scale_rows = scale_rows; p.group_rows = rows / scale_rows; p.zp_kind = zp_kind; p.is_signed = is_signed;
  const bool all_aligned = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scale) |
                              reinterpret_cast<uintptr_t>(packed)) & 15) == 0;
  if (!k_packed && out_dtype == B200Q_BF16 && zp_kind != B200Q_ZP_FLOAT && all_aligned) {
    p.col_blocks = (cols_packed + 255) / 256;
    const int64_t nblk = p.col_blocks * ((rows + kFastRows - 1) / kFastRows);
    if (nblk > 0x7FFFFFFFll) return B200Q_ERR_TOO_LARGE;
    if (is_signed) launch_or_fallback(dequant_rowpacked_bf16_kernel<true>, dim3((unsigned)nblk), st, p);
    else launch_or_fallback(dequant_rowpacked_bf16_kernel<false>, dim3((unsigned)nblk), st, p);
  } else if (!k_packed) {
    p.col_blocks = (cols_packed + 255) / 256;
    const int64_t nblk = p.col_blocks * ((rows + kRowsPerBlock - 1) / kRowsPerBlock);
    if (nblk > 0x7FFFFFFFll) return B200Q_ERR_TOO_LARGE;
    const unsigned grid = (unsigned)nblk;
    if (out_dtype == B200Q_BF16) {
      if (is_signed) launch_or_fallback(dequant_rowpacked_kernel<__nv_bfloat16, true>, dim3(grid), st, p);
      else launch_or_fallback(dequant_rowpacked_kernel<__nv_bfloat16, false>, dim3(grid), st, p);
    } else {
      if (is_signed) launch_or_fallback(dequant_rowpacked_kernel<float, true>, dim3(grid), st, p);
      else launch_or_fallback(dequant_rowpacked_kernel<float, false>, dim3(grid), st, p);
    }
  } else {
    if (rows % 8 || cols_packed % 8 || p.group_rows % 8 || zp_kind == B200Q_ZP_FLOAT) return B200Q_ERR_UNSUPPORTED;
    p.col_blocks = (cols_packed / 8 + 255) / 256;
    const int64_t nblk = p.col_blocks * (rows / 8);
    if (nblk > 0x7FFFFFFFll) return B200Q_ERR_TOO_LARGE;
    const unsigned grid = (unsigned)nblk;
    if (out_dtype == B200Q_BF16) {
      if (is_signed) launch_or_fallback(dequant_kpacked_kernel<__nv_bfloat16, true>, dim3(grid), st, p);
      else launch_or_fallback(dequant_kpacked_kernel<__nv_bfloat16, false>, dim3(grid), st, p);
    } else {
      if (is_signed) launch_or_fallback(dequant_kpacked_kernel<float, true>, dim3(grid), st, p);
      else launch_or_fallback(dequant_kpacked_kernel<float, false>, dim3(grid), st, p);
    }
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// ------------------------------------------------------------------ AutoGPTQ -> operator layout
// AutoGPTQ checkpoints pack the weight nibbles along K (qweight [K/8][N], nibble i of word (p, n)
// is W[8p+i][n]) and store zero points minus one (qzeros [K/g][N/8], packed along N).  The
// operator wants nibbles packed along N ([K][N/8]) and the true zero points.  One thread
// transposes an 8x8 nibble block: 8 consecutive words of a packed row in, one word for each
// of 8 consecutive rows out.
__global__ void __launch_bounds__(256) gptq_repack_weight_kernel(const int32_t* __restrict__ in, int32_t* __restrict__ out,
                                                                 int64_t K8, int64_t N8) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= K8 * N8) return;
  const int64_t p = t / N8, m = t % N8;
  const int64_t N = N8 * 8;
  uint32_t w[8];
  const uint4* src = reinterpret_cast<const uint4*>(in + p * N + m * 8);
  uint4 a = __ldcs(src), b = __ldcs(src + 1);
  w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t o = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) o |= ((w[j] >> (4 * i)) & 0xFu) << (4 * j);
    out[(p * 8 + i) * N8 + m] = (int32_t)o;
  }
}

// every nibble + 1 (mod 16)
__global__ void __launch_bounds__(256) gptq_zeros_plus_one_kernel(const int32_t* __restrict__ in, int32_t* __restrict__ out,
                                                                  int64_t n) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n) return;
  const uint32_t z = (uint32_t)in[t];
  const uint32_t lo = ((z & 0x0F0F0F0Fu) + 0x01010101u) & 0x0F0F0F0Fu;
  const uint32_t hi = (((z >> 4) & 0x0F0F0F0Fu) + 0x01010101u) & 0x0F0F0F0Fu;
  out[t] = (int32_t)(lo | (hi << 4));
}

int gptq_repack_impl(const int32_t* qweight, int32_t* qweight_out, int64_t K, int64_t N, const int32_t* qzeros,
                     int32_t* qzeros_out, int64_t zeros_words, cudaStream_t st) {
  if (K % 8 || N % 8) return B200Q_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(qweight) & 15) || (N % 4)) return B200Q_ERR_UNSUPPORTED;
  const int64_t items = (K / 8) * (N / 8);
  if (items > 0) {
    gptq_repack_weight_kernel<<<(unsigned)((items + 255) / 256), 256, 0, st>>>(qweight, qweight_out, K / 8, N / 8);
    B200Q_LAUNCH_CHECK();
  }
  if (qzeros && zeros_words > 0) {
    gptq_zeros_plus_one_kernel<<<(unsigned)((zeros_words + 255) / 256), 256, 0, st>>>(qzeros, qzeros_out, zeros_words);
    B200Q_LAUNCH_CHECK();
  }
  return B200Q_OK;
}

}  // namespace b200q
