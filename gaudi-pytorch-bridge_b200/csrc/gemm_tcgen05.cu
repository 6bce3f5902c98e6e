// FP8 GEMM on the 5th-generation tensor cores: out = (A[M][K] . B[N][K]^T) * scales + bias (+ D).
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0    TMA producer: 128-byte-swizzled K-major tiles of both operands into a
//             shared-memory ring (no multicast), completion on "full" mbarriers
//   warp 1    TMEM owner and MMA issuer: one thread issues tcgen05.mma.kind::f8f6f4
//             (128 x BN x 32 per instruction), tcgen05.commit releases ring stages
//             and publishes finished accumulators
//   warps 2-5 epilogue: tcgen05.ld the fp32 accumulator (each warp its 32 TMEM lanes),
//             apply (acc * sa) * sb + bias + D, round once, store
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// SWAP = false: lanes <- rows of A (tokens), columns <- rows of B (output channels).
// SWAP = true : lanes <- rows of B, columns <- rows of A: the small-M ("decode") form where
//               the weight stream fills the 128-lane dimension and the few tokens ride N.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "gemm_common.cuh"
#include "tcgen05_ptx.cuh"
#include "tma_host.cuh"

namespace b200q {

using namespace ptx;

constexpr int kBlockX = 128;  // rows of the lane-side operand per tile (UMMA M)
constexpr int kBlockK = 128;  // bytes (= fp8 elements) of K per ring stage: one swizzle row
constexpr int kUmmaK = 32;
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kTileOverheadCols = 590;  // width-independent part of a tile's cost, in columns (see the width choice)

enum { kErrProducer = 101, kErrMma = 102, kErrMmaTmem = 103, kErrEpilogue = 104 };

struct TcGemmParams {
  GemmParams g;
  int64_t x_rows, y_rows;  // extents of the lane-side / column-side operands
  int x_tiles, y_tiles, num_kb;
  // rows of the lane-side operand a tile covers (single-CTA kernel): 128, or fewer (a multiple of 8)
  // in the few-token form, where the tile count, not the tile height, must match the machine
  int x_tile_rows;
  int a_fmt_bits, b_fmt_bits;  // 0 = e4m3, 1 = e5m2 (lane-side, column-side)
  int x_mn, y_mn;              // 1 = that operand is stored MN-major ([K][rows], rows contiguous)
  int* status;                 // device status word (bounded waits report here)
  int no_probe;                // 1 = the MMA issuer ignores its look-ahead barrier probe (for comparison)
};

// KPS = k-blocks per ring stage.  A stage is KPS sub-stages [X tile][Y tile] of one k-block each;
// the barrier handshake (full / empty) is per stage.
template <int BN, int STAGES, int KPS = 1>
struct SmemLayout {
  static constexpr int kXBytes = kBlockX * kBlockK;
  static constexpr int kYBytes = BN * kBlockK;
  static constexpr int kSubBytes = kXBytes + kYBytes;
  static constexpr int kStageBytes = KPS * kSubBytes;
  static_assert(kSubBytes % 1024 == 0, "swizzled tiles need 1024-byte alignment");
  static constexpr int kRing = STAGES * kStageBytes;
  static constexpr int kEpiFloats = 2 * 3 * BN;  // per accumulator: col scale A, col scale B, col bias
  static constexpr int kBarOffset = kRing + kEpiFloats * 4;
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
};

// ---------------------------------------------------------------------------- epilogue pieces
// Per-thread (lane-side) and per-column epilogue operands of one tile.  Scales multiply in the
// order (acc * sa) * sb; a scalar or lane-side scale lives in rA / rB, a column-side one in
// shared memory (cA / cB), the other factor is 1.
struct EpiRow {
  float rA, rB, rBias;
  int64_t x;
  bool x_in;
};

template <int BN, bool SWAP>
__device__ __forceinline__ EpiRow epi_stage_operands(const GemmParams& g, int64_t x_rows, int64_t y_rows, int64_t x,
                                                     int64_t y0, int et, float* cA, float* cB, float* cBias) {
  // which output dimension the columns are: n (normal) or m (swapped)
  const int col_mode = SWAP ? B200Q_BCAST_PER_ROW : B200Q_BCAST_PER_COL;
  const int row_mode = SWAP ? B200Q_BCAST_PER_COL : B200Q_BCAST_PER_ROW;
  for (int c = et; c < BN; c += kEpiThreads) {
    const int64_t y = y0 + c;
    const bool in = y < y_rows;
    cA[c] = (g.a_scale_mode == col_mode && in) ? __ldg(g.a_scale + y) : 1.f;
    cB[c] = (g.b_scale_mode == col_mode && in) ? __ldg(g.b_scale + y) : 1.f;
    cBias[c] = (g.bias_mode == col_mode && in) ? ld_out_typed(g.bias, g.bias_dtype, y) : 0.f;
  }
  EpiRow r;
  r.x = x;
  r.x_in = x < x_rows;
  r.rA = 1.f; r.rB = 1.f; r.rBias = 0.f;
  if (g.a_scale_mode == B200Q_BCAST_SCALAR_HOST) r.rA = g.a_scale_host;
  else if (g.a_scale_mode == B200Q_BCAST_SCALAR_DEV) r.rA = __ldg(g.a_scale);
  else if (g.a_scale_mode == row_mode && r.x_in) r.rA = __ldg(g.a_scale + x);
  if (g.b_scale_mode == B200Q_BCAST_SCALAR_HOST) r.rB = g.b_scale_host;
  else if (g.b_scale_mode == B200Q_BCAST_SCALAR_DEV) r.rB = __ldg(g.b_scale);
  else if (g.b_scale_mode == row_mode && r.x_in) r.rB = __ldg(g.b_scale + x);
  if (g.bias_mode == row_mode && r.x_in) r.rBias = ld_out_typed(g.bias, g.bias_dtype, x);
  return r;
}

// Run-time choices of the epilogue that are the same for every element of a launch.
struct EpiFlags {
  bool full_extra, colA, colB, colBias;
  float s8;
};
template <bool SWAP>
__device__ __forceinline__ EpiFlags epi_flags(const GemmParams& g) {
  constexpr int kColMode = SWAP ? B200Q_BCAST_PER_ROW : B200Q_BCAST_PER_COL;
  EpiFlags f;
  f.full_extra = g.bias_mode == B200Q_BCAST_FULL || g.D != nullptr;
  f.colA = g.a_scale_mode == kColMode;
  f.colB = g.b_scale_mode == kColMode;
  f.colBias = g.bias_mode == kColMode;
  f.s8 = g.out8_dtype ? out8_scale_value(g) : 1.f;
  return f;
}

// CW accumulator values of this thread's lane (columns c0 .. c0 + CW of the tile) -> scaled,
// biased, rounded, stored.  The column-side operands come from shared memory as 16-byte vectors
// and only those that exist are read (a sixth of the shared-memory instructions of reading
// three scalars per element).
template <int CW>
__device__ __forceinline__ void epi_values(const uint32_t* r, int c0, const EpiRow& e, const float* cA, const float* cB,
                                           const float* cBias, const EpiFlags& f, float* v) {
  const float rA = e.rA, rB = e.rB, rBias = e.rBias;
  if (f.colA || f.colB || f.colBias) {
#pragma unroll
    for (int j = 0; j < CW; j += 4) {
      const float4 one = make_float4(1.f, 1.f, 1.f, 1.f), zero = make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 sa = f.colA ? *reinterpret_cast<const float4*>(cA + c0 + j) : one;
      const float4 sb = f.colB ? *reinterpret_cast<const float4*>(cB + c0 + j) : one;
      const float4 bb = f.colBias ? *reinterpret_cast<const float4*>(cBias + c0 + j) : zero;
      const float sav[4] = {sa.x, sa.y, sa.z, sa.w}, sbv[4] = {sb.x, sb.y, sb.z, sb.w}, bbv[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float a = __uint_as_float(r[j + q]);
        a = a * (rA * sav[q]);
        a = a * (rB * sbv[q]);
        v[j + q] = a + (rBias + bbv[q]);
      }
    }
  } else {
    // no column-side operand (the staged arrays hold 1, 1, 0): same arithmetic from registers
#pragma unroll
    for (int j = 0; j < CW; ++j) v[j] = (__uint_as_float(r[j]) * rA) * rB + rBias;
  }
}

template <int BN, bool SWAP>
__device__ __forceinline__ void epi_chunk(const GemmParams& g, const uint32_t* r, int c0, const EpiRow& e, int64_t y0,
                                          const float* cA, const float* cB, const float* cBias, const EpiFlags& f,
                                          uint32_t& code_max) {
  constexpr int CW = (BN % 32 == 0) ? 32 : 16;
  const int64_t x = e.x;
  const bool x_in = e.x_in;
  const float s8 = f.s8;
  const bool full_extra = f.full_extra;
  float v[CW];
  epi_values<CW>(r, c0, e, cA, cB, cBias, f, v);
  if (!SWAP) {
    // thread = output row m, registers = CW consecutive output columns n
    const int64_t m = x, n0 = y0 + c0;
    if (x_in) {
      if (full_extra) {
        // element-wise bias, then the accumulate input D: 16-byte loads of the thread's row segment where
        // the segment is whole and aligned (a 2-byte load per element and lane, each lane in another row,
        // made the accumulate form 3.5 times slower than the plain one), else element by element
        auto add_rowseg = [&](const void* base, int dtype, int64_t ld) {
          const int esz = dtype == B200Q_BF16 ? 2 : 4;
          const uint8_t* ptr = static_cast<const uint8_t*>(base) + (m * ld + n0) * esz;
          if (n0 + CW <= g.N && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0) {
            if (dtype == B200Q_BF16) {
#pragma unroll
              for (int j = 0; j < CW; j += 8) {
                const uint4 d = __ldg(reinterpret_cast<const uint4*>(ptr + 2 * j));
                const uint32_t w[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  v[j + 2 * k] += __uint_as_float(w[k] << 16);
                  v[j + 2 * k + 1] += __uint_as_float(w[k] & 0xFFFF0000u);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < CW; j += 4) {
                const float4 d = __ldg(reinterpret_cast<const float4*>(ptr + 4 * j));
                v[j] += d.x, v[j + 1] += d.y, v[j + 2] += d.z, v[j + 3] += d.w;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < CW; ++j)
              if (n0 + j < g.N) v[j] += ld_out_typed(base, dtype, m * ld + n0 + j);
          }
        };
        if (g.bias_mode == B200Q_BCAST_FULL) add_rowseg(g.bias, g.bias_dtype, g.bias_ld);
        if (g.D) add_rowseg(g.D, g.d_dtype, g.ldd);
      }
      if (g.out8_dtype) {
        uint8_t* o = static_cast<uint8_t*>(g.out) + m * g.ldo + n0;
        uint32_t w[CW / 4];
#pragma unroll
        for (int j = 0; j < CW; j += 4)
          w[j / 4] = out8_byte(g, v[j], s8) | (out8_byte(g, v[j + 1], s8) << 8) | (out8_byte(g, v[j + 2], s8) << 16) |
                     (out8_byte(g, v[j + 3], s8) << 24);
        if (n0 + CW <= g.N && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < CW / 4; j += 4) *reinterpret_cast<uint4*>(o + 4 * j) = make_uint4(w[j], w[j + 1], w[j + 2], w[j + 3]);
#pragma unroll
          for (int j = 0; j < CW / 4; ++j) code_max = __vmaxu4(code_max, w[j] & 0x7F7F7F7Fu);
        } else {
#pragma unroll
          for (int j = 0; j < CW; ++j)
            if (n0 + j < g.N) {
              o[j] = (uint8_t)(w[j / 4] >> (8 * (j & 3)));
              code_max = max(code_max, (w[j / 4] >> (8 * (j & 3))) & 0x7Fu);
            }
        }
      } else if (g.out_dtype == B200Q_BF16) {
        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(g.out) + m * g.ldo + n0;
        if (n0 + CW <= g.N && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < CW; j += 8)
            *reinterpret_cast<uint4*>(o + j) =
                make_uint4(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                           pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7]));
        } else if (n0 + CW <= g.N && (reinterpret_cast<uintptr_t>(o) & 7) == 0) {
          // a row pitch that is a multiple of 8 bytes only (N % 8 == 4): 8-byte stores
#pragma unroll
          for (int j = 0; j < CW; j += 4)
            *reinterpret_cast<uint2*>(o + j) = make_uint2(pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]));
        } else {
#pragma unroll
          for (int j = 0; j < CW; ++j)
            if (n0 + j < g.N) o[j] = __float2bfloat16_rn(v[j]);
        }
      } else {
        float* o = static_cast<float*>(g.out) + m * g.ldo + n0;
        if (n0 + CW <= g.N && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < CW; j += 4)
            *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < CW; ++j)
            if (n0 + j < g.N) o[j] = v[j];
        }
      }
    }
  } else {
    // thread = output column n (weight row), registers = CW consecutive tokens m
    const int64_t n = x;
    if (x_in && !full_extra && !g.out8_dtype) {
      // the common cases with every run-time choice hoisted out of the per-element loop (the
      // general loop below re-decides dtype, bias and accumulate input for every element and
      // runs several times slower)
      const int64_t left = g.M - (y0 + c0);
      if (g.out_dtype == B200Q_BF16) {
        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(g.out) + (y0 + c0) * g.ldo + n;
#pragma unroll
        for (int j = 0; j < CW; ++j)
          if (j < left) o[(int64_t)j * g.ldo] = __float2bfloat16_rn(v[j]);
      } else {
        float* o = static_cast<float*>(g.out) + (y0 + c0) * g.ldo + n;
#pragma unroll
        for (int j = 0; j < CW; ++j)
          if (j < left) o[(int64_t)j * g.ldo] = v[j];
      }
    } else if (x_in) {
#pragma unroll
      for (int j = 0; j < CW; ++j) {
        const int64_t m = y0 + c0 + j;
        if (m < g.M) {
          float o = v[j];
          if (g.bias_mode == B200Q_BCAST_FULL) o += ld_out_typed(g.bias, g.bias_dtype, m * g.bias_ld + n);
          if (g.D) o += ld_out_typed(g.D, g.d_dtype, m * g.ldd + n);
          if (g.out8_dtype) {
            const uint32_t byte = out8_byte(g, o, s8);
            static_cast<uint8_t*>(g.out)[m * g.ldo + n] = (uint8_t)byte;
            code_max = max(code_max, byte & 0x7Fu);
          } else if (g.out_dtype == B200Q_BF16) static_cast<__nv_bfloat16*>(g.out)[m * g.ldo + n] = __float2bfloat16_rn(o);
          else static_cast<float*>(g.out)[m * g.ldo + n] = o;
        }
      }
    }
  }
}

// TMEM accumulator (this warp's 32 lanes, BN columns from t_row) -> scaled, biased, rounded, stored.
template <int BN, bool SWAP>
__device__ __forceinline__ void epi_drain(const GemmParams& g, uint32_t t_row, const EpiRow& e, int64_t y0,
                                          const float* cA, const float* cB, const float* cBias) {
  const EpiFlags f = epi_flags<SWAP>(g);
  uint32_t code_max = 0;  // fused output cast: largest magnitude code (fp8 byte & 0x7F) this thread wrote, per byte lane
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 32) {
    uint32_t r[32];
    if (BN % 32 == 0) {
      tmem_ld_32x32(t_row + c0, r);
    } else {
      tmem_ld_32x16(t_row + c0, r);  // BN == 16
    }
    tmem_ld_wait();
    epi_chunk<BN, SWAP>(g, r, c0, e, y0, cA, cB, cBias, f, code_max);
  }
  if (g.out8_amax) {
    uint32_t m = max(max(code_max & 0xFFu, (code_max >> 8) & 0xFFu), max((code_max >> 16) & 0xFFu, code_max >> 24));
    m = __reduce_max_sync(0xFFFFFFFFu, m);
    if ((threadIdx.x & 31) == 0 && m) out8_amax_update(g, m);
  }
}

// Routed bf16 output (GemmParams::route_*): the rows of this CTA's tile belong to one destination
// buffer, possibly in another GPU's memory.  A thread's 64 output columns go through a 4 KB
// shared-memory patch of its warp (row per thread, 16-byte pieces XOR-swizzled by row so that
// neither side has bank conflicts) and leave as whole 128-byte row segments, four rows per store
// instruction: a peer write crosses NVLink as full lines instead of 32 scattered 16-byte pieces.
template <int BN>
__device__ __forceinline__ void epi_drain_routed(const GemmParams& g, uint32_t t_row, const EpiRow& e, int64_t row0,
                                                 int64_t y0, const float* cA, const float* cB, const float* cBias,
                                                 uint4* patch, int lane) {
  static_assert(BN % 64 == 0, "routed output is written in 64-column groups");
  const EpiFlags f = epi_flags<false>(g);
  // destination of this warp's 32 rows (row0 = first row; all of them in one route block)
  const int64_t blk = row0 / g.route_rows;
  __nv_bfloat16* dst0 = static_cast<__nv_bfloat16*>(g.route_out[blk]) +
                        (g.route_row_offset + (row0 - blk * g.route_rows)) * g.ldo;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 64) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t r[32];
      tmem_ld_32x32(t_row + c0 + 32 * h, r);
      tmem_ld_wait();
      float v[32];
      epi_values<32>(r, c0 + 32 * h, e, cA, cB, cBias, f, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int piece = 4 * h + k;
        patch[lane * 8 + (piece ^ (lane & 7))] =
            make_uint4(pack_bf16x2(v[8 * k], v[8 * k + 1]), pack_bf16x2(v[8 * k + 2], v[8 * k + 3]),
                       pack_bf16x2(v[8 * k + 4], v[8 * k + 5]), pack_bf16x2(v[8 * k + 6], v[8 * k + 7]));
      }
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int row = 4 * k + (lane >> 3), piece = lane & 7;
      const uint4 val = patch[row * 8 + (piece ^ (row & 7))];
      const int64_t n = y0 + c0 + piece * 8;
      if (row0 + row < g.M && n + 8 <= g.N)
        *reinterpret_cast<uint4*>(dst0 + (int64_t)row * g.ldo + n) = val;
    }
    __syncwarp();
  }
}

// Fused SwiGLU epilogue of a 256-column tile whose columns [0, 128) are gate and [128, 256) up
// projections of the same 128 hidden units (GemmParams::swiglu): both halves get the GEMM's
// scale / bias epilogue and its rounding to bf16, then silu(gate) * up -> bf16 -> * scale -> bf16
// -> e4m3, with the same device functions as swiglu_cast_kernel so that the bytes are those of
// the unfused pair of operators.  128 bytes per row and tile instead of 512 + a second pass.
__device__ __forceinline__ void epi_drain_swiglu(const GemmParams& g, uint32_t t_row, const EpiRow& e, int64_t y0,
                                                 const float* cA, const float* cB, const float* cBias) {
  const int64_t m = e.x;
  const float rA = e.rA, rB = e.rB, rBias = e.rBias;
  const float s_act = round_to_bf16(out8_scale_value(g));
  const int64_t f0 = (y0 >> 8) << 7;  // first hidden unit of the tile
  const int64_t F = g.N >> 1;
#pragma unroll 1
  for (int c0 = 0; c0 < 128; c0 += 32) {
    uint32_t rg[32], ru[32];
    tmem_ld_32x32(t_row + c0, rg);
    tmem_ld_32x32(t_row + 128 + c0, ru);
    tmem_ld_wait();
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      float y[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int cg = c0 + j + q, cu = 128 + cg;
        float a = __uint_as_float(rg[j + q]);
        a = a * (rA * cA[cg]);
        a = a * (rB * cB[cg]);
        a = round_to_bf16(a + (rBias + cBias[cg]));
        float b = __uint_as_float(ru[j + q]);
        b = b * (rA * cA[cu]);
        b = b * (rB * cB[cu]);
        b = round_to_bf16(b + (rBias + cBias[cu]));
        y[q] = round_to_bf16(silu_mul_bf16(a, b) * s_act);
      }
      o[j >> 2] = cvt_fp8x2<B200Q_E4M3>(clampf<B200Q_E4M3>(y[0]), clampf<B200Q_E4M3>(y[1])) |
                  (cvt_fp8x2<B200Q_E4M3>(clampf<B200Q_E4M3>(y[2]), clampf<B200Q_E4M3>(y[3])) << 16);
    }
    if (e.x_in) {
      uint8_t* dst = static_cast<uint8_t*>(g.out) + m * g.ldo + f0 + c0;
      if (f0 + c0 + 32 <= F && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(o[4], o[5], o[6], o[7]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (f0 + c0 + j < F) dst[j] = (uint8_t)(o[j >> 2] >> (8 * (j & 3)));
      }
    }
  }
}

template <int BN, int STAGES, bool SWAP, int KPS = 1>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                    const TcGemmParams p) {
  using L = SmemLayout<BN, STAGES, KPS>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up to the swizzle atom
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* epi_f = reinterpret_cast<float*>(smem + L::kRing);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_stop = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // TMEM is allocated in powers of two columns (two accumulators of BN columns each)
  constexpr uint32_t kTmemCols = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, kEpiThreads);
    }
    *abort_flag = 0;
    *epi_stop = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&map_x);
    tma_prefetch_desc(&map_y);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_tiles = p.x_tiles * p.y_tiles;
  const int num_kb = p.num_kb;
  // Everything above may run under the tail of the kernel in front of this one; nothing below may
  // touch global memory before pdl_enter() -- except, in the few-token form with weights that
  // nobody is writing (b_static), the producer's first ring-full of WEIGHT tiles, which it asks
  // for before it waits: the first memory round trip of the launch overlaps the predecessor too.
  int pre = 0;  // ring stages whose weight tiles were requested before the wait (producer thread only)
  const bool early_weights = SWAP && p.g.b_static && !p.x_mn && warp == 0 && lane == 0 && (int)blockIdx.x < num_tiles;
  if (early_weights) {
    const int xt = (int)blockIdx.x % p.x_tiles;
    for (int kb0 = 0; kb0 < num_kb && pre < STAGES; kb0 += KPS, ++pre) {
      const int nsub = num_kb - kb0 < KPS ? num_kb - kb0 : KPS;
      const uint32_t full = bar_full + 8 * pre;
      mbar_arrive_expect_tx(full, nsub * (L::kSubBytes - (kBlockX - p.x_tile_rows) * kBlockK));
#pragma unroll
      for (int j = 0; j < KPS; ++j)
        if (j < nsub)
          tma_load_2d(smem_base + pre * L::kStageBytes + j * L::kSubBytes, &map_x, full, (kb0 + j) * kBlockK, xt * p.x_tile_rows);
    }
  }
  pdl_enter();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      int nth = 0;  // stages issued so far
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int xt = tile % p.x_tiles, yt = tile / p.x_tiles;
        for (int kb0 = 0; kb0 < num_kb; kb0 += KPS, ++nth) {
          const int nsub = num_kb - kb0 < KPS ? num_kb - kb0 : KPS;
          const uint32_t full = bar_full + 8 * stage;
          if (nth < pre) {
            // weights already on their way (and the barrier armed): the token tiles follow now
#pragma unroll
            for (int j = 0; j < KPS; ++j)
              if (j < nsub)
                tma_load_2d(smem_base + stage * L::kStageBytes + j * L::kSubBytes + L::kXBytes, &map_y, full, (kb0 + j) * kBlockK, yt * BN);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, kErrProducer)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full, nsub * (L::kSubBytes - (kBlockX - p.x_tile_rows) * kBlockK));
          // K-major operand: box = 128 bytes of k x rows.  MN-major operand (stored [K][rows]):
          // box = 128 rows (bytes) x 128 k, one box per 128-row block; either way a 128-byte-
          // swizzled tile of the same size lands in the stage.
          // (a tile shorter than 128 rows leaves the stage's other rows as they were: the MMA
          // reads them into accumulator lanes that nobody stores)
#pragma unroll
          for (int j = 0; j < KPS; ++j) {
            if (j < nsub) {
              const int kb = kb0 + j;
              const uint32_t xs = smem_base + stage * L::kStageBytes + j * L::kSubBytes, ys = xs + L::kXBytes;
              if (!p.x_mn) tma_load_2d(xs, &map_x, full, kb * kBlockK, xt * p.x_tile_rows);
              else tma_load_2d(xs, &map_x, full, xt * kBlockX, kb * kBlockK);
              if (!p.y_mn) {
                tma_load_2d(ys, &map_y, full, kb * kBlockK, yt * BN);
              } else {
#pragma unroll
                for (int b = 0; b < BN / 128; ++b)
                  tma_load_2d(ys + b * (kBlockK * 128), &map_y, full, yt * BN + b * 128, kb * kBlockK);
              }
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_major(p.a_fmt_bits, p.b_fmt_bits, kBlockX, BN, p.x_mn, p.y_mn);
      // The issuing thread is a single dependent instruction stream: everything that does not
      // change per MMA is hoisted.  Descriptors of stage 0 are built once; a stage adds
      // kStageBytes >> 4 to the address field and a k-step adds 2 (K-major: 32 bytes inside the
      // 128-byte row) or 256 (MN-major: four 8-k atoms of 1024 bytes; 128-row blocks are a whole
      // k-block, 16 KB, apart).  The address field is 14 bits of (address >> 4), so the sums
      // never carry out of it.
      const uint64_t xd0 = p.x_mn ? smem_desc_mn_sw128(smem_base, kBlockK * 128, 1024) : smem_desc_k_sw128(smem_base);
      const uint64_t yd0 = p.y_mn ? smem_desc_mn_sw128(smem_base + L::kXBytes, kBlockK * 128, 1024)
                                  : smem_desc_k_sw128(smem_base + L::kXBytes);
      const uint32_t xstep = p.x_mn ? (4096u >> 4) : (kUmmaK >> 4), ystep = p.y_mn ? (4096u >> 4) : (kUmmaK >> 4);
      uint32_t stage = 0, phase = 0, ready = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.status, kErrMmaTmem)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb0 = 0; kb0 < num_kb; kb0 += KPS) {
          if (!ready && !mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, kErrMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const int nsub = num_kb - kb0 < KPS ? num_kb - kb0 : KPS;
          uint64_t xd = xd0 + (uint64_t)(stage * (uint32_t)(L::kStageBytes >> 4));
          uint64_t yd = yd0 + (uint64_t)(stage * (uint32_t)(L::kStageBytes >> 4));
          // all but the last k-block of the stage: MMAs only
#pragma unroll
          for (int j = 0; j + 1 < KPS; ++j) {
            if (j + 1 < nsub) {
              umma_f8(d_tmem, xd, yd, idesc, (kb0 + j) != 0);
#pragma unroll
              for (int k = 1; k < kBlockK / kUmmaK; ++k) umma_f8(d_tmem, xd + k * xstep, yd + k * ystep, idesc, 1u);
              xd += (uint32_t)(L::kSubBytes >> 4);
              yd += (uint32_t)(L::kSubBytes >> 4);
            }
          }
          const int kb = kb0 + nsub - 1;
          // the last k-block's four MMAs and the stage's commit (the stage is reusable once the
          // MMAs have read it), with a probe of the next stage's barrier issued before and read
          // after them
          const uint32_t nstage = stage + 1 == STAGES ? 0 : stage + 1;
          const uint32_t nphase = nstage == 0 ? phase ^ 1 : phase;
          static_assert(kBlockK / kUmmaK == 4, "umma_stage4_probe issues 4 MMAs");
          if (p.no_probe) {
            umma_f8(d_tmem, xd, yd, idesc, kb != 0);
#pragma unroll
            for (int k = 1; k < kBlockK / kUmmaK; ++k) umma_f8(d_tmem, xd + k * xstep, yd + k * ystep, idesc, 1u);
            umma_commit(bar_empty + 8 * stage);
          } else {
            ready = umma_stage4_probe<false, false>(d_tmem, xd, yd, idesc, kb != 0, bar_empty + 8 * stage,
                                                    bar_full + 8 * nstage, nphase, xstep, ystep);
          }
          stage = nstage;
          phase = nphase;
        }
        if (ok) umma_commit(bar_tfull + 8 * acc);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const GemmParams& g = p.g;
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int et = threadIdx.x - 64;     // 0..127
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int xt = tile % p.x_tiles, yt = tile / p.x_tiles;
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      const int64_t x0 = (int64_t)xt * p.x_tile_rows, y0 = (int64_t)yt * BN;
      const int64_t x_end = x0 + p.x_tile_rows < p.x_rows ? x0 + p.x_tile_rows : p.x_rows;  // rows of this tile only
      // column-side (per-y) epilogue operands for this tile -> shared memory
      float* cA = epi_f + acc * 3 * BN;
      float* cB = cA + BN;
      float* cBias = cB + BN;
      const EpiRow er = epi_stage_operands<BN, SWAP>(g, x_end, p.y_rows, x0 + q * 32 + lane, y0, et, cA, cB, cBias);
      // The wait can give up for some threads only; the decision to stop must be the same for
      // all 128 epilogue threads because they meet at named barriers: one thread samples the
      // abort flag between two barriers and everybody follows that sample.
      mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, kErrEpilogue, 128);
      named_bar_sync(1, kEpiThreads);
      if (et == 0) *epi_stop = *abort_flag;
      named_bar_sync(1, kEpiThreads);
      if (*epi_stop) break;
      tc_fence_after();
      epi_drain<BN, SWAP>(g, tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN, er, y0, cA, cB, cBias);
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();  // lanes 1..31 of the single-thread roles rejoin lane 0 here
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a bounded wait ran out: give copies that are still in flight time to land before the
    // shared memory and TMEM are released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}


// ------------------------------------------------------------------------ CTA-pair kernel
// Large-M form: two CTAs of a cluster (one per SM of a TPC) share a 256 x BN output tile.  Each
// CTA loads its own 128 rows of A and its own BN/2 rows of B per ring stage (no multicast: every
// byte is fetched by exactly one CTA), the even CTA's MMA thread issues
// tcgen05.mma.cta_group::2 (M = 256), which reads both CTAs' shared memory and writes 128
// accumulator rows into each CTA's TMEM.  Per flop the pair moves a third less data from L2
// into shared memory than two independent 128 x BN tiles, which is what bounds the
// single-CTA kernel.  Barrier traffic: both producers' TMA bytes complete on the even CTA's
// "full" barrier; tcgen05.commit (multicast to both CTAs) releases ring stages and publishes
// accumulators; both CTAs' epilogue threads arrive on the even CTA's "accumulator free" barrier.
template <int BN, int STAGES>
struct PairSmem {
  static constexpr int kXBytes = kBlockX * kBlockK;
  static constexpr int kYBytes = (BN / 2) * kBlockK;
  static constexpr int kStageBytes = kXBytes + kYBytes;
  static constexpr int kRing = STAGES * kStageBytes;
  static constexpr int kEpiFloats = 2 * 3 * BN;
  static constexpr int kPatchOffset = kRing + kEpiFloats * 4;  // 4 epilogue warps x 4 KB (routed output)
  static constexpr int kPatchBytes = (BN % 64 == 0) ? 4 * 4096 : 0;
  static constexpr int kBarOffset = kPatchOffset + kPatchBytes;
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
};

template <int BN, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                         const TcGemmParams p) {
  using L = PairSmem<BN, STAGES>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* epi_f = reinterpret_cast<float*>(smem + L::kRing);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_stop = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const uint32_t rank = cluster_ctarank();  // 0 = even CTA (issues the MMAs), 1 = its peer
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = 2 * BN <= 256 ? 256 : 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);   // the even CTA's expect_tx arrival; bytes of both CTAs
      mbar_init(bar_empty + 8 * s, 1);  // one multicast commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 2 * kEpiThreads);  // used in the even CTA only
    }
    *abort_flag = 0;
    *epi_stop = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&map_x);
    tma_prefetch_desc(&map_y);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // both CTAs' barriers are initialised before anything signals them remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();  // everything above may run under the tail of the kernel in front of this one

  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_tiles = p.x_tiles * p.y_tiles;  // x_tiles counts 256-row tiles here
  const int num_kb = p.num_kb;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int xt = tile % p.x_tiles, yt = tile / p.x_tiles;
        const int x_row = xt * 2 * kBlockX + (int)rank * kBlockX;
        const int y_row = yt * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, kErrProducer)) {
            ok = false;
            break;
          }
          const uint32_t full_leader = (bar_full + 8 * stage) & kPeerBitMask;
          if (rank == 0) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * L::kStageBytes);
          tma_load_2d_pair(smem_base + stage * L::kStageBytes, &map_x, full_leader, kb * kBlockK, x_row);
          tma_load_2d_pair(smem_base + stage * L::kStageBytes + L::kXBytes, &map_y, full_leader, kb * kBlockK, y_row);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(p.a_fmt_bits, p.b_fmt_bits, 2 * kBlockX, BN);
      // hoisted descriptors: see the single-CTA kernel
      const uint64_t xd0 = smem_desc_k_sw128(smem_base), yd0 = smem_desc_k_sw128(smem_base + L::kXBytes);
      uint32_t stage = 0, phase = 0, ready = 0;
      const bool no_probe = p.no_probe != 0;
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.status, kErrMmaTmem)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ready && !mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, kErrMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t xd = xd0 + (uint64_t)(stage * (uint32_t)(L::kStageBytes >> 4));
          const uint64_t yd = yd0 + (uint64_t)(stage * (uint32_t)(L::kStageBytes >> 4));
          // the stage's MMAs and commit, with a probe of the next stage's barrier around them
          const uint32_t nstage = stage + 1 == STAGES ? 0 : stage + 1;
          const uint32_t nphase = nstage == 0 ? phase ^ 1 : phase;
          static_assert(kBlockK / kUmmaK == 4 && (kUmmaK >> 4) == 2, "umma_stage4_probe issues 4 MMAs 32 bytes apart");
          if (no_probe) {
            umma_f8_pair(d_tmem, xd, yd, idesc, kb != 0);
#pragma unroll
            for (int k = 1; k < kBlockK / kUmmaK; ++k)
              umma_f8_pair(d_tmem, xd + k * (kUmmaK >> 4), yd + k * (kUmmaK >> 4), idesc, 1u);
            umma_commit_pair_both(bar_empty + 8 * stage);
          } else {
            ready = umma_stage4_probe<false, true>(d_tmem, xd, yd, idesc, kb != 0, bar_empty + 8 * stage,
                                                   bar_full + 8 * nstage, nphase, 2, 2);
          }
          stage = nstage;
          phase = nphase;
        }
        if (ok) umma_commit_pair_both(bar_tfull + 8 * acc);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const GemmParams& g = p.g;
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    int it = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
      const int xt = tile % p.x_tiles, yt = tile / p.x_tiles;
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      const int64_t x0 = (int64_t)xt * 2 * kBlockX + (int64_t)rank * kBlockX, y0 = (int64_t)yt * BN;
      float* cA = epi_f + acc * 3 * BN;
      float* cB = cA + BN;
      float* cBias = cB + BN;
      const EpiRow er = epi_stage_operands<BN, false>(g, p.x_rows, p.y_rows, x0 + q * 32 + lane, y0, et, cA, cB, cBias);
      mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, kErrEpilogue, 128);
      named_bar_sync(1, kEpiThreads);
      if (et == 0) *epi_stop = *abort_flag;
      named_bar_sync(1, kEpiThreads);
      if (*epi_stop) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      if (BN == 256 && g.swiglu) {
        epi_drain_swiglu(g, t_row, er, y0, cA, cB, cBias);
      } else if (BN % 64 == 0 && g.route_count > 0) {
        if constexpr (BN % 64 == 0)
          epi_drain_routed<BN>(g, t_row, er, x0 + q * 32, y0, cA, cB, cBias,
                               reinterpret_cast<uint4*>(smem + L::kPatchOffset) + q * 256, lane);
      } else {
        epi_drain<BN, false>(g, t_row, er, y0, cA, cB, cBias);
      }
      tc_fence_before();
      mbar_arrive_cluster((bar_tempty + 8 * acc) & kPeerBitMask);  // the even CTA's barrier
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  cluster_sync_all();  // neither CTA leaves while the other may still touch its shared memory, barriers or TMEM
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <int BN, int STAGES>
static int launch_pair(const CUtensorMap& mx, const CUtensorMap& my, const TcGemmParams& tp, cudaStream_t st) {
  using L = PairSmem<BN, STAGES>;
  constexpr int smem = L::kTotal + 1024;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  static_assert(smem > 116 * 1024, "one CTA per SM: two CTAs must never contend for TMEM");
  auto kern = gemm_tcgen05_pair_kernel<BN, STAGES>;
  // per device, once: raise the dynamic shared-memory limit and ask how many CTA pairs can be
  // resident at once (a pair needs both SMs of a TPC); -1 = pairs not available on this device
  static std::atomic<int> resident_pairs[kMaxDevices];
  const int dev = current_device_index();
  if (dev < 0) return B200Q_ERR_CUDA;
  int clusters = resident_pairs[dev].load(std::memory_order_acquire);
  if (clusters == 0) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kNumSMs, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaError_t oe = cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg);
    if (oe != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = -1;
    }
    resident_pairs[dev].store(clusters, std::memory_order_release);
  }
  if (clusters < 0) return B200Q_ERR_UNSUPPORTED;
  int tiles = tp.x_tiles * tp.y_tiles;
  int pairs = tiles < clusters ? tiles : clusters;
  static const bool no_pdl = std::getenv("B200Q_GEMM_NO_PDL") != nullptr;  // comparison switch
  if (no_pdl || launch_overlapped(kern, dim3((unsigned)(2 * pairs)), dim3(kThreads), smem, st, mx, my, tp) != cudaSuccess) {
    if (!no_pdl) (void)cudaGetLastError();
    kern<<<2 * pairs, kThreads, smem, st>>>(mx, my, tp);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// ------------------------------------------------------------------------ host side
// 2-D map over a row-major byte matrix [rows][kbytes] with row stride ld bytes; box = 128 bytes x box_rows.
int make_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t kbytes, int64_t ld_bytes,
                     int box_rows) {
  return make_tma_map_2d(map, base, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, kbytes, rows, ld_bytes, kBlockK, box_rows,
                         CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int BN, int STAGES, bool SWAP, int KPS = 1>
static int launch_cfg(const CUtensorMap& mx, const CUtensorMap& my, const TcGemmParams& tp, cudaStream_t st) {
  using L = SmemLayout<BN, STAGES, KPS>;
  constexpr int smem = L::kTotal + 1024;  // slack for the manual 1024-byte alignment
  static_assert(smem <= 227 * 1024, "shared memory budget");
  static_assert(smem > 116 * 1024, "one CTA per SM: two CTAs must never contend for TMEM");
  auto kern = gemm_tcgen05_kernel<BN, STAGES, SWAP, KPS>;
  static std::atomic<int> configured[kMaxDevices];
  const int dev = current_device_index();
  if (dev < 0) return B200Q_ERR_CUDA;
  if (!configured[dev].load(std::memory_order_acquire)) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev].store(1, std::memory_order_release);
  }
  int tiles = tp.x_tiles * tp.y_tiles;
  int grid = tiles < kNumSMs ? tiles : kNumSMs;
  // the kernel's set-up (barriers, TMEM, descriptors) may run under the tail of its predecessor: with a few
  // tokens it lasts 10-20 us and a launch gap of 2-3 us between two of them counts
  static const bool no_pdl = std::getenv("B200Q_GEMM_NO_PDL") != nullptr;  // comparison switch
  if (no_pdl || launch_overlapped(kern, dim3((unsigned)grid), dim3(kThreads), smem, st, mx, my, tp) != cudaSuccess) {
    if (!no_pdl) (void)cudaGetLastError();
    kern<<<grid, kThreads, smem, st>>>(mx, my, tp);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

static inline int fmt_bits(int dtype) { return dtype == B200Q_E5M2 ? 1 : 0; }

// Operand map: K-major = row-major [rows][K] (box 128 k-bytes x box_rows); MN-major = row-major
// [K][rows] (box 128 row-bytes x 128 k).
static int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, bool mn, int box_rows) {
  if (!mn) return make_operand_map(map, base, rows, K, ld, box_rows);
  return make_tma_map_2d(map, base, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, K, ld, 128, kBlockK, CU_TENSOR_MAP_SWIZZLE_128B);
}

int gemm_tcgen05_launch(const GemmParams& g, cudaStream_t st) {
  // eligibility: TMA-compatible strides and bases, one problem per launch.  A is K-major when
  // stored [M][K] (trans_a = 0), B when stored [N][K] (trans_b = 1); the other storage orders
  // are MN-major operands, which the tensor core reads through MN-major descriptors.
  const bool a_mn = g.trans_a != 0, b_mn = g.trans_b == 0;
  if (g.batch != 1 || g.K < 1 || (g.lda % 16) || (g.ldb % 16)) return B200Q_ERR_UNSUPPORTED;
  if ((!a_mn || !b_mn) && (g.K % 16)) return B200Q_ERR_UNSUPPORTED;  // a K-major row must be 16-byte granular
  if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B)) & 15) return B200Q_ERR_UNSUPPORTED;
  if (g.a_scale_mode == B200Q_BCAST_FULL || g.b_scale_mode == B200Q_BCAST_FULL) return B200Q_ERR_UNSUPPORTED;
  if (g.M <= 0 || g.N <= 0) return B200Q_ERR_UNSUPPORTED;
  if (g.M > (1ll << 30) || g.N > (1ll << 30) || g.K > (1ll << 30)) return B200Q_ERR_UNSUPPORTED;

  // fused SwiGLU: CTA-pair kernel only, whole 256-column tiles, bf16 intermediate
  if (g.swiglu && (g.M <= 128 || (g.N % 256) || a_mn || b_mn || g.out_dtype != B200Q_BF16 || g.out8_dtype != B200Q_E4M3))
    return B200Q_ERR_UNSUPPORTED;

  // routed output: bf16 rows through the CTA-pair kernel, every 128-row block inside one route block
  const bool routed = g.route_count > 0;
  if (routed && (g.M <= 128 || g.N <= 128 || a_mn || b_mn || g.out_dtype != B200Q_BF16 || g.out8_dtype || g.swiglu || g.D ||
                 g.bias_mode == B200Q_BCAST_FULL || (g.N % 8) || (g.ldo % 8) || g.route_rows <= 0 || (g.route_rows % 128) ||
                 g.route_count > 8 || (g.M + g.route_rows - 1) / g.route_rows > g.route_count))
    return B200Q_ERR_UNSUPPORTED;

  TcGemmParams tp;
  tp.g = g;
  static const bool no_probe = std::getenv("B200Q_GEMM_NO_PROBE") != nullptr;
  tp.no_probe = no_probe;
  tp.status = device_status_ptr();
  if (!tp.status) return B200Q_ERR_CUDA;
  tp.num_kb = (int)((g.K + kBlockK - 1) / kBlockK);
  // small M: weights on the lanes, tokens on the columns -- unless the tokens are MN-major (their
  // column tile would be narrower than the 128-byte MN-major row)
  const bool swap = g.M <= 128 && g.N >= 128 && !a_mn;
  CUtensorMap mx, my;
  if (!swap) {
    tp.x_rows = g.M; tp.y_rows = g.N;
    tp.a_fmt_bits = fmt_bits(g.a_dtype); tp.b_fmt_bits = fmt_bits(g.b_dtype);
    tp.x_mn = a_mn; tp.y_mn = b_mn;
    tp.x_tiles = (int)((g.M + kBlockX - 1) / kBlockX);
    tp.x_tile_rows = kBlockX;
    // Column-tile width: the one that minimises (waves over the 148 SMs) x (tile cost).  Measured
    // on 4096 x 14336 x 4096: a wave of 224-column tiles takes 96 % of the time of a wave of
    // 256-column tiles (the k-block time is dominated by operand traffic that does not shrink with
    // the width), i.e. a tile costs about (width + 590) units; narrower tiles only win when they
    // remove a whole wave.
    // An MN-major B operand comes in 128-column blocks: 256 or 128 only.
    static const int kWidths[] = {256, 224, 192, 160, 128};
    int bn = 128;
    double best = 1e30;
    for (int w : kWidths) {
      if (w > 128 && g.N <= 128) continue;
      if (b_mn && (w % 128)) continue;
      const int64_t tiles = (int64_t)tp.x_tiles * ((g.N + w - 1) / w);
      const double cost = (double)((tiles + kNumSMs - 1) / kNumSMs) * (w + kTileOverheadCols);
      if (cost < best) { best = cost; bn = w; }
    }
    tp.y_tiles = (int)((g.N + bn - 1) / bn);
    int rc = make_map(&mx, g.A, g.M, g.K, g.lda, a_mn, kBlockX);
    if (rc) return rc;
    // CTA pairs (256-row tiles) when there are enough rows to fill them (K-major operands)
    static const bool no_pairs = std::getenv("B200Q_GEMM_NO_PAIRS") != nullptr;
    if (g.M > 128 && g.N > 128 && !no_pairs && !a_mn && !b_mn) {
      TcGemmParams pp = tp;
      pp.x_tiles = (int)((g.M + 2 * kBlockX - 1) / (2 * kBlockX));
      int bp = 256;
      double bestp = 1e30;
      static const int kPairWidths[] = {256, 224, 192};
      for (int w : kPairWidths) {
        if (routed && (w % 64)) continue;
        const int64_t tiles = (int64_t)pp.x_tiles * ((g.N + w - 1) / w);
        const double cost = (double)((tiles + kNumSMs / 2 - 1) / (kNumSMs / 2)) * (w + kTileOverheadCols);
        if (cost < bestp) { bestp = cost; bp = w; }
      }
      static const int forced = std::getenv("B200Q_GEMM_PAIR_BN") ? std::atoi(std::getenv("B200Q_GEMM_PAIR_BN")) : 0;
      if ((forced == 256 || forced == 224 || forced == 192) && !(routed && (forced % 64))) bp = forced;
      if (g.swiglu) bp = 256;  // gate and up halves of a tile
      pp.y_tiles = (int)((g.N + bp - 1) / bp);
      rc = make_operand_map(&my, g.B, g.N, g.K, g.ldb, bp / 2);
      if (rc) return rc;
      switch (bp) {
        case 256: rc = launch_pair<256, 6>(mx, my, pp, st); break;
        case 224: rc = launch_pair<224, 7>(mx, my, pp, st); break;
        default: rc = launch_pair<192, 7>(mx, my, pp, st); break;
      }
      if (rc != B200Q_ERR_UNSUPPORTED) return rc;
    }
    if (g.swiglu || routed) return B200Q_ERR_UNSUPPORTED;  // only the pair kernel has these epilogues
    rc = make_map(&my, g.B, g.N, g.K, g.ldb, b_mn, bn);
    if (rc) return rc;
    switch (bn) {
      case 256: return launch_cfg<256, 4, false>(mx, my, tp, st);
      case 224: return launch_cfg<224, 5, false>(mx, my, tp, st);
      case 192: return launch_cfg<192, 5, false>(mx, my, tp, st);
      case 160: return launch_cfg<160, 6, false>(mx, my, tp, st);
      default: return launch_cfg<128, 6, false>(mx, my, tp, st);
    }
  }
  tp.x_rows = g.N; tp.y_rows = g.M;
  tp.a_fmt_bits = fmt_bits(g.b_dtype); tp.b_fmt_bits = fmt_bits(g.a_dtype);
  tp.x_mn = b_mn; tp.y_mn = 0;
  const int bn = g.M <= 16 ? 16 : g.M <= 32 ? 32 : g.M <= 64 ? 64 : 128;
  tp.y_tiles = (int)((g.M + bn - 1) / bn);
  // Tile height.  The kernel is one pass over the weight bytes, and a CTA's share of them is
  // (rounds of tiles over the SMs) x (tile rows): 14336 weight rows in 128-row tiles are 112 tiles,
  // one round in which 36 SMs stay idle and the others stream 128 rows each; in 104-row tiles they
  // are 138 tiles of a fifth fewer bytes.  The tensor core still multiplies 128 lanes; the lanes
  // beyond the tile read whatever the stage holds and are not stored.  Heights are multiples of 8
  // (the swizzle atom) from 32 up (a stage shorter than that keeps too few bytes in flight); the
  // cost of a round has a height-independent part (pipeline fill, accumulator drain) of about 24 rows.
  int rows = kBlockX;
  if (!b_mn) {
    static const bool fixed_height = std::getenv("B200Q_GEMM_SWAP_128") != nullptr;  // comparison switch
    double best = 1e30;
    for (int r = kBlockX; r >= 32 && !fixed_height; r -= 8) {
      const int64_t tiles = ((g.N + r - 1) / r) * tp.y_tiles;
      const double cost = (double)((tiles + kNumSMs - 1) / kNumSMs) * (r + 24);
      if (cost < best) { best = cost; rows = r; }
    }
  }
  tp.x_tile_rows = rows;
  tp.x_tiles = (int)((g.N + rows - 1) / rows);
  int rc = make_map(&mx, g.B, g.N, g.K, g.ldb, b_mn, rows);
  if (rc) return rc;
  rc = make_operand_map(&my, g.A, g.M, g.K, g.lda, bn);
  if (rc) return rc;
  // Few tokens: neither the bytes nor the MMAs set the pace here -- measured, a k-block costs a CTA
  // 0.25-0.3 us whatever the tile height (32 or 128 rows), with one MMA or none in place of four,
  // with or without the token tile's load, with 7 ring stages or 10 -- so the per-stage work of
  // the two single-thread roles (barrier round trips, commit) is spread over two k-blocks
  // (-6 % at K = 4096, -16 % at K = 14336).
  static const bool one_kb = std::getenv("B200Q_GEMM_SWAP_KPS1") != nullptr;  // comparison switch
  if (!b_mn && !one_kb) {
    switch (bn) {
      case 16:  // long K: four k-blocks per stage (measured: 27 against 30 us at K = 14336; no gain at 4096)
        if (tp.num_kb >= 64) return launch_cfg<16, 3, true, 4>(mx, my, tp, st);
        return launch_cfg<16, 5, true, 2>(mx, my, tp, st);
      case 32: return launch_cfg<32, 5, true, 2>(mx, my, tp, st);
      case 64: return launch_cfg<64, 4, true, 2>(mx, my, tp, st);
      default: return launch_cfg<128, 3, true, 2>(mx, my, tp, st);
    }
  }
  switch (bn) {
    case 16: return launch_cfg<16, 10, true>(mx, my, tp, st);
    case 32: return launch_cfg<32, 9, true>(mx, my, tp, st);
    case 64: return launch_cfg<64, 8, true>(mx, my, tp, st);
    default: return launch_cfg<128, 6, true>(mx, my, tp, st);
  }
}

}  // namespace b200q

