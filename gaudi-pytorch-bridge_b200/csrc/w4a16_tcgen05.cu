// W4A16 GEMM: out[M][N] = x[M][K] (bf16) . W[K][N], W = (nibble - zero_point) * scale held as
// packed 4-bit words [K][N/8] with group scales -- the dequantisation is fused into the staging
// of the weight operand, so the bf16 weights never exist in global memory.
//
// Warp-specialised, persistent:
//   warp 0        TMA producer: per ring stage the activation tile (bf16, K-major, 128-byte
//                 swizzle), the raw packed-weight tile [64 k][W words], and the k-group's scales
//                 and packed zero points
//   warps 6..     expanders: each thread takes packed words (k, column group) from the ring and
//                 expands them with packed bf16x2 arithmetic ((128+q)-(128+z) exact, one rounding
//                 in the multiply by the scale: bit-identical to the stand-alone dequant kernel).
//                 A word is eight neighbouring COLUMNS of one k, so the expanded tile is written
//                 MN-major (columns contiguous, 64 per 128-byte row, 8 k per swizzle atom) and the
//                 tensor core reads it through an MN-major descriptor: no transpose.  The nibble
//                 pairs come out as columns (i, i+4); they are stored in that order and the
//                 epilogue undoes the permutation when it writes the output columns.
//   warp 1        MMA issuer: tcgen05.mma.kind::f16 (bf16 x bf16 -> fp32 in TMEM)
//   warps 2..5    epilogue: tcgen05.ld, convert, store (or fp32 partials for split-K)
//
// Lanes <- 128 tokens, columns <- BN weight columns.  Small M (<= 128): only AR token rows are
// loaded (see Cfg), K is split over several CTAs per tile so that every SM streams weights, and
// the fp32 partial tiles are summed by a second kernel (deterministic: no atomics).
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "tcgen05_ptx.cuh"
#include "tma_host.cuh"

namespace b200q {

using namespace ptx;

namespace w4 {

constexpr int kK = 64;               // k per ring stage: 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaKBytes = 32;      // 16 bf16 per tcgen05.mma.kind::f16
constexpr int kUnit = 128;           // weight columns expanded by one 4-warp group per stage
constexpr int kRawUnit = kK * 64;    // packed words of one unit and stage: 64 k-rows x 16 words
constexpr int kEpiThreads = 128;

enum { kErrProducer = 201, kErrMma = 202, kErrMmaTmem = 203, kErrEpilogue = 204, kErrExpand = 205 };

struct Params {
  const __nv_bfloat16* scale;  // [K/group][N]
  const int32_t* zp;           // [K/group][N/8] or null
  void* out;                   // [M][N] out_dtype (splits == 1)
  float* partial;              // [splits][M][N] fp32 (splits > 1)
  int64_t M, N, K, ldo;
  int group, out_dtype;
  int group_shift;  // log2(group / 64) when that is a power of two, else -1 (the kernels then divide)
  int x_tiles, y_tiles, num_kb, splits, kb_per_split;
  int* status;
};

// Shared memory of the single-CTA kernel is two rings, because the two things a k-block needs
// live for very different times:
//   raw ring  (RS slots)  packed weights [64 k][W words] + the k-group's scales / zero points.
//                         Small (4.5 KB per 128 columns) and in flight for a whole DRAM round
//                         trip: many slots, so that enough bytes are outstanding per SM.
//   work ring (WS slots)  activations (bf16, K-major, 128-byte swizzle) + the expanded bf16
//                         tile (MN-major, 128-byte swizzle).  Large (16 KB per 128 columns) and
//                         live only from the expansion to the MMAs that read it: few slots.
template <int BN, int RS, int WS, int GROUPS, int AR = 0, int EW = 0>
struct Cfg {
  static constexpr int kUnits = BN / kUnit;
  // Activation rows held per work slot.  The MMA always reads 128 rows through its descriptor;
  // with AR < 128 the rows beyond AR are whatever follows in the slot (the expanded tile).  Each
  // output row depends on its own operand row only, and rows >= M are never stored, so for
  // M <= AR nothing needs to be there.
  static constexpr int kActRows = AR ? AR : 128;
  static_assert(AR == 0 || (AR <= 128 && AR % 8 == 0), "narrow activation tile: a multiple of 8 rows");
  static constexpr int kActBytes = kActRows * 128;
  static constexpr int kWCols = kUnits * kUnit;
  // work slot
  static constexpr int kWOffset = (kActBytes + 1023) / 1024 * 1024;  // expanded tile, 1024-byte aligned
  static constexpr int kWBytes = kWCols * 128;
  static constexpr int kWorkSlotBytes = kWOffset + kWBytes;
  // raw slot: packed weights, then scales (bf16) at +0 and packed zero points at +512 of a 1 KB block
  static constexpr int kRawBytes = kUnits * kRawUnit;
  static constexpr int kMetaOffset = kRawBytes;
  static constexpr int kScaleBytes = kWCols * 2, kZpBytes = kWCols / 2;
  static constexpr int kZpOffset = kMetaOffset + 512;
  static constexpr int kRawSlotBytes = kRawBytes + 1024;
  static constexpr int kRawRowWords = kUnits * 16;  // packed words per k-row of the slot's tile
  static constexpr int kRawRing = WS * kWorkSlotBytes;  // offset of the raw ring
  static constexpr int kBarOffset = kRawRing + RS * kRawSlotBytes;
  static constexpr int kNumBars = 2 * RS + 2 * WS + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
  // 8 expander warps per 128 weight columns and k-block (4 packed words per thread), in GROUPS
  // groups that take alternate k-blocks
  static constexpr int kExpandWarps = EW ? EW : 8 * kUnits;
  static constexpr int kExpandGroups = GROUPS;
  // Warp roles are placed by scheduler (warp % 4): the three producers (warps 0, 12, 16) and the
  // MMA issuer (warp 4) have scheduler 0 to themselves; their per-k-block instruction chains
  // (barrier wait, copies, MMAs, commit) run 25-40 % faster than when they compete with
  // expander warps for issue slots and the shared-memory instruction queue.  Epilogue: warps
  // 1, 2, 3 and 8 (TMEM lane quarters 1, 2, 3, 0; asleep during the main loop).  Expanders: the
  // warps >= 5 with warp % 4 != 0, in order (21 of them in a 32-warp CTA); a configuration with
  // more expander warps than that also takes warps 20, 24 and 28 of scheduler 0.
  static constexpr int kNumExpanders = kExpandWarps * kExpandGroups;
  static constexpr int kOffS0 = 21;  // expander warps available outside scheduler 0
  static constexpr int kLastExpander = (kNumExpanders <= kOffS0 ? kNumExpanders : kOffS0) - 1;
  static constexpr int kExpWarpsEnd = 5 + (kLastExpander / 3) * 4 + kLastExpander % 3 + 1;
  static constexpr int kWarps = kNumExpanders > kOffS0 ? 32 : (kExpWarpsEnd < 17 ? 17 : kExpWarpsEnd);
  static_assert(kNumExpanders <= kOffS0 + 3, "too many expander warps for one CTA");
  static constexpr int kThreads = 32 * kWarps;
  static_assert(kWorkSlotBytes % 1024 == 0 && kRawSlotBytes % 1024 == 0, "swizzled tiles need 1024-byte alignment");
  static_assert(kWorkSlotBytes >= 128 * 128, "the 128-row operand read must stay inside the slot");
  static_assert(kK % (kExpandWarps * 32 / kRawRowWords) == 0, "expander passes");
  static_assert(WS >= GROUPS, "every expander group needs a work slot of its own");
  static constexpr uint32_t kTmemCols = (2 * BN) < 32 ? 32 : 2 * BN;
};

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
// nibbles i and i+4 of a word as the bf16x2 {128 + q_i, 128 + q_{i+4}}
__device__ __forceinline__ uint32_t nib_pair(uint32_t w, int i) {
  return ((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
}

struct GroupRegs {
  uint32_t sp[4];  // {s_i, s_{i+4}}
  uint32_t zr[4];  // {128 + z_i, 128 + z_{i+4}}
};
__device__ __forceinline__ void make_group(GroupRegs& g, uint4 s, uint32_t zw, bool has_zp) {
  g.sp[0] = __byte_perm(s.x, s.z, 0x5410);
  g.sp[1] = __byte_perm(s.x, s.z, 0x7632);
  g.sp[2] = __byte_perm(s.y, s.w, 0x5410);
  g.sp[3] = __byte_perm(s.y, s.w, 0x7632);
#pragma unroll
  for (int i = 0; i < 4; ++i) g.zr[i] = has_zp ? nib_pair(zw, i) : 0x43004300u;
}

template <int BN, int RS, int WS, int GROUPS, int AR = 0, int EW = 0>
__global__ void __launch_bounds__((Cfg<BN, RS, WS, GROUPS, AR, EW>::kThreads), 1)
w4a16_kernel(const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CUtensorMap map_raw,
             const __grid_constant__ CUtensorMap map_scale, const __grid_constant__ CUtensorMap map_zp, const Params p) {
  using C = Cfg<BN, RS, WS, GROUPS, AR, EW>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBarOffset);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_stop = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const uint32_t smem_base = smem_u32(smem);
  // raw_full[r]   packed weights + scales of a k-block landed in raw slot r      -> expanders
  // raw_empty[r]  the k-block of raw slot r is done (tcgen05.commit after its MMAs: a second
  //               commit by the MMA issuer costs less than an arrival by every expander warp,
  //               whose chain per k-block is the longest in the kernel)                -> raw producers
  // w_ready[w]    activations landed in work slot w and the tile is expanded        -> MMA issuer
  // w_empty[w]    the MMAs that read work slot w retired (tcgen05.commit)           -> act producer, expanders
  const uint32_t raw_base = smem_base + C::kRawRing;
  const uint32_t bar_raw_full = smem_u32(bars), bar_raw_empty = bar_raw_full + 8 * RS;
  const uint32_t bar_w_ready = bar_raw_empty + 8 * RS, bar_w_empty = bar_w_ready + 8 * WS;
  const uint32_t bar_tfull = bar_w_empty + 8 * WS, bar_tempty = bar_tfull + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  enum { kProducer, kProducerMeta, kProducerAct, kMma, kEpilogue, kExpander, kIdle };
  // expander warp index (valid when that role): warps off scheduler 0 first, then 20, 24, 28
  const int ewarp = (warp & 3) != 0 ? ((warp - 5) >> 2) * 3 + ((warp & 3) - 1) : C::kOffS0 + ((warp - 20) >> 2);
  const int role = warp == 0    ? kProducer
                   : warp == 4  ? kMma
                   : warp == 12 ? kProducerMeta
                   : warp == 16 ? kProducerAct
                   : (warp < 4 || warp == 8) ? kEpilogue
                   : (((warp & 3) != 0 || warp >= 20) && ewarp < C::kNumExpanders) ? kExpander
                                                                                    : kIdle;

  if (threadIdx.x == 0) {
    for (int r = 0; r < RS; ++r) {
      mbar_init(bar_raw_full + 8 * r, 2);                  // the two raw-ring producer warps
      mbar_init(bar_raw_empty + 8 * r, 1);                 // one commit (see the MMA issuer)
    }
    for (int w = 0; w < WS; ++w) {
      mbar_init(bar_w_ready + 8 * w, 1 + C::kExpandWarps);  // act producer + one arrival per expander warp
      mbar_init(bar_w_empty + 8 * w, 1);                    // one commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, kEpiThreads);
    }
    *abort_flag = 0;
    *epi_stop = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&map_act);
    tma_prefetch_desc(&map_raw);
    tma_prefetch_desc(&map_scale);
    if (p.zp) tma_prefetch_desc(&map_zp);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();  // everything above overlaps the tail of the kernel in front; global memory is touched from here on

  const int num_work = p.x_tiles * p.y_tiles * p.splits;
  // work item -> (lane-side tile, column-side tile, k range).  Consecutive items (CTAs that run
  // at the same time) are neighbouring tiles of the same k range: together they read whole rows
  // of the packed weight matrix, which keeps the DRAM pages they open fully used.
  auto decode = [&](int w, int& xt, int& yt, int& kb0, int& kb1, int& split) {
    const int tiles = p.x_tiles * p.y_tiles;
    split = w / tiles;
    const int tile = w % tiles;
    xt = tile % p.x_tiles;
    yt = tile / p.x_tiles;
    kb0 = split * p.kb_per_split;
    kb1 = min(p.num_kb, kb0 + p.kb_per_split);
  };

  if (role == kProducer || role == kProducerMeta) {
    // ------------------------------------------------------------ raw-ring producers
    // Two warps, because one thread that waits for the slot and issues three copies and the
    // expect_tx needs more cycles per k-block than anything else in the kernel at small M:
    //   warp 0   packed weights
    //   warp 12  scales and zero points; every k-block carries them because consecutive
    //            k-blocks go to different expander warps
    if (lane == 0) {
      const bool meta = role == kProducerMeta;
      uint32_t slot = 0, phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        int xt, yt, kb0, kb1, split;
        decode(w, xt, yt, kb0, kb1, split);
        const int n0 = yt * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_raw_empty + 8 * slot, phase ^ 1, abort_flag, p.status, kErrProducer)) {
            ok = false;
            break;
          }
          const uint32_t sbase = raw_base + slot * C::kRawSlotBytes;
          const uint32_t full = bar_raw_full + 8 * slot;
          if (meta) {
            const int grp = p.group_shift >= 0 ? (kb >> p.group_shift) : (kb * kK) / p.group;
            mbar_arrive_expect_tx(full, C::kScaleBytes + (p.zp ? C::kZpBytes : 0));
            tma_load_2d(sbase + C::kMetaOffset, &map_scale, full, n0, grp);
            if (p.zp) tma_load_2d(sbase + C::kZpOffset, &map_zp, full, n0 / 8, grp);
          } else {
            mbar_arrive_expect_tx(full, C::kRawBytes);
            tma_load_2d(sbase, &map_raw, full, n0 / 8, kb * kK);
          }
          if (++slot == RS) { slot = 0; phase ^= 1; }
        }
      }
    }
  } else if (role == kProducerAct) {
    // ------------------------------------------------------------ activation producer (work ring)
    if (lane == 0) {
      uint32_t slot = 0, phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        int xt, yt, kb0, kb1, split;
        decode(w, xt, yt, kb0, kb1, split);
        const int act_row0 = xt * 128;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_w_empty + 8 * slot, phase ^ 1, abort_flag, p.status, kErrProducer)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(bar_w_ready + 8 * slot, C::kActBytes);
          tma_load_2d(smem_base + slot * C::kWorkSlotBytes, &map_act, bar_w_ready + 8 * slot, kb * kK, act_row0);
          if (++slot == WS) { slot = 0; phase ^= 1; }
        }
      }
    }
  } else if (role == kMma) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // bf16 x bf16; the expanded weights are the MN-major B operand
      const uint32_t idesc = umma_idesc_major(1u, 1u, 128, BN, 0u, 1u);
      const uint64_t da0 = smem_desc_k_sw128(smem_base);
      const uint64_t dw0 = smem_desc_mn_sw128(smem_base + C::kWOffset, (kK / 8) * 1024, 1024);
      uint32_t stage = 0, phase = 0, ready = 0;  // work-ring slot
      constexpr int STAGES = WS;
      uint32_t rslot = 0;
      int it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
        int xt, yt, kb0, kb1, split;
        decode(w, xt, yt, kb0, kb1, split);
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.status, kErrMmaTmem)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ready && !mbar_wait(bar_w_ready + 8 * stage, phase, abort_flag, p.status, kErrMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          // activations: K-major, 32 bytes per k-step inside the 128-byte row; weights: MN-major,
          // two 8-k atoms (2048 bytes) per k-step, column blocks 8 atoms apart (descriptors of
          // slot 0 are hoisted out of the loop).  Four MMAs and the commit in one sequence, with
          // a probe of the next slot's barrier issued before and read after them.
          const uint64_t soff = (uint64_t)(stage * (uint32_t)(C::kWorkSlotBytes >> 4));
          const uint64_t da = da0 + soff, dw = dw0 + soff;
          const uint32_t nstage = stage + 1 == STAGES ? 0 : stage + 1;
          const uint32_t nphase = nstage == 0 ? phase ^ 1 : phase;
          static_assert(kK / 16 == 4, "umma_stage4_probe issues 4 MMAs");
          constexpr uint64_t kActStep = kUmmaKBytes >> 4, kWStep = 2048 >> 4;
          ready = umma_stage4_probe<true, false>(d_tmem, da, dw, idesc, kb != kb0, bar_w_empty + 8 * stage,
                                                 bar_w_ready + 8 * nstage, nphase, kActStep, kWStep);
          umma_commit(bar_raw_empty + 8 * rslot);  // the expanders read raw slot rslot before they arrived on w_ready
          if (++rslot == RS) rslot = 0;
          stage = nstage;
          phase = nphase;
        }
        if (ok) umma_commit(bar_tfull + 8 * acc);
      }
    }
  } else if (role == kEpilogue) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int et = q * 32 + lane;
    int it = 0;
    for (int w = blockIdx.x; w < num_work; w += gridDim.x, ++it) {
      int xt, yt, kb0, kb1, split;
      decode(w, xt, yt, kb0, kb1, split);
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, kErrEpilogue, 128);
      named_bar_sync(1, kEpiThreads);
      if (et == 0) *epi_stop = *abort_flag;
      named_bar_sync(1, kEpiThreads);
      if (*epi_stop) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      // The weight columns inside every group of 8 sit at tile positions (0,4,1,5,2,6,3,7) (the
      // order the nibble pairs were stored in): position p holds column (p >> 1) + 4 * (p & 1);
      // the registers read from TMEM are renamed into column order below.
      const int64_t m = (int64_t)xt * 128 + q * 32 + lane;  // this thread's token
      const int64_t y0 = (int64_t)yt * BN;
      constexpr int CW = (BN % 32 == 0) ? 32 : 16;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        if (BN % 32 == 0) tmem_ld_32x32(t_row + c0, r);
        else tmem_ld_32x16(t_row + c0, r);
        tmem_ld_wait();
        // registers are in tile-position order: rename them into column order (free: all static)
        {
          uint32_t t[32];
#pragma unroll
          for (int j = 0; j < CW; ++j) t[(j & ~7) + ((j & 7) >> 1) + 4 * (j & 1)] = r[j];
#pragma unroll
          for (int j = 0; j < CW; ++j) r[j] = t[j];
        }
        const int64_t n0 = y0 + c0;
        if (m < p.M) {
          if (p.splits > 1) {
            float* o = p.partial + ((int64_t)split * p.M + m) * p.N + n0;
            if (n0 + CW <= p.N && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < CW; j += 4)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < CW; ++j)
                if (n0 + j < p.N) o[j] = __uint_as_float(r[j]);
            }
          } else if (p.out_dtype == B200Q_BF16) {
            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + m * p.ldo + n0;
            if (n0 + CW <= p.N && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < CW; j += 8)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(
                    pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                    pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                    pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])),
                    pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
            } else {
#pragma unroll
              for (int j = 0; j < CW; ++j)
                if (n0 + j < p.N) o[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          } else {
            float* o = static_cast<float*>(p.out) + m * p.ldo + n0;
            if (n0 + CW <= p.N && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < CW; j += 4)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < CW; ++j)
                if (n0 + j < p.N) o[j] = __uint_as_float(r[j]);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
    }
  } else if (role == kExpander) {
    // ------------------------------------------------------------ expanders
    const int et = (ewarp % C::kExpandWarps) * 32 + lane;  // position inside the group
    const int my_group = ewarp / C::kExpandWarps;          // the stages this warp takes
    constexpr int W = C::kRawRowWords;                      // packed words per k-row (16 per 128 columns)
    constexpr int kRowsPerPass = C::kExpandWarps * 32 / W;  // k-rows covered by the group at once (16)
    constexpr int kPasses = kK / kRowsPerPass;
    const int ngl = et % W;                                 // column group (8 columns) inside the stage's tile
    const int kr = et / W;                                  // first k-row of this thread; then every kRowsPerPass
    const bool has_zp = p.zp != nullptr;
    // Raw tile: row k holds W consecutive words, so a warp reads 32 consecutive words.
    // Expanded tile: column block b = ngl / 8 (64 columns), 16-byte chunk c = ngl % 8 of the
    // 128-byte row k % 8 of atom (b, k / 8), chunk XOR-swizzled with the row: the 8 lanes of
    // a quarter warp write the 8 chunks of one row.
    const uint32_t krow = kr & 7;
    const uint32_t raw_off = (kr * W + ngl) * 4;
    const uint32_t wt_off = C::kWOffset + ((ngl >> 3) * (kK / 8) + (kr >> 3)) * 1024 + krow * 128 + (((ngl & 7) ^ krow) << 4);
    // This warp takes every kExpandGroups-th k-block of the CTA's sequence (which runs on across
    // work items), starting with number my_group: the ring positions advance by that many slots.
    uint32_t rslot = 0, rphase = 0, wslot = 0, wphase = 0;
    auto advance = [](uint32_t& slot, uint32_t& phase, int n, int size) {
      slot += n;
      while (slot >= (uint32_t)size) { slot -= size; phase ^= 1; }
    };
    advance(rslot, rphase, my_group, RS);
    advance(wslot, wphase, my_group, WS);
    int lead = my_group;  // k-blocks of the next work item that belong to other groups before ours
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
      int xt, yt, kb0, kb1, split;
      decode(w, xt, yt, kb0, kb1, split);
      GroupRegs g;
      int g_cur = -1;
      int kb = kb0 + lead;
      for (; kb < kb1; kb += C::kExpandGroups) {
        {
          // the packed weights have landed and the work slot's previous tile has been consumed
          if (!mbar_wait(bar_raw_full + 8 * rslot, rphase, abort_flag, p.status, kErrExpand) ||
              !mbar_wait(bar_w_empty + 8 * wslot, wphase ^ 1, abort_flag, p.status, kErrExpand)) {
            ok = false;
            break;
          }
          const uint32_t rbase = raw_base + rslot * C::kRawSlotBytes;
          const uint32_t wbase = smem_base + wslot * C::kWorkSlotBytes;
          const int grp = p.group_shift >= 0 ? (kb >> p.group_shift) : (kb * kK) / p.group;
          if (grp != g_cur) {  // scales / zero points stay in registers while the k-group lasts
            uint4 sv;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(sv.x), "=r"(sv.y), "=r"(sv.z), "=r"(sv.w)
                         : "r"(rbase + C::kMetaOffset + ngl * 16));
            const uint32_t zw = has_zp ? lds32(rbase + C::kZpOffset + ngl * 4) : 0u;
            make_group(g, sv, zw, has_zp);
            g_cur = grp;
          }
          uint32_t wv[kPasses];
#pragma unroll
          for (int j = 0; j < kPasses; ++j) wv[j] = lds32(rbase + raw_off + j * kRowsPerPass * W * 4);
#pragma unroll
          for (int j = 0; j < kPasses; ++j) {
            // pair i = columns (i, i+4): stored in that order, the epilogue restores the column order
            sts128(wbase + wt_off + j * (kRowsPerPass / 8) * 1024, bf2_mul(bf2_sub(nib_pair(wv[j], 0), g.zr[0]), g.sp[0]),
                   bf2_mul(bf2_sub(nib_pair(wv[j], 1), g.zr[1]), g.sp[1]),
                   bf2_mul(bf2_sub(nib_pair(wv[j], 2), g.zr[2]), g.sp[2]),
                   bf2_mul(bf2_sub(nib_pair(wv[j], 3), g.zr[3]), g.sp[3]));
          }
          // every thread publishes its own writes to the async proxy (the tensor core's view of
          // shared memory); the warp then arrives once -- an arrival per thread would put hundreds
          // of serialised shared-memory atomics on the barrier every k-block
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_w_ready + 8 * wslot);
        }
        advance(rslot, rphase, C::kExpandGroups, RS);
        advance(wslot, wphase, C::kExpandGroups, WS);
      }
      lead = kb - kb1;  // how far the stride overshot this work item's range
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}


// ------------------------------------------------------------------------ CTA-pair form (large M)
// Two CTAs of a cluster share a 256-token x 256-column tile.  Each CTA loads its own 128 token
// rows and expands its own 128 weight columns per stage (half the expansion work and half the
// expanded-tile stores per CTA for the same tensor-core work as a 128 x 256 tile); the even CTA
// issues tcgen05.mma.cta_group::2 (M = 256, N = 256), which reads both CTAs' shared memory.
//
// A ring stage holds everything of one 64-deep k-block: activations, packed weights, scales /
// zero points and the expanded bf16 weight tile.  Per stage there are three barriers:
//   raw[s]    (each CTA)  this CTA's packed weights and scales landed           -> expanders
//   ready[s]  (even CTA)  activations of both CTAs landed (transaction bytes) and the
//                         expander warps of both CTAs finished the tile        -> MMA issuer
//   empty[s]  (each CTA)  the MMAs that read the stage retired (multicast commit) -> producer
// The expanders need no "tile free" barrier: raw[s] completes only after this CTA's producer
// saw empty[s] and refilled the stage.  The MMA issuer waits on one barrier per stage, and
// commits once.  Expander warps come in kExpandGroups groups that take alternate stages: the
// chain wait -> load -> expand -> store -> fence -> arrive of one stage is several times
// longer than the tensor-core time of a stage, so several stages are expanded concurrently.
template <int STAGES, int GROUPS>
struct PairCfg {
  static constexpr int kActBytes = 128 * 128;
  static constexpr int kRawOffset = kActBytes;
  static constexpr int kRawBytes = kRawUnit;  // 64 k x 16 words
  static constexpr int kMetaOffset = kRawOffset + kRawBytes;
  static constexpr int kScaleBytes = kUnit * 2, kZpBytes = kUnit / 2;
  static constexpr int kZpOffset = kMetaOffset + 512;
  static constexpr int kWOffset = kMetaOffset + 1024;  // 1024-byte aligned (swizzle atom)
  static constexpr int kWBytes = kUnit * 128;          // 128 columns x 64 k bf16
  static constexpr int kStageBytes = kWOffset + kWBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kNumBars = 3 * STAGES + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kExpandWarps = 8;  // per stage
  static constexpr int kExpandGroups = GROUPS;
  // Warp roles are placed by scheduler (warp % 4): the producer (warp 0) and the MMA issuer
  // (warp 4) share scheduler 0 with no expander warp; their per-stage instruction chains
  // (barrier wait, copies, MMAs, commit) run 25-40 % faster than when they compete with
  // expander warps for issue slots and the shared-memory instruction queue.  Epilogue: warps
  // 1, 2, 3 and 8 (TMEM lane quarters 1, 2, 3, 0; asleep during the main loop).  Expanders: the
  // warps >= 5 with warp % 4 != 0, in order.  Other warps of scheduler 0 idle.
  static constexpr int kLastExpander = kExpandWarps * kExpandGroups - 1;
  static constexpr int kWarps = 5 + (kLastExpander / 3) * 4 + kLastExpander % 3 + 1;
  static_assert(kWarps <= 32, "too many expander warps for one CTA");
  static constexpr int kThreads = 32 * kWarps;
  static_assert(kWOffset % 1024 == 0 && kStageBytes % 1024 == 0, "swizzled tiles need 1024-byte alignment");
};

template <int STAGES, int GROUPS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((PairCfg<STAGES, GROUPS>::kThreads), 1)
w4a16_pair_kernel(const __grid_constant__ CUtensorMap map_act, const __grid_constant__ CUtensorMap map_raw,
                  const __grid_constant__ CUtensorMap map_scale, const __grid_constant__ CUtensorMap map_zp, const Params p) {
  using C = PairCfg<STAGES, GROUPS>;
  constexpr int BN = 256;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBarOffset);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_stop = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const uint32_t rank = cluster_ctarank();
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_ready = smem_u32(bars), bar_empty = bar_ready + 8 * STAGES, bar_raw = bar_empty + 8 * STAGES;
  const uint32_t bar_tfull = bar_raw + 8 * STAGES, bar_tempty = bar_tfull + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  enum { kProducer, kMma, kEpilogue, kExpander, kIdle };
  const int ewarp = ((warp - 5) >> 2) * 3 + ((warp & 3) - 1);  // expander warp index (valid when that role)
  const int role = warp == 0 ? kProducer
                   : warp == 4 ? kMma
                   : (warp < 4 || warp == 8) ? kEpilogue
                   : ((warp & 3) != 0 && ewarp < C::kExpandWarps * C::kExpandGroups) ? kExpander
                                                                                      : kIdle;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_ready + 8 * s, 1 + 2 * C::kExpandWarps);  // producer + expander warps of both CTAs
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_raw + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 2 * kEpiThreads);
    }
    *abort_flag = 0;
    *epi_stop = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&map_act);
    tma_prefetch_desc(&map_raw);
    tma_prefetch_desc(&map_scale);
    if (p.zp) tma_prefetch_desc(&map_zp);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();  // everything above may run under the tail of the kernel in front of this one

  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_tiles = p.x_tiles * p.y_tiles;  // 256-token x 256-column tiles
  const int num_kb = p.num_kb;

  if (role == kProducer) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      const uint32_t meta_bytes = C::kScaleBytes + (p.zp ? C::kZpBytes : 0);
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int xt = tile % p.x_tiles, yt = tile / p.x_tiles;
        const int act_row0 = xt * 256 + (int)rank * 128;
        const int n0 = yt * BN + (int)rank * kUnit;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, kErrProducer)) {
            ok = false;
            break;
          }
          const uint32_t sbase = smem_base + stage * C::kStageBytes;
          const int grp = p.group_shift >= 0 ? (kb >> p.group_shift) : (kb * kK) / p.group;
          // packed weights and scales first: the expanders are the longer chain
          const uint32_t rawb = bar_raw + 8 * stage;
          mbar_arrive_expect_tx(rawb, C::kRawBytes + meta_bytes);
          tma_load_2d(sbase + C::kRawOffset, &map_raw, rawb, n0 / 8, kb * kK);
          tma_load_2d(sbase + C::kMetaOffset, &map_scale, rawb, n0, grp);
          if (p.zp) tma_load_2d(sbase + C::kZpOffset, &map_zp, rawb, n0 / 8, grp);
          // activations of both CTAs complete on the even CTA's barrier
          if (rank == 0) mbar_arrive_expect_tx(bar_ready + 8 * stage, 2 * C::kActBytes);
          tma_load_2d_pair(sbase, &map_act, (bar_ready + 8 * stage) & kPeerBitMask, kb * kK, act_row0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (role == kMma) {
    // ------------------------------------------------------------ MMA issuer (even CTA)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc_major(1u, 1u, 256, BN, 0u, 1u);
      const uint64_t da0 = smem_desc_k_sw128(smem_base);
      const uint64_t dw0 = smem_desc_mn_sw128(smem_base + C::kWOffset, (kK / 8) * 1024, 1024);
      uint32_t stage = 0, phase = 0, ready = 0;
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
        const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.status, kErrMmaTmem)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ready && !mbar_wait(bar_ready + 8 * stage, phase, abort_flag, p.status, kErrMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t soff = (uint64_t)(stage * (uint32_t)(C::kStageBytes >> 4));
          const uint64_t da = da0 + soff, dw = dw0 + soff;
          // four MMAs and the commit in one sequence, with a probe of the next stage's barrier
          // issued before and read after them
          const uint32_t nstage = stage + 1 == STAGES ? 0 : stage + 1;
          const uint32_t nphase = nstage == 0 ? phase ^ 1 : phase;
          static_assert(kK / 16 == 4, "umma_stage4_probe issues 4 MMAs");
          ready = umma_stage4_probe<true, true>(d_tmem, da, dw, idesc, kb != 0, bar_empty + 8 * stage,
                                                bar_ready + 8 * nstage, nphase, kUmmaKBytes >> 4, 2048 >> 4);
          stage = nstage;
          phase = nphase;
        }
        if (ok) umma_commit_pair_both(bar_tfull + 8 * acc);
      }
    }
  } else if (role == kEpilogue) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const int et = q * 32 + lane;
    int it = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++it) {
      const int xt = tile % p.x_tiles, yt = tile / p.x_tiles;
      const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
      mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, kErrEpilogue, 128);
      named_bar_sync(1, kEpiThreads);
      if (et == 0) *epi_stop = *abort_flag;
      named_bar_sync(1, kEpiThreads);
      if (*epi_stop) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      const int64_t m = (int64_t)xt * 256 + (int64_t)rank * 128 + q * 32 + lane;
      const int64_t y0 = (int64_t)yt * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c0, r);
        tmem_ld_wait();
        {  // tile-position order -> column order (see the single-CTA kernel)
          uint32_t t[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) t[(j & ~7) + ((j & 7) >> 1) + 4 * (j & 1)] = r[j];
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = t[j];
        }
        const int64_t n0 = y0 + c0;
        if (m < p.M) {
          if (p.out_dtype == B200Q_BF16) {
            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + m * p.ldo + n0;
            if (n0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(
                    pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                    pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                    pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])),
                    pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) o[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          } else {
            float* o = static_cast<float*>(p.out) + m * p.ldo + n0;
            if (n0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<uint4*>(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < p.N) o[j] = __uint_as_float(r[j]);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive_remote((bar_tempty + 8 * acc) & kPeerBitMask);  // the even CTA's barrier
    }
  } else if (role == kExpander) {
    // ------------------------------------------------------------ expanders
    // this CTA's 128 columns: 8 warps per stage, 4 packed words per thread
    const int et = (ewarp % C::kExpandWarps) * 32 + lane;
    const int my_group = ewarp / C::kExpandWarps;
    constexpr int W = 16;
    constexpr int kRowsPerPass = C::kExpandWarps * 32 / W;  // 16
    constexpr int kPasses = kK / kRowsPerPass;              // 4
    const int ngl = et % W, kr = et / W;
    const bool has_zp = p.zp != nullptr;
    const uint32_t krow = kr & 7;
    const uint32_t raw_off = C::kRawOffset + (kr * W + ngl) * 4;
    const uint32_t wt_off = C::kWOffset + ((ngl >> 3) * (kK / 8) + (kr >> 3)) * 1024 + krow * 128 + (((ngl & 7) ^ krow) << 4);
    uint32_t stage = 0, phase = 0;
    int turn = 0;  // whose stage this is
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      GroupRegs g;
      int g_cur = -1;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (turn == my_group) {
          if (!mbar_wait(bar_raw + 8 * stage, phase, abort_flag, p.status, kErrExpand)) {
            ok = false;
            break;
          }
          const uint32_t sbase = smem_base + stage * C::kStageBytes;
          const int grp = p.group_shift >= 0 ? (kb >> p.group_shift) : (kb * kK) / p.group;
          if (grp != g_cur) {
            uint4 sv;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(sv.x), "=r"(sv.y), "=r"(sv.z), "=r"(sv.w)
                         : "r"(sbase + C::kMetaOffset + ngl * 16));
            const uint32_t zw = has_zp ? lds32(sbase + C::kZpOffset + ngl * 4) : 0u;
            make_group(g, sv, zw, has_zp);
            g_cur = grp;
          }
          uint32_t wv[kPasses];
#pragma unroll
          for (int j = 0; j < kPasses; ++j) wv[j] = lds32(sbase + raw_off + j * kRowsPerPass * W * 4);
#pragma unroll
          for (int j = 0; j < kPasses; ++j) {
            sts128(sbase + wt_off + j * (kRowsPerPass / 8) * 1024, bf2_mul(bf2_sub(nib_pair(wv[j], 0), g.zr[0]), g.sp[0]),
                   bf2_mul(bf2_sub(nib_pair(wv[j], 1), g.zr[1]), g.sp[1]),
                   bf2_mul(bf2_sub(nib_pair(wv[j], 2), g.zr[2]), g.sp[2]),
                   bf2_mul(bf2_sub(nib_pair(wv[j], 3), g.zr[3]), g.sp[3]));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (rank == 0) mbar_arrive(bar_ready + 8 * stage);
            else mbar_arrive_remote((bar_ready + 8 * stage) & kPeerBitMask);  // the even CTA's barrier
          }
        }
        if (++turn == C::kExpandGroups) turn = 0;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int STAGES, int GROUPS>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mr, const CUtensorMap& ms, const CUtensorMap& mz,
                       const Params& p, cudaStream_t st) {
  using C = PairCfg<STAGES, GROUPS>;
  constexpr int smem = C::kTotal + 1024;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  static_assert(smem > 116 * 1024, "one CTA per SM: two CTAs must never contend for TMEM");
  auto kern = w4a16_pair_kernel<STAGES, GROUPS>;
  static std::atomic<int> resident_pairs[kMaxDevices];
  const int dev = current_device_index();
  if (dev < 0) return B200Q_ERR_CUDA;
  int clusters = resident_pairs[dev].load(std::memory_order_acquire);
  if (clusters == 0) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kNumSMs, 1, 1);
    cfg.blockDim = dim3(C::kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = -1;
    }
    resident_pairs[dev].store(clusters, std::memory_order_release);
  }
  if (clusters < 0) return B200Q_ERR_UNSUPPORTED;
  const int tiles = p.x_tiles * p.y_tiles;
  const int pairs = tiles < clusters ? tiles : clusters;
  if (launch_overlapped(kern, dim3((unsigned)(2 * pairs)), dim3(C::kThreads), smem, st, ma, mr, ms, mz, p) != cudaSuccess) {
    (void)cudaGetLastError();
    kern<<<2 * pairs, C::kThreads, smem, st>>>(ma, mr, ms, mz, p);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

// Sum the fp32 partial tiles of a split-K run (in split order) and round once to the output dtype.
// VEC = 4: four neighbouring columns per thread (N and ldo multiples of 4, 16-byte aligned
// pointers): 16-byte loads of the partials, one division per four outputs, an 8- or 16-byte
// store.  Launched under the tail of the GEMM kernel; it waits for that grid before it reads.
template <int VEC>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, void* out, int out_dtype,
                                                            int64_t M, int64_t N, int64_t ldo, int splits) {
  pdl_enter();
  const int64_t total = M * N / VEC;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = i * VEC, m = e / N, n = e - m * N;
    if (VEC == 4) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < splits; ++s) {
        const float4 t = __ldcs(reinterpret_cast<const float4*>(partial + (int64_t)s * M * N + e));
        v.x += t.x, v.y += t.y, v.z += t.z, v.w += t.w;
      }
      if (out_dtype == B200Q_BF16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + m * ldo + n) =
            make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      } else {
        *reinterpret_cast<float4*>(static_cast<float*>(out) + m * ldo + n) = v;
      }
    } else {
      float v = 0.f;
      for (int s = 0; s < splits; ++s) v += partial[(int64_t)s * M * N + e];
      if (out_dtype == B200Q_BF16) static_cast<__nv_bfloat16*>(out)[m * ldo + n] = __float2bfloat16_rn(v);
      else static_cast<float*>(out)[m * ldo + n] = v;
    }
  }
}

template <int BN, int RS, int WS, int GROUPS, int AR = 0, int EW = 0>
static int launch(const CUtensorMap& ma, const CUtensorMap& mr, const CUtensorMap& ms, const CUtensorMap& mz, const Params& p,
                  cudaStream_t st) {
  using C = Cfg<BN, RS, WS, GROUPS, AR, EW>;
  constexpr int smem = C::kTotal + 1024;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  // TMEM: CTAs that share an SM must never ask for more than 512 columns together
  static_assert(C::kTmemCols * (227 * 1024 / smem) <= 512, "TMEM over-subscription");
  auto kern = w4a16_kernel<BN, RS, WS, GROUPS, AR, EW>;
  static std::atomic<int> configured[kMaxDevices];
  const int dev = current_device_index();
  if (dev < 0) return B200Q_ERR_CUDA;
  if (!configured[dev].load(std::memory_order_acquire)) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev].store(1, std::memory_order_release);
  }
  int work = p.x_tiles * p.y_tiles * p.splits;
  int per_sm = 227 * 1024 / smem;
  int grid = work < kNumSMs * per_sm ? work : kNumSMs * per_sm;
  if (launch_overlapped(kern, dim3((unsigned)grid), dim3(C::kThreads), (size_t)smem, st, ma, mr, ms, mz, p) != cudaSuccess) {
    (void)cudaGetLastError();
    kern<<<grid, C::kThreads, smem, st>>>(ma, mr, ms, mz, p);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // namespace w4

// Number of K splits the small-M path uses (every split gets at least one k-block), and the
// fp32 workspace that goes with it.
static int w4a16_splits(int64_t M, int64_t N, int64_t K) {
  if (M > 128) return 1;
  // 128-token x 256-column tiles; the split count that minimises the busiest CTA's k-blocks
  // (plus a few per work item for its pipeline fill and its partial-tile epilogue)
  const int64_t tiles = (N + 255) / 256;
  const int64_t num_kb = K / w4::kK;
  if (num_kb <= 0) return 1;  // K below one k-block: nothing to split (and nothing to divide by below)
  int64_t best_cost = 0;
  int best = 1;
  for (int s = 1; s <= 16 && s * 4 <= num_kb; ++s) {
    const int64_t rounds = (tiles * s + kNumSMs - 1) / kNumSMs;
    const int64_t cost = rounds * ((num_kb + s - 1) / s + 4);
    if (s == 1 || cost < best_cost) { best_cost = cost; best = s; }
  }
  const int64_t per = (num_kb + best - 1) / best;
  return (int)((num_kb + per - 1) / per);  // drop splits that would be empty
}

// few-token kernel (w4a16_smallm.cu)
bool w4a16_smallm_eligible(int64_t M, int64_t N, int64_t K, int64_t group, int k_packed);
int w4a16_smallm_launch(const void* x, int64_t ldx, const int32_t* qweight, const void* scale, const int32_t* zp,
                        int k_packed, int64_t M, int64_t N, int64_t K, int64_t group, void* out, int out_dtype,
                        int64_t ldo, cudaStream_t st);

size_t w4a16_workspace_bytes_impl(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0 || K % w4::kK || N % 32) return 0;  // shapes the fused kernel does not take
  if (w4a16_smallm_eligible(M, N, K, w4::kK, 0)) return 0;  // reduced inside its clusters: no scratch
  const int s = w4a16_splits(M, N, K);
  return s > 1 ? (size_t)s * (size_t)M * (size_t)N * sizeof(float) : 0;
}

int w4a16_gemm_impl(const void* x, int64_t ldx, const int32_t* qweight, const void* scale, const int32_t* zp,
                    int zp_kind, int k_packed, int64_t M, int64_t N, int64_t K, int64_t group, void* out,
                    int out_dtype, int64_t ldo, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (K == 0) {
    // an empty contraction: the result is all zeros (rows may be strided)
    const size_t esz = out_dtype == B200Q_BF16 ? 2 : 4;
    B200Q_CUDA_OK(cudaMemset2DAsync(out, (size_t)ldo * esz, 0, (size_t)N * esz, (size_t)M, st));
    return B200Q_OK;
  }
  // a handful of tokens: the streaming kernel (either weight layout)
  if (w4a16_smallm_eligible(M, N, K, group, k_packed)) {
    const int rc = w4a16_smallm_launch(x, ldx, qweight, scale, zp_kind == B200Q_ZP_PACKED ? zp : nullptr, k_packed, M, N, K,
                                       group, out, out_dtype, ldo, st);
    if (rc != B200Q_ERR_UNSUPPORTED) return rc;
  }
  if (k_packed) return B200Q_ERR_UNSUPPORTED;  // the tcgen05 kernels take the operator layout [K][N/8]
  if (K % w4::kK || group % w4::kK || K % group || N % 32 || ldx % 8) return B200Q_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(qweight) | reinterpret_cast<uintptr_t>(scale)) & 15)
    return B200Q_ERR_UNSUPPORTED;
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return B200Q_ERR_TOO_LARGE;
  w4::Params p;
  p.scale = static_cast<const __nv_bfloat16*>(scale);
  p.zp = zp_kind == B200Q_ZP_PACKED ? zp : nullptr;
  p.out = out; p.partial = nullptr; p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.group = (int)group;
  {
    const int64_t gk = group / w4::kK;
    p.group_shift = -1;
    for (int sh = 0; sh < 24; ++sh)
      if (gk == (1ll << sh)) p.group_shift = sh;
  }
  p.out_dtype = out_dtype; p.num_kb = (int)(K / w4::kK);
  p.status = device_status_ptr();
  if (!p.status) return B200Q_ERR_CUDA;
  const bool small_m = M <= 128;
  p.splits = small_m ? w4a16_splits(M, N, K) : 1;
  p.kb_per_split = (p.num_kb + p.splits - 1) / p.splits;
  if (p.splits > 1) {
    const size_t need = (size_t)p.splits * (size_t)M * (size_t)N * sizeof(float);
    if (!workspace || workspace_bytes < need) return B200Q_ERR_BAD_ARGUMENT;
    p.partial = static_cast<float*>(workspace);
  }
  CUtensorMap ma, mr;
  int rc = 0;
  const int bn_w = (!small_m && N > 128) ? 256 : 128;  // weight columns per stage tile
  rc = make_tma_map_2d(&mr, qweight, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, N / 8, K, (N / 8) * 4, bn_w / 8, w4::kK,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  CUtensorMap ms, mz;
  rc = make_tma_map_2d(&ms, scale, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K / group, N * 2, bn_w, 1, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  if (p.zp) {
    if (reinterpret_cast<uintptr_t>(p.zp) & 15) return B200Q_ERR_UNSUPPORTED;
    rc = make_tma_map_2d(&mz, p.zp, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, N / 8, K / group, (N / 8) * 4, bn_w / 8, 1,
                         CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  } else {
    mz = ms;  // never dereferenced
  }
  static const bool no_pairs = std::getenv("B200Q_W4A16_NO_PAIRS") != nullptr;
  if (bn_w == 256 && !no_pairs) {
    // CTA pairs: 256-token x 256-column tiles, each CTA expands 128 columns
    w4::Params pp = p;
    pp.x_tiles = (int)((M + 255) / 256);
    pp.y_tiles = (int)((N + 255) / 256);
    CUtensorMap mr1, ms1, mz1;
    rc = make_tma_map_2d(&mr1, qweight, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, N / 8, K, (N / 8) * 4, 16, w4::kK,
                         CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = make_tma_map_2d(&ms1, scale, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K / group, N * 2, 128, 1, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    mz1 = ms1;
    if (p.zp) {
      rc = make_tma_map_2d(&mz1, p.zp, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, N / 8, K / group, (N / 8) * 4, 16, 1,
                           CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rc) return rc;
    }
    rc = make_tma_map_2d(&ma, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, ldx * 2, w4::kK, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = w4::launch_pair<6, 2>(ma, mr1, ms1, mz1, pp, st);
    if (rc != B200Q_ERR_UNSUPPORTED) return rc;
  }
  if (!small_m) {
    p.x_tiles = (int)((M + 127) / 128);
    const int bn = bn_w;
    p.y_tiles = (int)((N + bn - 1) / bn);
    rc = make_tma_map_2d(&ma, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, ldx * 2, w4::kK, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    if (bn == 256) rc = w4::launch<256, 8, 3, 1>(ma, mr, ms, mz, p, st);
    else rc = w4::launch<128, 12, 4, 2>(ma, mr, ms, mz, p, st);
  } else {
    // small M, token-major with a narrow activation tile: 128 x 256 MMAs cover twice the weight
    // columns per instruction of the weight-major form, whose issue rate is what bounds it
    p.x_tiles = 1;
    p.y_tiles = (int)((N + 255) / 256);
    CUtensorMap mr2, ms2, mz2;
    rc = make_tma_map_2d(&mr2, qweight, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, N / 8, K, (N / 8) * 4, 32, w4::kK,
                         CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = make_tma_map_2d(&ms2, scale, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K / group, N * 2, 256, 1, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    mz2 = ms2;
    if (p.zp) {
      rc = make_tma_map_2d(&mz2, p.zp, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, N / 8, K / group, (N / 8) * 4, 32, 1,
                           CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rc) return rc;
    }
    const int ar = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    rc = make_tma_map_2d(&ma, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, ldx * 2, w4::kK, ar, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    // three expander groups over four work slots (24 expander warps, 32 warps in all): the
    // expand -> MMA -> release round trip of a work slot is what paces small M
    switch (ar) {
      case 16: rc = w4::launch<256, 8, 4, 3, 16, 8>(ma, mr2, ms2, mz2, p, st); break;
      case 32: rc = w4::launch<256, 8, 4, 3, 32, 8>(ma, mr2, ms2, mz2, p, st); break;
      case 64: rc = w4::launch<256, 6, 4, 3, 64, 8>(ma, mr2, ms2, mz2, p, st); break;
      default: rc = w4::launch<256, 7, 3, 3, 0, 8>(ma, mr2, ms2, mz2, p, st); break;
    }
  }
  if (rc) return rc;
  if (p.splits > 1) {
    const int esz = out_dtype == B200Q_BF16 ? 2 : 4;
    const bool vec4 = (N % 4) == 0 && (ldo % 4) == 0 && (reinterpret_cast<uintptr_t>(out) % (4 * esz)) == 0 &&
                      (reinterpret_cast<uintptr_t>(p.partial) & 15) == 0;
    const int64_t total = vec4 ? M * N / 4 : M * N;
    int grid = (int)((total + 255) / 256);
    if (grid > kNumSMs * 8) grid = kNumSMs * 8;
    auto kern = vec4 ? w4::splitk_reduce_kernel<4> : w4::splitk_reduce_kernel<1>;
    if (launch_overlapped(kern, dim3((unsigned)grid), dim3(256), 0, st, (const float*)p.partial, out, out_dtype, M, N, ldo,
                          p.splits) != cudaSuccess) {
      (void)cudaGetLastError();
      kern<<<grid, 256, 0, st>>>(p.partial, out, out_dtype, M, N, ldo, p.splits);
    }
    B200Q_LAUNCH_CHECK();
  }
  return B200Q_OK;
}

// ------------------------------------------------------------------------ allocation-free variant
// Scratch for b200q_w4a16_gemm_noalloc: it lives in the library image, so every GPU that loads
// the library carries these 8 MiB until the process exits, and the caller never has to hand in
// (or allocate) a workspace.  Only device code may use the name directly; host code must ask the
// runtime for the device address (below).
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) float g_w4a16_static_scratch[kStaticScratchBytes / sizeof(float)];

// Device address of the static scratch on the current device.  In host code the array's name
// is only a stand-in for the symbol, not a pointer the GPU can follow, so the address is
// looked up with cudaGetSymbolAddress -- once per device, with that device current -- and kept.
static int static_scratch_ptr(float** out) {
  static std::atomic<float*> cache[kMaxDevices];
  const int dev = current_device_index();
  if (dev < 0) return B200Q_ERR_CUDA;
  float* p = cache[dev].load(std::memory_order_acquire);
  if (!p) {
    void* addr = nullptr;
    B200Q_CUDA_OK(cudaGetSymbolAddress(&addr, g_w4a16_static_scratch));
    p = static_cast<float*>(addr);
    cache[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return B200Q_OK;
}

int w4a16_gemm_noalloc_impl(const void* x, int64_t ldx, const int32_t* qweight, const void* scale, const int32_t* zp,
                            int zp_kind, int k_packed, int64_t M, int64_t N, int64_t K, int64_t group, void* out,
                            int out_dtype, int64_t ldo, cudaStream_t st) {
  // (shapes the fused kernel rejects report a zero workspace here and are refused, with their
  // own code, by the argument checks of w4a16_gemm_impl)
  const size_t need = w4a16_workspace_bytes_impl(M, N, K);
  if (need > kStaticScratchBytes) return B200Q_ERR_TOO_LARGE;
  float* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc) return rc;
  // Nothing in the scratch has to start at zero: every (split, row, column) cell that the
  // reduction reads is written by exactly one CTA of this call first.
  return w4a16_gemm_impl(x, ldx, qweight, scale, zp, zp_kind, k_packed, M, N, K, group, out, out_dtype, ldo, scratch,
                         kStaticScratchBytes, st);
}

size_t w4a16_noalloc_max_bytes_impl() { return kStaticScratchBytes; }

}  // namespace b200q



