// W4A16 GEMM for a handful of tokens (M <= 16): out[M][N] = x[M][K] . W[K][N] with W held as
// packed 4-bit words.  At this size the operator is a stream over the packed weights (0.5 byte
// per weight against 32 flop), so the kernel is built around bytes in flight, contiguous DRAM
// accesses and instructions per weight, not around the tensor pipe:
//
//   * a CTA of 16 warps covers 256 output columns: warp w streams the 64-column strip w % 4 over
//     k-part w / 4 of the CTA's k-slice.  A thread-block cluster of 4 CTAs splits K into 4 slices
//     (16 with the k-parts): N / 256 clusters, 128 CTAs for N = 8192, all resident at once
//     (clusters of 8 left a sixth of the SMs unused: 15 of them fit on the GPU).
//   * every warp copies its part with cp.async into a ring of its own (6 - 8 KB in flight per warp,
//     about 100 KB per SM) and shares no barrier with any other warp in the main loop; the 16 tokens'
//     activations of a k-part are staged in shared memory 512 k-rows at a time by its four warps
//     (one barrier among them per 512 rows), in the order the MMA fragments read them.
//   * a thread reads whole packed words from the ring, expands them in registers with packed
//     bf16x2 arithmetic -- (128 + q) - (128 + z) exact, one rounding in the multiply by the scale:
//     the bytes of the stand-alone dequant kernel -- and feeds mma.sync.m16n8k16 with the weights
//     as the 16-row operand (two output columns per thread and instruction) and 8 tokens as the
//     8-column operand.  About 3 instructions per weight.
//   * the four k-parts of a CTA add their fp32 partial tiles through shared memory, the 4 CTAs of
//     the cluster add theirs through distributed shared memory (CTA r finishes 64 of the 256
//     columns), always in the same order: no global scratch, no second kernel, the same bits on
//     every run.
//
// Two weight layouts: the operator's [K][N/8] (a word = 8 neighbouring columns of one k; k-pairs
// for the MMA operand are built with two byte permutes per four weights) and AutoGPTQ's [K/8][N]
// (a word = 8 consecutive k of one column; a word's nibble pairs are used as k-pairs directly and
// the activations are permuted to match, which costs nothing per weight).
#include <cuda.h>

#include "common.cuh"

namespace b200q {
namespace w4s {

constexpr int kWarps = 16;
constexpr int kThreads = 32 * kWarps;
constexpr int kCluster = 4;
constexpr int kStrips = 4;            // 64-column strips per CTA
constexpr int kParts = kWarps / kStrips;  // k-parts per CTA
constexpr int kStrip = 64;            // output columns per warp
constexpr int kCols = kStrips * kStrip;   // output columns per CTA / cluster
constexpr int kSlices = kParts * kCluster;  // k-slices: cluster rank x k-part
constexpr int kRingBytes = 8192;      // per warp
constexpr int kBatch = 4;             // operator layout: k-steps per ring slot (one wait, one refill per slot)
constexpr int kSlotBytes = kBatch * 512;
constexpr int kSlots = kRingBytes / kSlotBytes;
constexpr int kXChunkRows = 512;      // k-rows of activations staged at a time per k-part
constexpr int kXBytes = kXChunkRows * 16 * 2;             // 16 tokens x 512 k, bf16 = 16 KB
constexpr int kXOffset = kWarps * kRingBytes;
constexpr int kPartOffset = kXOffset + kParts * kXBytes;  // CTA partial tile [16][256] fp32
constexpr int kSmemBytes = kPartOffset + 16 * kCols * 4;  // 208 KB

struct Params {
  const int32_t* qw;
  const __nv_bfloat16* scale;  // [K/group][N]
  const int32_t* zp;           // [K/group][N/8] or null
  const __nv_bfloat16* x;      // [M][K], row stride ldx
  void* out;
  int64_t M, N, K, ldx, ldo;
  int group, out_dtype;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait(int pending) {  // the count must be an immediate
  switch (pending) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    case 7: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    case 8: asm volatile("cp.async.wait_group 8;" ::: "memory"); break;
    case 9: asm volatile("cp.async.wait_group 9;" ::: "memory"); break;
    case 10: asm volatile("cp.async.wait_group 10;" ::: "memory"); break;
    case 11: asm volatile("cp.async.wait_group 11;" ::: "memory"); break;
    case 12: asm volatile("cp.async.wait_group 12;" ::: "memory"); break;
    case 13: asm volatile("cp.async.wait_group 13;" ::: "memory"); break;
    case 14: asm volatile("cp.async.wait_group 14;" ::: "memory"); break;
    case 15: asm volatile("cp.async.wait_group 15;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 16;" ::: "memory"); break;
  }
}
__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
// nibbles i and i + 4 of a word as the bf16x2 {128 + q_i, 128 + q_{i+4}}
__device__ __forceinline__ uint32_t nib_pair(uint32_t w, int i) { return ((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u; }
__device__ __forceinline__ void named_bar(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// MT = token blocks of 8 (M <= 8 * MT).  KP = 0: operator layout [K][N/8]; 1: AutoGPTQ layout [K/8][N].
//
// Thread (g = lane / 4, q = lane % 4) owns 8 of its warp's 64 columns and feeds 4 MMAs per k-step
// whose 16 operand rows are output columns:
//   KP = 0  step = 16 k-rows; the thread's word column g (columns 8g .. 8g + 7) of k-rows
//           {2q, 2q+1, 2q+8, 2q+9}; MMA i: operand row g = column 8g + i, row g + 8 = column 8g + i + 4
//   KP = 1  step = 64 k-rows = 8 word-rows; columns g + 8j (j = 0..7) of word-rows q and q + 4; MMA
//           i of accumulator a takes its k labels (2q, 2q+1) from nibbles (i, i+4) of word-row q
//           and (2q+8, 2q+9) from the same nibbles of word-row q + 4 -- over q and i every nibble
//           of the 8 word-rows once -- with the activation fragment gathered the same way;
//           accumulator a = columns g + 16a (operand row g) and g + 16a + 8 (row g + 8)
template <int MT, int KP>
__global__ void __cluster_dims__(kCluster, 1, 1) __launch_bounds__(kThreads, 1) w4a16_smallm_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_enter();  // launched under the tail of the kernel in front of it
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const int strip = warp & (kStrips - 1), khalf = warp / kStrips;  // (khalf: the warp's k-part)
  const uint32_t crank = cluster_rank();
  const int cg = blockIdx.x / kCluster;
  const int64_t n0 = (int64_t)cg * kCols + strip * kStrip;  // first column of this warp's strip
  constexpr int kStepRows = KP ? 64 : 16;
  constexpr int kStageBytes = 2048;                 // KP = 1: a ring stage is one k-step
  constexpr int kDepth = kRingBytes / kStageBytes;  // 4 steps in flight
  const int64_t rows_per_slice = p.K / kSlices;
  const int64_t k_begin = ((int64_t)crank * kParts + khalf) * rows_per_slice;
  const int steps = (int)(rows_per_slice / kStepRows);
  const int64_t nw = KP ? p.N : p.N / 8;  // words per row of the packed matrix
  uint8_t* ring = smem + warp * kRingBytes;
  const uint32_t ring_u = smem_addr(ring);

  // One k-step in the ring.  KP = 0: 16 rows x 8 words, one 16-byte copy per lane (row
  // lane / 2, words 4 (lane % 2) ..); rows are stored in the order [load L = (row & 1) + 2 (row >> 3)]
  // [(row >> 1) & 3] so that load L of thread (g, q) -- word g of row 2q (+1, +8, +9) -- is
  // conflict-free.  KP = 1: 8 word-rows x 64 columns, 16-byte pieces XOR-swizzled by word-row so
  // that the column-strided reads are conflict-free.
  // this lane's source of the next step to be issued, and where its copy goes inside a stage
  const int32_t* w_src;
  uint32_t w_dst = 0;
  if (KP == 0) {
    const int row = lane >> 1, hf = lane & 1;
    w_dst = (((row & 1) + 2 * (row >> 3)) * 4 + ((row >> 1) & 3)) * 32 + hf * 16;
    w_src = p.qw + (k_begin + row) * nw + n0 / 8 + 4 * hf;
  } else {
    w_src = p.qw + (k_begin / 8) * nw + n0 + (lane & 15) * 4;  // (word-row offsets are added per copy)
  }
  // KP = 0: k-steps 4t .. 4t + 3 (those that exist) into slot t % kSlots, as one group -- committed
  // even when empty, so that the number of groups that may stay pending is the same at every t
  auto issue_batch = [&](int t) {
    const uint32_t dst = ring_u + (t & (kSlots - 1)) * kSlotBytes + w_dst;
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
      if (t * kBatch + j < steps) cp_async16(dst + j * 512, w_src + (int64_t)j * 16 * nw);
    w_src += (int64_t)kBatch * 16 * nw;
    cp_async_commit();
  };
  auto issue = [&](int s) {  // KP = 1: one k-step into stage s % kDepth
    const uint32_t dst = ring_u + (s & (kDepth - 1)) * kStageBytes;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int id = c * 32 + lane, w = id >> 4, piece = id & 15;
      cp_async16(dst + w * 256 + ((piece * 16) ^ ((w & 3) * 32)), w_src + (int64_t)w * nw);
    }
    w_src += 8 * nw;
    cp_async_commit();
  };
  // The activations of k-rows [k_begin + 512 c, + 512) of this k-part, copied by its 4 warps (8
  // pieces of 16 bytes per thread) in fragment order.  KP = 0: per step of 16 rows
  // [k half][token][16 bytes]; KP = 1: per step of 64 rows [token][128 bytes] with the 16-byte
  // pieces XOR-swizzled by token parity.  Tokens beyond M read the last real token's row.
  const uint32_t xs_u = smem_addr(smem + kXOffset + khalf * kXBytes);
  const uint8_t* xs = smem + kXOffset + khalf * kXBytes;
  auto stage_x = [&](int chunk) {
    const int64_t kc = k_begin + (int64_t)chunk * kXChunkRows;
    const int64_t rows = rows_per_slice - (int64_t)chunk * kXChunkRows < kXChunkRows
                             ? rows_per_slice - (int64_t)chunk * kXChunkRows : kXChunkRows;
    const int tid = strip * 32 + lane;  // 0..127 inside the k-part
#pragma unroll
    for (int c = 0; c < kXBytes / 16 / (32 * kStrips); ++c) {
      const int id = c * (32 * kStrips) + tid;  // 16-byte piece of the chunk
      if (KP == 0) {
        const int step = id >> 5, tok = (id & 31) >> 1, hf = id & 1;
        if (step * 16 < rows)
          cp_async16(xs_u + step * 512 + hf * 256 + tok * 16, p.x + (tok < p.M ? tok : p.M - 1) * p.ldx + kc + step * 16 + 8 * hf);
      } else {
        const int step = id >> 7, tok = (id & 127) >> 3, piece = id & 7;
        if (step * 64 < rows)
          cp_async16(xs_u + step * 2048 + tok * 128 + ((piece ^ ((tok & 1) << 2)) * 16),
                     p.x + (tok < p.M ? tok : p.M - 1) * p.ldx + kc + step * 64 + 8 * piece);
      }
    }
    cp_async_commit();
  };
  constexpr int kStepsPerChunk = kXChunkRows / kStepRows;

  stage_x(0);
  if (KP == 0) {
    for (int t = 0; t < kSlots - 1; ++t) issue_batch(t);
  } else {
    for (int t = 0; t < kDepth - 1; ++t) {
      if (t < steps) issue(t);
      else cp_async_commit();
    }
  }

  float acc[4][MT][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[a][t][e] = 0.f;

  // group bookkeeping without divisions in the loop: steps until the next group begins (+1: the
  // counter is decremented before step 0 as well)
  int64_t cur_grp = k_begin / p.group;
  const int steps_per_group = p.group / kStepRows;
  int to_next_group = steps_per_group - (int)((k_begin % p.group) / kStepRows) + 1;
  if (KP == 0) {
    // scales and 128 + zero point of the thread's 8 columns, each twice in a register: lo[i] column
    // 8g + i, hi[i] column 8g + i + 4 (an operand register holds two k of one column)
    uint32_t slo[4], shi[4], zlo[4], zhi[4];
    // The scales and zero points of a group are fetched one group ahead: a load that is consumed at
    // once comes back behind the cp.async traffic this warp has queued, i.e. after a full memory
    // latency, once per group.
    uint4 nsv;
    uint32_t nz;
    const int64_t last_grp = (p.K - 1) / p.group;
    auto fetch_group = [&](int64_t grp) {
      if (grp > last_grp) grp = last_grp;  // (never used then)
      nsv = __ldg(reinterpret_cast<const uint4*>(p.scale + grp * p.N + n0 + 8 * g));
      nz = p.zp ? (uint32_t)__ldg(p.zp + grp * (p.N / 8) + n0 / 8 + g) : 0u;
    };
    auto load_group = [&](int64_t grp) {  // takes what fetch_group(grp) asked for, asks for grp + 1
      const uint4 sv = nsv;
      const uint32_t z = nz;
      fetch_group(grp + 1);
      slo[0] = __byte_perm(sv.x, 0u, 0x1010); slo[1] = __byte_perm(sv.x, 0u, 0x3232);
      slo[2] = __byte_perm(sv.y, 0u, 0x1010); slo[3] = __byte_perm(sv.y, 0u, 0x3232);
      shi[0] = __byte_perm(sv.z, 0u, 0x1010); shi[1] = __byte_perm(sv.z, 0u, 0x3232);
      shi[2] = __byte_perm(sv.w, 0u, 0x1010); shi[3] = __byte_perm(sv.w, 0u, 0x3232);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        zlo[i] = (((z >> (4 * i)) & 15u) * 0x00010001u) | 0x43004300u;
        zhi[i] = (((z >> (4 * i + 16)) & 15u) * 0x00010001u) | 0x43004300u;
      }
    };
    // One k-step: the lane's four packed words (word g of k-rows 2q, 2q + 1, 2q + 8, 2q + 9) are
    // transposed while still packed -- two byte permutes per pair of rows put the same four
    // columns of both rows into one word -- so that a nibble pair (i, i + 4) of such a word is
    // one column at two consecutive k: the operand register the MMA wants, with nothing to
    // shuffle after the expansion.
    auto k_step = [&](const uint8_t* wp, const uint8_t* xp) {
      uint32_t b[MT][2];
#pragma unroll
      for (int tk = 0; tk < MT; ++tk) {
        b[tk][0] = *reinterpret_cast<const uint32_t*>(xp + tk * 128);
        b[tk][1] = *reinterpret_cast<const uint32_t*>(xp + 256 + tk * 128);
      }
      uint32_t w[4];
#pragma unroll
      for (int L = 0; L < 4; ++L) w[L] = *reinterpret_cast<const uint32_t*>(wp + L * 128);
      const uint32_t m0 = __byte_perm(w[0], w[1], 0x5410), m1 = __byte_perm(w[0], w[1], 0x7632);
      const uint32_t m2 = __byte_perm(w[2], w[3], 0x5410), m3 = __byte_perm(w[2], w[3], 0x7632);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t a0 = bf2_mul(bf2_sub(nib_pair(m0, i), zlo[i]), slo[i]);
        const uint32_t a1 = bf2_mul(bf2_sub(nib_pair(m1, i), zhi[i]), shi[i]);
        const uint32_t a2 = bf2_mul(bf2_sub(nib_pair(m2, i), zlo[i]), slo[i]);
        const uint32_t a3 = bf2_mul(bf2_sub(nib_pair(m3, i), zhi[i]), shi[i]);
#pragma unroll
        for (int tk = 0; tk < MT; ++tk) mma_bf16(acc[i][tk], a0, a1, a2, a3, b[tk][0], b[tk][1]);
      }
    };
    fetch_group(cur_grp);
    load_group(cur_grp);  // before the first wait: its latency hides under the weights'
    // A ring slot holds kBatch k-steps: per slot one wait, one warp barrier (which also says that
    // every lane is done with the slot before), one refill of that slot and one set of addresses;
    // per k-step only 4 + 2 MT shared loads, the expansion and the MMAs (plus the group countdown
    // in a slot that a group boundary or the end of the slice cuts).
    constexpr int kBatchesPerChunk = kXChunkRows / (16 * kBatch);
    const int batches = (steps + kBatch - 1) / kBatch;
    for (int t = 0; t < batches; ++t) {
      if ((t & (kBatchesPerChunk - 1)) == 0) {
        // a new chunk of activations: the first one was issued before the weights (it is the
        // oldest group), a later one is issued here, after every warp of the k-half is done
        // with the old chunk, and waited for at once
        if (t > 0) {
          named_bar(1 + khalf, 32 * kStrips);
          stage_x(t / kBatchesPerChunk);
          cp_async_wait(0);
        } else {
          asm volatile("cp.async.wait_group %0;" ::"n"(kSlots - 1) : "memory");  // all but the weights: the chunk
        }
        named_bar(1 + khalf, 32 * kStrips);
      }
      asm volatile("cp.async.wait_group %0;" ::"n"(kSlots - 2) : "memory");
      __syncwarp();
      issue_batch(t + kSlots - 1);
      const uint8_t* sl = ring + (t & (kSlots - 1)) * kSlotBytes + q * 32 + g * 4;
      const uint8_t* xb = xs + (t & (kBatchesPerChunk - 1)) * (kBatch * 512) + g * 16 + 4 * q;
      const int nst = steps - t * kBatch;
      if (to_next_group == 1) {  // a group begins with this slot's first step
        to_next_group = steps_per_group + 1;
        load_group(++cur_grp);
      }
      if (nst >= kBatch && to_next_group > kBatch) {  // a whole slot inside one group: nothing to test per step
        to_next_group -= kBatch;
#pragma unroll
        for (int j = 0; j < kBatch; ++j) k_step(sl + j * 512, xb + j * 512);
      } else {
#pragma unroll 1
        for (int j = 0; j < kBatch && j < nst; ++j) {
          if (--to_next_group == 0) {  // (a division per step costs more than the step's arithmetic)
            to_next_group = steps_per_group;
            load_group(++cur_grp);
          }
          k_step(sl + j * 512, xb + j * 512);
        }
      }
    }
  } else {
    // per accumulator a the two columns g + 16a and g + 16a + 8: scale and 128 + zero point, each
    // twice in a register (an operand register holds two k of one column), set up once per group
    uint32_t sc2[4][2], zc2[4][2];
    auto load_group = [&](int64_t grp) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        sc2[j >> 1][j & 1] = (uint32_t)__bfloat16_as_ushort(p.scale[grp * p.N + n0 + g + 8 * j]) * 0x00010001u;
        // column n0 + g + 8j is nibble g of zero-point word n0 / 8 + j
        const uint32_t z = p.zp ? ((uint32_t)__ldg(p.zp + grp * (p.N / 8) + n0 / 8 + j) >> (4 * g)) & 15u : 0u;
        zc2[j >> 1][j & 1] = (z * 0x00010001u) | 0x43004300u;
      }
    };
    load_group(cur_grp);
    // A stage is refilled one step after it was read (after the warp barrier of the next step),
    // so its words are loaded where they are used instead of all in front of the refill; every
    // step commits a group, an empty one past the end, so that the wait is the same at every step.
    auto issue_or_empty = [&](int s) {
      if (s < steps) issue(s);
      else cp_async_commit();
    };
    const uint32_t lane_off = q * 256 + g * 4, q32 = q * 32;
    for (int s = 0; s < steps; ++s) {
      if ((s & (kStepsPerChunk - 1)) == 0) {
        if (s > 0) {
          named_bar(1 + khalf, 32 * kStrips);
          stage_x(s / kStepsPerChunk);
          cp_async_wait(0);
        } else {
          asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 1) : "memory");  // all but the weights: the chunk
        }
        named_bar(1 + khalf, 32 * kStrips);
      }
      asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 2) : "memory");
      __syncwarp();  // step s has landed for every lane, and every lane is done with the stage of step s - 1
      issue_or_empty(s + kDepth - 1);
      if (--to_next_group == 0) {
        to_next_group = steps_per_group;
        load_group(++cur_grp);
      }
      // [token block][word-row q / q + 4][nibble pair i]: (x[k_i], x[k_{i+4}]) of that word-row's 8 k
      uint32_t bx[MT][2][4];
      const uint8_t* xf = xs + (s & (kStepsPerChunk - 1)) * 2048;
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        const int tok = 8 * t + g;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xf + tok * 128 + (((q + 4 * h) ^ ((tok & 1) << 2)) * 16));
          bx[t][h][0] = __byte_perm(xv.x, xv.z, 0x5410);
          bx[t][h][1] = __byte_perm(xv.x, xv.z, 0x7632);
          bx[t][h][2] = __byte_perm(xv.y, xv.w, 0x5410);
          bx[t][h][3] = __byte_perm(xv.y, xv.w, 0x7632);
        }
      }
      // word (word-row wr, column g + 8j) sits at wr * 256 + ((g + 8j) * 4 ^ (wr & 3) * 32); with wr = q or
      // q + 4 that is lane_off (+ 1024) + 32 (j ^ q)
      const uint8_t* st = ring + (s & (kDepth - 1)) * kStageBytes + lane_off;
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const uint32_t o0 = (uint32_t)(64 * a) ^ q32, o1 = (uint32_t)(64 * a + 32) ^ q32;
        const uint32_t w00 = *reinterpret_cast<const uint32_t*>(st + o0), w01 = *reinterpret_cast<const uint32_t*>(st + o1);
        const uint32_t w10 = *reinterpret_cast<const uint32_t*>(st + 1024 + o0),
                       w11 = *reinterpret_cast<const uint32_t*>(st + 1024 + o1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t a0 = bf2_mul(bf2_sub(nib_pair(w00, i), zc2[a][0]), sc2[a][0]);
          const uint32_t a1 = bf2_mul(bf2_sub(nib_pair(w01, i), zc2[a][1]), sc2[a][1]);
          const uint32_t a2 = bf2_mul(bf2_sub(nib_pair(w10, i), zc2[a][0]), sc2[a][0]);
          const uint32_t a3 = bf2_mul(bf2_sub(nib_pair(w11, i), zc2[a][1]), sc2[a][1]);
#pragma unroll
          for (int t = 0; t < MT; ++t) mma_bf16(acc[a][t], a0, a1, a2, a3, bx[t][0][i], bx[t][1][i]);
        }
      }
    }
  }

  // ---------------------------------------------------------------- reduction
  // warp partial tile -> this warp's ring (all of its copies have landed and been read):
  // red[warp][token 0..15][column 0..63] fp32 = 4 KB
  cp_async_wait(0);
  __syncwarp();
  float* red = reinterpret_cast<float*>(ring);
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int col_lo = KP ? g + 16 * a : 8 * g + a, col_hi = KP ? col_lo + 8 : col_lo + 4;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      const int tok = 8 * t + 2 * q;
      red[tok * kStrip + col_lo] = acc[a][t][0];
      red[(tok + 1) * kStrip + col_lo] = acc[a][t][1];
      red[tok * kStrip + col_hi] = acc[a][t][2];
      red[(tok + 1) * kStrip + col_hi] = acc[a][t][3];
    }
  }
  __syncthreads();
  // CTA partial tile part[token][256 columns] = the k-parts' tiles in part order
  float* part = reinterpret_cast<float*>(smem + kPartOffset);
  for (int e = threadIdx.x; e < 8 * MT * kCols; e += kThreads) {
    const int tok = e / kCols, col = e % kCols, st = col / kStrip, c = col % kStrip;
    float v = 0.f;
#pragma unroll
    for (int kp = 0; kp < kParts; ++kp)
      v += reinterpret_cast<const float*>(smem + (kp * kStrips + st) * kRingBytes)[tok * kStrip + c];
    part[e] = v;
  }
  cluster_sync();
  // CTA r of the cluster finishes columns [64 r, 64 r + 64): the CTA partials in rank order
  const uint32_t part_u = smem_addr(part);
  for (int e = threadIdx.x; e < 8 * MT * kStrip; e += kThreads) {
    const int tok = e / kStrip, col = (int)crank * kStrip + e % kStrip;
    float v = 0.f;
#pragma unroll
    for (uint32_t r = 0; r < (uint32_t)kCluster; ++r) v += ld_cluster_f32(part_u + (tok * kCols + col) * 4, r);
    if (tok < p.M) {
      const int64_t idx = (int64_t)tok * p.ldo + (int64_t)cg * kCols + col;
      if (p.out_dtype == B200Q_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(v);
      else static_cast<float*>(p.out)[idx] = v;
    }
  }
  cluster_sync();  // no CTA leaves while another may still read its partial tile
}

template <int MT, int KP>
static int launch(const Params& p, cudaStream_t st) {
  auto kern = w4a16_smallm_kernel<MT, KP>;
  static std::atomic<int> configured[kMaxDevices];
  const int dev = current_device_index();
  if (dev < 0) return B200Q_ERR_CUDA;
  if (!configured[dev].load(std::memory_order_acquire)) {
    B200Q_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[dev].store(1, std::memory_order_release);
  }
  const int grid = (int)(p.N / kCols) * kCluster;
  if (launch_overlapped(kern, dim3((unsigned)grid), dim3(kThreads), kSmemBytes, st, p) != cudaSuccess) {
    (void)cudaGetLastError();
    kern<<<grid, kThreads, kSmemBytes, st>>>(p);
  }
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // namespace w4s

// Whether the few-token kernel takes this problem: M <= 16, whole 256-column blocks, K divisible
// into 16 slices of whole k-steps (16 rows; 64 for the AutoGPTQ layout), groups that k-steps do
// not straddle.
bool w4a16_smallm_eligible(int64_t M, int64_t N, int64_t K, int64_t group, int k_packed) {
  const int64_t step = k_packed ? 64 : 16;
  return M >= 1 && M <= 16 && N >= w4s::kCols && N % w4s::kCols == 0 && K >= w4s::kSlices * step &&
         K % (w4s::kSlices * step) == 0 && group % step == 0 && K % group == 0;
}

int w4a16_smallm_launch(const void* x, int64_t ldx, const int32_t* qweight, const void* scale, const int32_t* zp,
                        int k_packed, int64_t M, int64_t N, int64_t K, int64_t group, void* out, int out_dtype,
                        int64_t ldo, cudaStream_t st) {
  if (!w4a16_smallm_eligible(M, N, K, group, k_packed)) return B200Q_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(qweight) | reinterpret_cast<uintptr_t>(scale)) & 15)
    return B200Q_ERR_UNSUPPORTED;
  if (ldx % 8) return B200Q_ERR_UNSUPPORTED;
  w4s::Params p;
  p.qw = qweight; p.scale = static_cast<const __nv_bfloat16*>(scale); p.zp = zp;
  p.x = static_cast<const __nv_bfloat16*>(x); p.out = out;
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldo = ldo; p.group = (int)group; p.out_dtype = out_dtype;
  if (k_packed) return M <= 8 ? w4s::launch<1, 1>(p, st) : w4s::launch<2, 1>(p, st);
  return M <= 8 ? w4s::launch<1, 0>(p, st) : w4s::launch<2, 0>(p, st);
}

}  // namespace b200q
