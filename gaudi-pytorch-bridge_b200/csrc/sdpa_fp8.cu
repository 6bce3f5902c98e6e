// FP8 scaled-dot-product attention, forward: out = softmax(q k^T * scale + mask) v with q, k, v in
// e4m3 and the probabilities re-quantised to e4m3 for the second product.
//
// tcgen05 kernel (head dimension 128), one CTA per (batch x head, block of 128 queries), 320 threads:
//   warp 0    TMA producer: the query tile once, then the key tiles (twice, see below) and value
//             tiles through two shared-memory rings (128-byte swizzle, no multicast)
//   warp 1    TMEM owner and MMA issuer: S = Q K^T (kind::f8f6f4, 128 x 128 x 32 per instruction)
//             into one of two score buffers in TMEM, and O += P V with P read from shared memory
//             (K-major) and V through an MN-major descriptor (V is stored [key][d]: no transpose)
//   warps 2-9 softmax, two groups of four warps; a group owns one of the two score buffers (it takes
//             every other key block) and thread = query row: tcgen05.ld of its score row, scale /
//             mask / exp2, the e4m3 probabilities written into the swizzled P tile for the second
//             product.  Blocks with nothing to mask take a path of one instruction per score in
//             the first pass and 3.5 in the second (FFMA, ex2.approx, add, half a convert: the
//             probability scale is folded into the exponent and divided out of the row sum).
// Two passes over the keys: the first only takes the row maxima, the second recomputes the
// scores and forms exp(S - max) against the final maximum.  The probabilities are therefore
// quantised exactly where the CPU restatement quantises them (no running-maximum rescaling of
// an accumulator that already holds rounded products), the accumulator in TMEM is never read
// back and corrected, and the price is one extra Q K^T per block on a tensor pipe that the
// softmax arithmetic leaves half idle anyway.
//
// Every wait is bounded (tcgen05_ptx.cuh); a wait that runs out sets the device status word.
// Other head dimensions, and anything else the fast path does not take, run a plain CUDA kernel.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05_ptx.cuh"
#include "tma_host.cuh"

namespace b200q {

using namespace ptx;

namespace sdpa {

constexpr int kD = 128;        // head dimension of the tcgen05 path (bytes per row)
constexpr int kBM = 128;       // queries per CTA
constexpr int kBN = 128;       // keys per block
constexpr int kStages = 3;     // key / value ring depth
constexpr int kTile = 128 * 128;  // bytes of every tile here
constexpr int kThreads = 320;   // producer warp, MMA warp, two softmax warpgroups
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kMasked = -1.0e30f;

enum { kErrProducer = 301, kErrMma = 302, kErrSoftmax = 303 };

struct Params {
  void* out;               // bf16 or e4m3 [BH][L][D]
  int out_fp8;
  __nv_bfloat16* m_out;    // [BH][L] or null
  __nv_bfloat16* linv_out; // [BH][L] or null
  float* amax_s;           // or null; zeroed by the caller
  float* amax_o;
  const void* mask;        // additive (bf16 / f32) or boolean (1 = keep), or null
  int mask_kind;           // 0 none, 1 bf16, 2 f32, 3 bool
  int64_t mask_sb, mask_sl;  // element strides of the flattened batch x head index and of the query row
  int64_t BH, L, S;
  int kv_rep;              // query heads per key/value head: kv index = bh / kv_rep
  int causal;
  // the six scales of the operator: a device scalar when the pointer is set, else the host value
  const float* scale_dev[6];  // d_scale_q, d_scale_k, d_scale_v, q_scale_s, q_scale_o, d_scale_s
  float scale_host[6];
  int d_scale_s_given;     // 0: d_scale_s = 1 / q_scale_s
  float softmax_scale;
  int* status;
  // derived in the kernel (Scales::load)
  float c_log2, q_scale_s, o_scale, q_scale_o;
};

// c_log2 = d_scale_q * d_scale_k * softmax scale * log2(e); o_scale = d_scale_s * d_scale_v
__device__ __forceinline__ void load_scales(Params& p) {
  float s[6];
#pragma unroll
  for (int i = 0; i < 6; ++i) s[i] = p.scale_dev[i] ? __ldg(p.scale_dev[i]) : p.scale_host[i];
  p.c_log2 = (s[0] * s[1]) * p.softmax_scale * kLog2e;
  p.q_scale_s = s[3];
  p.q_scale_o = s[4];
  p.o_scale = (p.d_scale_s_given ? s[5] : 1.f / s[3]) * s[2];
}

// warp maximum of a non-negative float (bit patterns of non-negative floats order like the values)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float warp_max_f32_bits(float x) { return __uint_as_float(warp_max_u32(__float_as_uint(x))); }

// mask term of (row, key) in the log2 domain
__device__ __forceinline__ float mask_term(const Params& p, int64_t bh, int64_t row, int64_t key) {
  if (p.mask_kind == 0) return 0.f;
  const int64_t idx = bh * p.mask_sb + row * p.mask_sl + key;
  if (p.mask_kind == 1) return __bfloat162float(static_cast<const __nv_bfloat16*>(p.mask)[idx]) * kLog2e;
  if (p.mask_kind == 2) return static_cast<const float*>(p.mask)[idx] * kLog2e;
  return static_cast<const uint8_t*>(p.mask)[idx] ? 0.f : kMasked;
}

struct Smem {
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kP = kV + kStages * kTile;
  static constexpr int kRowStats = kP + 2 * kTile;        // [2 groups][128 rows] fp32: maxima, then sums
  static constexpr int kBars = kRowStats + 2 * 128 * 4;
  // barriers: q_full, k_full[3], k_empty[3], v_full[3], v_empty[3], s_full[2], s_empty[2], p_full[2], p_empty[2], o_full
  static constexpr int kNumBars = 1 + 4 * kStages + 8 + 1;
  static constexpr int kTotal = kBars + kNumBars * 8 + 16;
};

__global__ void __launch_bounds__(kThreads, 1)
sdpa_fp8_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const Params p_in) {
  Params p = p_in;
  load_scales(p);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* sm_stop = reinterpret_cast<volatile int*>(tmem_slot + 2);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_q = b0, bar_kf = b0 + 8, bar_ke = bar_kf + 8 * kStages, bar_vf = bar_ke + 8 * kStages,
                 bar_ve = bar_vf + 8 * kStages, bar_sf = bar_ve + 8 * kStages, bar_se = bar_sf + 16, bar_pf = bar_se + 16,
                 bar_pe = bar_pf + 16, bar_of = bar_pe + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int64_t bh = blockIdx.y;
  // (the last query blocks first: under a causal mask they have the most key blocks, and a long
  // CTA that starts late is what the kernel ends on)
  const int64_t q0 = (int64_t)(gridDim.x - 1 - blockIdx.x) * kBM;
  const int64_t kv = bh / p.kv_rep;
  // key blocks this query block needs (causal: keys beyond its last query are all masked)
  int64_t keys = p.S;
  if (p.causal && q0 + kBM < keys) keys = q0 + kBM;
  const int nblk = (int)((keys + kBN - 1) / kBN);

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_kf + 8 * s, 1); mbar_init(bar_ke + 8 * s, 1);
      mbar_init(bar_vf + 8 * s, 1); mbar_init(bar_ve + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_sf + 8 * a, 1); mbar_init(bar_se + 8 * a, 128);
      mbar_init(bar_pf + 8 * a, 128); mbar_init(bar_pe + 8 * a, 1);
    }
    mbar_init(bar_of, 1);
    *abort_flag = 0;
    *sm_stop = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_k); tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;  // columns [0,128) S0, [128,256) S1, [256,384) O

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      mbar_arrive_expect_tx(bar_q, kTile);
      tma_load_3d(sbase + Smem::kQ, &map_q, bar_q, 0, (int)q0, (int)bh);
      uint32_t ks = 0, kph = 0, vs = 0, vph = 0;
      bool ok = true;
      for (int t = 0; t < 2 * nblk && ok; ++t) {
        const int j = t < nblk ? t : t - nblk;
        if (!mbar_wait(bar_ke + 8 * ks, kph ^ 1, abort_flag, p.status, kErrProducer)) break;
        mbar_arrive_expect_tx(bar_kf + 8 * ks, kTile);
        tma_load_3d(sbase + Smem::kK + ks * kTile, &map_k, bar_kf + 8 * ks, 0, j * kBN, (int)kv);
        if (++ks == kStages) { ks = 0; kph ^= 1; }
        if (t >= nblk) {
          if (!mbar_wait(bar_ve + 8 * vs, vph ^ 1, abort_flag, p.status, kErrProducer)) { ok = false; break; }
          mbar_arrive_expect_tx(bar_vf + 8 * vs, kTile);
          tma_load_3d(sbase + Smem::kV + vs * kTile, &map_v, bar_vf + 8 * vs, 0, j * kBN, (int)kv);
          if (++vs == kStages) { vs = 0; vph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(0, 0, kBM, kBN);                      // Q, K both K-major e4m3
      const uint32_t idesc_o = umma_idesc_major(0, 0, kBM, kD, 0, 1);           // P K-major, V MN-major
      const uint64_t qd = smem_desc_k_sw128(sbase + Smem::kQ);
      uint32_t ks = 0, kph = 0, vs = 0, vph = 0;
      bool ok = mbar_wait(bar_q, 0, abort_flag, p.status, kErrMma);
      // O += P_j V_j
      auto pv = [&](int j) {
        const uint32_t pb = j & 1, pph = (j >> 1) & 1;
        if (!mbar_wait(bar_pf + 8 * pb, pph, abort_flag, p.status, kErrMma)) return false;
        if (!mbar_wait(bar_vf + 8 * vs, vph, abort_flag, p.status, kErrMma)) return false;
        tc_fence_after();
        const uint64_t pd = smem_desc_k_sw128(sbase + Smem::kP + pb * kTile);
        const uint64_t vd = smem_desc_mn_sw128(sbase + Smem::kV + vs * kTile, 128 * 128, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f8(tmem + 256, pd + 2 * k, vd + 256 * k, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(bar_ve + 8 * vs);
        umma_commit(bar_pe + 8 * pb);
        if (++vs == kStages) { vs = 0; vph ^= 1; }
        return true;
      };
      for (int t = 0; t < 2 * nblk && ok; ++t) {
        const uint32_t sb = t & 1, sph = (t >> 1) & 1;
        if (!mbar_wait(bar_kf + 8 * ks, kph, abort_flag, p.status, kErrMma)) break;
        if (!mbar_wait(bar_se + 8 * sb, sph ^ 1, abort_flag, p.status, kErrMma)) break;
        tc_fence_after();
        const uint64_t kd = smem_desc_k_sw128(sbase + Smem::kK + ks * kTile);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f8(tmem + sb * 128, qd + 2 * k, kd + 2 * k, idesc_s, k > 0 ? 1u : 0u);
        umma_commit(bar_ke + 8 * ks);
        umma_commit(bar_sf + 8 * sb);
        if (++ks == kStages) { ks = 0; kph ^= 1; }
        // the second product of the block before: its probabilities are ready by now
        if (t >= nblk + 1) ok = pv(t - nblk - 1);
      }
      if (ok && nblk > 0) ok = pv(nblk - 1);
      if (ok) umma_commit(bar_of);
    }
  } else {
    // ------------------------------------------------------------ softmax (warps 2..9)
    const int grp = (warp - 2) >> 2;          // 0 / 1: the score buffer (and key blocks t = grp mod 2) of this group
    const int qtr = warp & 3;                 // TMEM lane quarter of this warp
    const int row = qtr * 32 + lane;          // query row inside the block = TMEM lane
    const int64_t qi = q0 + row;              // query index
    const int st = (threadIdx.x - 64) & 127;  // 0..127 inside the group
    const int bar_id = 1 + grp;               // named barrier of the group; 3 = both groups
    const uint32_t t_lane = tmem + ((uint32_t)(qtr * 32) << 16);
    float* stats = reinterpret_cast<float*>(smem + Smem::kRowStats);
    float mx = kMasked;                       // row maximum, log2 domain
    float off = 0.f;                          // log2(q_scale_s) - mx (second pass)
    float ls[4] = {0.f, 0.f, 0.f, 0.f};       // partial row sums of the scaled probabilities
    const float lq = log2f(p.q_scale_s);
    bool stop = false;
    // nothing to mask in a block: no mask tensor, all of its keys exist and (causal) lie at or
    // before the first query of this block
    auto block_plain = [&](int j) {
      const int64_t key0 = (int64_t)j * kBN;
      return p.mask_kind == 0 && key0 + kBN <= p.S && (!p.causal || key0 + kBN - 1 <= q0);
    };
    // One key block of this group: scores -> row maximum (first pass) or e4m3 probabilities and
    // row sum (second pass).  Returns false when a wait ran out.
    auto do_tile = [&](int t) {
      const bool second = t >= nblk;
      const int j = second ? t - nblk : t;
      const uint32_t sb = grp, sph = (t >> 1) & 1;
      mbar_wait(bar_sf + 8 * sb, sph, abort_flag, p.status, kErrSoftmax, 32);
      if (second && j >= 2) mbar_wait(bar_pe + 8 * (j & 1), ((j >> 1) - 1) & 1, abort_flag, p.status, kErrSoftmax, 32);
      named_bar_sync(bar_id, 128);
      if (st == 0) sm_stop[grp] = *abort_flag;
      named_bar_sync(bar_id, 128);
      if (sm_stop[grp]) return false;
      tc_fence_after();
      const int64_t key0 = (int64_t)j * kBN;
      const bool plain = block_plain(j);
      uint8_t* prow = smem + Smem::kP + (j & 1) * kTile + row * 128;
      // the row in two halves of 64 scores: both loads of a half are in flight together
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
      uint32_t rr[2][32];
      tmem_ld_32x32(t_lane + sb * 128 + half * 64, rr[0]);
      tmem_ld_32x32(t_lane + sb * 128 + half * 64 + 32, rr[1]);
      tmem_ld_wait();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * half + cc;
        const uint32_t* r = rr[cc];
        float x[32];
        if (plain) {
#pragma unroll
          for (int e = 0; e < 32; ++e) x[e] = __uint_as_float(r[e]) * p.c_log2;
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int64_t key = key0 + c * 32 + e;
            float v = __uint_as_float(r[e]) * p.c_log2;
            if (p.mask_kind) v += mask_term(p, bh, qi < p.L ? qi : p.L - 1, key < p.S ? key : p.S - 1);
            if (key >= p.S || (p.causal && key > qi)) v = kMasked;
            x[e] = v;
          }
        }
        if (!second) {
          float m4[4] = {mx, kMasked, kMasked, kMasked};
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            m4[0] = fmaxf(m4[0], x[e]); m4[1] = fmaxf(m4[1], x[e + 1]);
            m4[2] = fmaxf(m4[2], x[e + 2]); m4[3] = fmaxf(m4[3], x[e + 3]);
          }
          mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        } else {
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            float pr[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              pr[u] = ex2_approx(x[e + u] + off);  // = exp(S - max) * q_scale_s
              ls[u] += pr[u];
            }
            // (the conversion saturates at 448: a probability scale beyond that cannot overflow)
            w[e >> 2] = cvt_fp8x2<B200Q_E4M3>(pr[0], pr[1]) | (cvt_fp8x2<B200Q_E4M3>(pr[2], pr[3]) << 16);
          }
          // 32 keys = two 16-byte pieces (2c, 2c + 1) of the row, XOR-swizzled by the row
          *reinterpret_cast<uint4*>(prow + (((2 * c) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(prow + (((2 * c + 1) ^ (row & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
      }
      tc_fence_before();
      mbar_arrive(bar_se + 8 * sb);  // the score buffer may be overwritten
      if (second) {
        fence_proxy_async_smem();    // the P tile is read by the tensor core (async proxy)
        mbar_arrive(bar_pf + 8 * (j & 1));
      }
      return true;
    };
    // first pass: this group's blocks t = grp, grp + 2, ... < nblk
    for (int t = grp; t < nblk && !stop; t += 2) stop = !do_tile(t);
    // between the passes both groups meet (stopped or not, exactly once): the row maximum over
    // all blocks
    stats[grp * 128 + row] = mx;
    named_bar_sync(3, 256);
    mx = fmaxf(stats[row], stats[128 + row]);
    off = lq - mx;
    named_bar_sync(3, 256);
    // second pass: tiles t = nblk .. 2 nblk - 1 with t = grp (mod 2)
    for (int t = nblk + ((nblk & 1) == grp ? 0 : 1); t < 2 * nblk && !stop; t += 2) stop = !do_tile(t);
    // ---- output: O / l, scaled.  The row sums of both groups are added, then group 0 writes the
    // first 64 output columns of its rows and group 1 the other 64.
    float lsum = (ls[0] + ls[1]) + (ls[2] + ls[3]);
    if (!stop && nblk > 0) {
      mbar_wait(bar_of, 0, abort_flag, p.status, kErrSoftmax, 64);
      named_bar_sync(bar_id, 128);
      if (st == 0) sm_stop[grp] = *abort_flag;
      named_bar_sync(bar_id, 128);
      stop = sm_stop[grp] != 0;
    }
    // (both groups reach these two barriers exactly once, stopped or not)
    stats[grp * 128 + row] = lsum;
    named_bar_sync(3, 256);
    lsum = (stats[row] + stats[128 + row]) / p.q_scale_s;
    if (!stop) {
      tc_fence_after();
      const float linv = lsum > 0.f ? 1.f / lsum : 0.f;
      const float osc = p.o_scale * linv;
      float amax_o = 0.f;
      const bool in = qi < p.L;
#pragma unroll 1
      for (int c = 2 * grp; c < 2 * grp + 2; ++c) {
        uint32_t r[32];
        if (nblk > 0) {
          tmem_ld_32x32(t_lane + 256 + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0u;
        }
        float o[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          o[e] = __uint_as_float(r[e]) * osc;
          amax_o = fmaxf(amax_o, fabsf(o[e]));
        }
        if (in) {
          if (p.out_fp8) {
            uint8_t* dst = static_cast<uint8_t*>(p.out) + (bh * p.L + qi) * kD + c * 32;
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              w[e >> 2] = cvt_fp8x2<B200Q_E4M3>(clampf<B200Q_E4M3>(o[e] * p.q_scale_o), clampf<B200Q_E4M3>(o[e + 1] * p.q_scale_o)) |
                          (cvt_fp8x2<B200Q_E4M3>(clampf<B200Q_E4M3>(o[e + 2] * p.q_scale_o), clampf<B200Q_E4M3>(o[e + 3] * p.q_scale_o)) << 16);
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(dst + 16) = make_uint4(w[4], w[5], w[6], w[7]);
          } else {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + (bh * p.L + qi) * kD + c * 32;
#pragma unroll
            for (int e = 0; e < 32; e += 8)
              *reinterpret_cast<uint4*>(dst + e) = make_uint4(pack_bf16x2(o[e], o[e + 1]), pack_bf16x2(o[e + 2], o[e + 3]),
                                                            pack_bf16x2(o[e + 4], o[e + 5]), pack_bf16x2(o[e + 6], o[e + 7]));
          }
        }
      }
      if (in && grp == 0) {
        if (p.m_out) p.m_out[bh * p.L + qi] = __float2bfloat16_rn(mx / kLog2e);
        if (p.linv_out) p.linv_out[bh * p.L + qi] = __float2bfloat16_rn(linv);
      }
      // amax of the probabilities (1 / l of a row is its largest probability) and of the output
      if (p.amax_s && grp == 0) {
        const float a = warp_max_f32_bits(in ? linv : 0.f);
        if (lane == 0 && a > 0.f) atomicMax(reinterpret_cast<unsigned int*>(p.amax_s), __float_as_uint(a));
      }
      if (p.amax_o) {
        const float a = warp_max_f32_bits(in ? amax_o : 0.f);
        if (lane == 0 && a > 0.f) atomicMax(reinterpret_cast<unsigned int*>(p.amax_o), __float_as_uint(a));
      }
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
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------ plain kernel
// Any head dimensions up to 256: one block of 128 threads per (batch x head, query).  Same two
// passes, same quantisation points; scores of a block of 128 keys go through shared memory.
__global__ void __launch_bounds__(128) sdpa_fp8_plain_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ k,
                                                             const uint8_t* __restrict__ v, int dqk, int dv, const Params p_in) {
  Params p = p_in;
  load_scales(p);
  __shared__ float s_q[256];
  __shared__ float s_p[128];
  __shared__ float s_red[4];
  const int64_t bh = blockIdx.y, qi = blockIdx.x, kvh = bh / p.kv_rep;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  for (int d = tid; d < dqk; d += 128) s_q[d] = fp8_to_float<B200Q_E4M3>(q[(bh * p.L + qi) * dqk + d]);
  __syncthreads();
  int64_t keys = p.S;
  if (p.causal && qi + 1 < keys) keys = qi + 1;
  auto score = [&](int64_t key) {
    float acc = 0.f;
    const uint8_t* kr = k + (kvh * p.S + key) * dqk;
    for (int d = 0; d < dqk; ++d) acc += s_q[d] * fp8_to_float<B200Q_E4M3>(kr[d]);
    float x = acc * p.c_log2;
    if (p.mask_kind) x += mask_term(p, bh, qi, key);
    return x;
  };
  auto block_max = [&](float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xFFFFFFFFu, x, o));
    __syncthreads();
    if (lane == 0) s_red[wid] = x;
    __syncthreads();
    return fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
  };
  float mx = kMasked;
  for (int64_t k0 = 0; k0 < keys; k0 += 128)
    if (k0 + tid < keys) mx = fmaxf(mx, score(k0 + tid));
  mx = block_max(mx);
  float lsum = 0.f;
  float acc0 = 0.f, acc1 = 0.f;  // output elements tid and tid + 128
  for (int64_t k0 = 0; k0 < keys; k0 += 128) {
    float pr = 0.f;
    if (k0 + tid < keys) pr = exp2f(score(k0 + tid) - mx);
    lsum += pr;
    const float p8 = fp8_to_float<B200Q_E4M3>(cvt_fp8x2<B200Q_E4M3>(fminf(pr * p.q_scale_s, 448.f), 0.f) & 0xFFu);
    __syncthreads();
    s_p[tid] = p8;
    __syncthreads();
    const int n = (int)(keys - k0 < 128 ? keys - k0 : 128);
    for (int j = 0; j < n; ++j) {
      const uint8_t* vr = v + (kvh * p.S + k0 + j) * dv;
      if (tid < dv) acc0 += s_p[j] * fp8_to_float<B200Q_E4M3>(vr[tid]);
      if (tid + 128 < dv) acc1 += s_p[j] * fp8_to_float<B200Q_E4M3>(vr[tid + 128]);
    }
  }
  // row sum over the block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xFFFFFFFFu, lsum, o);
  __syncthreads();
  if (lane == 0) s_red[wid] = lsum;
  __syncthreads();
  lsum = (s_red[0] + s_red[1]) + (s_red[2] + s_red[3]);
  const float linv = lsum > 0.f ? 1.f / lsum : 0.f;
  const float osc = p.o_scale * linv;
  float amax_o = 0.f;
  for (int h = 0; h < 2; ++h) {
    const int d = tid + 128 * h;
    if (d >= dv) continue;
    const float o = (h ? acc1 : acc0) * osc;
    amax_o = fmaxf(amax_o, fabsf(o));
    const int64_t idx = (bh * p.L + qi) * dv + d;
    if (p.out_fp8) static_cast<uint8_t*>(p.out)[idx] = (uint8_t)(cvt_fp8x2<B200Q_E4M3>(clampf<B200Q_E4M3>(o * p.q_scale_o), 0.f) & 0xFFu);
    else static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(o);
  }
  if (tid == 0) {
    if (p.m_out) p.m_out[bh * p.L + qi] = __float2bfloat16_rn(mx / kLog2e);
    if (p.linv_out) p.linv_out[bh * p.L + qi] = __float2bfloat16_rn(linv);
    if (p.amax_s && linv > 0.f) atomicMax(reinterpret_cast<unsigned int*>(p.amax_s), __float_as_uint(linv));
  }
  if (p.amax_o) {
    const float a = warp_max_f32_bits(amax_o);
    if (lane == 0 && a > 0.f) atomicMax(reinterpret_cast<unsigned int*>(p.amax_o), __float_as_uint(a));
  }
}

static int make_map_3d(CUtensorMap* map, const void* base, int64_t d_bytes, int64_t rows, int64_t batch) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return B200Q_ERR_CUDA;
  cuuint64_t dims[3] = {(cuuint64_t)d_bytes, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)d_bytes, (cuuint64_t)(d_bytes * rows)};
  cuuint32_t box[3] = {128, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200Q_OK : B200Q_ERR_CUDA;
}

}  // namespace sdpa

int sdpa_fp8_fwd_impl(const b200q_sdpa_args& a, cudaStream_t st) {
  const void *q = a.q, *k = a.k, *v = a.v;
  void* out = a.out;
  const int64_t BH = a.BH, L = a.L, S = a.S;
  const int dqk = a.dqk, dv = a.dv, kv_rep = a.kv_rep, force_plain = a.force_plain;
  sdpa::Params p;
  p.out = out; p.out_fp8 = a.out_dtype == B200Q_E4M3;
  p.m_out = static_cast<__nv_bfloat16*>(a.m_out); p.linv_out = static_cast<__nv_bfloat16*>(a.linv_out);
  p.amax_s = a.amax_s; p.amax_o = a.amax_o;
  p.mask = a.mask; p.mask_kind = a.mask ? a.mask_kind : 0; p.mask_sb = a.mask_sb; p.mask_sl = a.mask_sl;
  p.BH = BH; p.L = L; p.S = S; p.kv_rep = kv_rep; p.causal = a.causal;
  const float* devs[6] = {a.d_scale_q, a.d_scale_k, a.d_scale_v, a.q_scale_s, a.q_scale_o, a.d_scale_s};
  const float hosts[6] = {a.d_scale_q_host, a.d_scale_k_host, a.d_scale_v_host, a.q_scale_s_host, a.q_scale_o_host, a.d_scale_s_host};
  for (int i = 0; i < 6; ++i) { p.scale_dev[i] = devs[i]; p.scale_host[i] = hosts[i]; }
  p.d_scale_s_given = a.d_scale_s_given;
  p.softmax_scale = a.softmax_scale;
  p.c_log2 = p.q_scale_s = p.o_scale = p.q_scale_o = 0.f;
  p.status = device_status_ptr();
  if (!p.status) return B200Q_ERR_CUDA;
  if (BH > 65535) return B200Q_ERR_TOO_LARGE;
  const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                         reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (!force_plain && dqk == sdpa::kD && dv == sdpa::kD && aligned && S >= 1) {
    CUtensorMap mq, mk, mv;
    int rc = sdpa::make_map_3d(&mq, q, dqk, L, BH);
    if (!rc) rc = sdpa::make_map_3d(&mk, k, dqk, S, BH / kv_rep);
    if (!rc) rc = sdpa::make_map_3d(&mv, v, dv, S, BH / kv_rep);
    if (rc) return rc;
    constexpr int smem = sdpa::Smem::kTotal + 1024;
    static_assert(smem <= 227 * 1024 && smem > 116 * 1024, "one CTA per SM");
    static std::atomic<int> configured[kMaxDevices];
    const int dev = current_device_index();
    if (dev < 0) return B200Q_ERR_CUDA;
    if (!configured[dev].load(std::memory_order_acquire)) {
      B200Q_CUDA_OK(cudaFuncSetAttribute(sdpa::sdpa_fp8_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      configured[dev].store(1, std::memory_order_release);
    }
    dim3 grid((unsigned)((L + sdpa::kBM - 1) / sdpa::kBM), (unsigned)BH);
    sdpa::sdpa_fp8_tcgen05_kernel<<<grid, sdpa::kThreads, smem, st>>>(mq, mk, mv, p);
    B200Q_LAUNCH_CHECK();
    return B200Q_OK;
  }
  if (dqk > 256 || dv > 256 || dqk < 1 || dv < 1) return B200Q_ERR_UNSUPPORTED;
  dim3 grid((unsigned)L, (unsigned)BH);
  sdpa::sdpa_fp8_plain_kernel<<<grid, 128, 0, st>>>(static_cast<const uint8_t*>(q), static_cast<const uint8_t*>(k),
                                                    static_cast<const uint8_t*>(v), dqk, dv, p);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // namespace b200q
