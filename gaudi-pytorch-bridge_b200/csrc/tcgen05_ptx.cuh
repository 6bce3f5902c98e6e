// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor, no multicast),
// tcgen05 (TMEM allocation, UMMA issue/commit, TMEM loads) and the descriptor encodings.
// Every wait is bounded: a wait that runs out records a code and tells the caller to stop.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// try_wait with a suspend-time hint (nanoseconds): the hardware may park the thread for up to
// that long while the phase is incomplete, instead of returning to a polling loop that takes
// issue slots from the other warps of its scheduler.
__device__ __forceinline__ uint32_t mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok;
}
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                 int code, uint32_t hint_ns, uint32_t limit = 1u << 22) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait_hint(bar, parity, hint_ns)) return true;
    if ((i & 63u) == 63u) {
      if (*abort_flag) return false;
    }
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}

// Bounded wait.  `abort_flag` is a shared-memory word any role may set; the wait gives up
// when it is set or after kWaitLimit polls (seconds of wall time), and then sets it itself.
// `backoff_ns` > 0 makes a waiter that is not on the critical path (an epilogue warp waiting
// for the whole main loop of its tile) sleep between polls, so that it does not take issue
// slots from the warps that feed the tensor core.
constexpr uint32_t kWaitLimit = 1u << 24;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code, uint32_t backoff_ns = 0, uint32_t limit = kWaitLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff_ns) __nanosleep(backoff_ns);
    if ((i & 255u) == 255u) {
      if (*abort_flag) return false;
      if (i > 4096u) __nanosleep(64);
    }
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}

// ---- TMA: 2-D tiled load global -> shared, completion on an mbarrier (never multicast) ----
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tcgen05 ----
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues.  kind::f8f6f4: K = 32 per instruction.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::f16 (bf16 / fp16 operands): K = 16 per instruction.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every previously issued MMA of this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}


// ---- CTA pairs (cta_group::2): two CTAs of a cluster drive one 256-row MMA ----
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address: the even CTA

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// All threads of all CTAs of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t ncols) {  // the same warp in both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMA load into this CTA's shared memory whose completion bytes are counted on the barrier of
// the pair's even CTA (`bar` must already have the rank bit cleared).  Not a multicast: each CTA
// fetches only its own tile.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// 256 x N x 32 MMA over both CTAs' shared memory and TMEM; issued by one thread of the even CTA.
__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One ring stage in a single instruction sequence: a non-blocking probe of the NEXT stage's
// barrier is issued first and its result is read only after the stage's four MMAs (operand
// descriptors advancing by astep / bstep 16-byte units) and its commit have been issued.  A
// probe that succeeds lets the issuer skip the blocking wait of the next stage: the round trip
// of the wait -- a few hundred cycles when shared memory is busy -- then overlaps the MMA issue
// instead of adding to it.  Returns 1 when the next stage is already complete.
// F16: kind::f16 (bf16 operands), else kind::f8f6f4.  PAIR: cta_group::2 with a commit
// multicast to both CTAs of the pair, else cta_group::1.
template <bool F16, bool PAIR>
__device__ __forceinline__ uint32_t umma_stage4_probe(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                      uint32_t accumulate, uint32_t commit_bar, uint32_t next_bar,
                                                      uint32_t next_parity, uint64_t astep, uint64_t bstep) {
  uint32_t ready;
#define B200Q_MMA_OP(G, KIND) "tcgen05.mma.cta_group::" G ".kind::" KIND " "
#define B200Q_STAGE4(G, KIND, COMMIT)                                                    \
  asm volatile(                                                                          \
      "{\n"                                                                              \
      ".reg .pred p, q, t;\n"                                                            \
      ".reg .b64 a1, b1, a2, b2, a3, b3;\n"                                              \
      ".reg .b16 m;\n"                                                                   \
      "mbarrier.test_wait.parity.shared::cta.b64 q, [%7], %8;\n"                         \
      "setp.ne.b32 p, %5, 0;\n"                                                          \
      "setp.eq.b32 t, 0, 0;\n"                                                           \
      "add.u64 a1, %2, %9;\n"                                                            \
      "add.u64 b1, %3, %10;\n"                                                           \
      "add.u64 a2, a1, %9;\n"                                                            \
      "add.u64 b2, b1, %10;\n"                                                           \
      "add.u64 a3, a2, %9;\n"                                                            \
      "add.u64 b3, b2, %10;\n"                                                           \
      B200Q_MMA_OP(G, KIND) "[%1], %2, %3, %4, p;\n"                                     \
      B200Q_MMA_OP(G, KIND) "[%1], a1, b1, %4, t;\n"                                     \
      B200Q_MMA_OP(G, KIND) "[%1], a2, b2, %4, t;\n"                                     \
      B200Q_MMA_OP(G, KIND) "[%1], a3, b3, %4, t;\n"                                     \
      "mov.b16 m, 3;\n"                                                                  \
      COMMIT                                                                             \
      "selp.u32 %0, 1, 0, q;\n"                                                          \
      "}\n"                                                                              \
      : "=r"(ready)                                                                      \
      : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(commit_bar), "r"(next_bar), \
        "r"(next_parity), "l"(astep), "l"(bstep)                                         \
      : "memory")
#define B200Q_COMMIT_PAIR "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%6], m;\n"
#define B200Q_COMMIT_ONE "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n"
  if constexpr (PAIR && !F16) B200Q_STAGE4("2", "f8f6f4", B200Q_COMMIT_PAIR);
  else if constexpr (PAIR && F16) B200Q_STAGE4("2", "f16", B200Q_COMMIT_PAIR);
  else if constexpr (!PAIR && !F16) B200Q_STAGE4("1", "f8f6f4", B200Q_COMMIT_ONE);
  else B200Q_STAGE4("1", "f16", B200Q_COMMIT_ONE);
#undef B200Q_COMMIT_ONE
#undef B200Q_COMMIT_PAIR
#undef B200Q_STAGE4
#undef B200Q_MMA_OP
  return ready;
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Bounded wait on a barrier that threads of the peer CTA arrive on (cluster-scope acquire, so
// that what they wrote to their shared memory before arriving is ordered before what follows).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                  int code) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((i & 255u) == 255u) {
      if (*abort_flag) return false;
      if (i > 4096u) __nanosleep(64);
    }
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}
// Completion of the pair's MMAs signalled on the barrier at the same offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair_both(uint32_t bar) {
  asm volatile(
      "{\n"
      ".reg .b16 m;\n"
      "mov.b16 m, 3;\n"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n"
      "}\n" ::"r"(bar)
      : "memory");
}
// Arrive on a barrier addressed in the cluster window (own CTA or the peer).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The same with the default (CTA-scope) release: no cluster-wide fence is executed, which on
// B200 costs about a thousand cycles per arrival.  Enough when what the arrival publishes is
// this CTA's own shared memory, already made visible to the async proxy by
// fence.proxy.async, and read there by the tensor core of this same SM.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Named barrier among a subset of the CTA's warps.
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- descriptors ----
// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle, rows of 128 bytes:
// 8-row groups are 1024 bytes apart (SBO); LBO is unused for swizzled K-major layouts (1).
// The tile base must be 1024-byte aligned; stepping K inside the 128-byte row adds bytes
// to the start address.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);       // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                         // leading byte offset (16 B units), bits [16,30)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                         // descriptor version (Blackwell), bits [46,48)
  d |= (uint64_t)2 << 61;                         // layout: SWIZZLE_128B, bits [61,64)
  return d;
}

// MN-major operand (the M or N index is contiguous in memory), 128-byte swizzle: 64 bf16 along
// MN form a 128-byte row, 8 consecutive k form a 1024-byte atom; `lbo` is the byte distance
// between 64-element MN blocks and `sbo` the distance between 8-k groups.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor (dense, fp32 accumulate, both operands K-major).
// fmt for kind::f8f6f4: 0 = e4m3, 1 = e5m2; for kind::f16: 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Same with the operands' major-ness: bit 15 = A is MN-major, bit 16 = B is MN-major.
__host__ __device__ constexpr uint32_t umma_idesc_major(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n,
                                                        uint32_t a_mn, uint32_t b_mn) {
  return umma_idesc(a_fmt, b_fmt, m, n) | (a_mn << 15) | (b_mn << 16);
}

}  // namespace ptx
}  // namespace b200q
