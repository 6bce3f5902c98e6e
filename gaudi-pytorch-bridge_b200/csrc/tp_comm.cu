// Second half of the row-parallel projection of a tensor-parallel layer, after the GEMM has
// delivered every rank's partial sums to the ranks that own the rows (routed output of the FP8
// GEMM): the owner adds the tp partial sums of its rows and writes the result into every
// rank's output.  All addresses other than `stage` may be memory of other GPUs mapped into
// this process (plain stores; no multicast object is involved).
#include "common.cuh"

namespace b200q {

struct OutPtrs {
  __nv_bfloat16* p[8];
};

// One 16-byte vector (8 bf16) per thread and step.  Partial sums are added in slot order in
// fp32 and rounded once, so every rank ends up with the same bytes whatever the timing.
__global__ void __launch_bounds__(256) tp_reduce_bcast_kernel(const uint4* __restrict__ stage, OutPtrs outs, int tp, int me,
                                                              int64_t vecs_per_slot, int64_t out_vec0) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs_per_slot; i += stride) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    uint4 v[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
      if (s < tp) v[s] = __ldcg(stage + (int64_t)s * vecs_per_slot + i);  // written by other GPUs: read past L1
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < tp) {
        const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += bf16_bits_to_float(w[j] & 0xFFFFu);
          acc[2 * j + 1] += bf16_bits_to_float(w[j] >> 16);
        }
      }
    }
    const uint4 r = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                               pack_bf16x2(acc[6], acc[7]));
    // own copy last, the peers starting with the next rank, so that the ranks do not all write
    // to the same destination at once
#pragma unroll
    for (int k = 1; k <= 8; ++k) {
      if (k <= tp) {
        const int dst = (me + k) % tp;
        reinterpret_cast<uint4*>(outs.p[dst])[out_vec0 + i] = r;
      }
    }
  }
}

int tp_reduce_bcast_impl(const void* stage, void* const* out_ptrs_host, int tp, int me, int64_t rows, int64_t d,
                         cudaStream_t st) {
  if (tp < 1 || tp > 8 || me < 0 || me >= tp || (d % 8)) return B200Q_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(stage) & 15) return B200Q_ERR_UNSUPPORTED;
  OutPtrs outs;
  for (int i = 0; i < 8; ++i) {
    outs.p[i] = i < tp ? static_cast<__nv_bfloat16*>(out_ptrs_host[i]) : nullptr;
    if (i < tp && (!out_ptrs_host[i] || (reinterpret_cast<uintptr_t>(out_ptrs_host[i]) & 15))) return B200Q_ERR_BAD_ARGUMENT;
  }
  const int64_t vecs = rows * d / 8;
  if (vecs == 0) return B200Q_OK;
  int64_t blocks = (vecs + 255) / 256;
  if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
  tp_reduce_bcast_kernel<<<(int)blocks, 256, 0, st>>>(static_cast<const uint4*>(stage), outs, tp, me, vecs,
                                                      (int64_t)me * vecs);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

}  // namespace b200q
