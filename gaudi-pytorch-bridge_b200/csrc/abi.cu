// extern "C" entry points of libb200q: argument validation, dispatch, status reporting.
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "fp8_misc.cuh"
#include "gemm_common.cuh"
#include "tcgen05_ptx.cuh"

namespace b200q {

std::atomic<uint64_t> g_launches{0};
static thread_local char t_cuda_error[256] = "";

__device__ int g_device_status = 0;

int record_cuda_error(cudaError_t e, const char* where) {
  snprintf(t_cuda_error, sizeof(t_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
  return B200Q_ERR_CUDA;
}

// The status word is a __device__ variable: in host code its name is only a handle, so the
// device address is looked up once per device (with that device current) and cached.
int* device_status_ptr() {
  constexpr int kMaxDev = 64;
  static std::atomic<int*> cache[kMaxDev];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  int* p = cache[dev].load(std::memory_order_acquire);
  if (p) return p;
  void* addr = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&addr, g_device_status);
  if (e != cudaSuccess) {
    record_cuda_error(e, "cudaGetSymbolAddress(g_device_status)");
    return nullptr;
  }
  cache[dev].store(static_cast<int*>(addr), std::memory_order_release);
  return static_cast<int*>(addr);
}

// Self-test of the bounded-wait mechanism: one warp waits on an mbarrier that nothing ever
// arrives at, with a short poll limit.  The wait must give up, record `code` in the status
// word and let the kernel finish normally -- the same path a production kernel takes when a
// producer or a peer never shows up.
__global__ void wait_timeout_selftest_kernel(int* status, int code, uint32_t limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  const uint32_t b = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    ptx::mbar_init(b, 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  ptx::mbar_wait(b, 0, &abort_flag, status, code, 0, limit);  // phase 0 never completes
  __syncthreads();
}

int cast_to_fp8_impl(const void*, int, void*, int, const float*, float, int, int64_t, int64_t, float*, int, uint64_t,
                     uint64_t, uint64_t, int, cudaStream_t);
int cast_hybrid_impl(const void*, int, void*, void*, const float*, float, int, const float*, float, int, int64_t, float*, int,
                     uint64_t, uint64_t, uint64_t, int, cudaStream_t);
int cast_from_fp8_impl(const void*, int, void*, int, const float*, float, int, int64_t, int64_t, cudaStream_t);
int swiglu_cast_impl(const void*, int64_t, const void*, int64_t, void*, float, int64_t, int64_t, float*, cudaStream_t);
int softmax_fp8_impl(const SoftmaxParams&, cudaStream_t);
int sum_fp8_impl(const void*, int, void*, int, int64_t, int64_t, int64_t, void*, size_t, cudaStream_t);
size_t sum_fp8_workspace_bytes_impl(int64_t, int64_t, int64_t);
int in_place_interleave_impl(void*, int64_t, int64_t, cudaStream_t);
int im2col_u8_impl(const void*, void*, int64_t, int64_t, int64_t, int64_t, int, int, int, int, int, int, int, int, int64_t, int64_t,
                   int64_t, cudaStream_t);
int nchw_to_nhwc_u8_impl(const void*, void*, int64_t, int64_t, int64_t, int64_t, cudaStream_t);
int im2col_nhwc_u8_impl(const void*, void*, int64_t, int64_t, int64_t, int64_t, int, int, int, int, int, int, int, int, int64_t,
                        int64_t, int64_t, cudaStream_t);
int amax_impl(const void*, int, int64_t, float*, cudaStream_t);
int scale_from_amax_impl(const float*, float*, float*, float, int, int, cudaStream_t);
int amax_history_impl(float*, int, int, const float*, int, float*, float*, float, int, int, cudaStream_t);
int dequant_int4_impl(const int32_t*, const void*, const void*, int, int, int, void*, int64_t, int64_t, int64_t, int,
                      cudaStream_t);
int w4a16_gemm_impl(const void*, int64_t, const int32_t*, const void*, const int32_t*, int, int, int64_t, int64_t,
                    int64_t, int64_t, void*, int, int64_t, void*, size_t, cudaStream_t);
size_t w4a16_workspace_bytes_impl(int64_t, int64_t, int64_t);
int tp_reduce_bcast_impl(const void*, void* const*, int, int, int64_t, int64_t, cudaStream_t);
int sdpa_fp8_fwd_impl(const b200q_sdpa_args&, cudaStream_t);
int gptq_repack_impl(const int32_t*, int32_t*, int64_t, int64_t, const int32_t*, int32_t*, int64_t, cudaStream_t);
int w4a16_gemm_noalloc_impl(const void*, int64_t, const int32_t*, const void*, const int32_t*, int, int, int64_t, int64_t,
                            int64_t, int64_t, void*, int, int64_t, cudaStream_t);

static bool is_fp8(int d) { return d == B200Q_E4M3 || d == B200Q_E5M2; }
static bool is_wide(int d) { return d == B200Q_F32 || d == B200Q_BF16; }
static bool scale_args_ok(const float* dev, int mode) {
  if (mode < B200Q_BCAST_NONE || mode > B200Q_BCAST_FULL) return false;
  if (mode >= B200Q_BCAST_SCALAR_DEV && !dev) return false;
  return true;
}

}  // namespace b200q

using namespace b200q;

extern "C" {

const char* b200q_strerror(int status) {
  switch (status) {
    case B200Q_OK: return "ok";
    case B200Q_ERR_BAD_ARGUMENT: return "bad argument (null pointer, negative size or unknown enum value)";
    case B200Q_ERR_UNSUPPORTED: return "argument combination not supported by this build";
    case B200Q_ERR_CUDA: return "CUDA call failed (see b200q_last_cuda_error)";
    case B200Q_ERR_TOO_LARGE: return "size beyond the documented maximum";
    case B200Q_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out";
    default: return "unknown b200q status";
  }
}

const char* b200q_last_cuda_error(void) { return t_cuda_error; }

uint64_t b200q_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

size_t b200q_sizeof_args(int which) {
  return which == 0 ? sizeof(b200q_gemm_args) : which == 1 ? sizeof(b200q_sdpa_args) : 0;
}

int b200q_device_status(int* code_out) {
  int* p = device_status_ptr();
  if (!p) return B200Q_ERR_CUDA;
  B200Q_CUDA_OK(cudaDeviceSynchronize());
  int code = 0;
  B200Q_CUDA_OK(cudaMemcpy(&code, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (code != 0) {
    int zero = 0;
    B200Q_CUDA_OK(cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice));
  }
  if (code_out) *code_out = code;
  return code == 0 ? B200Q_OK : B200Q_ERR_DEVICE_TIMEOUT;
}

int b200q_selftest_wait_timeout(int code, void* stream) {
  int* status = device_status_ptr();
  if (!status) return B200Q_ERR_CUDA;
  if (code == 0) return B200Q_ERR_BAD_ARGUMENT;
  wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, code, 1u << 12);
  B200Q_LAUNCH_CHECK();
  return B200Q_OK;
}

int b200q_cast_to_fp8(const void* in, int in_dtype, void* out, int out_dtype, const float* scale, float scale_host,
                      int scale_mode, int64_t rows, int64_t cols, float* amax, int rounding, uint64_t seed,
                      uint64_t offset, uint64_t first_index, int flags, void* stream) {
  if (rows < 0 || cols < 0) return B200Q_ERR_BAD_ARGUMENT;
  if (rows * cols > 0 && (!in || !out)) return B200Q_ERR_BAD_ARGUMENT;
  if (!is_fp8(out_dtype) || !(is_wide(in_dtype) || is_fp8(in_dtype))) return B200Q_ERR_BAD_ARGUMENT;
  if (!scale_args_ok(scale, scale_mode)) return B200Q_ERR_BAD_ARGUMENT;
  if (rounding != B200Q_ROUND_RNE && rounding != B200Q_ROUND_STOCHASTIC) return B200Q_ERR_BAD_ARGUMENT;
  return cast_to_fp8_impl(in, in_dtype, out, out_dtype, scale, scale_host, scale_mode, rows, cols, amax, rounding,
                          seed, offset, first_index, flags, static_cast<cudaStream_t>(stream));
}

int b200q_cast_to_fp8_hybrid(const void* in, int in_dtype, void* out_e5m2, void* out_e4m3, const float* scale_e5m2,
                             float scale_e5m2_host, int scale_e5m2_mode, const float* scale_e4m3, float scale_e4m3_host,
                             int scale_e4m3_mode, int64_t n, float* amax, int rounding_e5m2, uint64_t seed,
                             uint64_t offset, uint64_t first_index, int flags, void* stream) {
  if (n < 0 || (n > 0 && (!in || !out_e5m2 || !out_e4m3))) return B200Q_ERR_BAD_ARGUMENT;
  if (!is_wide(in_dtype)) return B200Q_ERR_BAD_ARGUMENT;
  for (int m : {scale_e5m2_mode, scale_e4m3_mode})
    if (m != B200Q_BCAST_NONE && m != B200Q_BCAST_SCALAR_HOST && m != B200Q_BCAST_SCALAR_DEV) return B200Q_ERR_UNSUPPORTED;
  if ((scale_e5m2_mode == B200Q_BCAST_SCALAR_DEV && !scale_e5m2) || (scale_e4m3_mode == B200Q_BCAST_SCALAR_DEV && !scale_e4m3))
    return B200Q_ERR_BAD_ARGUMENT;
  if (rounding_e5m2 != B200Q_ROUND_RNE && rounding_e5m2 != B200Q_ROUND_STOCHASTIC) return B200Q_ERR_BAD_ARGUMENT;
  return cast_hybrid_impl(in, in_dtype, out_e5m2, out_e4m3, scale_e5m2, scale_e5m2_host, scale_e5m2_mode, scale_e4m3,
                          scale_e4m3_host, scale_e4m3_mode, n, amax, rounding_e5m2, seed, offset, first_index, flags,
                          static_cast<cudaStream_t>(stream));
}

int b200q_cast_from_fp8(const void* in, int in_dtype, void* out, int out_dtype, const float* scale, float scale_host,
                        int scale_mode, int64_t rows, int64_t cols, void* stream) {
  if (rows < 0 || cols < 0) return B200Q_ERR_BAD_ARGUMENT;
  if (rows * cols > 0 && (!in || !out)) return B200Q_ERR_BAD_ARGUMENT;
  if (!is_fp8(in_dtype) || !is_wide(out_dtype)) return B200Q_ERR_BAD_ARGUMENT;
  if (!scale_args_ok(scale, scale_mode)) return B200Q_ERR_BAD_ARGUMENT;
  return cast_from_fp8_impl(in, in_dtype, out, out_dtype, scale, scale_host, scale_mode, rows, cols,
                            static_cast<cudaStream_t>(stream));
}

int b200q_swiglu_cast_fp8(const void* gate, int64_t ld_gate, const void* up, int64_t ld_up, void* out,
                          float scale_host, int64_t rows, int64_t cols, float* amax, void* stream) {
  if (rows < 0 || cols < 0 || ld_gate < cols || ld_up < cols) return B200Q_ERR_BAD_ARGUMENT;
  if (rows * cols > 0 && (!gate || !up || !out)) return B200Q_ERR_BAD_ARGUMENT;
  return swiglu_cast_impl(gate, ld_gate, up, ld_up, out, scale_host, rows, cols, amax,
                          static_cast<cudaStream_t>(stream));
}

int b200q_softmax_fp8(const void* in, int in_dtype, void* out, int out_fp8, int64_t rows, int64_t cols, float pre_scale_host,
                      const float* input_scale, const float* inv_attn_heads, const float* output_scale,
                      float output_scale_host, const void* fused_add, int nd, const int64_t* lead_sizes,
                      const int64_t* fused_add_strides, void* stream) {
  if (rows < 0 || cols < 0 || nd < 0 || nd > 7) return B200Q_ERR_BAD_ARGUMENT;
  if (in_dtype != B200Q_BF16 && in_dtype != B200Q_E4M3) return B200Q_ERR_BAD_ARGUMENT;
  if (rows * cols > 0 && (!in || !out)) return B200Q_ERR_BAD_ARGUMENT;
  if (fused_add && (!lead_sizes || !fused_add_strides)) return B200Q_ERR_BAD_ARGUMENT;
  SoftmaxParams p;
  p.in = in; p.in_dtype = in_dtype; p.out = out; p.out_fp8 = out_fp8; p.rows = rows; p.cols = cols;
  p.pre_scale = pre_scale_host; p.input_scale = input_scale; p.inv_attn_heads = inv_attn_heads;
  p.output_scale = output_scale; p.output_scale_host = output_scale_host;
  p.fused_add = static_cast<const __nv_bfloat16*>(fused_add);
  p.nd = fused_add ? nd : 0;
  int64_t prod = 1;
  for (int d = 0; d < 7; ++d) {
    p.size[d] = (fused_add && d < nd) ? lead_sizes[d] : 1;
    p.fa_stride[d] = (fused_add && d < nd) ? fused_add_strides[d] : 0;
    if (p.size[d] < 1 && rows > 0) return B200Q_ERR_BAD_ARGUMENT;
    prod *= p.size[d];
  }
  if (fused_add && prod != rows) return B200Q_ERR_BAD_ARGUMENT;
  return softmax_fp8_impl(p, static_cast<cudaStream_t>(stream));
}

size_t b200q_sum_fp8_workspace_bytes(int64_t outer, int64_t reduce, int64_t inner) {
  if (outer < 0 || reduce < 0 || inner < 0) return 0;
  return sum_fp8_workspace_bytes_impl(outer, reduce, inner);
}

int b200q_sum_fp8(const void* in, int in_dtype, void* out, int out_dtype, int64_t outer, int64_t reduce, int64_t inner,
                  void* workspace, size_t workspace_bytes, void* stream) {
  if (out_dtype != B200Q_F32 && out_dtype != B200Q_BF16 && out_dtype != B200Q_E4M3 && out_dtype != B200Q_E5M2)
    return B200Q_ERR_BAD_ARGUMENT;
  return sum_fp8_impl(in, in_dtype, out, out_dtype, outer, reduce, inner, workspace, workspace_bytes,
                      static_cast<cudaStream_t>(stream));
}

int b200q_in_place_interleave(void* data, int64_t n_rows, int64_t row_bytes, void* stream) {
  return in_place_interleave_impl(data, n_rows, row_bytes, static_cast<cudaStream_t>(stream));
}

int b200q_im2col_fp8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W, int kh, int kw, int sh, int sw,
                     int ph, int pw, int dh, int dw, int64_t c0, int64_t cg, int64_t ld_out, void* stream) {
  return im2col_u8_impl(in, out, N, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, c0, cg, ld_out, static_cast<cudaStream_t>(stream));
}

int b200q_nchw_to_nhwc_u8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W, void* stream) {
  return nchw_to_nhwc_u8_impl(in, out, N, C, H, W, static_cast<cudaStream_t>(stream));
}

int b200q_im2col_nhwc_fp8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W, int kh, int kw, int sh, int sw,
                          int ph, int pw, int dh, int dw, int64_t c0, int64_t cg, int64_t ld_out, void* stream) {
  return im2col_nhwc_u8_impl(in, out, N, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, c0, cg, ld_out,
                             static_cast<cudaStream_t>(stream));
}

int b200q_amax(const void* in, int in_dtype, int64_t n, float* amax, void* stream) {
  return amax_impl(in, in_dtype, n, amax, static_cast<cudaStream_t>(stream));
}

int b200q_scale_from_amax(const float* amax, float* scale, float* scale_inv, float fp8_max, int pow2, int margin,
                          void* stream) {
  return scale_from_amax_impl(amax, scale, scale_inv, fp8_max, pow2, margin, static_cast<cudaStream_t>(stream));
}

int b200q_amax_history_update(float* history, int len, int pos, const float* new_amax, int use_max, float* scale,
                              float* scale_inv, float fp8_max, int pow2, int margin, void* stream) {
  return amax_history_impl(history, len, pos, new_amax, use_max, scale, scale_inv, fp8_max, pow2, margin,
                           static_cast<cudaStream_t>(stream));
}

int b200q_dequant_int4(const int32_t* packed, const void* scale, const void* zp, int zp_kind, int is_signed,
                       int out_dtype, void* out, int64_t rows, int64_t cols_packed, int64_t scale_rows, int k_packed,
                       void* stream) {
  if (rows < 0 || cols_packed < 0) return B200Q_ERR_BAD_ARGUMENT;
  if (rows * cols_packed > 0 && (!packed || !scale || !out)) return B200Q_ERR_BAD_ARGUMENT;
  if (!is_wide(out_dtype)) return B200Q_ERR_BAD_ARGUMENT;
  if (zp_kind < B200Q_ZP_NONE || zp_kind > B200Q_ZP_FLOAT) return B200Q_ERR_BAD_ARGUMENT;
  if (zp_kind != B200Q_ZP_NONE && !zp && rows * cols_packed > 0) return B200Q_ERR_BAD_ARGUMENT;
  return dequant_int4_impl(packed, scale, zp, zp_kind, is_signed, out_dtype, out, rows, cols_packed, scale_rows,
                           k_packed, static_cast<cudaStream_t>(stream));
}

int b200q_fp8_gemm(const b200q_gemm_args* a) {
  if (!a) return B200Q_ERR_BAD_ARGUMENT;
  if (a->M < 0 || a->N < 0 || a->K < 0 || a->batch < 0) return B200Q_ERR_BAD_ARGUMENT;
  if (!is_fp8(a->a_dtype) || !is_fp8(a->b_dtype) || !is_wide(a->out_dtype)) return B200Q_ERR_BAD_ARGUMENT;
  if (!scale_args_ok(a->a_scale, a->a_scale_mode) || !scale_args_ok(a->b_scale, a->b_scale_mode))
    return B200Q_ERR_BAD_ARGUMENT;
  if (a->bias_mode < B200Q_BCAST_NONE || a->bias_mode > B200Q_BCAST_FULL || a->bias_mode == B200Q_BCAST_SCALAR_HOST)
    return B200Q_ERR_BAD_ARGUMENT;
  if (a->bias_mode != B200Q_BCAST_NONE && (!a->bias || !is_wide(a->bias_dtype))) return B200Q_ERR_BAD_ARGUMENT;
  if (a->D && !is_wide(a->d_dtype)) return B200Q_ERR_BAD_ARGUMENT;
  const int64_t work = a->M * a->N * a->batch;
  if (work == 0) return B200Q_OK;
  if ((!a->out && a->route_count <= 0) || (a->K > 0 && (!a->A || !a->B))) return B200Q_ERR_BAD_ARGUMENT;
  GemmParams g;
  g.A = a->A; g.B = a->B; g.a_dtype = a->a_dtype; g.b_dtype = a->b_dtype; g.trans_a = a->trans_a; g.trans_b = a->trans_b;
  g.M = a->M; g.N = a->N; g.K = a->K; g.lda = a->lda; g.ldb = a->ldb;
  g.batch = a->batch; g.a_batch_stride = a->a_batch_stride; g.b_batch_stride = a->b_batch_stride;
  g.out_batch_stride = a->out_batch_stride; g.out = a->out; g.out_dtype = a->out_dtype; g.ldo = a->ldo;
  g.a_scale = a->a_scale; g.a_scale_host = a->a_scale_host; g.a_scale_mode = a->a_scale_mode;
  g.b_scale = a->b_scale; g.b_scale_host = a->b_scale_host; g.b_scale_mode = a->b_scale_mode;
  g.bias = a->bias; g.bias_dtype = a->bias_dtype; g.bias_mode = a->bias_mode; g.bias_ld = a->bias_ld;
  g.bias_batch_stride = a->bias_batch_stride; g.D = a->D; g.d_dtype = a->d_dtype; g.ldd = a->ldd;
  g.d_batch_stride = a->d_batch_stride;
  g.out8_dtype = a->out8_dtype; g.out8_scale = a->out8_scale; g.out8_scale_host = a->out8_scale_host;
  if (g.out8_dtype != 0 && !is_fp8(g.out8_dtype)) return B200Q_ERR_BAD_ARGUMENT;
  g.swiglu = a->swiglu;
  g.out8_amax = g.out8_dtype ? a->out8_amax : nullptr;
  g.b_static = a->b_static ? 1 : 0;
  g.route_count = a->route_count; g.route_rows = a->route_rows; g.route_row_offset = a->route_row_offset;
  for (int i = 0; i < 8; ++i) g.route_out[i] = a->route_out[i];
  if (g.route_count < 0 || g.route_count > 8) return B200Q_ERR_BAD_ARGUMENT;
  for (int i = 0; i < g.route_count; ++i)
    if (!g.route_out[i] || (reinterpret_cast<uintptr_t>(g.route_out[i]) & 15)) return B200Q_ERR_BAD_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(a->stream);
  if (g.route_count > 0) {
    if (g.batch != 1 || a->force_generic || g.route_row_offset < 0) return B200Q_ERR_UNSUPPORTED;
    return gemm_tcgen05_launch(g, st);  // B200Q_ERR_UNSUPPORTED when the shape has no routed kernel
  }
  if (g.swiglu) {
    if (g.out8_dtype != B200Q_E4M3) return B200Q_ERR_BAD_ARGUMENT;
    if (g.batch != 1 || g.D || g.trans_a || !g.trans_b || a->force_generic) return B200Q_ERR_UNSUPPORTED;
    return gemm_tcgen05_launch(g, st);  // B200Q_ERR_UNSUPPORTED when the shape has no fused kernel
  }
  if (!a->force_generic) {
    if (g.batch == 1) {
      int rc = gemm_tcgen05_launch(g, st);
      if (rc != B200Q_ERR_UNSUPPORTED) return rc;
    } else if (g.batch <= 1024) {
      // batched problems: one tensor-core launch per batch item (same eligibility for all of them)
      auto elem = [](int dtype) { return dtype == B200Q_BF16 ? 2 : 4; };
      for (int64_t b = 0; b < g.batch; ++b) {
        GemmParams gb = g;
        gb.batch = 1;
        gb.A = static_cast<const uint8_t*>(g.A) + b * g.a_batch_stride;
        gb.B = static_cast<const uint8_t*>(g.B) + b * g.b_batch_stride;
        gb.out = static_cast<uint8_t*>(g.out) + b * g.out_batch_stride * (g.out8_dtype ? 1 : elem(g.out_dtype));
        if (g.bias_mode == B200Q_BCAST_FULL)
          gb.bias = static_cast<const uint8_t*>(g.bias) + b * g.bias_batch_stride * elem(g.bias_dtype);
        if (g.D) gb.D = static_cast<const uint8_t*>(g.D) + b * g.d_batch_stride * elem(g.d_dtype);
        int rc = gemm_tcgen05_launch(gb, st);
        if (rc == B200Q_ERR_UNSUPPORTED && b == 0) break;  // not eligible: the generic kernel takes the whole batch
        if (rc != B200Q_OK) return rc;
        if (b == g.batch - 1) return B200Q_OK;
      }
    }
  }
  return gemm_generic_launch(g, st);
}

int b200q_gptq_repack(const int32_t* qweight, int32_t* qweight_out, int64_t K, int64_t N, const int32_t* qzeros,
                      int32_t* qzeros_out, int64_t zeros_words, void* stream) {
  if (K < 0 || N < 0 || zeros_words < 0) return B200Q_ERR_BAD_ARGUMENT;
  if (K * N > 0 && (!qweight || !qweight_out)) return B200Q_ERR_BAD_ARGUMENT;
  if (qzeros && zeros_words > 0 && !qzeros_out) return B200Q_ERR_BAD_ARGUMENT;
  return gptq_repack_impl(qweight, qweight_out, K, N, qzeros, qzeros_out, zeros_words, static_cast<cudaStream_t>(stream));
}

int b200q_fp8_sdpa_fwd(const b200q_sdpa_args* a) {
  if (!a) return B200Q_ERR_BAD_ARGUMENT;
  if (a->BH < 0 || a->L < 0 || a->S < 1 || a->kv_rep < 1 || a->dqk < 1 || a->dv < 1) return B200Q_ERR_BAD_ARGUMENT;
  if (a->BH * a->L == 0) return B200Q_OK;
  if (!a->q || !a->k || !a->v || !a->out || a->BH % a->kv_rep) return B200Q_ERR_BAD_ARGUMENT;
  if (a->out_dtype != B200Q_BF16 && a->out_dtype != B200Q_E4M3) return B200Q_ERR_BAD_ARGUMENT;
  if (a->mask && (a->mask_kind < 1 || a->mask_kind > 3)) return B200Q_ERR_BAD_ARGUMENT;
  return sdpa_fp8_fwd_impl(*a, static_cast<cudaStream_t>(a->stream));
}

int b200q_tp_reduce_bcast(const void* stage, void* const* out_ptrs_host, int tp, int me, int64_t rows, int64_t d,
                          void* stream) {
  if (!stage || !out_ptrs_host || rows < 0 || d < 0) return B200Q_ERR_BAD_ARGUMENT;
  return tp_reduce_bcast_impl(stage, out_ptrs_host, tp, me, rows, d, static_cast<cudaStream_t>(stream));
}

size_t b200q_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return w4a16_workspace_bytes_impl(M, N, K);
}

int b200q_w4a16_gemm(const void* x, int64_t ldx, const int32_t* qweight, const void* scale, const int32_t* zp,
                     int zp_kind, int k_packed, int64_t M, int64_t N, int64_t K, int64_t group, void* out,
                     int out_dtype, int64_t ldo, void* workspace, size_t workspace_bytes, void* stream) {
  if (M < 0 || N < 0 || K < 0 || group <= 0) return B200Q_ERR_BAD_ARGUMENT;
  if (M * N == 0) return B200Q_OK;
  if (!x || !qweight || !scale || !out || !is_wide(out_dtype)) return B200Q_ERR_BAD_ARGUMENT;
  if (zp_kind != B200Q_ZP_NONE && zp_kind != B200Q_ZP_PACKED) return B200Q_ERR_UNSUPPORTED;
  if (zp_kind == B200Q_ZP_PACKED && !zp) return B200Q_ERR_BAD_ARGUMENT;
  return w4a16_gemm_impl(x, ldx, qweight, scale, zp, zp_kind, k_packed, M, N, K, group, out, out_dtype, ldo, workspace,
                         workspace_bytes, static_cast<cudaStream_t>(stream));
}

int b200q_w4a16_gemm_noalloc(const void* x, int64_t ldx, const int32_t* qweight, const void* scale, const int32_t* zp,
                             int zp_kind, int k_packed, int64_t M, int64_t N, int64_t K, int64_t group, void* out,
                             int out_dtype, int64_t ldo, void* stream) {
  if (M < 0 || N < 0 || K < 0 || group <= 0) return B200Q_ERR_BAD_ARGUMENT;
  if (M * N == 0) return B200Q_OK;
  if (!x || !qweight || !scale || !out || !is_wide(out_dtype)) return B200Q_ERR_BAD_ARGUMENT;
  if (zp_kind != B200Q_ZP_NONE && zp_kind != B200Q_ZP_PACKED) return B200Q_ERR_UNSUPPORTED;
  if (zp_kind == B200Q_ZP_PACKED && !zp) return B200Q_ERR_BAD_ARGUMENT;
  return w4a16_gemm_noalloc_impl(x, ldx, qweight, scale, zp, zp_kind, k_packed, M, N, K, group, out, out_dtype, ldo,
                                 static_cast<cudaStream_t>(stream));
}

}  // extern "C"
