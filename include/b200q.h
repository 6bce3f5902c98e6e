/*
 * b200q -- C ABI of the B200 (sm_100a) kernels behind the quantized-inference
 * operator family torch.ops.hpu.{cast_to_fp8_v2, cast_from_fp8, fp8_gemm_v2,
 * convert_from_int4, convert_from_uint4} plus the fused W4A16 GEMM.
 *
 * Conventions
 *  - every pointer is a caller-owned DEVICE pointer unless its name ends in _host;
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *  - nothing here allocates, synchronises or throws; a call validates its
 *    arguments on the host, enqueues kernels on `stream` and returns;
 *  - the return value is B200Q_OK (0) or a negative B200Q_ERR_* code, and
 *    b200q_strerror() turns it into text;
 *  - kernels that wait on barriers bound every wait; a wait that runs out sets a
 *    device status word that b200q_device_status() reads back (it synchronises).
 *
 * Each entry point names the reference interface it replaces, by the file's
 * path inside the reference project.
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum b200q_status {
  B200Q_OK = 0,
  B200Q_ERR_BAD_ARGUMENT = -1,  /* null pointer, negative size, unknown enum value */
  B200Q_ERR_UNSUPPORTED = -2,   /* a combination this build has no kernel for */
  B200Q_ERR_CUDA = -3,          /* a CUDA runtime / driver call failed; see b200q_last_cuda_error() */
  B200Q_ERR_TOO_LARGE = -4,     /* size beyond a documented maximum */
  B200Q_ERR_DEVICE_TIMEOUT = -5 /* a bounded wait inside a kernel ran out (b200q_device_status) */
};

enum b200q_dtype {
  B200Q_F32 = 0,
  B200Q_BF16 = 1,
  B200Q_E4M3 = 2, /* float8_e4m3fn: no inf, max 448 */
  B200Q_E5M2 = 3  /* float8_e5m2: max finite 57344 */
};

/* How a scale (or bias) operand lines up with the [rows, cols] problem. */
enum b200q_bcast {
  B200Q_BCAST_NONE = 0,        /* operand absent */
  B200Q_BCAST_SCALAR_HOST = 1, /* one value, passed by value in the *_host field */
  B200Q_BCAST_SCALAR_DEV = 2,  /* one value in device memory */
  B200Q_BCAST_PER_COL = 3,     /* cols values: operand[c] applies to column c */
  B200Q_BCAST_PER_ROW = 4,     /* rows values: operand[r] applies to row r */
  B200Q_BCAST_FULL = 5         /* rows x cols values */
};

enum b200q_rounding {
  B200Q_ROUND_RNE = 0,       /* round half to nearest even, saturating */
  B200Q_ROUND_STOCHASTIC = 1 /* Philox4x32-10 keyed by (seed, element index), saturating */
};

/* flag bits of b200q_cast_to_fp8 */
#define B200Q_CAST_MUL_IN_FP32 1 /* form input*scale in fp32 instead of in the input dtype */

const char* b200q_strerror(int status);
/* Text of the last CUDA error a b200q call saw on this thread ("" if none). */
const char* b200q_last_cuda_error(void);
/* Synchronises the current device, reads and clears the device status word.
 * 0 = every bounded wait completed; otherwise a kernel-specific code. */
int b200q_device_status(int* code_out);
/* Launches a one-warp kernel whose only wait can never be satisfied and has a short poll limit:
 * the wait gives up, stores `code` (non-zero) in the device status word and the kernel ends
 * normally.  b200q_device_status() then reports B200Q_ERR_DEVICE_TIMEOUT with that code and the
 * context stays usable.  Exercises the path every tcgen05 kernel here takes when a barrier is
 * never signalled (the reference maps device errors to exceptions in
 * backend/synapse_helpers/synapse_error.h). */
int b200q_selftest_wait_timeout(int code, void* stream);
/* Number of kernels this library has launched in this process (all threads). */
uint64_t b200q_launch_count(void);
/* sizeof of an argument struct as this library was built: which = 0 b200q_gemm_args, 1 b200q_sdpa_args; 0 for
 * any other value.  A binding that mirrors the structs (ctypes, cgo, JNI) checks its own layout against it. */
size_t b200q_sizeof_args(int which);

/*
 * cast_to_fp8: out = fp8(in * scale), optional amax = max|in| (of the unscaled input).
 * Replaces the node `convert_to_fp8_{f32,bf16}` emitted by CastToFp8V2::AddNode,
 * hpu_ops/backend/fp8_ops.cpp:192-258 (rounding choice :105-119, scales :63-96).
 *
 * in        [rows*cols] contiguous, in_dtype F32 or BF16 (E4M3/E5M2 input = byte copy,
 *           out_dtype must equal in_dtype, amax must be NULL)
 * out       [rows*cols] bytes, out_dtype E4M3 or E5M2
 * scale     per b200q_bcast, fp32; the product is formed in the input dtype (the scale
 *           is first rounded to it) unless B200Q_CAST_MUL_IN_FP32 is set
 * amax      NULL or one fp32; written by the call (zeroed on `stream` first)
 * rounding  b200q_rounding; for STOCHASTIC, element i draws from Philox4x32-10 (key = seed,
 *           counter = (block, offset)) at global index first_index + i: 8 random bits per
 *           element, 16 elements per block, when the product is a bf16 value (bf16 input and
 *           no B200Q_CAST_MUL_IN_FP32), else 16 bits per element, 8 elements per block
 */
int b200q_cast_to_fp8(const void* in, int in_dtype, void* out, int out_dtype,
                      const float* scale, float scale_host, int scale_mode,
                      int64_t rows, int64_t cols, float* amax, int rounding,
                      uint64_t seed, uint64_t offset, uint64_t first_index, int flags,
                      void* stream);

/*
 * cast_to_fp8_hybrid: one pass over the input, two outputs: e5m2 = fp8(in * scale_e5m2) (RNE or
 * stochastic) and e4m3 = fp8(in * scale_e4m3) (always RNE), plus the optional amax.
 * Replaces the node emitted by CastToFp8Hybrid::AddNode,
 * hpu_ops/backend/cast_to_fp8_hybrid_gen.cpp:39-100 (schema scripts/hpu_op.yaml:7365-7366).
 * Scales are per tensor: B200Q_BCAST_NONE, _SCALAR_HOST or _SCALAR_DEV.  Other arguments as
 * b200q_cast_to_fp8.
 */
int b200q_cast_to_fp8_hybrid(const void* in, int in_dtype, void* out_e5m2, void* out_e4m3,
                             const float* scale_e5m2, float scale_e5m2_host, int scale_e5m2_mode,
                             const float* scale_e4m3, float scale_e4m3_host, int scale_e4m3_mode,
                             int64_t n, float* amax, int rounding_e5m2, uint64_t seed,
                             uint64_t offset, uint64_t first_index, int flags, void* stream);

/*
 * cast_from_fp8: out = T(in) * T(scale), rounded once in T = out_dtype (F32 or BF16).
 * Replaces `convert_from_fp8_{f32,bf16}`, CastFromFp8::AddNode,
 * hpu_ops/backend/fp8_ops.cpp:265-308.
 */
int b200q_cast_from_fp8(const void* in, int in_dtype, void* out, int out_dtype,
                        const float* scale, float scale_host, int scale_mode,
                        int64_t rows, int64_t cols, void* stream);

/* zero-point kinds of b200q_dequant_int4 / b200q_w4a16_gemm */
enum b200q_zp_kind {
  B200Q_ZP_NONE = 0,
  B200Q_ZP_PACKED = 1, /* int32 words, 8 nibbles each, same nibble order and signedness as the input */
  B200Q_ZP_FLOAT = 2   /* out_dtype values, subtracted in out_dtype */
};

/*
 * dequant_int4: out[r][8p+i] = (nibble_i(packed[r][p]) - zp) * scale, nibble i = bits [4i,4i+4).
 * Replaces `dequantize_4_bit_{bf16,f32}`, Int4BaseOp::AddNode,
 * hpu_ops/backend/int4_ops.cpp:40-56 (int4/uint4 typing backend/habana_operator.cpp:376-386).
 *
 * packed      int32 [rows][cols_packed]
 * out         out_dtype (F32/BF16) [rows][8*cols_packed]
 * scale       out_dtype [scale_rows][8*cols_packed]; scale_rows divides rows and row r uses
 *             scale row r / (rows/scale_rows)   (scale_rows == rows: one scale per element)
 * zp          per zp_kind; PACKED: int32 [scale_rows][cols_packed]; FLOAT: like scale
 * is_signed   1 = int4 (nibbles above 7 are negative), 0 = uint4
 * k_packed    0 = the operator's layout above.  1 = AutoGPTQ layout: packed is
 *             [rows/8][cols] with the 8 nibbles of a word going down 8 consecutive ROWS,
 *             out is [rows][cols], scale [scale_rows][cols], PACKED zp [scale_rows][cols/8]
 *             (packed along columns); `cols_packed` then carries cols.
 */
int b200q_dequant_int4(const int32_t* packed, const void* scale, const void* zp, int zp_kind,
                       int is_signed, int out_dtype, void* out, int64_t rows, int64_t cols_packed,
                       int64_t scale_rows, int k_packed, void* stream);

/*
 * gptq_repack: AutoGPTQ checkpoint tensors -> the operator's layout, on the device.
 * qweight int32 [K/8][N] (nibbles packed along K) -> qweight_out int32 [K][N/8] (packed along N);
 * qzeros (stored minus one, any shape, `zeros_words` int32 words) -> qzeros_out = every nibble + 1.
 * Replaces the host-side repack the reference's test does before calling convert_from_uint4
 * (tests/pytest_working/any_mode/test_hpu_convert_from_int4.py:380-395, hpu_preprocessing).
 * qzeros may be NULL.  Needs K % 8 == 0, N % 8 == 0 and a 16-byte aligned qweight.
 */
int b200q_gptq_repack(const int32_t* qweight, int32_t* qweight_out, int64_t K, int64_t N,
                      const int32_t* qzeros, int32_t* qzeros_out, int64_t zeros_words, void* stream);

/*
 * fp8_gemm: out = (op(A) @ op(B)) * a_scale * b_scale [+ bias] [+ D], fp32 accumulation.
 * Replaces `fp8_gemm_{f32,bf16}`, Fp8GemmV2::AddNode, hpu_ops/backend/fp8_ops.cpp:403-496
 * (node inputs [A, B, A_scale_inv, B_scale_inv, bias, D]).
 *
 * op(A) is M x K: A is stored [M][K] (trans_a = 0) or [K][M] (trans_a = 1), row stride lda.
 * op(B) is K x N: B is stored [K][N] (trans_b = 0) or [N][K] (trans_b = 1), row stride ldb.
 * Scales and bias line up with the M x N output per b200q_bcast (rows = M, cols = N).
 * `batch` independent problems are `*_batch_stride` elements apart (0 = shared operand).
 * The tcgen05 path takes all four storage orders (a transposed operand is read through an
 * MN-major shared-memory descriptor); it needs batch == 1, 16-byte aligned bases and row
 * strides, and K % 16 == 0 unless both operands are stored [K][rows]; everything else runs a
 * generic CUDA kernel, which is two to three orders of magnitude slower on large problems.  This
 * entry point allocates nothing: a caller with K % 16 != 0 and an operand stored [rows][K] gets
 * the tcgen05 path by passing copies whose rows are padded with zero bytes to K rounded up to 16
 * (fp8 0x00 is +0 and adds nothing), as the torch operator does above 2^26 multiply-adds.
 */
typedef struct b200q_gemm_args {
  const void* A;
  const void* B;
  int a_dtype, b_dtype; /* E4M3 / E5M2, may differ */
  int trans_a, trans_b;
  int64_t M, N, K;
  int64_t lda, ldb;
  int64_t batch, a_batch_stride, b_batch_stride, out_batch_stride;
  void* out;
  int out_dtype; /* F32 / BF16 */
  int64_t ldo;
  const float* a_scale;
  float a_scale_host;
  int a_scale_mode;
  const float* b_scale;
  float b_scale_host;
  int b_scale_mode;
  const void* bias; /* bias_dtype F32 / BF16 */
  int bias_dtype, bias_mode;
  int64_t bias_ld, bias_batch_stride; /* bias_ld: row stride when bias_mode == FULL */
  const void* D; /* NULL = no accumulate */
  int d_dtype;
  int64_t ldd, d_batch_stride;
  int force_generic; /* 1 = skip the tcgen05 path (testing) */
  void* stream;
  /* Fused output cast (0 = off): with out8_dtype = E4M3 / E5M2, `out` receives fp8 bytes (ldo in
   * bytes = elements) equal to cast_to_fp8(out_dtype(result), out8_scale) -- the GEMM result is
   * rounded to out_dtype first, then scaled and rounded to fp8 (RNE, saturating), which is the
   * cast -> MME fusion of the reference's graph compiler (hpu_ops/backend/fp8_ops.cpp:478-480)
   * with the numerics of the unfused pair of operators. */
  int out8_dtype;
  const float* out8_scale; /* device scalar or NULL */
  float out8_scale_host;   /* used when out8_scale is NULL */
  /* Fused SwiGLU (0 = off; needs out8_dtype = E4M3, trans_a = 0, trans_b = 1, batch = 1, no D,
   * N % 256 == 0, M > 128; other cases return B200Q_ERR_UNSUPPORTED): B holds the gate and up
   * projection weights interleaved in blocks of 128 rows -- rows [256 b, 256 b + 128) are gate
   * rows, the next 128 up rows, both of hidden units [128 b, 128 b + 128), and the per-channel
   * scales / bias follow the same order.  `out` receives e4m3 [M][N / 2] (ldo in elements):
   * cast(bf16(silu(gate) * up), out8 scale) with gate / up rounded to out_dtype first, i.e. the
   * bytes of this GEMM followed by b200q_swiglu_cast_fp8, without the [M][N] round trip. */
  int swiglu;
  /* Routed output (route_count = 0: off).  With route_count = r in 1..8, block i = m / route_rows of
   * the token rows is written to route_out[i] (bf16, row stride ldo) at row
   * route_row_offset + m % route_rows instead of to `out`; the buffers may be memory of other
   * GPUs mapped into this process (peer access enabled), which are then written with plain
   * stores of whole 128-byte row segments.  This is how the row-parallel projection of a
   * tensor-parallel layer hands each block of partial sums to the rank that reduces it while
   * the GEMM is still running; b200q_tp_reduce_bcast finishes the job.  Needs M > 128, bf16
   * output, K-major operands, no D / element-wise bias / fused cast, N % 8 == 0,
   * route_rows % 128 == 0, 16-byte aligned buffers; otherwise B200Q_ERR_UNSUPPORTED.  The
   * reference has no counterpart: its collective is a separate call on the finished tensor
   * (python_packages/habana_frameworks/torch/distributed/hccl/process_group_hccl_base.cpp:412-497). */
  void* route_out[8];
  int route_count;
  int64_t route_rows, route_row_offset;
  /* With a fused output cast (out8_dtype != 0): NULL, or one fp32 that receives max |out|, the
   * largest magnitude among the fp8 values written (as aten::_scaled_mm returns it for float8
   * outputs in the reference, hpu_ops/backend/scaled_mm_gen.cpp:283-320: abs + reduce_max over
   * the casted result), taken in the epilogue while the values are in registers.  The caller
   * zeroes it before the call; it is updated with atomic max, a NaN output makes it NaN. */
  float* out8_amax;
  /* 1 = B (the weights) is not written by anything still in flight on the stream, as the weights of
   * an inference engine are not: the few-token kernel (M <= 128) may then start to read B while the
   * kernel in front of it in the stream is still finishing (it is launched with programmatic stream
   * serialization and waits for that kernel only before it touches A, the scales, bias, D and out).
   * 0 (default) = nothing is read before the preceding kernel is complete.  No counterpart in the
   * reference (a graph compiler orders its loads). */
  int b_static;
} b200q_gemm_args;

int b200q_fp8_gemm(const b200q_gemm_args* args);

/*
 * fp8_sdpa_fwd: scaled-dot-product attention forward on e4m3 tensors,
 *   out = softmax(q k^T * score_scale + mask) v,  probabilities re-quantised to e4m3 in between.
 * Replaces the node `sdpa_recomp_fwd_*` emitted for hpu::fp8_sdpa_recomp_fwd,
 * hpu_ops/backend/sdpa_gen.cpp:820-1000 (output shapes :600-702, fp8 scale inputs :875-882), forward
 * only, no dropout, no valid_seq_len.  Quantisation points (the reference's are inside its closed
 * kernel library; its test bounds the result against unquantised attention with atol 0.4):
 *   S = (q k^T) * score_scale [+ mask] [causal: key <= query];  m = rowmax S;  Pt = exp(S - m);
 *   l = rowsum Pt (fp32);  P8 = e4m3(min(Pt * q_scale_s, 448));  O = (P8 v) * o_scale / l;
 *   out = bf16(O) or e4m3(O * q_scale_o).
 * q [BH][L][dqk], k [BH / kv_rep][S][dqk], v [BH / kv_rep][S][dv], out [BH][L][dv] contiguous;
 * query head bh reads key/value head bh / kv_rep (grouped- and multi-query attention).
 * score_scale = d_scale_q * d_scale_k * softmax_scale;  o_scale = d_scale_s * d_scale_v, with
 * d_scale_s = 1 / q_scale_s unless d_scale_s_given.  Each of the six scales is a device scalar
 * (pointer set) or the *_host value (absent scales: pass 1).
 * mask: NULL, or values addressed as mask[bh * mask_sb + row * mask_sl + key] (strides in
 * elements, 0 = broadcast); mask_kind 1 = bf16 additive, 2 = fp32 additive, 3 = bytes, non-zero =
 * keep.  m_out / linv_out: NULL or bf16 [BH][L] (row maximum of S and 1 / l).  amax_s / amax_o:
 * NULL or one fp32 each, zeroed by the caller: largest probability (max over rows of 1 / l) and
 * max |O|.  dqk = dv = 128 with 16-byte aligned tensors runs the tcgen05 kernel; other head
 * dimensions (<= 256), or force_plain = 1, a plain CUDA kernel with the same arithmetic.
 */
typedef struct b200q_sdpa_args {
  const void *q, *k, *v;
  void* out;
  int out_dtype; /* BF16 or E4M3 */
  int64_t BH, L, S;
  int dqk, dv, kv_rep;
  const void* mask;
  int mask_kind;
  int64_t mask_sb, mask_sl;
  int causal;
  float softmax_scale;
  const float *d_scale_q, *d_scale_k, *d_scale_v, *q_scale_s, *q_scale_o, *d_scale_s;
  float d_scale_q_host, d_scale_k_host, d_scale_v_host, q_scale_s_host, q_scale_o_host, d_scale_s_host;
  int d_scale_s_given;
  void *m_out, *linv_out;
  float *amax_s, *amax_o;
  int force_plain;
  void* stream;
} b200q_sdpa_args;

int b200q_fp8_sdpa_fwd(const b200q_sdpa_args* args);

/*
 * tp_reduce_bcast: the reduction half of a SUM all-reduce whose scatter half was done by the
 * producer (routed GEMM output above).  Stands in for ProcessGroupHcclBase::allreduce,
 * python_packages/habana_frameworks/torch/distributed/hccl/process_group_hccl_base.cpp:412-497,
 * on the output of a row-parallel projection.
 *
 * stage          this rank's staging buffer, bf16 [tp][rows][d]: slot s holds rank s's partial sums
 *                of the `rows` token rows this rank owns
 * out_ptrs_host  HOST array of tp device pointers: the full output bf16 [tp*rows][d] of every rank,
 *                in rank order (own buffer included; the others are peer mappings)
 * The tp slots are added in slot order in fp32 and rounded once to bf16; rows
 * [me*rows, (me+1)*rows) of every output receive the same bytes.  The caller orders this call
 * after every rank's producer (a barrier across the ranks) and the consumers of the outputs
 * after every rank's call.
 */
int b200q_tp_reduce_bcast(const void* stage, void* const* out_ptrs_host, int tp, int me, int64_t rows,
                          int64_t d, void* stream);

/*
 * w4a16_gemm: out[M][N] = x[M][K] @ W[K][N], W = (nibble - zp) * scale rounded to bf16 exactly
 * as b200q_dequant_int4 would produce it, bf16 tensor-core product, fp32 accumulation.
 * No counterpart node in the reference: there `dequantize_4_bit` -> `gemm` are two nodes
 * that the graph compiler fuses (hpu_ops/backend/int4_ops.cpp:48-53); the contract is the
 * composition matmul(x, convert_from_uint4(...)).
 *
 * x        bf16 [M][K], row stride ldx
 * qweight  k_packed = 0: int32 [K][N/8] (operator layout); 1: int32 [K/8][N] (AutoGPTQ)
 * scale    bf16 [K/group][N];  zp: NONE or PACKED int32 [K/group][N/8]
 * out      out_dtype F32/BF16 [M][N], row stride ldo
 * workspace  caller-owned device scratch of at least b200q_w4a16_workspace_bytes(M, N, K) bytes
 *            (0 for M > 128): for small M the K dimension is split over several CTAs per
 *            output tile and the fp32 partial tiles are summed by a second kernel.  May be
 *            NULL when the required size is 0.  Needs 16-byte alignment; contents are scratch.
 * The fused kernel takes k_packed = 0 with K % 64 == 0, group % 64 == 0, K % group == 0,
 * N % 32 == 0 and 16-byte aligned bases; other cases return B200Q_ERR_UNSUPPORTED.
 */
size_t b200q_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K);
int b200q_w4a16_gemm(const void* x, int64_t ldx, const int32_t* qweight, const void* scale,
                     const int32_t* zp, int zp_kind, int k_packed, int64_t M, int64_t N, int64_t K,
                     int64_t group, void* out, int out_dtype, int64_t ldo, void* workspace,
                     size_t workspace_bytes, void* stream);

/*
 * w4a16_gemm_noalloc: b200q_w4a16_gemm for callers that cannot supply a workspace.
 * It has no counterpart in the reference.
 *
 * Who needs it: code that runs where device memory must not be requested -- a serving loop
 * whose memory plan was frozen at start-up (all of HBM already handed to weights and KV
 * cache, so a cudaMalloc could fail or stall the device while it synchronises), a plug-in
 * called from inside another framework's stream callback or memory-pool critical section,
 * or a host language binding that owns no allocator at all.  Such callers pass only their
 * inputs and the output; the split-K scratch that the small-M path needs sits in an 8 MiB
 * array that is part of the library image (every GPU that loads the library keeps it until
 * the process exits).
 *
 * Same arguments and results as b200q_w4a16_gemm without the workspace pair.  Limits and rules:
 *  - the call fails with B200Q_ERR_TOO_LARGE when b200q_w4a16_workspace_bytes(M, N, K) exceeds
 *    8 MiB (for K = N = 8192 that admits M <= 32; M > 128 needs no scratch and always fits);
 *  - it calls no cudaMalloc / cudaFree and no allocating library routine;
 *  - the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and keeps it; make that first call before any stream capture;
 *  - all calls share the one array and it keeps the previous call's contents (nothing in it
 *    needs clearing: each cell is written before it is read within a call), so two calls
 *    that overlap on the GPU -- different streams, or different threads -- race.  Serialise them.
 */
int b200q_w4a16_gemm_noalloc(const void* x, int64_t ldx, const int32_t* qweight, const void* scale,
                             const int32_t* zp, int zp_kind, int k_packed, int64_t M, int64_t N,
                             int64_t K, int64_t group, void* out, int out_dtype, int64_t ldo,
                             void* stream);

/*
 * swiglu_cast_fp8: out8 = e4m3(bf16(silu(gate) * up) * scale), the activation step between the
 * column-parallel and the row-parallel GEMMs of an FP8 MLP, in one pass.
 * No single counterpart in the reference (silu, mul and CastToFp8V2 are separate nodes there,
 * fused by its graph compiler; cast semantics as b200q_cast_to_fp8 with RNE).
 * gate/up bf16 [rows][cols] with row strides ld_gate / ld_up; out e4m3 [rows][cols] contiguous.
 */
int b200q_swiglu_cast_fp8(const void* gate, int64_t ld_gate, const void* up, int64_t ld_up,
                          void* out, float scale_host, int64_t rows, int64_t cols, float* amax,
                          void* stream);

/*
 * FP8 scale management (current and delayed scaling) with all state on the device.
 * Follows the composition the reference builds from ATen ops for its FP8 optimizer state,
 * habana_kernels/lazy_optimizer_kernels.cpp:113-126 (CastMomentToFp8WithScale):
 *   amax = max(abs(x)); exp = floor(log2(fp8_max / amax)); sf = 2^exp;
 *   scale = where(amax > 0, sf, scale); cast_to_fp8_v2(x, scale, true, false, dtype, {1}).
 *
 * b200q_amax: *amax = max |in[i]| over n contiguous bf16 / fp32 elements (NaN propagates;
 *   0 for n == 0).  `in` 16-byte aligned.
 * b200q_scale_from_amax: when *amax > 0, *scale = 2^floor(log2(fp8_max / *amax)) (pow2 != 0;
 *   the exponent is taken exactly from the quotient's bit pattern) or (fp8_max / *amax) / 2^margin
 *   (pow2 == 0); otherwise *scale is kept.  scale_inv (may be NULL) receives 1 / *scale.
 * b200q_amax_history_update: delayed scaling.  history[len] is a ring of earlier amax values:
 *   history[pos] = *new_amax, then the scale as above from max(history) (use_max != 0) or from
 *   the newest entry.
 */
int b200q_amax(const void* in, int in_dtype, int64_t n, float* amax, void* stream);
int b200q_scale_from_amax(const float* amax, float* scale, float* scale_inv, float fp8_max, int pow2,
                          int margin, void* stream);
int b200q_amax_history_update(float* history, int len, int pos, const float* new_amax, int use_max,
                              float* scale, float* scale_inv, float fp8_max, int pow2, int margin,
                              void* stream);

/*
 * softmax_fp8 (hpu_ops/backend/softmax_fp8_gen.cpp:65-160, node softmax_fwd in its HF8 modes):
 *   x = in * inv_attn_heads * input_scale + fused_add   (fp32; absent factors are 1, absent addend 0)
 *   y = softmax over the last dimension, rounded to bf16
 *   out = y as bf16 (out_fp8 == 0) or e4m3(bf16(y * output_scale)) (out_fp8 != 0; RNE, saturating)
 * in: bf16 or e4m3, [rows][cols] contiguous.  The three scales are device scalars or NULL; a
 * NULL input_scale / inv_attn_heads contributes the host factor `pre_scale_host` instead (pass 1
 * when neither is given), a NULL output_scale the host value `output_scale_host`.
 * fused_add (bf16 or NULL) broadcasts over the leading dimensions: `nd` leading sizes in
 * `lead_sizes` (their product is `rows`) and its strides in elements in `fused_add_strides` (0
 * where it broadcasts); its last dimension is `cols`, contiguous.  nd <= 7.
 */
int b200q_softmax_fp8(const void* in, int in_dtype, void* out, int out_fp8, int64_t rows,
                      int64_t cols, float pre_scale_host, const float* input_scale,
                      const float* inv_attn_heads, const float* output_scale,
                      float output_scale_host, const void* fused_add, int nd,
                      const int64_t* lead_sizes, const int64_t* fused_add_strides, void* stream);

/*
 * sum_fp8 (hpu_ops/backend/fp8_ops_gen.cpp:20-49, node reduce_sum): the e4m3 / e5m2 input viewed
 * as [outer][reduce][inner] (contiguous) is summed over `reduce` in fp32, in a fixed order, and
 * written as out_dtype (fp32, bf16, or an fp8 format: RNE, saturating) to [outer][inner].
 * `workspace`: b200q_sum_fp8_workspace_bytes(outer, reduce, inner) bytes of device memory.
 */
size_t b200q_sum_fp8_workspace_bytes(int64_t outer, int64_t reduce, int64_t inner);
int b200q_sum_fp8(const void* in, int in_dtype, void* out, int out_dtype, int64_t outer,
                  int64_t reduce, int64_t inner, void* workspace, size_t workspace_bytes,
                  void* stream);

/*
 * in_place_interleave_ (hpu_ops/backend/fp8_ops.cpp:498-545, node in_place_interleave_fwd):
 * row j of `data` ([n_rows][row_bytes], n_rows % 4 == 0) becomes the old row j / 4, in place --
 * every one of the first n_rows / 4 rows repeated four times.  Any element type.
 */
int b200q_in_place_interleave(void* data, int64_t n_rows, int64_t row_bytes, void* stream);

/*
 * im2col for conv2d_fp8 (hpu_ops/backend/fp8_ops.cpp:547-705: the reference hands the convolution
 * to one MME node; here it is this gather followed by b200q_fp8_gemm against the weight viewed as
 * [C_out][C_g * kh * kw]).  in: one-byte elements [N][C][H][W]; out: [N * Ho * Wo][ld_out] with
 * column k = (c - c0, i, j) over the channels [c0, c0 + cg) and the kh x kw window (stride sh/sw,
 * padding ph/pw, dilation dh/dw), zero outside the image and for k >= cg * kh * kw.
 * ld_out: a multiple of 16, >= cg * kh * kw.  Ho = (H + 2 ph - dh (kh - 1) - 1) / sh + 1, Wo alike.
 */
int b200q_im2col_fp8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W, int kh,
                     int kw, int sh, int sw, int ph, int pw, int dh, int dw, int64_t c0, int64_t cg,
                     int64_t ld_out, void* stream);

/*
 * The same matrix built from a channels-last copy of the input (same reference interface,
 * hpu_ops/backend/fp8_ops.cpp:547-705).  b200q_nchw_to_nhwc_u8: out[n][h][w][c] = in[n][c][h][w],
 * one-byte elements, C a multiple of 4.  b200q_im2col_nhwc_fp8: in is that copy [N][H][W][C];
 * out: [N * Ho * Wo][ld_out] with column k = (i, j, c - c0) -- the window position first, then the
 * channel -- so the weight operand is viewed as [C_out][kh][kw][C_g]; C, c0, cg and ld_out are
 * multiples of 16, in and out 16-byte aligned; zero outside the image and for k >= kh * kw * cg.
 */
int b200q_nchw_to_nhwc_u8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W, void* stream);
int b200q_im2col_nhwc_fp8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W, int kh,
                          int kw, int sh, int sw, int ph, int pw, int dh, int dw, int64_t c0,
                          int64_t cg, int64_t ld_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */
