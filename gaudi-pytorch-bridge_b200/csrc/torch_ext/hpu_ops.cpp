// torch.ops.hpu.* for CUDA tensors on B200: the operator schemas of the reference
// (habana_kernels/kernels_register.cpp:2427-2451, identical in
// habana_eager/eager_custom_op_register.cpp:2146-2171) registered verbatim, with CUDA and
// Meta implementations.  Argument checks and error strings follow
// hpu_ops/backend/fp8_ops.cpp and hpu_ops/common/batched_matmul_output_shape.cpp; the
// wrappers mirror habana_eager/eager_custom_op_register.cpp:59-322,1272-1306.  All device
// work goes through the C ABI in b200q.h on the current CUDA stream; there is no fallback.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <atomic>
#include <cstdlib>
#include <sstream>
#include <variant>

#include "b200q.h"

namespace {

using OptTensor = c10::optional<at::Tensor>;
using OptShape = at::OptionalIntArrayRef;
using ScaleArg = std::variant<std::monostate, at::Tensor, double, std::vector<double>>;

// ---- process-wide knobs (out-of-band: the operator schemas have no argument for them) ----
std::atomic<int64_t> g_sr_seed{[] {
  const char* e = std::getenv("B200Q_SR_SEED");
  return e ? std::atoll(e) : 1234ll;
}()};
std::atomic<int64_t> g_sr_offset{0};
std::atomic<bool> g_mul_in_fp32{[] {
  const char* e = std::getenv("B200Q_CAST_MUL_IN_FP32");
  return e && e[0] == '1';
}()};

void check_status(int rc, const char* op) {
  if (rc == B200Q_OK) return;
  TORCH_CHECK(false, op, ": ", b200q_strerror(rc), rc == B200Q_ERR_CUDA ? std::string(" -- ") + b200q_last_cuda_error()
                                                                        : std::string());
}

int to_b200q_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return B200Q_F32;
    case at::kBFloat16: return B200Q_BF16;
    case at::kFloat8_e4m3fn: return B200Q_E4M3;
    case at::kFloat8_e5m2: return B200Q_E5M2;
    default: TORCH_CHECK(false, "unsupported dtype ", t); return -1;
  }
}
bool is_fp8(at::ScalarType t) { return t == at::kFloat8_e5m2 || t == at::kFloat8_e4m3fn; }

void* current_stream() { return static_cast<void*>(c10::cuda::getCurrentCUDAStream().stream()); }

int64_t numel_of(c10::IntArrayRef s) {
  int64_t n = 1;
  for (auto d : s) n *= d;
  return n;
}

// hpu_ops/backend/fp8_ops.cpp:29-53
void validate_scale_shape(const ScaleArg& scale, OptShape scale_shape) {
  if (!scale_shape.has_value()) return;
  int64_t n = 0;
  if (auto t = std::get_if<at::Tensor>(&scale)) n = t->numel();
  else if (auto l = std::get_if<std::vector<double>>(&scale)) n = (int64_t)l->size();
  else return;
  int64_t m = numel_of(*scale_shape);
  TORCH_CHECK(n == m, "Number of scale elements (", n, ") is not equal to number of scale_shape elements (", m, ").");
}

// A scale resolved against a [rows, cols] problem.
struct ResolvedScale {
  int mode = B200Q_BCAST_NONE;
  float host = 1.f;
  at::Tensor dev;  // fp32, contiguous, on the problem's device (keeps the storage alive)
  const float* ptr() const { return dev.defined() ? dev.data_ptr<float>() : nullptr; }
};

// Scale as an fp32 tensor of its final shape (fp8_ops.cpp:63-96), or undefined for None/float.
at::Tensor scale_tensor(const ScaleArg& scale, OptShape scale_shape, const at::Device& dev) {
  if (auto t = std::get_if<at::Tensor>(&scale)) {
    at::Tensor s = t->to(dev, at::kFloat);
    if (s.numel() > 1 && scale_shape.has_value() && s.sizes() != *scale_shape) s = s.reshape(*scale_shape);
    return s;
  }
  if (auto l = std::get_if<std::vector<double>>(&scale)) {
    at::Tensor s = at::tensor(*l, at::TensorOptions().dtype(at::kDouble)).to(at::kFloat);
    if (scale_shape.has_value()) s = s.reshape(*scale_shape);
    return s.to(dev);
  }
  return at::Tensor();
}

// Classify how `s` (already of its final shape) broadcasts against `shape`; on return rows*cols ==
// numel(shape) and the mode says how s lines up with that 2-D view.
ResolvedScale classify_against(const at::Tensor& s_in, c10::IntArrayRef shape, int64_t* rows, int64_t* cols,
                               const char* what) {
  ResolvedScale r;
  const int64_t n = numel_of(shape);
  *rows = 1;
  *cols = n;
  at::Tensor s = s_in;
  if (s.numel() == 1) {
    r.mode = B200Q_BCAST_SCALAR_DEV;
    r.dev = s.reshape({1}).contiguous();
    return r;
  }
  const int64_t rank = (int64_t)shape.size();
  TORCH_CHECK(s.dim() <= rank, what, " of shape ", s.sizes(), " does not broadcast against ", shape);
  std::vector<int64_t> ss(rank, 1);
  for (int64_t i = 0; i < s.dim(); ++i) ss[rank - s.dim() + i] = s.size(i);
  for (int64_t i = 0; i < rank; ++i)
    TORCH_CHECK(ss[i] == 1 || ss[i] == shape[i], what, " of shape ", s.sizes(), " does not broadcast against ", shape);
  int64_t first_full = rank, last_full = -1;
  bool all_full = true;
  for (int64_t i = 0; i < rank; ++i) {
    bool full = ss[i] == shape[i] && shape[i] != 1;
    bool one = ss[i] == 1 && shape[i] != 1;
    if (full) { first_full = std::min(first_full, i); last_full = std::max(last_full, i); }
    if (one) all_full = false;
  }
  if (all_full) {
    r.mode = B200Q_BCAST_FULL;
    r.dev = s.contiguous();
    return r;
  }
  // trailing block: ones before first_full, matches from first_full to the end
  bool trailing = true, leading = true;
  for (int64_t i = 0; i < rank; ++i) {
    if (shape[i] == 1) continue;
    bool full = ss[i] == shape[i];
    if (i >= first_full && !full) trailing = false;
    if (i <= last_full && !full) leading = false;
  }
  if (trailing && first_full < rank) {
    *cols = 1;
    for (int64_t i = first_full; i < rank; ++i) *cols *= shape[i];
    *rows = n / *cols;
    r.mode = B200Q_BCAST_PER_COL;
    r.dev = s.contiguous().reshape({*cols});
    return r;
  }
  if (leading && last_full >= 0) {
    *rows = 1;
    for (int64_t i = 0; i <= last_full; ++i) *rows *= shape[i];
    *cols = n / *rows;
    r.mode = B200Q_BCAST_PER_ROW;
    r.dev = s.contiguous().reshape({*rows});
    return r;
  }
  r.mode = B200Q_BCAST_FULL;  // mixed pattern: materialise
  r.dev = s.reshape(ss).expand(shape).contiguous();
  return r;
}

ResolvedScale resolve_cast_scale(const ScaleArg& scale, OptShape scale_shape, const at::Tensor& input, int64_t* rows,
                                 int64_t* cols) {
  validate_scale_shape(scale, scale_shape);
  *rows = 1;
  *cols = input.numel();
  ResolvedScale r;
  if (std::holds_alternative<std::monostate>(scale)) return r;
  if (auto d = std::get_if<double>(&scale)) {
    r.mode = B200Q_BCAST_SCALAR_HOST;
    r.host = (float)*d;
    return r;
  }
  return classify_against(scale_tensor(scale, scale_shape, input.device()), input.sizes(), rows, cols, "scale");
}

// ------------------------------------------------------------------ cast_to_fp8_v2
std::tuple<at::Tensor, at::Tensor> cast_to_fp8_v2_common(const at::Tensor& input, const ScaleArg& scale,
                                                         bool stochastic_rounding, bool is_amax, at::ScalarType dtype,
                                                         OptShape scale_shape) {
  const auto src = input.scalar_type();
  const bool fp8_in = is_fp8(src);
  TORCH_CHECK(fp8_in || src == at::kFloat || src == at::kBFloat16,
              "CastToFp8V2 input dtype must be one of [float, bfloat16, float8_e5m2, float8_e4m3fn].");
  if (fp8_in) {
    TORCH_CHECK(!is_amax, "CastToFp8V2 must have no amax for float8.");
    TORCH_CHECK(src == dtype, "CastToFp8V2 input and output must have the same dtype for float8, but are ", src,
                " and ", dtype);
  }
  TORCH_CHECK(is_fp8(dtype), "CastToFp8V2 output dtype must be float8_e5m2 or float8_e4m3fn, got ", dtype);
  c10::cuda::CUDAGuard guard(input.device());
  at::Tensor in = input.contiguous();
  int64_t rows, cols;
  ResolvedScale s = resolve_cast_scale(scale, scale_shape, in, &rows, &cols);
  at::Tensor out = at::empty(in.sizes(), in.options().dtype(dtype));
  at::Tensor amax = is_amax ? at::empty({}, in.options().dtype(at::kFloat)) : at::empty({0}, in.options().dtype(at::kFloat));
  uint64_t seed = (uint64_t)g_sr_seed.load(), offset = 0;
  if (stochastic_rounding && !fp8_in) offset = (uint64_t)g_sr_offset.fetch_add(1);
  int flags = g_mul_in_fp32.load() ? B200Q_CAST_MUL_IN_FP32 : 0;
  check_status(b200q_cast_to_fp8(in.data_ptr(), to_b200q_dtype(src), out.data_ptr(), to_b200q_dtype(dtype), s.ptr(),
                                 s.host, fp8_in ? B200Q_BCAST_NONE : s.mode, rows, cols,
                                 is_amax ? amax.data_ptr<float>() : nullptr,
                                 stochastic_rounding ? B200Q_ROUND_STOCHASTIC : B200Q_ROUND_RNE, seed, offset, 0, flags,
                                 current_stream()),
               "cast_to_fp8_v2");
  return {out, amax};
}

std::tuple<at::Tensor, at::Tensor> cast_to_fp8_v2(const at::Tensor& input, const OptTensor& scale,
                                                  bool stochastic_rounding, bool is_amax, at::ScalarType dtype,
                                                  OptShape scale_shape) {
  ScaleArg s;
  if (scale.has_value() && scale->defined()) s = *scale;
  return cast_to_fp8_v2_common(input, s, stochastic_rounding, is_amax, dtype, scale_shape);
}
std::tuple<at::Tensor, at::Tensor> cast_to_fp8_v2_scalar(const at::Tensor& input, double scale,
                                                         bool stochastic_rounding, bool is_amax, at::ScalarType dtype,
                                                         OptShape) {
  return cast_to_fp8_v2_common(input, ScaleArg(scale), stochastic_rounding, is_amax, dtype, c10::nullopt);
}
std::tuple<at::Tensor, at::Tensor> cast_to_fp8_v2_scalar_list(const at::Tensor& input, c10::ArrayRef<double> scale,
                                                              bool stochastic_rounding, bool is_amax,
                                                              at::ScalarType dtype, OptShape scale_shape) {
  return cast_to_fp8_v2_common(input, ScaleArg(scale.vec()), stochastic_rounding, is_amax, dtype, scale_shape);
}

// legacy out-variant (kernels_register.cpp:2427; fp8_ops.cpp:123-166)
std::tuple<at::Tensor&, at::Tensor&> cast_to_fp8(const at::Tensor& input, const OptTensor& scale,
                                                 bool stochastic_rounding, at::Tensor& out, at::Tensor& amax) {
  const auto src = input.scalar_type();
  TORCH_CHECK(src == at::kFloat || src == at::kBFloat16, "CastToFp8 input must be of float or bfloat16 dtype.");
  TORCH_CHECK(input.sizes() == out.sizes(), "Input and output must have the same shape");
  TORCH_CHECK(out.is_contiguous() && is_fp8(out.scalar_type()), "CastToFp8 out must be a contiguous float8 tensor");
  auto r = cast_to_fp8_v2(input, scale, stochastic_rounding, amax.numel() != 0, out.scalar_type(), c10::nullopt);
  out.copy_(std::get<0>(r));
  if (amax.numel() != 0) amax.copy_(std::get<1>(r).reshape(amax.sizes()));
  return {out, amax};
}

// ------------------------------------------------------------------ cast_to_fp8_hybrid
// scripts/hpu_op.yaml:7365-7366, hpu_ops/backend/cast_to_fp8_hybrid_gen.cpp:39-100
std::tuple<at::Tensor, at::Tensor, at::Tensor> cast_to_fp8_hybrid(const at::Tensor& input, const OptTensor& scale_152,
                                                                  const OptTensor& scale_143, bool stochastic_rounding,
                                                                  bool is_amax) {
  const auto src = input.scalar_type();
  TORCH_CHECK(src == at::kFloat || src == at::kBFloat16, "CastToFp8Hybrid input must be of float or bfloat16 dtype.");
  c10::cuda::CUDAGuard guard(input.device());
  at::Tensor in = input.contiguous();
  auto one_scale = [&](const OptTensor& s, at::Tensor& keep, int* mode) -> const float* {
    *mode = B200Q_BCAST_NONE;
    if (!s.has_value() || !s->defined()) return nullptr;
    TORCH_CHECK(s->numel() == 1, "CastToFp8Hybrid scales must have one element, got ", s->sizes());
    keep = s->to(in.device(), at::kFloat).reshape({1}).contiguous();
    *mode = B200Q_BCAST_SCALAR_DEV;
    return keep.data_ptr<float>();
  };
  at::Tensor k152, k143;
  int m152, m143;
  const float* p152 = one_scale(scale_152, k152, &m152);
  const float* p143 = one_scale(scale_143, k143, &m143);
  at::Tensor o152 = at::empty(in.sizes(), in.options().dtype(at::kFloat8_e5m2));
  at::Tensor o143 = at::empty(in.sizes(), in.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor amax = is_amax ? at::empty({}, in.options().dtype(at::kFloat)) : at::empty({0}, in.options().dtype(at::kFloat));
  uint64_t seed = (uint64_t)g_sr_seed.load(), offset = 0;
  if (stochastic_rounding) offset = (uint64_t)g_sr_offset.fetch_add(1);
  check_status(b200q_cast_to_fp8_hybrid(in.data_ptr(), to_b200q_dtype(src), o152.data_ptr(), o143.data_ptr(), p152, 1.f, m152,
                                        p143, 1.f, m143, in.numel(), is_amax ? amax.data_ptr<float>() : nullptr,
                                        stochastic_rounding ? B200Q_ROUND_STOCHASTIC : B200Q_ROUND_RNE, seed, offset, 0,
                                        g_mul_in_fp32.load() ? B200Q_CAST_MUL_IN_FP32 : 0, current_stream()),
               "cast_to_fp8_hybrid");
  return {o152, o143, amax};
}

// ------------------------------------------------------------------ cast_from_fp8
at::Tensor cast_from_fp8_common(const at::Tensor& input, const ScaleArg& scale, at::ScalarType out_dtype,
                                OptShape scale_shape) {
  validate_scale_shape(scale, scale_shape);
  TORCH_CHECK(out_dtype == at::kFloat || out_dtype == at::kBFloat16,
              "CastFromFp8 output dtype must be equal to float or bfloat16.");
  TORCH_CHECK(is_fp8(input.scalar_type()), "CastFromFp8 input must be float8_e5m2 or float8_e4m3fn, got ",
              input.scalar_type());
  c10::cuda::CUDAGuard guard(input.device());
  at::Tensor in = input.contiguous();
  int64_t rows, cols;
  ResolvedScale s = resolve_cast_scale(scale, scale_shape, in, &rows, &cols);
  at::Tensor out = at::empty(in.sizes(), in.options().dtype(out_dtype));
  check_status(b200q_cast_from_fp8(in.data_ptr(), to_b200q_dtype(in.scalar_type()), out.data_ptr(),
                                   to_b200q_dtype(out_dtype), s.ptr(), s.host, s.mode, rows, cols, current_stream()),
               "cast_from_fp8");
  return out;
}
at::Tensor cast_from_fp8(const at::Tensor& input, const OptTensor& scale, at::ScalarType out_dtype,
                         OptShape scale_shape) {
  ScaleArg s;
  if (scale.has_value() && scale->defined()) s = *scale;
  return cast_from_fp8_common(input, s, out_dtype, scale_shape);
}
at::Tensor cast_from_fp8_scalar(const at::Tensor& input, double scale, at::ScalarType out_dtype, OptShape) {
  return cast_from_fp8_common(input, ScaleArg(scale), out_dtype, c10::nullopt);
}
at::Tensor cast_from_fp8_scalar_list(const at::Tensor& input, c10::ArrayRef<double> scale, at::ScalarType out_dtype,
                                     OptShape scale_shape) {
  return cast_from_fp8_common(input, ScaleArg(scale.vec()), out_dtype, scale_shape);
}

// ------------------------------------------------------------------ convert_from_{int4,uint4}
at::Tensor convert_from_4bit(const at::Tensor& input, const at::Tensor& scale, const OptTensor& zero_point,
                             at::ScalarType out_dtype, bool is_signed) {
  TORCH_CHECK(input.scalar_type() == at::kInt, "convert_from_int4 input must be int32 (8 packed nibbles per element)");
  TORCH_CHECK(out_dtype == at::kFloat || out_dtype == at::kBFloat16,
              "convert_from_int4 output dtype must be float or bfloat16, got ", out_dtype);
  TORCH_CHECK(input.dim() >= 1, "convert_from_int4 input must have at least one dimension");
  c10::cuda::CUDAGuard guard(input.device());
  at::Tensor in = input.contiguous();
  auto out_shape = in.sizes().vec();
  out_shape.back() *= 8;
  const int64_t cols_packed = in.size(-1), cols = cols_packed * 8;
  const int64_t rows = cols_packed ? in.numel() / cols_packed : 0;
  // scale: out_dtype, either the full output shape or [..., K/g, N]
  at::Tensor sc = scale.to(in.device(), out_dtype).contiguous();
  int64_t scale_rows = rows;
  if (sc.sizes() != c10::IntArrayRef(out_shape)) {
    bool grouped = sc.dim() == (int64_t)out_shape.size() && sc.dim() >= 2 && sc.size(-1) == cols &&
                   sc.size(-2) > 0 && out_shape[out_shape.size() - 2] % sc.size(-2) == 0;
    for (int64_t i = 0; grouped && i < sc.dim() - 2; ++i) grouped = sc.size(i) == out_shape[i];
    if (grouped) scale_rows = sc.numel() / cols;
    else {
      sc = sc.expand(out_shape).contiguous();
    }
  }
  int zp_kind = B200Q_ZP_NONE;
  at::Tensor zp;
  if (zero_point.has_value() && zero_point->defined()) {
    if (zero_point->scalar_type() == at::kInt) {
      zp_kind = B200Q_ZP_PACKED;
      zp = zero_point->to(in.device()).contiguous();
      TORCH_CHECK(zp.numel() == scale_rows * cols_packed, "packed zero_point must have the scale's shape with the last "
                  "dimension divided by 8, got ", zp.sizes(), " for scale ", sc.sizes());
    } else {
      zp_kind = B200Q_ZP_FLOAT;
      zp = zero_point->to(in.device(), out_dtype);
      if (zp.numel() != scale_rows * cols) zp = zp.expand(sc.sizes());
      zp = zp.contiguous();
    }
  }
  at::Tensor out = at::empty(out_shape, in.options().dtype(out_dtype));
  check_status(b200q_dequant_int4(in.data_ptr<int32_t>(), sc.data_ptr(), zp.defined() ? zp.data_ptr() : nullptr, zp_kind,
                                  is_signed ? 1 : 0, to_b200q_dtype(out_dtype), out.data_ptr(), rows, cols_packed,
                                  scale_rows, 0, current_stream()),
               "convert_from_int4");
  return out;
}
at::Tensor convert_from_int4(const at::Tensor& input, const at::Tensor& scale, const OptTensor& zp, at::ScalarType dt) {
  return convert_from_4bit(input, scale, zp, dt, true);
}
at::Tensor convert_from_uint4(const at::Tensor& input, const at::Tensor& scale, const OptTensor& zp,
                              at::ScalarType dt) {
  return convert_from_4bit(input, scale, zp, dt, false);
}

// AutoGPTQ layout (packed along K) -> [K, N]; b200q namespace: not a reference operator.
at::Tensor dequant_kpacked(const at::Tensor& qweight, const at::Tensor& scales, const OptTensor& qzeros,
                           at::ScalarType out_dtype) {
  TORCH_CHECK(qweight.dim() == 2 && qweight.scalar_type() == at::kInt, "qweight must be int32 [K/8, N]");
  c10::cuda::CUDAGuard guard(qweight.device());
  at::Tensor q = qweight.contiguous();
  const int64_t K = q.size(0) * 8, N = q.size(1);
  at::Tensor sc = scales.to(q.device(), out_dtype).contiguous();
  TORCH_CHECK(sc.dim() == 2 && sc.size(1) == N && K % sc.size(0) == 0, "scales must be [K/g, N]");
  at::Tensor zp;
  int zp_kind = B200Q_ZP_NONE;
  if (qzeros.has_value() && qzeros->defined()) {
    zp = qzeros->contiguous();
    TORCH_CHECK(zp.scalar_type() == at::kInt && zp.numel() == sc.size(0) * (N / 8), "qzeros must be int32 [K/g, N/8]");
    zp_kind = B200Q_ZP_PACKED;
  }
  at::Tensor out = at::empty({K, N}, q.options().dtype(out_dtype));
  check_status(b200q_dequant_int4(q.data_ptr<int32_t>(), sc.data_ptr(), zp.defined() ? zp.data_ptr() : nullptr, zp_kind, 0,
                                  to_b200q_dtype(out_dtype), out.data_ptr(), K, N, sc.size(0), 1, current_stream()),
               "dequant_kpacked");
  return out;
}

// AutoGPTQ checkpoint tensors -> operator layout (the reference's test repacks on the host,
// tests/pytest_working/any_mode/test_hpu_convert_from_int4.py:380-395).
std::tuple<at::Tensor, at::Tensor> gptq_repack(const at::Tensor& qweight, const OptTensor& qzeros) {
  TORCH_CHECK(qweight.dim() == 2 && qweight.scalar_type() == at::kInt, "gptq_repack: qweight must be int32 [K/8, N]");
  c10::cuda::CUDAGuard guard(qweight.device());
  at::Tensor q = qweight.contiguous();
  const int64_t K = q.size(0) * 8, N = q.size(1);
  TORCH_CHECK(N % 8 == 0, "gptq_repack: N must be a multiple of 8");
  at::Tensor out = at::empty({K, N / 8}, q.options());
  at::Tensor z, zout;
  if (qzeros.has_value() && qzeros->defined()) {
    TORCH_CHECK(qzeros->scalar_type() == at::kInt, "gptq_repack: qzeros must be int32");
    z = qzeros->contiguous();
    zout = at::empty_like(z);
  } else {
    zout = at::empty({0}, q.options());
  }
  check_status(b200q_gptq_repack(q.data_ptr<int32_t>(), out.data_ptr<int32_t>(), K, N,
                                 z.defined() ? z.data_ptr<int32_t>() : nullptr,
                                 z.defined() ? zout.data_ptr<int32_t>() : nullptr, z.defined() ? z.numel() : 0,
                                 current_stream()),
               "gptq_repack");
  return {out, zout};
}

// ------------------------------------------------------------------ fp8_gemm_v2
// hpu_ops/common/batched_matmul_output_shape.cpp:34-88
std::vector<int64_t> matmul_out_shape(c10::IntArrayRef a, c10::IntArrayRef b, bool ta, bool tb) {
  std::vector<int64_t> out;
  const size_t ra = a.size(), rb = b.size();
  TORCH_CHECK(ra >= 1 && rb >= 1, "matmul inputs must have at least one dimension");
  size_t ca = 0, cb = 0;
  if (rb > 1) {
    out.push_back(b[tb ? rb - 2 : rb - 1]);
    cb = tb ? rb - 1 : rb - 2;
  }
  if (ra > 1) {
    out.push_back(a[ta ? ra - 1 : ra - 2]);
    ca = ta ? ra - 2 : ra - 1;
  }
  TORCH_CHECK(a[ca] == b[cb], "Common dimension sizes of matmul inputs should be the same. Got ", a[ca], " and ", b[cb]);
  const size_t mr = std::max(ra, rb);
  for (size_t i = 3; i <= mr; ++i) {
    int64_t da = i > ra ? 1 : a[ra - i], db = i > rb ? 1 : b[rb - i];
    TORCH_CHECK(da == db || da == 1 || db == 1, "Batch dimension ", mr - i,
                " of matmul inputs should be the same or at least one of them should be equal to 1. Got ", da, " and ",
                db);
    out.push_back(da == db ? da : da * db);
  }
  std::reverse(out.begin(), out.end());
  return out;
}

struct EpiOperand {
  int mode = B200Q_BCAST_NONE;
  float host = 1.f;
  at::Tensor t;
  int64_t ld = 0, batch_stride = 0;
};

// Line a scale / bias tensor up with the output, seen canonically as bshape + [M, N]
// (has_m / has_n say whether the output really has those dimensions: 1-D operands drop them).
EpiOperand classify_epi(const at::Tensor& t_in, c10::IntArrayRef bshape, int64_t M, int64_t N, bool has_m, bool has_n,
                        c10::IntArrayRef out_shape, bool want_float, const char* what) {
  EpiOperand e;
  at::Tensor t = want_float ? t_in.to(at::kFloat) : t_in;
  if (t.numel() == 1) {
    e.mode = B200Q_BCAST_SCALAR_DEV;
    e.t = t.reshape({1}).contiguous();
    return e;
  }
  const int64_t orank = (int64_t)out_shape.size();
  TORCH_CHECK(t.dim() <= orank, what, " of shape ", t.sizes(), " does not broadcast against the output ", out_shape);
  // right-align with the output, then insert the dropped M / N dimensions as size 1
  std::vector<int64_t> ts(orank, 1);
  for (int64_t i = 0; i < t.dim(); ++i) ts[orank - t.dim() + i] = t.size(i);
  for (int64_t i = 0; i < orank; ++i)
    TORCH_CHECK(ts[i] == 1 || ts[i] == out_shape[i], what, " of shape ", t.sizes(),
                " does not broadcast against the output ", out_shape);
  std::vector<int64_t> can(ts.begin(), ts.begin() + (int64_t)bshape.size());
  int64_t pos = (int64_t)bshape.size();
  can.push_back(has_m ? ts[pos++] : 1);
  can.push_back(has_n ? ts[pos++] : 1);
  bool batch_ones = true;
  for (size_t i = 0; i < bshape.size(); ++i) batch_ones = batch_ones && can[i] == 1;
  const int64_t tm = can[can.size() - 2], tn = can[can.size() - 1];
  if (batch_ones && tm == 1 && tn == N) {
    e.mode = B200Q_BCAST_PER_COL;
    e.t = t.reshape({N}).contiguous();
    return e;
  }
  if (batch_ones && tn == 1 && tm == M) {
    e.mode = B200Q_BCAST_PER_ROW;
    e.t = t.reshape({M}).contiguous();
    return e;
  }
  std::vector<int64_t> full(bshape.begin(), bshape.end());
  full.push_back(M);
  full.push_back(N);
  int64_t batch = numel_of(bshape);
  e.mode = B200Q_BCAST_FULL;
  e.t = t.reshape(can).expand(full).contiguous().reshape({batch, M, N});
  e.ld = N;
  e.batch_stride = M * N;
  return e;
}

ScaleArg to_scale_arg(const OptTensor& t) {
  ScaleArg s;
  if (t.has_value() && t->defined()) s = *t;
  return s;
}

// out8_dtype / out8_scale: fused output cast (b200q::fp8_gemm_cast); Undefined = plain fp8_gemm_v2.
at::Tensor fp8_gemm_v2_common(const at::Tensor& A, bool trans_A, const at::Tensor& B, bool trans_B, const OptTensor& D,
                              at::ScalarType out_dtype, const ScaleArg& A_scale_inv, const ScaleArg& B_scale_inv,
                              const OptTensor& bias, bool accumulate, OptShape B_scale_shape,
                              at::ScalarType out8_dtype = at::ScalarType::Undefined, double out8_scale = 1.0,
                              const OptTensor& out8_scale_dev = c10::nullopt, at::Tensor* out8_amax = nullptr) {
  TORCH_CHECK(is_fp8(A.scalar_type()) && is_fp8(B.scalar_type()), "fp8_gemm_v2 inputs must be float8 tensors, got ",
              A.scalar_type(), " and ", B.scalar_type());
  TORCH_CHECK(out_dtype == at::kFloat || out_dtype == at::kBFloat16,
              "fp8_gemm_v2 output dtype must be float or bfloat16, got ", out_dtype);
  validate_scale_shape(B_scale_inv, B_scale_shape);
  const bool has_D = D.has_value() && D->defined();
  TORCH_CHECK(!accumulate || has_D,
              "Accumulation tensor must be provided at index 4 for Fp8GemmV2, when accumulate is true");
  const std::vector<int64_t> out_shape = matmul_out_shape(A.sizes(), B.sizes(), trans_A, trans_B);
  c10::cuda::CUDAGuard guard(A.device());

  // 2-D (or batched 3-D) operand views; 1-D operands become a row / a column
  at::Tensor a = A, b = B;
  bool ta = trans_A, tb = trans_B;
  const bool has_m = A.dim() > 1, has_n = B.dim() > 1;
  if (a.dim() == 1) { a = a.unsqueeze(0); ta = false; }
  if (b.dim() == 1) { b = b.unsqueeze(1); tb = false; }
  const int64_t M = ta ? a.size(-1) : a.size(-2), K = ta ? a.size(-2) : a.size(-1);
  const int64_t N = tb ? b.size(-2) : b.size(-1);
  // batch dims
  std::vector<int64_t> bshape;
  {
    auto ab = a.sizes().slice(0, a.dim() - 2), bb = b.sizes().slice(0, b.dim() - 2);
    bshape = at::infer_size(ab, bb);
  }
  int64_t batch = numel_of(bshape);
  const bool fused_cast = out8_dtype != at::ScalarType::Undefined;
  at::Tensor out8_scale_keep;
  TORCH_CHECK(!fused_cast || is_fp8(out8_dtype), "fp8_gemm_cast: the output dtype must be float8_e5m2 or float8_e4m3fn");
  at::Tensor out = at::empty(out_shape, A.options().dtype(fused_cast ? out8_dtype : out_dtype));
  if (out.numel() == 0) return out;

  b200q_gemm_args g{};
  if (fused_cast) {
    g.out8_dtype = to_b200q_dtype(out8_dtype);
    g.out8_scale = nullptr;
    g.out8_scale_host = (float)out8_scale;
    if (out8_scale_dev.has_value() && out8_scale_dev->defined()) {  // a device scalar: no read-back to the host
      TORCH_CHECK(out8_scale_dev->numel() == 1, "the output scale must have one element");
      out8_scale_keep = out8_scale_dev->to(A.device(), at::kFloat).reshape({1}).contiguous();
      g.out8_scale = out8_scale_keep.data_ptr<float>();
    }
    if (out8_amax) {
      *out8_amax = at::zeros({}, A.options().dtype(at::kFloat));
      g.out8_amax = out8_amax->data_ptr<float>();
    }
  }
  int64_t Mk = M;  // M as the kernel sees it (batch may be folded in)
  bool folded = false;
  if (batch > 1 && b.dim() == 2 && !ta) {
    // [.., M, K] x [K, N]: fold the batch into M
    a = a.contiguous().reshape({batch * M, K});
    Mk = batch * M;
    folded = true;
  } else if (batch > 1 || a.dim() > 2 || b.dim() > 2) {
    std::vector<int64_t> as = bshape, bs = bshape;
    as.push_back(a.size(-2)); as.push_back(a.size(-1));
    bs.push_back(b.size(-2)); bs.push_back(b.size(-1));
    a = a.expand(as).contiguous().reshape({batch, a.size(-2), a.size(-1)});
    b = b.expand(bs).contiguous().reshape({batch, b.size(-2), b.size(-1)});
  }
  auto as_matrix = [](at::Tensor& t) {
    // row-major with unit inner stride (a transposed view counts as a copy here)
    if (t.stride(-1) != 1 || (t.dim() >= 2 && t.size(-2) > 1 && t.stride(-2) < t.size(-1))) t = t.contiguous();
  };
  as_matrix(a);
  as_matrix(b);
  // K not a multiple of 16 with an operand stored [rows][K]: its row pitch is not 16-byte granular and
  // the tensor-core kernels (TMA) cannot take it; the CUDA-core kernel that can is two to three orders
  // of magnitude slower.  For problems large enough to matter both operands are copied into
  // buffers with K rounded up to 16, the extra k filled with zeros (fp8 0x00 = +0 adds nothing).
  int64_t Kk = K;
  if ((K % 16) != 0 && (!ta || tb) && (double)Mk * (double)N * (double)K >= (double)(1 << 26)) {
    Kk = (K + 15) / 16 * 16;
    auto pad_k = [&](at::Tensor& t, int64_t kdim) {
      auto sizes = t.sizes().vec();
      sizes[t.dim() + kdim] = Kk;
      at::Tensor padded = at::zeros(sizes, t.options().dtype(at::kByte));
      padded.narrow(kdim, 0, K).copy_(t.view(at::kByte));
      t = padded.view(t.scalar_type());
    };
    pad_k(a, ta ? -2 : -1);
    pad_k(b, tb ? -1 : -2);
  }
  const int64_t kbatch = folded ? 1 : batch;
  g.A = a.data_ptr(); g.B = b.data_ptr();
  g.a_dtype = to_b200q_dtype(a.scalar_type()); g.b_dtype = to_b200q_dtype(b.scalar_type());
  g.trans_a = ta; g.trans_b = tb; g.M = Mk; g.N = N; g.K = Kk;
  g.lda = a.size(-2) > 1 ? a.stride(-2) : a.size(-1);
  g.ldb = b.size(-2) > 1 ? b.stride(-2) : b.size(-1);
  g.batch = kbatch;
  g.a_batch_stride = a.dim() == 3 ? a.stride(0) : 0;
  g.b_batch_stride = b.dim() == 3 ? b.stride(0) : 0;
  g.out_batch_stride = M * N;
  g.out = out.data_ptr(); g.out_dtype = to_b200q_dtype(out_dtype); g.ldo = N;

  // epilogue operands are classified against the un-folded output, then adapted if folded
  std::vector<at::Tensor> keep;
  auto setup_scale = [&](const ScaleArg& s, OptShape shape, const float** dev, float* host, int* mode) {
    *mode = B200Q_BCAST_NONE; *dev = nullptr; *host = 1.f;
    if (std::holds_alternative<std::monostate>(s)) return;
    if (auto d = std::get_if<double>(&s)) { *mode = B200Q_BCAST_SCALAR_HOST; *host = (float)*d; return; }
    at::Tensor t = scale_tensor(s, shape, A.device());
    EpiOperand e = classify_epi(t, bshape, M, N, has_m, has_n, out_shape, true, "scale");
    if (folded && e.mode == B200Q_BCAST_PER_ROW) e.t = e.t.repeat({batch});
    if (e.mode == B200Q_BCAST_FULL) {
      TORCH_CHECK(folded || batch == 1, "fp8_gemm_v2: an element-wise scale with batched operands is not supported");
    }
    keep.push_back(e.t);
    *dev = e.t.data_ptr<float>(); *mode = e.mode;
  };
  setup_scale(A_scale_inv, c10::nullopt, &g.a_scale, &g.a_scale_host, &g.a_scale_mode);
  setup_scale(B_scale_inv, B_scale_shape, &g.b_scale, &g.b_scale_host, &g.b_scale_mode);
  if (bias.has_value() && bias->defined()) {
    at::Tensor bt = bias->to(A.device());
    if (bt.scalar_type() != at::kFloat && bt.scalar_type() != at::kBFloat16) bt = bt.to(at::kFloat);
    EpiOperand e = classify_epi(bt, bshape, M, N, has_m, has_n, out_shape, false, "bias");
    if (e.mode == B200Q_BCAST_SCALAR_DEV) {  // one value: treat as a per-column vector
      e.t = e.t.expand({N}).contiguous();
      e.mode = B200Q_BCAST_PER_COL;
    }
    if (folded && e.mode == B200Q_BCAST_PER_ROW) e.t = e.t.repeat({batch});
    keep.push_back(e.t);
    g.bias = e.t.data_ptr(); g.bias_dtype = to_b200q_dtype(e.t.scalar_type()); g.bias_mode = e.mode;
    g.bias_ld = N; g.bias_batch_stride = folded ? 0 : M * N;
  }
  if (accumulate) {
    at::Tensor d = D->to(A.device());
    if (d.scalar_type() != at::kFloat && d.scalar_type() != at::kBFloat16) d = d.to(at::kFloat);
    d = d.expand(out_shape).contiguous();
    keep.push_back(d);
    g.D = d.data_ptr(); g.d_dtype = to_b200q_dtype(d.scalar_type()); g.ldd = N; g.d_batch_stride = folded ? 0 : M * N;
  }
  g.stream = current_stream();
  check_status(b200q_fp8_gemm(&g), "fp8_gemm_v2");
  return out;
}

at::Tensor fp8_gemm_v2(const at::Tensor& A, bool trans_A, const at::Tensor& B, bool trans_B, const OptTensor& D,
                       at::ScalarType out_dtype, const OptTensor& A_scale_inv, const OptTensor& B_scale_inv,
                       const OptTensor& bias, bool accumulate, OptShape B_scale_shape) {
  return fp8_gemm_v2_common(A, trans_A, B, trans_B, D, out_dtype, to_scale_arg(A_scale_inv), to_scale_arg(B_scale_inv),
                            bias, accumulate, B_scale_shape);
}
at::Tensor fp8_gemm_v2_scalar(const at::Tensor& A, bool trans_A, const at::Tensor& B, bool trans_B, const OptTensor& D,
                              at::ScalarType out_dtype, double A_scale_inv, double B_scale_inv, const OptTensor& bias,
                              bool accumulate, OptShape) {
  return fp8_gemm_v2_common(A, trans_A, B, trans_B, D, out_dtype, ScaleArg(A_scale_inv), ScaleArg(B_scale_inv), bias,
                            accumulate, c10::nullopt);
}
at::Tensor fp8_gemm_v2_scalar_list(const at::Tensor& A, bool trans_A, const at::Tensor& B, bool trans_B,
                                   const OptTensor& D, at::ScalarType out_dtype, c10::ArrayRef<double> A_scale_inv,
                                   c10::ArrayRef<double> B_scale_inv, const OptTensor& bias, bool accumulate,
                                   OptShape B_scale_shape) {
  return fp8_gemm_v2_common(A, trans_A, B, trans_B, D, out_dtype, ScaleArg(A_scale_inv.vec()),
                            ScaleArg(B_scale_inv.vec()), bias, accumulate, B_scale_shape);
}

// legacy out-variant (kernels_register.cpp:2445; fp8_ops.cpp:312-366)
at::Tensor& fp8_gemm(const at::Tensor& A, bool trans_A, const at::Tensor& B, bool trans_B, const at::Tensor& D,
                     at::ScalarType out_dtype, const OptTensor& A_scale_inv, const OptTensor& B_scale_inv,
                     const OptTensor& bias, bool accumulate, at::Tensor& out) {
  at::Tensor r = fp8_gemm_v2(A, trans_A, B, trans_B, D, out_dtype, A_scale_inv, B_scale_inv, bias, accumulate,
                             c10::nullopt);
  out.copy_(r);
  return out;
}

// GEMM with the cast of its result fused into the epilogue: cast_to_fp8_v2(fp8_gemm_v2(...), out_scale, RNE).
at::Tensor fp8_gemm_cast(const at::Tensor& A, bool trans_A, const at::Tensor& B, bool trans_B, const OptTensor& D,
                         at::ScalarType mid_dtype, const OptTensor& A_scale_inv, const OptTensor& B_scale_inv,
                         const OptTensor& bias, bool accumulate, OptShape B_scale_shape, double out_scale,
                         at::ScalarType out_dtype) {
  return fp8_gemm_v2_common(A, trans_A, B, trans_B, D, mid_dtype, to_scale_arg(A_scale_inv), to_scale_arg(B_scale_inv), bias,
                            accumulate, B_scale_shape, out_dtype, out_scale);
}

// aten::_scaled_mm-shaped entry (the reference lowers _scaled_mm to the same fp8_gemm node,
// hpu_ops/backend/scaled_mm_gen.cpp:66-140): out = (a @ b) * scale_a * scale_b + bias; b is usually the
// transposed view of an [N, K] weight, which is recognised and passed as a K-major operand.
// Returns (out, amax): for a float8 out_dtype amax = max |out| of the values written (taken in the
// GEMM's epilogue, scaled_mm_gen.cpp:283-320); for other output dtypes the reference computes no
// amax and a zero is returned.
std::tuple<at::Tensor, at::Tensor> scaled_mm(const at::Tensor& a, const at::Tensor& b, const at::Tensor& scale_a,
                                             const at::Tensor& scale_b, const OptTensor& bias,
                                             const OptTensor& scale_result, at::ScalarType out_dtype) {
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "scaled_mm: 2-D operands expected");
  const bool b_is_transposed_view = b.stride(0) == 1 && b.stride(1) >= b.size(0) && b.size(0) > 1;
  at::Tensor bb = b_is_transposed_view ? b.t() : b;
  at::Tensor sb = scale_b;
  OptShape shape = c10::nullopt;
  std::vector<int64_t> shp;
  if (sb.numel() > 1) {  // row-wise scaling: scale_b is [1, N]
    shp = {1, sb.numel()};
    shape = shp;
  }
  if (is_fp8(out_dtype)) {
    at::Tensor amax;
    at::Tensor out = fp8_gemm_v2_common(a, false, bb, b_is_transposed_view, c10::nullopt, at::kBFloat16, ScaleArg(scale_a),
                                        ScaleArg(sb), bias, false, shape, out_dtype, 1.0, scale_result, &amax);
    return {out, amax};
  }
  at::Tensor out = fp8_gemm_v2_common(a, false, bb, b_is_transposed_view, c10::nullopt, out_dtype, ScaleArg(scale_a),
                                      ScaleArg(sb), bias, false, shape);
  return {out, at::zeros({}, a.options().dtype(at::kFloat))};
}

// ------------------------------------------------------------------ fp8_sdpa_recomp_fwd
// habana_kernels/kernels_register.cpp:2525,2533; node hpu_ops/backend/sdpa_gen.cpp:820-1000; shapes
// sdpa_gen.cpp:600-702; meta python_packages/habana_frameworks/torch/dynamo/_custom_op_meta_registrations.py:636-657.
// Forward without dropout.  q / k / v: e4m3 [..., L, D]; the batch dimensions of k / v equal those of
// q or broadcast along the LAST of them (multi-query [B, 1, S, D]; grouped-query as the reference's
// caller reshapes it, q [B, G, R, L, D] against k / v [B, G, 1, S, D]).
struct SdpaScale {
  at::Tensor dev;  // one-element fp32 on the device, or undefined
  float host = 1.f;
  bool given = false;
};
static SdpaScale sdpa_scale(const OptTensor& t, const at::Device& d) {
  SdpaScale s;
  if (t.has_value() && t->defined() && t->numel() > 0) {
    s.dev = t->to(d, at::kFloat).reshape(-1).slice(0, 0, 1).contiguous();
    s.given = true;
  }
  return s;
}
static SdpaScale sdpa_scale(double v) {
  SdpaScale s;
  if (v != 0.) {  // the reference treats a scalar 0 as "not given" (sdpa_gen.cpp:893-905)
    s.host = (float)v;
    s.given = true;
  }
  return s;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> fp8_sdpa_recomp_fwd_common(
    const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const OptTensor& attention_mask, double p, double scale,
    bool is_causal, bool requires_backward, c10::string_view softmax_mode, const SdpaScale& d_q, const SdpaScale& d_k,
    const SdpaScale& d_v, const SdpaScale& q_s, const SdpaScale& q_o, const SdpaScale& d_s, bool is_amax_s, bool is_amax_o,
    const OptTensor& valid_seq_len, c10::string_view seq_padding_type) {
  (void)softmax_mode; (void)seq_padding_type;
  TORCH_CHECK(q.scalar_type() == at::kFloat8_e4m3fn && k.scalar_type() == at::kFloat8_e4m3fn && v.scalar_type() == at::kFloat8_e4m3fn,
              "fp8_sdpa_recomp_fwd: q, k and v must be float8_e4m3fn tensors");
  TORCH_CHECK(p == 0.0, "fp8_sdpa_recomp_fwd: dropout is not supported");
  TORCH_CHECK(!(valid_seq_len.has_value() && valid_seq_len->defined()), "fp8_sdpa_recomp_fwd: valid_seq_len is not supported");
  const int64_t rank = q.dim();
  TORCH_CHECK(rank >= 3 && k.dim() == rank && v.dim() == rank, "fp8_sdpa_recomp_fwd: q, k, v must have the same rank >= 3");
  const int64_t L = q.size(-2), D = q.size(-1), S = k.size(-2), Dv = v.size(-1);
  TORCH_CHECK(k.size(-1) == D && v.size(-2) == S, "fp8_sdpa_recomp_fwd: k / v do not match q");
  TORCH_CHECK(S >= 1, "fp8_sdpa_recomp_fwd: no keys");
  c10::cuda::CUDAGuard guard(q.device());
  // batch layout: BH query heads, each reading key/value head bh / kv_rep
  int64_t BH = 1, BHkv = 1;
  for (int64_t d = 0; d < rank - 2; ++d) { BH *= q.size(d); BHkv *= k.size(d); }
  at::Tensor kc = k, vc = v;
  bool pattern_ok = BHkv > 0 && BH % BHkv == 0;
  for (int64_t d = 0; d < rank - 2 && pattern_ok; ++d) {
    const bool same = k.size(d) == q.size(d) && v.size(d) == q.size(d);
    const bool last_bcast = d == rank - 3 && k.size(d) == 1 && v.size(d) == 1;
    pattern_ok = same || last_bcast;
  }
  if (!pattern_ok) {  // any other broadcast: materialise it
    std::vector<int64_t> ks(q.sizes().begin(), q.sizes().end() - 2), vs = ks;
    ks.push_back(S); ks.push_back(D); vs.push_back(S); vs.push_back(Dv);
    kc = k.expand(ks); vc = v.expand(vs);
    BHkv = BH;
  }
  const int kv_rep = (int)(BH / BHkv);
  at::Tensor qc = q.contiguous();
  kc = kc.contiguous(); vc = vc.contiguous();
  std::vector<int64_t> out_shape(q.sizes().begin(), q.sizes().end() - 1);
  out_shape.push_back(Dv);
  std::vector<int64_t> stat_shape(q.sizes().begin(), q.sizes().end() - 1);
  stat_shape.push_back(1);
  const bool fp8_out = q_o.given;
  at::Tensor out = at::empty(out_shape, q.options().dtype(fp8_out ? at::kFloat8_e4m3fn : at::kBFloat16));
  at::Tensor m = requires_backward ? at::empty(stat_shape, q.options().dtype(at::kBFloat16)) : at::zeros({1}, q.options().dtype(at::kBFloat16));
  at::Tensor linv = requires_backward ? at::empty(stat_shape, q.options().dtype(at::kBFloat16)) : at::zeros({1}, q.options().dtype(at::kBFloat16));
  at::Tensor seed = at::zeros({1}, q.options().dtype(at::kInt));
  at::Tensor amax_s = at::zeros({1}, q.options().dtype(at::kFloat)), amax_o = at::zeros({1}, q.options().dtype(at::kFloat));
  if (out.numel() == 0) return {out, m, linv, seed, amax_s, amax_o};

  b200q_sdpa_args a{};
  a.q = qc.data_ptr(); a.k = kc.data_ptr(); a.v = vc.data_ptr(); a.out = out.data_ptr();
  a.out_dtype = fp8_out ? B200Q_E4M3 : B200Q_BF16;
  a.BH = BH; a.L = L; a.S = S; a.dqk = (int)D; a.dv = (int)Dv; a.kv_rep = kv_rep;
  a.causal = is_causal ? 1 : 0;
  a.softmax_scale = (float)scale;
  at::Tensor mask_keep;
  if (attention_mask.has_value() && attention_mask->defined()) {
    // broadcast the mask against [batch dims..., L, S]; batch-invariant / row-invariant masks keep stride 0
    at::Tensor mk = attention_mask->to(q.device());
    if (mk.scalar_type() == at::kBool) mk = mk.to(at::kByte);
    else if (mk.scalar_type() != at::kBFloat16 && mk.scalar_type() != at::kFloat) mk = mk.to(at::kFloat);
    TORCH_CHECK(mk.dim() <= rank && mk.size(-1) == S, "fp8_sdpa_recomp_fwd: the attention mask does not broadcast against [.., L, S]");
    while (mk.dim() < rank) mk = mk.unsqueeze(0);
    bool batch_invariant = true;
    for (int64_t d = 0; d < rank - 2; ++d) {
      TORCH_CHECK(mk.size(d) == 1 || mk.size(d) == q.size(d), "fp8_sdpa_recomp_fwd: the attention mask does not broadcast");
      batch_invariant = batch_invariant && mk.size(d) == 1;
    }
    TORCH_CHECK(mk.size(-2) == 1 || mk.size(-2) == L, "fp8_sdpa_recomp_fwd: the attention mask does not broadcast");
    const bool row_invariant = mk.size(-2) == 1;
    if (!batch_invariant) {
      std::vector<int64_t> full(q.sizes().begin(), q.sizes().end() - 2);
      full.push_back(mk.size(-2)); full.push_back(S);
      mk = mk.expand(full);
    }
    mask_keep = mk.contiguous();
    a.mask = mask_keep.data_ptr();
    a.mask_kind = mask_keep.scalar_type() == at::kBFloat16 ? 1 : mask_keep.scalar_type() == at::kFloat ? 2 : 3;
    a.mask_sl = row_invariant ? 0 : S;
    a.mask_sb = batch_invariant ? 0 : (row_invariant ? S : L * S);
  }
  const SdpaScale* sc[6] = {&d_q, &d_k, &d_v, &q_s, &q_o, &d_s};
  const float** devs[6] = {&a.d_scale_q, &a.d_scale_k, &a.d_scale_v, &a.q_scale_s, &a.q_scale_o, &a.d_scale_s};
  float* hosts[6] = {&a.d_scale_q_host, &a.d_scale_k_host, &a.d_scale_v_host, &a.q_scale_s_host, &a.q_scale_o_host, &a.d_scale_s_host};
  for (int i = 0; i < 6; ++i) {
    *hosts[i] = sc[i]->given ? sc[i]->host : 1.f;
    *devs[i] = sc[i]->dev.defined() ? sc[i]->dev.data_ptr<float>() : nullptr;
  }
  a.d_scale_s_given = d_s.given ? 1 : 0;
  if (requires_backward) { a.m_out = m.data_ptr(); a.linv_out = linv.data_ptr(); }
  if (is_amax_s) a.amax_s = amax_s.data_ptr<float>();
  if (is_amax_o) a.amax_o = amax_o.data_ptr<float>();
  static const bool force_plain = std::getenv("B200Q_SDPA_PLAIN") != nullptr;  // comparison switch
  a.force_plain = force_plain ? 1 : 0;
  a.stream = current_stream();
  check_status(b200q_fp8_sdpa_fwd(&a), "fp8_sdpa_recomp_fwd");
  return {out, m, linv, seed, amax_s, amax_o};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> fp8_sdpa_recomp_fwd(
    const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const OptTensor& attention_mask, double p, double scale,
    bool is_causal, bool requires_backward, c10::string_view softmax_mode, const OptTensor& d_scale_q, const OptTensor& d_scale_k,
    const OptTensor& d_scale_v, const OptTensor& q_scale_s, const OptTensor& q_scale_o, const OptTensor& d_scale_s, bool is_amax_s,
    bool is_amax_o, const OptTensor& valid_seq_len, c10::string_view seq_padding_type) {
  const auto dev = q.device();
  return fp8_sdpa_recomp_fwd_common(q, k, v, attention_mask, p, scale, is_causal, requires_backward, softmax_mode,
                                    sdpa_scale(d_scale_q, dev), sdpa_scale(d_scale_k, dev), sdpa_scale(d_scale_v, dev),
                                    sdpa_scale(q_scale_s, dev), sdpa_scale(q_scale_o, dev), sdpa_scale(d_scale_s, dev), is_amax_s,
                                    is_amax_o, valid_seq_len, seq_padding_type);
}
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> fp8_sdpa_recomp_fwd_scalar(
    const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const OptTensor& attention_mask, double p, double scale,
    bool is_causal, bool requires_backward, c10::string_view softmax_mode, double d_scale_q, double d_scale_k, double d_scale_v,
    double q_scale_s, double q_scale_o, double d_scale_s, bool is_amax_s, bool is_amax_o, const OptTensor& valid_seq_len,
    c10::string_view seq_padding_type) {
  return fp8_sdpa_recomp_fwd_common(q, k, v, attention_mask, p, scale, is_causal, requires_backward, softmax_mode,
                                    sdpa_scale(d_scale_q), sdpa_scale(d_scale_k), sdpa_scale(d_scale_v), sdpa_scale(q_scale_s),
                                    sdpa_scale(q_scale_o), sdpa_scale(d_scale_s), is_amax_s, is_amax_o, valid_seq_len,
                                    seq_padding_type);
}

// Meta: shapes and dtypes of the six outputs (_custom_op_meta_registrations.py:636-657)
static std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> meta_sdpa_outputs(
    const at::Tensor& q, const at::Tensor& v, bool fp8_out, bool requires_backward) {
  std::vector<int64_t> out_shape(q.sizes().begin(), q.sizes().end() - 1);
  out_shape.push_back(v.size(-1));
  std::vector<int64_t> stat_shape(q.sizes().begin(), q.sizes().end() - 1);
  stat_shape.push_back(1);
  if (!requires_backward) stat_shape = {1};
  auto o = q.options();
  return {at::empty(out_shape, o.dtype(fp8_out ? at::kFloat8_e4m3fn : at::kBFloat16)), at::empty(stat_shape, o.dtype(at::kBFloat16)),
          at::empty(stat_shape, o.dtype(at::kBFloat16)), at::empty({1}, o.dtype(at::kInt)), at::empty({1}, o.dtype(at::kFloat)),
          at::empty({1}, o.dtype(at::kFloat))};
}
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> meta_fp8_sdpa_recomp_fwd(
    const at::Tensor& q, const at::Tensor&, const at::Tensor& v, const OptTensor&, double, double, bool, bool requires_backward,
    c10::string_view, const OptTensor&, const OptTensor&, const OptTensor&, const OptTensor&, const OptTensor& q_scale_o,
    const OptTensor&, bool, bool, const OptTensor&, c10::string_view) {
  return meta_sdpa_outputs(q, v, q_scale_o.has_value() && q_scale_o->defined() && q_scale_o->numel() > 0, requires_backward);
}
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> meta_fp8_sdpa_recomp_fwd_scalar(
    const at::Tensor& q, const at::Tensor&, const at::Tensor& v, const OptTensor&, double, double, bool, bool requires_backward,
    c10::string_view, double, double, double, double, double q_scale_o, double, bool, bool, const OptTensor&, c10::string_view) {
  return meta_sdpa_outputs(q, v, q_scale_o != 0., requires_backward);
}

// ------------------------------------------------------------------ b200q:: extras
at::Tensor w4a16_gemm(const at::Tensor& x, const at::Tensor& qweight, const at::Tensor& scales, const OptTensor& qzeros,
                      int64_t group_size, bool k_packed, at::ScalarType out_dtype) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2, "w4a16_gemm: x must be bf16 [M, K]");
  TORCH_CHECK(qweight.scalar_type() == at::kInt && qweight.dim() == 2, "w4a16_gemm: qweight must be int32 2-D");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor xc = x.contiguous(), q = qweight.contiguous(), sc = scales.to(at::kBFloat16).contiguous();
  const int64_t M = xc.size(0), K = xc.size(1);
  const int64_t N = k_packed ? q.size(1) : q.size(1) * 8;
  TORCH_CHECK((k_packed ? q.size(0) * 8 : q.size(0)) == K, "w4a16_gemm: qweight does not match K = ", K);
  TORCH_CHECK(group_size > 0 && K % group_size == 0 && sc.dim() == 2 && sc.size(0) == K / group_size && sc.size(1) == N,
              "w4a16_gemm: scales must be [K/group, N]");
  at::Tensor zp;
  int zp_kind = B200Q_ZP_NONE;
  if (qzeros.has_value() && qzeros->defined()) {
    zp = qzeros->contiguous();
    TORCH_CHECK(zp.scalar_type() == at::kInt && zp.numel() == sc.size(0) * (N / 8), "w4a16_gemm: qzeros must be int32 [K/group, N/8]");
    zp_kind = B200Q_ZP_PACKED;
  }
  at::Tensor out = at::empty({M, N}, xc.options().dtype(out_dtype));
  if (k_packed && M > 16) {
    // The AutoGPTQ layout [K/8, N] is read directly only by the few-token kernel; more tokens go
    // through one repack pass into the operator layout [K, N/8] (a weight-sized copy: callers
    // that keep weights resident should call b200q::gptq_repack once instead).
    TORCH_CHECK(K % 8 == 0 && N % 8 == 0, "w4a16_gemm: K and N must be multiples of 8");
    at::Tensor q2 = at::empty({K, N / 8}, q.options());
    check_status(b200q_gptq_repack(q.data_ptr<int32_t>(), q2.data_ptr<int32_t>(), K, N, nullptr, nullptr, 0, current_stream()),
                 "w4a16_gemm (repack)");
    q = q2;
    k_packed = false;
  }
  const size_t ws_bytes = b200q_w4a16_workspace_bytes(M, N, K);
  at::Tensor ws;
  if (ws_bytes) ws = at::empty({(int64_t)ws_bytes}, xc.options().dtype(at::kByte));
  check_status(b200q_w4a16_gemm(xc.data_ptr(), K, q.data_ptr<int32_t>(), sc.data_ptr(),
                                zp.defined() ? zp.data_ptr<int32_t>() : nullptr, zp_kind, k_packed ? 1 : 0, M, N, K,
                                group_size, out.data_ptr(), to_b200q_dtype(out_dtype), N,
                                ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, current_stream()),
               "w4a16_gemm");
  return out;
}

std::tuple<at::Tensor, at::Tensor> swiglu_cast_fp8(const at::Tensor& gate, const at::Tensor& up, double scale, bool is_amax);

// Gate / up projection GEMM with the SwiGLU + cast in its epilogue.  w_gate_up: e4m3 [2f, d] with
// gate and up rows interleaved in blocks of 128 (rows [256 b, 256 b + 128) gate, next 128 up, of
// hidden units [128 b, 128 b + 128)); w_scale_inv [2f] in the same order.  Returns e4m3 [M, f] =
// swiglu_cast_fp8 of fp8_gemm_v2(x8, w_gate_up^T) -- the same bytes -- without writing the bf16
// [M, 2f] intermediate when the shape has a fused kernel (M > 128, 2f % 256 == 0).
at::Tensor fp8_gemm_swiglu_cast(const at::Tensor& x8, const at::Tensor& w_gate_up, const OptTensor& x_scale_inv,
                                const OptTensor& w_scale_inv, double act_scale) {
  TORCH_CHECK(is_fp8(x8.scalar_type()) && is_fp8(w_gate_up.scalar_type()) && x8.dim() == 2 && w_gate_up.dim() == 2 &&
                  x8.size(1) == w_gate_up.size(1) && w_gate_up.size(0) % 256 == 0,
              "fp8_gemm_swiglu_cast: x8 [M, d] and w_gate_up [2f, d] float8, 2f a multiple of 256");
  c10::cuda::CUDAGuard guard(x8.device());
  const int64_t M = x8.size(0), N = w_gate_up.size(0), K = x8.size(1), F = N / 2;
  at::Tensor a = x8.contiguous(), b = w_gate_up.contiguous();
  at::Tensor out = at::empty({M, F}, x8.options().dtype(at::kFloat8_e4m3fn));
  if (out.numel() == 0) return out;
  b200q_gemm_args g{};
  g.A = a.data_ptr(); g.B = b.data_ptr();
  g.a_dtype = to_b200q_dtype(a.scalar_type()); g.b_dtype = to_b200q_dtype(b.scalar_type());
  g.trans_a = 0; g.trans_b = 1;
  g.M = M; g.N = N; g.K = K; g.lda = K; g.ldb = K; g.batch = 1;
  g.out = out.data_ptr(); g.out_dtype = B200Q_BF16; g.ldo = F;
  at::Tensor sa, sb;
  if (x_scale_inv.has_value() && x_scale_inv->defined()) {
    TORCH_CHECK(x_scale_inv->numel() == 1, "fp8_gemm_swiglu_cast: x_scale_inv must have one element");
    sa = x_scale_inv->to(at::kFloat).contiguous();
    g.a_scale = sa.data_ptr<float>(); g.a_scale_mode = B200Q_BCAST_SCALAR_DEV;
  }
  if (w_scale_inv.has_value() && w_scale_inv->defined()) {
    TORCH_CHECK(w_scale_inv->numel() == 1 || w_scale_inv->numel() == N, "fp8_gemm_swiglu_cast: w_scale_inv must have 1 or 2f elements");
    sb = w_scale_inv->to(at::kFloat).contiguous();
    g.b_scale = sb.data_ptr<float>(); g.b_scale_mode = sb.numel() == 1 ? B200Q_BCAST_SCALAR_DEV : B200Q_BCAST_PER_COL;
  }
  g.out8_dtype = B200Q_E4M3; g.out8_scale = nullptr; g.out8_scale_host = (float)act_scale;
  g.swiglu = 1;
  g.stream = current_stream();
  const int rc = b200q_fp8_gemm(&g);
  if (rc == B200Q_ERR_UNSUPPORTED) {
    // no fused kernel for this shape: the two operators, on the de-interleaved halves
    std::vector<int64_t> one_n{1, N};
    at::Tensor gu = fp8_gemm_v2(a, false, b, true, c10::nullopt, at::kBFloat16, x_scale_inv, w_scale_inv, c10::nullopt, false,
                                sb.defined() && sb.numel() == N ? OptShape(at::IntArrayRef(one_n)) : OptShape(c10::nullopt));
    at::Tensor v = gu.view({M, F / 128, 2, 128});
    at::Tensor gate = v.select(2, 0).reshape({M, F}), up = v.select(2, 1).reshape({M, F});
    return std::get<0>(swiglu_cast_fp8(gate, up, act_scale, false));
  }
  check_status(rc, "fp8_gemm_swiglu_cast");
  return out;
}

std::tuple<at::Tensor, at::Tensor> swiglu_cast_fp8(const at::Tensor& gate, const at::Tensor& up, double scale,
                                                   bool is_amax) {
  TORCH_CHECK(gate.scalar_type() == at::kBFloat16 && up.scalar_type() == at::kBFloat16 && gate.dim() == 2 &&
                  gate.sizes() == up.sizes() && gate.stride(1) == 1 && up.stride(1) == 1,
              "swiglu_cast_fp8: gate/up must be bf16 [rows, cols] with unit inner stride");
  c10::cuda::CUDAGuard guard(gate.device());
  at::Tensor out = at::empty(gate.sizes(), gate.options().dtype(at::kFloat8_e4m3fn));
  at::Tensor amax = is_amax ? at::empty({}, gate.options().dtype(at::kFloat)) : at::empty({0}, gate.options().dtype(at::kFloat));
  check_status(b200q_swiglu_cast_fp8(gate.data_ptr(), gate.stride(0), up.data_ptr(), up.stride(0), out.data_ptr(),
                                     (float)scale, gate.size(0), gate.size(1),
                                     is_amax ? amax.data_ptr<float>() : nullptr, current_stream()),
               "swiglu_cast_fp8");
  return {out, amax};
}

// ---- softmax_fp8 (hpu_ops/backend/softmax_fp8_gen.cpp:65-160; schemas scripts/hpu_op.yaml:7399-7418) ----
struct SoftmaxScale {  // absent | device scalar | host scalar
  const float* dev = nullptr;
  float host = 1.f;
  bool given = false;
  at::Tensor keep;
};
static SoftmaxScale softmax_scale(const OptTensor& t, const at::Tensor& like) {
  SoftmaxScale s;
  if (t.has_value() && t->defined()) {
    TORCH_CHECK(t->scalar_type() == at::kFloat, "Input scale must be of dtype: ", at::kFloat);
    TORCH_CHECK(t->numel() == 1, "softmax_fp8 scales must have one element");
    s.keep = t->to(like.device()).contiguous();
    s.dev = s.keep.data_ptr<float>();
    s.given = true;
  }
  return s;
}
static SoftmaxScale softmax_scale(double v) {
  SoftmaxScale s;
  s.host = (float)v;
  s.given = true;
  return s;
}

at::Tensor softmax_fp8_common(const at::Tensor& input, int64_t dim, const SoftmaxScale& in_s, const SoftmaxScale& out_s,
                              const SoftmaxScale& heads, const OptTensor& fused_add) {
  const auto dt = input.scalar_type();
  TORCH_CHECK(dt == at::kBFloat16 || dt == at::kFloat8_e4m3fn,
              "Input tensor must be of torch.bfloat16 or torch.float8_e4m3fn dtype.");
  TORCH_CHECK(in_s.given == out_s.given, "Output and input scales must be both given or None");
  TORCH_CHECK(dt != at::kFloat8_e4m3fn || in_s.given, "If Input is of torch.float8_e4m3fn dtype then input scale must be given.");
  const int64_t rank = input.dim();
  TORCH_CHECK(rank >= 1 && rank <= 8, "softmax_fp8: input rank must be 1..8");
  dim = at::maybe_wrap_dim(dim, rank, /*wrap_scalar=*/true);
  if (dim != rank - 1) {
    // the row kernel reduces over the last dimension: move `dim` there, run, move it back (the
    // reference passes any dim to its kernel, softmax_fp8_gen.cpp:65-160); fused_add's layout
    // rules are stated for the last dimension only
    TORCH_CHECK(!(fused_add.has_value() && fused_add->defined()), "softmax_fp8: fused_add needs dim = -1");
    at::Tensor moved = input.transpose(dim, rank - 1).contiguous();
    return softmax_fp8_common(moved, rank - 1, in_s, out_s, heads, fused_add).transpose(dim, rank - 1).contiguous();
  }
  c10::cuda::CUDAGuard guard(input.device());
  at::Tensor in = input.contiguous();
  const bool fp8_out = in_s.given;
  at::Tensor out = at::empty(in.sizes(), in.options().dtype(fp8_out ? at::kFloat8_e4m3fn : at::kBFloat16));
  at::Tensor fa;
  std::vector<int64_t> lead(in.sizes().begin(), in.sizes().end() - 1), fa_strides(lead.size(), 0);
  if (fused_add.has_value() && fused_add->defined()) {
    TORCH_CHECK(in_s.given, "FusedAdd available only for Float8 output, but input scale is not given.");
    TORCH_CHECK(fused_add->scalar_type() == at::kBFloat16, "Input fused_add must be of dtype: ", at::kBFloat16);
    TORCH_CHECK(fused_add->dim() == rank, "FusedAdd tensor must have the same rank as the input tensor");
    TORCH_CHECK(fused_add->size(0) == in.size(0) && fused_add->size(rank - 1) == in.size(rank - 1),
                "FusedAdd tensor must have the same first and last dim as the input tensor");
    for (int64_t d = 1; d < rank - 1; ++d)
      TORCH_CHECK(fused_add->size(d) == 1 || fused_add->size(d) == in.size(d),
                  "FusedAdd tensor's dim other than first and last should be equal to 1 or the same as the input tensor");
    fa = fused_add->contiguous();
    for (int64_t d = 0; d < rank - 1; ++d) fa_strides[d] = fa.size(d) == 1 && in.size(d) != 1 ? 0 : fa.stride(d);
  }
  const int64_t cols = rank ? in.size(rank - 1) : 1;
  const int64_t rows = cols ? in.numel() / cols : 0;
  float pre = 1.f;
  if (in_s.given && !in_s.dev) pre *= in_s.host;
  if (heads.given && !heads.dev) pre *= heads.host;
  check_status(b200q_softmax_fp8(in.data_ptr(), to_b200q_dtype(dt), out.data_ptr(), fp8_out, rows, cols, pre, in_s.dev, heads.dev,
                                 out_s.dev, out_s.given ? out_s.host : 1.f, fa.defined() ? fa.data_ptr() : nullptr,
                                 (int)lead.size(), lead.data(), fa_strides.data(), current_stream()),
               "softmax_fp8");
  return out;
}
at::Tensor softmax_fp8(const at::Tensor& input, int64_t dim, const OptTensor& input_scale, const OptTensor& output_scale,
                       const OptTensor& inv_attn_heads, const OptTensor& fused_add) {
  return softmax_fp8_common(input, dim, softmax_scale(input_scale, input), softmax_scale(output_scale, input),
                            softmax_scale(inv_attn_heads, input), fused_add);
}
at::Tensor softmax_fp8_scalar_scales(const at::Tensor& input, int64_t dim, double input_scale, double output_scale,
                                     const OptTensor& inv_attn_heads, const OptTensor& fused_add) {
  return softmax_fp8_common(input, dim, softmax_scale(input_scale), softmax_scale(output_scale),
                            softmax_scale(inv_attn_heads, input), fused_add);
}
at::Tensor softmax_fp8_scalar(const at::Tensor& input, int64_t dim, double input_scale, double output_scale,
                              double inv_attn_heads, const OptTensor& fused_add) {
  return softmax_fp8_common(input, dim, softmax_scale(input_scale), softmax_scale(output_scale), softmax_scale(inv_attn_heads),
                            fused_add);
}

// ---- sum_fp8 (hpu_ops/backend/fp8_ops_gen.cpp:20-49; schema scripts/hpu_op.yaml:7448-7449) ----
at::Tensor sum_fp8(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> out_dtype) {
  TORCH_CHECK(is_fp8(self.scalar_type()), "sum_fp8: input must be float8_e5m2 or float8_e4m3fn");
  const at::ScalarType odt = out_dtype.value_or(self.scalar_type());
  TORCH_CHECK(is_fp8(odt) || odt == at::kFloat || odt == at::kBFloat16, "sum_fp8: unsupported out_dtype ", odt);
  c10::cuda::CUDAGuard guard(self.device());
  const int64_t rank = self.dim();
  std::vector<bool> red(rank, false);
  if (!dim.has_value() || dim->empty()) {
    std::fill(red.begin(), red.end(), true);
  } else {
    for (int64_t d : *dim) red[at::maybe_wrap_dim(d, rank)] = true;
  }
  // kept dims first, reduced dims last: [outer][reduce][1]; when the reduced dims already are a
  // leading / trailing / middle block of the contiguous tensor no copy is made
  std::vector<int64_t> kept, reduced, out_shape;
  for (int64_t d = 0; d < rank; ++d) {
    (red[d] ? reduced : kept).push_back(d);
    if (!red[d]) out_shape.push_back(self.size(d));
    else if (keepdim) out_shape.push_back(1);
  }
  int64_t outer = 1, reduce = 1, inner = 1;
  at::Tensor src = self.contiguous();
  bool block = true;  // reduced dims contiguous in index space?
  for (size_t i = 1; i < reduced.size(); ++i) block = block && reduced[i] == reduced[i - 1] + 1;
  if (block) {
    const int64_t first = reduced.empty() ? rank : reduced.front(), last = reduced.empty() ? rank - 1 : reduced.back();
    for (int64_t d = 0; d < first; ++d) outer *= self.size(d);
    for (int64_t d : reduced) reduce *= self.size(d);
    for (int64_t d = last + 1; d < rank; ++d) inner *= self.size(d);
  } else {
    std::vector<int64_t> perm = kept;
    perm.insert(perm.end(), reduced.begin(), reduced.end());
    src = self.view(at::kByte).permute(perm).contiguous();
    for (int64_t d : kept) outer *= self.size(d);
    for (int64_t d : reduced) reduce *= self.size(d);
  }
  at::Tensor out = at::empty(out_shape, self.options().dtype(odt));
  const size_t ws_bytes = b200q_sum_fp8_workspace_bytes(outer, reduce, inner);
  at::Tensor ws = at::empty({(int64_t)((ws_bytes + 3) / 4)}, self.options().dtype(at::kFloat));
  check_status(b200q_sum_fp8(src.data_ptr(), to_b200q_dtype(self.scalar_type()), out.data_ptr(), to_b200q_dtype(odt), outer, reduce,
                             inner, ws.data_ptr(), ws_bytes, current_stream()),
               "sum_fp8");
  return out;
}

// ---- in_place_interleave_ (hpu_ops/backend/fp8_ops.cpp:498-545; kernels_register.cpp:2548) ----
at::Tensor& in_place_interleave_(at::Tensor& self) {
  TORCH_CHECK(self.dim() == 4, "Input has to be a 4D tensor.");
  TORCH_CHECK(self.size(0) % 4 == 0, "Batch size has to be a multiple of 4.");
  TORCH_CHECK(self.is_contiguous(), "in_place_interleave_: input must be contiguous");
  c10::cuda::CUDAGuard guard(self.device());
  const int64_t rows = self.size(0);
  const int64_t row_bytes = rows ? (int64_t)(self.numel() / rows) * (int64_t)self.element_size() : 0;
  check_status(b200q_in_place_interleave(self.data_ptr(), rows, row_bytes, current_stream()), "in_place_interleave_");
  return self;
}

// ---- conv2d_fp8 (hpu_ops/backend/fp8_ops.cpp:547-705; schemas scripts/hpu_op.yaml:7371-7391) ----
static std::vector<int64_t> expand2(at::IntArrayRef v, const char* name) {
  TORCH_CHECK(v.size() == 1 || v.size() == 2, "conv2d_fp8: ", name, " must have 1 or 2 elements");
  return v.size() == 1 ? std::vector<int64_t>{v[0], v[0]} : std::vector<int64_t>{v[0], v[1]};
}
static std::vector<int64_t> conv2d_out_shape(at::IntArrayRef in, at::IntArrayRef wt, const std::vector<int64_t>& stride,
                                             const std::vector<int64_t>& padding, const std::vector<int64_t>& dilation) {
  std::vector<int64_t> o{in[0], wt[0]};
  for (int i = 0; i < 2; ++i) o.push_back((in[i + 2] + 2 * padding[i] - dilation[i] * (wt[i + 2] - 1) - 1) / stride[i] + 1);
  return o;
}

// scale: absent, a one-element tensor, or a host scalar
struct ConvScale {
  OptTensor t;
  double v = 1.0;
  bool is_tensor = false;
};

at::Tensor conv2d_fp8_common(const at::Tensor& input, const at::Tensor& weight, const OptTensor& bias, at::IntArrayRef stride_,
                             at::IntArrayRef padding_, at::IntArrayRef dilation_, int64_t groups,
                             c10::optional<at::ScalarType> out_dtype_, const ConvScale& s_in, const ConvScale& s_w) {
  TORCH_CHECK(input.dim() == 4 && weight.dim() == 4, "Input and weight must be 4D tensors");
  if (bias.has_value() && bias->defined())
    TORCH_CHECK(bias->dim() == 1 && bias->size(0) == weight.size(0), "Bias must be 1D tensor with size equal to weight dim0");
  TORCH_CHECK(is_fp8(input.scalar_type()) && is_fp8(weight.scalar_type()), "conv2d_fp8: input and weight must be float8 tensors");
  for (const ConvScale* sc : {&s_in, &s_w})
    if (sc->is_tensor) TORCH_CHECK(sc->t->numel() == 1, "Multi-element scale tensors are not supported yet.");
  const auto stride = expand2(stride_, "stride"), padding = expand2(padding_, "padding"), dilation = expand2(dilation_, "dilation");
  const at::ScalarType odt = out_dtype_.value_or(at::kBFloat16);
  TORCH_CHECK(odt == at::kBFloat16 || odt == at::kFloat, "conv2d_fp8: out_dtype must be bfloat16 or float");
  const int64_t N = input.size(0), C = input.size(1), H = input.size(2), W = input.size(3);
  const int64_t Co = weight.size(0), Cg = weight.size(1), kh = weight.size(2), kw = weight.size(3);
  TORCH_CHECK(groups >= 1 && C == Cg * groups && Co % groups == 0, "conv2d_fp8: channels do not match groups");
  const auto oshape = conv2d_out_shape(input.sizes(), weight.sizes(), stride, padding, dilation);
  const int64_t Ho = oshape[2], Wo = oshape[3];
  TORCH_CHECK(Ho > 0 && Wo > 0, "conv2d_fp8: empty output");
  c10::cuda::CUDAGuard guard(input.device());
  at::Tensor in = input.contiguous(), w = weight.contiguous();
  const int64_t K = Cg * kh * kw, Kp = (K + 15) / 16 * 16, rows = N * Ho * Wo, Cog = Co / groups;
  // scales: both host scalars -> the .scalar GEMM entry; otherwise one-element tensors
  auto as_tensor = [&](const ConvScale& sc) {
    if (sc.is_tensor) return sc.t->to(in.device()).to(at::kFloat).reshape({1});
    return at::full({1}, sc.v, in.options().dtype(at::kFloat));
  };
  const bool host_scales = !s_in.is_tensor && !s_w.is_tensor;
  at::Tensor ts_in, ts_w;
  if (!host_scales) { ts_in = as_tensor(s_in); ts_w = as_tensor(s_w); }
  std::vector<at::Tensor> parts;
  // Channel groups of whole 16-byte pieces: the matrix is built from a channels-last copy of the
  // input, 16 bytes at a time, with its columns ordered (i, j, c); the weight is permuted to match.
  const bool channels_last = (C % 16) == 0 && (Cg % 16) == 0;
  at::Tensor nhwc;
  if (channels_last) {
    nhwc = at::empty({N, H, W, C}, in.options());
    check_status(b200q_nchw_to_nhwc_u8(in.data_ptr(), nhwc.data_ptr(), N, C, H, W, current_stream()), "conv2d_fp8 (channels-last copy)");
  }
  for (int64_t g = 0; g < groups && channels_last; ++g) {
    at::Tensor cols = at::empty({rows, K}, in.options());
    check_status(b200q_im2col_nhwc_fp8(nhwc.data_ptr(), cols.data_ptr(), N, C, H, W, (int)kh, (int)kw, (int)stride[0],
                                       (int)stride[1], (int)padding[0], (int)padding[1], (int)dilation[0], (int)dilation[1],
                                       g * Cg, Cg, K, current_stream()),
                 "conv2d_fp8 (im2col)");
    at::Tensor wg = w.narrow(0, g * Cog, Cog).view(at::kByte).permute({0, 2, 3, 1}).contiguous().reshape({Cog, K}).view(w.scalar_type());
    OptTensor bg;
    if (bias.has_value() && bias->defined()) bg = bias->narrow(0, g * Cog, Cog).to(odt);
    parts.push_back(host_scales ? fp8_gemm_v2_scalar(cols, false, wg, true, c10::nullopt, odt, s_in.v, s_w.v, bg, false, c10::nullopt)
                                : fp8_gemm_v2(cols, false, wg, true, c10::nullopt, odt, ts_in, ts_w, bg, false, c10::nullopt));
  }
  for (int64_t g = 0; g < groups && !channels_last; ++g) {
    at::Tensor cols = at::empty({rows, Kp}, in.options());
    check_status(b200q_im2col_fp8(in.data_ptr(), cols.data_ptr(), N, C, H, W, (int)kh, (int)kw, (int)stride[0], (int)stride[1],
                                  (int)padding[0], (int)padding[1], (int)dilation[0], (int)dilation[1], g * Cg, Cg, Kp,
                                  current_stream()),
                 "conv2d_fp8 (im2col)");
    at::Tensor wg = w.narrow(0, g * Cog, Cog).reshape({Cog, K});
    if (Kp != K) {
      at::Tensor wp = at::zeros({Cog, Kp}, w.options().dtype(at::kByte));
      wp.narrow(1, 0, K).copy_(wg.view(at::kByte));
      wg = wp.view(w.scalar_type());
    }
    OptTensor bg;
    if (bias.has_value() && bias->defined()) bg = bias->narrow(0, g * Cog, Cog).to(odt);
    at::Tensor o2 = host_scales ? fp8_gemm_v2_scalar(cols, false, wg, true, c10::nullopt, odt, s_in.v, s_w.v, bg, false, c10::nullopt)
                                : fp8_gemm_v2(cols, false, wg, true, c10::nullopt, odt, ts_in, ts_w, bg, false, c10::nullopt);
    parts.push_back(o2);
  }
  at::Tensor out2d = groups == 1 ? parts[0] : at::cat(parts, 1);
  // [N*Ho*Wo, Co] is the channels-last image: return it as an NCHW-shaped view
  return out2d.view({N, Ho, Wo, Co}).permute({0, 3, 1, 2});
}
at::Tensor conv2d_fp8(const at::Tensor& input, const at::Tensor& weight, const OptTensor& bias, at::IntArrayRef stride,
                      at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups, c10::optional<at::ScalarType> out_dtype,
                      const OptTensor& scale_input, const OptTensor& scale_weight) {
  ConvScale a, b;
  if (scale_input.has_value() && scale_input->defined()) { a.t = scale_input; a.is_tensor = true; }
  if (scale_weight.has_value() && scale_weight->defined()) { b.t = scale_weight; b.is_tensor = true; }
  return conv2d_fp8_common(input, weight, bias, stride, padding, dilation, groups, out_dtype, a, b);
}
at::Tensor conv2d_fp8_scalar(const at::Tensor& input, const at::Tensor& weight, const OptTensor& bias, at::IntArrayRef stride,
                             at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups,
                             c10::optional<at::ScalarType> out_dtype, double scale_input, double scale_weight) {
  ConvScale a, b;
  a.v = scale_input;
  b.v = scale_weight;
  return conv2d_fp8_common(input, weight, bias, stride, padding, dilation, groups, out_dtype, a, b);
}

// ---- FP8 scale management (lazy_optimizer_kernels.cpp:113-126) ----
static float fp8_max_of(at::ScalarType dtype) {
  TORCH_CHECK(is_fp8(dtype), "fp8 dtype must be float8_e5m2 or float8_e4m3fn, got ", dtype);
  return dtype == at::kFloat8_e4m3fn ? 448.f : 57344.f;
}

at::Tensor amax_op(const at::Tensor& input) {
  TORCH_CHECK(input.scalar_type() == at::kFloat || input.scalar_type() == at::kBFloat16, "amax: input must be float or bfloat16");
  c10::cuda::CUDAGuard guard(input.device());
  at::Tensor in = input.contiguous();
  at::Tensor amax = at::empty({}, in.options().dtype(at::kFloat));
  check_status(b200q_amax(in.data_ptr(), to_b200q_dtype(in.scalar_type()), in.numel(), amax.data_ptr<float>(), current_stream()), "amax");
  return amax;
}

at::Tensor& scale_from_amax_(at::Tensor& scale, const at::Tensor& amax, double fp8_max, bool pow2, int64_t margin) {
  TORCH_CHECK(scale.scalar_type() == at::kFloat && amax.scalar_type() == at::kFloat && scale.numel() == 1 && amax.numel() == 1,
              "scale_from_amax_: scale and amax must be one-element float tensors");
  c10::cuda::CUDAGuard guard(scale.device());
  check_status(b200q_scale_from_amax(amax.data_ptr<float>(), scale.data_ptr<float>(), nullptr, (float)fp8_max, pow2, (int)margin,
                                     current_stream()),
               "scale_from_amax_");
  return scale;
}

at::Tensor& amax_history_update_(at::Tensor& scale, at::Tensor& history, int64_t pos, const at::Tensor& new_amax, bool use_max,
                                 double fp8_max, bool pow2, int64_t margin) {
  TORCH_CHECK(scale.scalar_type() == at::kFloat && history.scalar_type() == at::kFloat && new_amax.scalar_type() == at::kFloat &&
                  scale.numel() == 1 && new_amax.numel() == 1 && history.dim() == 1 && history.is_contiguous(),
              "amax_history_update_: float tensors, one-element scale / new_amax, contiguous 1-D history");
  TORCH_CHECK(pos >= 0 && pos < history.numel(), "amax_history_update_: pos out of range");
  c10::cuda::CUDAGuard guard(scale.device());
  check_status(b200q_amax_history_update(history.data_ptr<float>(), (int)history.numel(), (int)pos, new_amax.data_ptr<float>(),
                                         use_max, scale.data_ptr<float>(), nullptr, (float)fp8_max, pow2, (int)margin,
                                         current_stream()),
               "amax_history_update_");
  return scale;
}

// CastMomentToFp8WithScale: amax -> power-of-two scale (kept when amax == 0) -> stochastic cast
// with that scale; three launches on the current stream, nothing read back to the host.
at::Tensor cast_moment_to_fp8(const at::Tensor& moment, at::Tensor& scale, at::ScalarType dtype) {
  const float fmax = fp8_max_of(dtype);
  at::Tensor amax = amax_op(moment);
  scale_from_amax_(scale, amax, fmax, true, 0);
  const std::vector<int64_t> one{1};
  auto r = cast_to_fp8_v2(moment, scale, true, false, dtype, at::IntArrayRef(one));
  return std::get<0>(r);
}

void set_sr_seed(int64_t seed) {
  g_sr_seed.store(seed);
  g_sr_offset.store(0);
}
void set_cast_mul_in_fp32(bool on) { g_mul_in_fp32.store(on); }
int64_t launch_count() { return (int64_t)b200q_launch_count(); }
int64_t device_status() {
  int code = 0;
  int rc = b200q_device_status(&code);
  TORCH_CHECK(rc == B200Q_OK || rc == B200Q_ERR_DEVICE_TIMEOUT, "device_status: ", b200q_strerror(rc), " ",
              b200q_last_cuda_error());
  return code;
}

// ------------------------------------------------------------------ Meta
// python_packages/habana_frameworks/torch/dynamo/_custom_op_meta_registrations.py:56-217
std::tuple<at::Tensor, at::Tensor> meta_cast_to(const at::Tensor& input, bool is_amax, at::ScalarType dtype) {
  at::Tensor out = at::empty(input.sizes(), input.options().dtype(dtype));
  at::Tensor amax = is_amax ? at::empty({}, input.options().dtype(at::kFloat)) : at::empty({0}, input.options().dtype(at::kFloat));
  return {out, amax};
}
std::tuple<at::Tensor, at::Tensor> meta_cast_to_fp8_v2(const at::Tensor& i, const OptTensor&, bool, bool a,
                                                       at::ScalarType d, OptShape) { return meta_cast_to(i, a, d); }
std::tuple<at::Tensor, at::Tensor> meta_cast_to_fp8_v2_scalar(const at::Tensor& i, double, bool, bool a,
                                                              at::ScalarType d, OptShape) { return meta_cast_to(i, a, d); }
std::tuple<at::Tensor, at::Tensor> meta_cast_to_fp8_v2_list(const at::Tensor& i, c10::ArrayRef<double>, bool, bool a,
                                                            at::ScalarType d, OptShape) { return meta_cast_to(i, a, d); }
std::tuple<at::Tensor, at::Tensor, at::Tensor> meta_cast_to_fp8_hybrid(const at::Tensor& i, const OptTensor&, const OptTensor&,
                                                                       bool, bool is_amax) {
  return {at::empty(i.sizes(), i.options().dtype(at::kFloat8_e5m2)), at::empty(i.sizes(), i.options().dtype(at::kFloat8_e4m3fn)),
          is_amax ? at::empty({}, i.options().dtype(at::kFloat)) : at::empty({0}, i.options().dtype(at::kFloat))};
}
at::Tensor meta_cast_from(const at::Tensor& i, at::ScalarType d) { return at::empty(i.sizes(), i.options().dtype(d)); }
at::Tensor meta_cast_from_fp8(const at::Tensor& i, const OptTensor&, at::ScalarType d, OptShape) { return meta_cast_from(i, d); }
at::Tensor meta_cast_from_fp8_scalar(const at::Tensor& i, double, at::ScalarType d, OptShape) { return meta_cast_from(i, d); }
at::Tensor meta_cast_from_fp8_list(const at::Tensor& i, c10::ArrayRef<double>, at::ScalarType d, OptShape) { return meta_cast_from(i, d); }
at::Tensor meta_convert_from_4bit(const at::Tensor& i, const at::Tensor&, const OptTensor&, at::ScalarType d) {
  auto s = i.sizes().vec();
  s.back() *= 8;
  return at::empty(s, i.options().dtype(d));
}
at::Tensor meta_gemm(const at::Tensor& A, bool ta, const at::Tensor& B, bool tb, at::ScalarType d) {
  return at::empty(matmul_out_shape(A.sizes(), B.sizes(), ta, tb), A.options().dtype(d));
}
at::Tensor meta_fp8_gemm_v2(const at::Tensor& A, bool ta, const at::Tensor& B, bool tb, const OptTensor&,
                            at::ScalarType d, const OptTensor&, const OptTensor&, const OptTensor&, bool, OptShape) {
  return meta_gemm(A, ta, B, tb, d);
}
at::Tensor meta_fp8_gemm_v2_scalar(const at::Tensor& A, bool ta, const at::Tensor& B, bool tb, const OptTensor&,
                                   at::ScalarType d, double, double, const OptTensor&, bool, OptShape) {
  return meta_gemm(A, ta, B, tb, d);
}
at::Tensor meta_fp8_gemm_v2_list(const at::Tensor& A, bool ta, const at::Tensor& B, bool tb, const OptTensor&,
                                 at::ScalarType d, c10::ArrayRef<double>, c10::ArrayRef<double>, const OptTensor&, bool,
                                 OptShape) {
  return meta_gemm(A, ta, B, tb, d);
}

}  // namespace

TORCH_LIBRARY(hpu, m) {
  m.def("cast_to_fp8(Tensor input, Tensor? scale, bool stochastic_rounding, Tensor(a!) out, Tensor(b!) amax) -> (Tensor(a!), Tensor(b!))");
  m.def("cast_to_fp8_v2(Tensor input, Tensor? scale=None, bool stochastic_rounding=False, bool is_amax=False, ScalarType dtype=None, int[]? scale_shape=None) -> (Tensor, Tensor)");
  m.def("cast_to_fp8_v2.scalar(Tensor input, float scale, bool stochastic_rounding=False, bool is_amax=False, ScalarType dtype=None, int[]? scale_shape=None) -> (Tensor, Tensor)");
  m.def("cast_to_fp8_v2.scalar_list(Tensor input, float[] scale, bool stochastic_rounding=False, bool is_amax=False, ScalarType dtype=None, int[]? scale_shape=None) -> (Tensor, Tensor)");
  m.def("cast_to_fp8_hybrid(Tensor input, Tensor? scale_152=None, Tensor? scale_143=None, bool stochastic_rounding=False, bool is_amax=False) -> (Tensor, Tensor, Tensor)");
  m.def("convert_from_int4(Tensor input, Tensor scale, Tensor? zero_point, ScalarType out_dtype) -> Tensor");
  m.def("convert_from_uint4(Tensor input, Tensor scale, Tensor? zero_point, ScalarType out_dtype) -> Tensor");
  m.def("cast_from_fp8(Tensor input, Tensor? scale, ScalarType out_dtype, int[]? scale_shape=None) -> Tensor");
  m.def("cast_from_fp8.scalar(Tensor input, float scale, ScalarType out_dtype, int[]? scale_shape=None) -> Tensor");
  m.def("cast_from_fp8.scalar_list(Tensor input, float[] scale, ScalarType out_dtype, int[]? scale_shape=None) -> Tensor");
  m.def("fp8_gemm(Tensor A, bool trans_A, Tensor B, bool trans_B, Tensor D, ScalarType out_dtype, Tensor? A_scale_inv, Tensor? B_scale_inv, Tensor? bias, bool accumulate, Tensor(a!) out) -> Tensor(a!)");
  m.def("fp8_gemm_v2(Tensor A, bool trans_A, Tensor B, bool trans_B, Tensor? D, ScalarType out_dtype, Tensor? A_scale_inv=None, Tensor? B_scale_inv=None, Tensor? bias=None, bool accumulate=False, int[]? B_scale_shape=None) -> Tensor");
  m.def("fp8_gemm_v2.scalar(Tensor A, bool trans_A, Tensor B, bool trans_B, Tensor? D, ScalarType out_dtype, float A_scale_inv, float B_scale_inv, Tensor? bias=None, bool accumulate=False, int[]? B_scale_shape=None) -> Tensor");
  m.def("conv2d_fp8(Tensor input, Tensor weight, Tensor? bias=None, SymInt[2] stride=1, SymInt[2] padding=0, SymInt[2] dilation=1, int groups=1, ScalarType? out_dtype=None, Tensor? scale_input=None, Tensor? scale_weight=None) -> Tensor");
  m.def("conv2d_fp8.scalar(Tensor input, Tensor weight, Tensor? bias=None, SymInt[2] stride=1, SymInt[2] padding=0, SymInt[2] dilation=1, int groups=1, ScalarType? out_dtype=None, float scale_input=1.0, float scale_weight=1.0) -> Tensor");
  m.def("softmax_fp8(Tensor input, int dim, Tensor? input_scale=None, Tensor? output_scale=None, Tensor? inv_attn_heads=None, Tensor? fused_add=None) -> Tensor");
  m.def("softmax_fp8.Scalar_scales(Tensor input, int dim, float input_scale, float output_scale, Tensor? inv_attn_heads=None, Tensor? fused_add=None) -> Tensor");
  m.def("softmax_fp8.Scalar(Tensor input, int dim, float input_scale, float output_scale, float inv_attn_heads, Tensor? fused_add=None) -> Tensor");
  m.def("sum_fp8(Tensor self, int[1]? dim=None, bool keepdim=False, ScalarType? out_dtype=None) -> Tensor");
  m.def("in_place_interleave_(Tensor(a!) self) -> (Tensor(a!))");
  m.def("fp8_sdpa_recomp_fwd(Tensor q, Tensor k, Tensor v, Tensor? attention_mask, float p, float scale, bool is_causal, bool requires_backward, str softmax_mode, Tensor? d_scale_q, Tensor? d_scale_k, Tensor? d_scale_v, Tensor? q_scale_s, Tensor? q_scale_o, Tensor? d_scale_s, bool is_amax_s, bool is_amax_0, Tensor? valid_seq_len, str seq_padding_type ) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("fp8_sdpa_recomp_fwd.scalar(Tensor q, Tensor k, Tensor v, Tensor? attention_mask, float p, float scale, bool is_causal, bool requires_backward, str softmax_mode, float d_scale_q, float d_scale_k, float d_scale_v, float q_scale_s, float q_scale_o, float d_scale_s, bool is_amax_s, bool is_amax_0, Tensor? valid_seq_len, str seq_padding_type ) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("fp8_gemm_v2.scalar_list(Tensor A, bool trans_A, Tensor B, bool trans_B, Tensor? D, ScalarType out_dtype, float[] A_scale_inv, float[] B_scale_inv, Tensor? bias=None, bool accumulate=False, int[]? B_scale_shape=None) -> Tensor");
}

TORCH_LIBRARY_IMPL(hpu, CUDA, m) {
  m.impl("cast_to_fp8", cast_to_fp8);
  m.impl("cast_to_fp8_hybrid", cast_to_fp8_hybrid);
  m.impl("cast_to_fp8_v2", cast_to_fp8_v2);
  m.impl("cast_to_fp8_v2.scalar", cast_to_fp8_v2_scalar);
  m.impl("cast_to_fp8_v2.scalar_list", cast_to_fp8_v2_scalar_list);
  m.impl("convert_from_int4", convert_from_int4);
  m.impl("convert_from_uint4", convert_from_uint4);
  m.impl("cast_from_fp8", cast_from_fp8);
  m.impl("cast_from_fp8.scalar", cast_from_fp8_scalar);
  m.impl("cast_from_fp8.scalar_list", cast_from_fp8_scalar_list);
  m.impl("conv2d_fp8", conv2d_fp8);
  m.impl("conv2d_fp8.scalar", conv2d_fp8_scalar);
  m.impl("softmax_fp8", softmax_fp8);
  m.impl("softmax_fp8.Scalar_scales", softmax_fp8_scalar_scales);
  m.impl("softmax_fp8.Scalar", softmax_fp8_scalar);
  m.impl("sum_fp8", sum_fp8);
  m.impl("in_place_interleave_", in_place_interleave_);
  m.impl("fp8_sdpa_recomp_fwd", fp8_sdpa_recomp_fwd);
  m.impl("fp8_sdpa_recomp_fwd.scalar", fp8_sdpa_recomp_fwd_scalar);
  m.impl("fp8_gemm", fp8_gemm);
  m.impl("fp8_gemm_v2", fp8_gemm_v2);
  m.impl("fp8_gemm_v2.scalar", fp8_gemm_v2_scalar);
  m.impl("fp8_gemm_v2.scalar_list", fp8_gemm_v2_scalar_list);
}

// softmax_fp8_gen.cpp:65-72 (SoftmaxFp8Meta), fp8_ops_gen.cpp:20-34 (SumFp8Meta)
at::Tensor meta_softmax_fp8(const at::Tensor& input, int64_t, const OptTensor& input_scale, const OptTensor&, const OptTensor&,
                            const OptTensor&) {
  const bool scaled = input_scale.has_value() && input_scale->defined();
  return at::empty(input.sizes(), input.options().dtype(scaled ? at::kFloat8_e4m3fn : at::kBFloat16));
}
at::Tensor meta_softmax_fp8_scalar_scales(const at::Tensor& input, int64_t, double, double, const OptTensor&, const OptTensor&) {
  return at::empty(input.sizes(), input.options().dtype(at::kFloat8_e4m3fn));
}
at::Tensor meta_softmax_fp8_scalar(const at::Tensor& input, int64_t, double, double, double, const OptTensor&) {
  return at::empty(input.sizes(), input.options().dtype(at::kFloat8_e4m3fn));
}
at::Tensor meta_sum_fp8(const at::Tensor& self, at::OptionalIntArrayRef dim, bool keepdim, c10::optional<at::ScalarType> out_dtype) {
  const int64_t rank = self.dim();
  std::vector<bool> red(rank, !dim.has_value() || dim->empty());
  if (dim.has_value())
    for (int64_t d : *dim) red[at::maybe_wrap_dim(d, rank)] = true;
  std::vector<int64_t> shape;
  for (int64_t d = 0; d < rank; ++d) {
    if (!red[d]) shape.push_back(self.size(d));
    else if (keepdim) shape.push_back(1);
  }
  return at::empty(shape, self.options().dtype(out_dtype.value_or(self.scalar_type())));
}
at::Tensor& meta_in_place_interleave_(at::Tensor& self) { return self; }
// fp8_ops.cpp:594-612 (Conv2dFp8Meta)
at::Tensor meta_conv2d_fp8(const at::Tensor& input, const at::Tensor& weight, const OptTensor&, at::IntArrayRef stride,
                           at::IntArrayRef padding, at::IntArrayRef dilation, int64_t, c10::optional<at::ScalarType> out_dtype,
                           const OptTensor&, const OptTensor&) {
  TORCH_CHECK(input.dim() == 4 && weight.dim() == 4, "Input and weight must be 4D tensors");
  return at::empty(conv2d_out_shape(input.sizes(), weight.sizes(), expand2(stride, "stride"), expand2(padding, "padding"),
                                    expand2(dilation, "dilation")),
                   input.options().dtype(out_dtype.value_or(at::kBFloat16)));
}
at::Tensor meta_conv2d_fp8_scalar(const at::Tensor& input, const at::Tensor& weight, const OptTensor& b, at::IntArrayRef stride,
                                  at::IntArrayRef padding, at::IntArrayRef dilation, int64_t g,
                                  c10::optional<at::ScalarType> out_dtype, double, double) {
  return meta_conv2d_fp8(input, weight, b, stride, padding, dilation, g, out_dtype, c10::nullopt, c10::nullopt);
}

TORCH_LIBRARY_IMPL(hpu, Meta, m) {
  m.impl("conv2d_fp8", meta_conv2d_fp8);
  m.impl("conv2d_fp8.scalar", meta_conv2d_fp8_scalar);
  m.impl("softmax_fp8", meta_softmax_fp8);
  m.impl("softmax_fp8.Scalar_scales", meta_softmax_fp8_scalar_scales);
  m.impl("softmax_fp8.Scalar", meta_softmax_fp8_scalar);
  m.impl("sum_fp8", meta_sum_fp8);
  m.impl("in_place_interleave_", meta_in_place_interleave_);
  m.impl("fp8_sdpa_recomp_fwd", meta_fp8_sdpa_recomp_fwd);
  m.impl("fp8_sdpa_recomp_fwd.scalar", meta_fp8_sdpa_recomp_fwd_scalar);
  m.impl("cast_to_fp8_hybrid", meta_cast_to_fp8_hybrid);
  m.impl("cast_to_fp8_v2", meta_cast_to_fp8_v2);
  m.impl("cast_to_fp8_v2.scalar", meta_cast_to_fp8_v2_scalar);
  m.impl("cast_to_fp8_v2.scalar_list", meta_cast_to_fp8_v2_list);
  m.impl("convert_from_int4", meta_convert_from_4bit);
  m.impl("convert_from_uint4", meta_convert_from_4bit);
  m.impl("cast_from_fp8", meta_cast_from_fp8);
  m.impl("cast_from_fp8.scalar", meta_cast_from_fp8_scalar);
  m.impl("cast_from_fp8.scalar_list", meta_cast_from_fp8_list);
  m.impl("fp8_gemm_v2", meta_fp8_gemm_v2);
  m.impl("fp8_gemm_v2.scalar", meta_fp8_gemm_v2_scalar);
  m.impl("fp8_gemm_v2.scalar_list", meta_fp8_gemm_v2_list);
}

TORCH_LIBRARY(b200q, m) {
  m.def("w4a16_gemm(Tensor x, Tensor qweight, Tensor scales, Tensor? qzeros, int group_size, bool k_packed, ScalarType out_dtype) -> Tensor");
  m.def("dequant_kpacked(Tensor qweight, Tensor scales, Tensor? qzeros, ScalarType out_dtype) -> Tensor");
  m.def("gptq_repack(Tensor qweight, Tensor? qzeros) -> (Tensor, Tensor)");
  m.def("fp8_gemm_cast(Tensor A, bool trans_A, Tensor B, bool trans_B, Tensor? D, ScalarType mid_dtype, Tensor? A_scale_inv, Tensor? B_scale_inv, Tensor? bias, bool accumulate, int[]? B_scale_shape, float out_scale, ScalarType out_dtype) -> Tensor");
  m.def("scaled_mm(Tensor a, Tensor b, Tensor scale_a, Tensor scale_b, Tensor? bias, Tensor? scale_result, ScalarType out_dtype) -> (Tensor, Tensor)");
  m.def("swiglu_cast_fp8(Tensor gate, Tensor up, float scale, bool is_amax) -> (Tensor, Tensor)");
  m.def("fp8_gemm_swiglu_cast(Tensor x8, Tensor w_gate_up, Tensor? x_scale_inv, Tensor? w_scale_inv, float act_scale) -> Tensor");
  m.def("amax(Tensor input) -> Tensor");
  m.def("scale_from_amax_(Tensor(a!) scale, Tensor amax, float fp8_max, bool pow2=True, int margin=0) -> Tensor(a!)");
  m.def("amax_history_update_(Tensor(a!) scale, Tensor(b!) history, int pos, Tensor new_amax, bool use_max, float fp8_max, bool pow2=True, int margin=0) -> Tensor(a!)");
  m.def("cast_moment_to_fp8(Tensor moment, Tensor(a!) scale, ScalarType dtype) -> Tensor");
  m.def("set_sr_seed(int seed) -> ()", set_sr_seed);
  m.def("set_cast_mul_in_fp32(bool on) -> ()", set_cast_mul_in_fp32);
  m.def("launch_count() -> int", launch_count);
  m.def("device_status() -> int", device_status);
}

TORCH_LIBRARY_IMPL(b200q, CUDA, m) {
  m.impl("w4a16_gemm", w4a16_gemm);
  m.impl("dequant_kpacked", dequant_kpacked);
  m.impl("gptq_repack", gptq_repack);
  m.impl("fp8_gemm_cast", fp8_gemm_cast);
  m.impl("scaled_mm", scaled_mm);
  m.impl("swiglu_cast_fp8", swiglu_cast_fp8);
  m.impl("fp8_gemm_swiglu_cast", fp8_gemm_swiglu_cast);
  m.impl("amax", amax_op);
  m.impl("scale_from_amax_", scale_from_amax_);
  m.impl("amax_history_update_", amax_history_update_);
  m.impl("cast_moment_to_fp8", cast_moment_to_fp8);
}
