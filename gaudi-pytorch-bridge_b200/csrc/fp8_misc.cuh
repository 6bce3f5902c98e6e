// Argument block of softmax_fp8_kernel (shared by the kernel file and the C ABI wrapper).
#pragma once

#include "common.cuh"

namespace b200q {

struct SoftmaxParams {
  const void* in;
  int in_dtype;  // B200Q_BF16 or B200Q_E4M3
  void* out;
  int out_fp8;
  int64_t rows, cols;
  float pre_scale;                // inv_attn_heads * input_scale folded on the host when both are host scalars
  const float* input_scale;       // device scalars (or null)
  const float* inv_attn_heads;
  const float* output_scale;
  float output_scale_host;
  const __nv_bfloat16* fused_add;  // or null
  int nd;                          // number of leading (row) dimensions
  int64_t size[7];                 // their sizes
  int64_t fa_stride[7];            // fused_add strides in elements (0 where it broadcasts)
};

}  // namespace b200q
