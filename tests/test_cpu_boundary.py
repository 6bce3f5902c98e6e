"""CPU-only checks of the drop-in boundary: the C-ABI library loads and exports every symbol
that include/b200q.h declares, the hpu::* schemas are registered verbatim, Meta kernels give the
reference's shapes/dtypes, and CPU tensors are refused (there is no fallback)."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT

import b200_hpu_ops
from b200_hpu_ops import abi


def test_header_symbols_are_exported():
    hdr = open(os.path.join(ROOT, "include", "b200q.h")).read()
    declared = set(re.findall(r"^(?:int|const char\*|uint64_t|size_t)\s+(b200q_[a-z0-9_]+)\s*\(", hdr, re.M))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(b200_hpu_ops.KERNEL_LIB)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in b200q.h but not exported"
    assert declared == set(abi.EXPORTS)
    assert abi.lib.b200q_strerror(0) == b"ok"
    assert b"bad argument" in abi.lib.b200q_strerror(-1)


SCHEMAS = {
    # legacy out-variants, habana_kernels/kernels_register.cpp:2427,2445
    "cast_to_fp8": "hpu::cast_to_fp8(Tensor input, Tensor? scale, bool stochastic_rounding, Tensor(a!) out, Tensor(b!) amax) -> (Tensor(a!), Tensor(b!))",
    "fp8_gemm": "hpu::fp8_gemm(Tensor A, bool trans_A, Tensor B, bool trans_B, Tensor D, ScalarType out_dtype, Tensor? A_scale_inv, Tensor? B_scale_inv, Tensor? bias, bool accumulate, Tensor(a!) out) -> Tensor(a!)",
    "cast_to_fp8_hybrid": "hpu::cast_to_fp8_hybrid(Tensor input, Tensor? scale_152=None, Tensor? scale_143=None, bool stochastic_rounding=False, bool is_amax=False) -> (Tensor, Tensor, Tensor)",
    "cast_to_fp8_v2": "hpu::cast_to_fp8_v2(Tensor input, Tensor? scale=None, bool stochastic_rounding=False, bool is_amax=False, ScalarType dtype=None, int[]? scale_shape=None) -> (Tensor, Tensor)",
    "cast_to_fp8_v2.scalar": "hpu::cast_to_fp8_v2.scalar(Tensor input, float scale, bool stochastic_rounding=False, bool is_amax=False, ScalarType dtype=None, int[]? scale_shape=None) -> (Tensor, Tensor)",
    "cast_to_fp8_v2.scalar_list": "hpu::cast_to_fp8_v2.scalar_list(Tensor input, float[] scale, bool stochastic_rounding=False, bool is_amax=False, ScalarType dtype=None, int[]? scale_shape=None) -> (Tensor, Tensor)",
    "convert_from_int4": "hpu::convert_from_int4(Tensor input, Tensor scale, Tensor? zero_point, ScalarType out_dtype) -> Tensor",
    "convert_from_uint4": "hpu::convert_from_uint4(Tensor input, Tensor scale, Tensor? zero_point, ScalarType out_dtype) -> Tensor",
    "cast_from_fp8": "hpu::cast_from_fp8(Tensor input, Tensor? scale, ScalarType out_dtype, int[]? scale_shape=None) -> Tensor",
    "cast_from_fp8.scalar": "hpu::cast_from_fp8.scalar(Tensor input, float scale, ScalarType out_dtype, int[]? scale_shape=None) -> Tensor",
    "cast_from_fp8.scalar_list": "hpu::cast_from_fp8.scalar_list(Tensor input, float[] scale, ScalarType out_dtype, int[]? scale_shape=None) -> Tensor",
    "fp8_gemm_v2": "hpu::fp8_gemm_v2(Tensor A, bool trans_A, Tensor B, bool trans_B, Tensor? D, ScalarType out_dtype, Tensor? A_scale_inv=None, Tensor? B_scale_inv=None, Tensor? bias=None, bool accumulate=False, int[]? B_scale_shape=None) -> Tensor",
    "fp8_gemm_v2.scalar": "hpu::fp8_gemm_v2.scalar(Tensor A, bool trans_A, Tensor B, bool trans_B, Tensor? D, ScalarType out_dtype, float A_scale_inv, float B_scale_inv, Tensor? bias=None, bool accumulate=False, int[]? B_scale_shape=None) -> Tensor",
    # scripts/hpu_op.yaml:7399-7418, 7448-7449; kernels_register.cpp:2548
    "conv2d_fp8": "hpu::conv2d_fp8(Tensor input, Tensor weight, Tensor? bias=None, SymInt[2] stride=[1, 1], SymInt[2] padding=[0, 0], SymInt[2] dilation=[1, 1], int groups=1, ScalarType? out_dtype=None, Tensor? scale_input=None, Tensor? scale_weight=None) -> Tensor",
    "conv2d_fp8.scalar": "hpu::conv2d_fp8.scalar(Tensor input, Tensor weight, Tensor? bias=None, SymInt[2] stride=[1, 1], SymInt[2] padding=[0, 0], SymInt[2] dilation=[1, 1], int groups=1, ScalarType? out_dtype=None, float scale_input=1., float scale_weight=1.) -> Tensor",
    "softmax_fp8": "hpu::softmax_fp8(Tensor input, int dim, Tensor? input_scale=None, Tensor? output_scale=None, Tensor? inv_attn_heads=None, Tensor? fused_add=None) -> Tensor",
    "softmax_fp8.Scalar_scales": "hpu::softmax_fp8.Scalar_scales(Tensor input, int dim, float input_scale, float output_scale, Tensor? inv_attn_heads=None, Tensor? fused_add=None) -> Tensor",
    "softmax_fp8.Scalar": "hpu::softmax_fp8.Scalar(Tensor input, int dim, float input_scale, float output_scale, float inv_attn_heads, Tensor? fused_add=None) -> Tensor",
    "sum_fp8": "hpu::sum_fp8(Tensor self, int[1]? dim=None, bool keepdim=False, ScalarType? out_dtype=None) -> Tensor",
    "in_place_interleave_": "hpu::in_place_interleave_(Tensor(a!) self) -> Tensor(a!)",
    # habana_kernels/kernels_register.cpp:2525,2533 (the reference's own spelling of is_amax_0)
    "fp8_sdpa_recomp_fwd": "hpu::fp8_sdpa_recomp_fwd(Tensor q, Tensor k, Tensor v, Tensor? attention_mask, float p, float scale, bool is_causal, bool requires_backward, str softmax_mode, Tensor? d_scale_q, Tensor? d_scale_k, Tensor? d_scale_v, Tensor? q_scale_s, Tensor? q_scale_o, Tensor? d_scale_s, bool is_amax_s, bool is_amax_0, Tensor? valid_seq_len, str seq_padding_type) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)",
    "fp8_sdpa_recomp_fwd.scalar": "hpu::fp8_sdpa_recomp_fwd.scalar(Tensor q, Tensor k, Tensor v, Tensor? attention_mask, float p, float scale, bool is_causal, bool requires_backward, str softmax_mode, float d_scale_q, float d_scale_k, float d_scale_v, float q_scale_s, float q_scale_o, float d_scale_s, bool is_amax_s, bool is_amax_0, Tensor? valid_seq_len, str seq_padding_type) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)",
    "fp8_gemm_v2.scalar_list": "hpu::fp8_gemm_v2.scalar_list(Tensor A, bool trans_A, Tensor B, bool trans_B, Tensor? D, ScalarType out_dtype, float[] A_scale_inv, float[] B_scale_inv, Tensor? bias=None, bool accumulate=False, int[]? B_scale_shape=None) -> Tensor",
}


@pytest.mark.parametrize("name", sorted(SCHEMAS))
def test_schema_strings_match_reference(name):
    # habana_kernels/kernels_register.cpp:2429-2451
    base, _, overload = name.partition(".")
    op = getattr(getattr(torch.ops.hpu, base), overload or "default")
    assert str(op._schema) == SCHEMAS[name]


def test_meta_shapes_follow_reference():
    # python_packages/habana_frameworks/torch/dynamo/_custom_op_meta_registrations.py:56-217
    x = torch.empty(6, 10, device="meta", dtype=torch.bfloat16)
    for is_amax in (False, True):
        o, a = torch.ops.hpu.cast_to_fp8_v2(x, None, False, is_amax, torch.float8_e5m2)
        assert o.shape == x.shape and o.dtype == torch.float8_e5m2
        assert a.dtype == torch.float32 and tuple(a.shape) == (() if is_amax else (0,))
    o, _ = torch.ops.hpu.cast_to_fp8_v2(x, 2.0, False, False, torch.float8_e4m3fn)
    assert o.dtype == torch.float8_e4m3fn
    o, _ = torch.ops.hpu.cast_to_fp8_v2(x, [1.0] * 10, False, False, torch.float8_e4m3fn, [1, 10])
    assert o.shape == x.shape
    r = torch.ops.hpu.cast_from_fp8(o, None, torch.bfloat16)
    assert r.dtype == torch.bfloat16 and r.shape == x.shape
    q = torch.empty(4, 6, 4, device="meta", dtype=torch.int32)
    for fn in (torch.ops.hpu.convert_from_int4, torch.ops.hpu.convert_from_uint4):
        assert tuple(fn(q, x, None, torch.float32).shape) == (4, 6, 32)
    f8 = torch.float8_e4m3fn
    cases = [((2, 1, 4, 2), (1, 3, 4, 8), True, False, (2, 3, 2, 8)), ((4, 2), (3, 4, 8), True, False, (3, 2, 8)),
             ((10,), (10,), False, False, ()), ((2, 10), (10,), False, False, (2,)),
             ((8,), (2, 4, 8, 16), False, False, (2, 4, 16)), ((4096, 4096), (14336, 4096), False, True, (4096, 14336))]
    for sa, sb, ta, tb, so in cases:
        A = torch.empty(sa, device="meta", dtype=f8)
        B = torch.empty(sb, device="meta", dtype=f8)
        assert tuple(torch.ops.hpu.fp8_gemm_v2(A, ta, B, tb, None, torch.bfloat16).shape) == so
        assert tuple(torch.ops.hpu.fp8_gemm_v2(A, ta, B, tb, None, torch.float32, 1.0, 1.0).shape) == so
    with pytest.raises(RuntimeError, match="Common dimension sizes of matmul inputs should be the same. Got 5 and 4"):
        torch.ops.hpu.fp8_gemm_v2(torch.empty(3, 5, device="meta", dtype=f8), False,
                                  torch.empty(4, 6, device="meta", dtype=f8), False, None, torch.bfloat16)
    with pytest.raises(RuntimeError, match="Batch dimension 0 of matmul inputs should be the same"):
        torch.ops.hpu.fp8_gemm_v2(torch.empty(2, 3, 5, device="meta", dtype=f8), False,
                                  torch.empty(3, 5, 6, device="meta", dtype=f8), False, None, torch.bfloat16)


def test_ctypes_mirrors_have_the_library_layout():
    """The ctypes mirrors of the argument structs are as large as the C structs the library was built
    with (a field added on one side only would shift everything behind it)."""
    import ctypes
    from b200_hpu_ops import abi
    assert abi.lib.b200q_sizeof_args(0) == ctypes.sizeof(abi.GemmArgs)
    assert abi.lib.b200q_sizeof_args(1) == ctypes.sizeof(abi.SdpaArgs)
    assert abi.lib.b200q_sizeof_args(7) == 0


def test_cpu_tensors_are_refused():
    with pytest.raises(NotImplementedError):
        torch.ops.hpu.cast_to_fp8_v2(torch.zeros(4), None, False, False, torch.float8_e4m3fn)


def test_abi_rejects_bad_arguments_without_a_gpu():
    # validation happens before any CUDA call
    assert abi.lib.b200q_cast_to_fp8(None, abi.BF16, None, abi.E4M3, None, 1.0, abi.BCAST_NONE, 4, 4, None, 0, 0, 0, 0,
                                     0, None) == -1
    assert abi.lib.b200q_cast_to_fp8(None, abi.BF16, None, abi.BF16, None, 1.0, abi.BCAST_NONE, 0, 0, None, 0, 0, 0, 0,
                                     0, None) == -1
    assert abi.lib.b200q_cast_from_fp8(None, abi.BF16, None, abi.BF16, None, 1.0, abi.BCAST_NONE, 0, 0, None) == -1
    assert abi.lib.b200q_fp8_gemm(None) == -1
    g = abi.GemmArgs()
    g.M = g.N = g.K = 4
    g.batch = 1
    g.a_dtype = g.b_dtype = abi.E4M3
    g.out_dtype = abi.BF16
    assert abi.lib.b200q_fp8_gemm(ctypes.byref(g)) == -1  # null operands
    g.a_dtype = abi.F32
    assert abi.lib.b200q_fp8_gemm(ctypes.byref(g)) == -1
    assert abi.lib.b200q_dequant_int4(None, None, None, 7, 0, abi.BF16, None, 1, 1, 1, 0, None) == -1


@pytest.mark.parametrize("K", [0, 1, 32, 63])
def test_w4a16_workspace_query_below_one_k_block(K):
    """Shapes the fused W4A16 kernel does not take (K not a multiple of its 64-deep k-block) ask for
    no workspace; the size query must not do arithmetic on them (it once divided by zero)."""
    from b200_hpu_ops import abi
    for M in (1, 4, 128, 4096):
        assert abi.lib.b200q_w4a16_workspace_bytes(M, 64, K) == 0
    assert abi.lib.b200q_w4a16_workspace_bytes(64, 8192, 8192) > 0   # split-K path
    assert abi.lib.b200q_w4a16_workspace_bytes(16, 8192, 8192) == 0  # few-token kernel: reduced inside its clusters
