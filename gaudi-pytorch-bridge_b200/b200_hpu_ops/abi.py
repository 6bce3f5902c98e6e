"""ctypes binding of the C ABI in include/b200q.h (the drop-in boundary), used by the
benchmarks and by tests that want to call the kernels without the torch dispatcher."""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libb200q.so")

F32, BF16, E4M3, E5M2 = 0, 1, 2, 3
BCAST_NONE, BCAST_SCALAR_HOST, BCAST_SCALAR_DEV, BCAST_PER_COL, BCAST_PER_ROW, BCAST_FULL = range(6)
ROUND_RNE, ROUND_STOCHASTIC = 0, 1
ZP_NONE, ZP_PACKED, ZP_FLOAT = 0, 1, 2
CAST_MUL_IN_FP32 = 1

EXPORTS = [
    "b200q_strerror", "b200q_last_cuda_error", "b200q_device_status", "b200q_selftest_wait_timeout", "b200q_launch_count", "b200q_sizeof_args",
    "b200q_cast_to_fp8", "b200q_cast_to_fp8_hybrid", "b200q_cast_from_fp8", "b200q_dequant_int4", "b200q_gptq_repack", "b200q_fp8_gemm", "b200q_tp_reduce_bcast", "b200q_fp8_sdpa_fwd",
    "b200q_w4a16_gemm", "b200q_w4a16_workspace_bytes", "b200q_w4a16_gemm_noalloc", "b200q_swiglu_cast_fp8",
    "b200q_amax", "b200q_scale_from_amax", "b200q_amax_history_update",
    "b200q_softmax_fp8", "b200q_sum_fp8_workspace_bytes", "b200q_sum_fp8", "b200q_in_place_interleave", "b200q_im2col_fp8",
    "b200q_nchw_to_nhwc_u8", "b200q_im2col_nhwc_fp8",
]

DTYPE = {torch.float32: F32, torch.bfloat16: BF16, torch.float8_e4m3fn: E4M3, torch.float8_e5m2: E5M2}


class GemmArgs(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("a_dtype", C.c_int), ("b_dtype", C.c_int),
        ("trans_a", C.c_int), ("trans_b", C.c_int),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("lda", C.c_int64), ("ldb", C.c_int64),
        ("batch", C.c_int64), ("a_batch_stride", C.c_int64), ("b_batch_stride", C.c_int64),
        ("out_batch_stride", C.c_int64),
        ("out", C.c_void_p), ("out_dtype", C.c_int), ("ldo", C.c_int64),
        ("a_scale", C.c_void_p), ("a_scale_host", C.c_float), ("a_scale_mode", C.c_int),
        ("b_scale", C.c_void_p), ("b_scale_host", C.c_float), ("b_scale_mode", C.c_int),
        ("bias", C.c_void_p), ("bias_dtype", C.c_int), ("bias_mode", C.c_int),
        ("bias_ld", C.c_int64), ("bias_batch_stride", C.c_int64),
        ("D", C.c_void_p), ("d_dtype", C.c_int), ("ldd", C.c_int64), ("d_batch_stride", C.c_int64),
        ("force_generic", C.c_int), ("stream", C.c_void_p),
        ("out8_dtype", C.c_int), ("out8_scale", C.c_void_p), ("out8_scale_host", C.c_float),
        ("swiglu", C.c_int),
        ("route_out", C.c_void_p * 8), ("route_count", C.c_int), ("route_rows", C.c_int64), ("route_row_offset", C.c_int64),
        ("out8_amax", C.c_void_p), ("b_static", C.c_int),
    ]


class SdpaArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("out_dtype", C.c_int),
        ("BH", C.c_int64), ("L", C.c_int64), ("S", C.c_int64), ("dqk", C.c_int), ("dv", C.c_int), ("kv_rep", C.c_int),
        ("mask", C.c_void_p), ("mask_kind", C.c_int), ("mask_sb", C.c_int64), ("mask_sl", C.c_int64), ("causal", C.c_int),
        ("softmax_scale", C.c_float),
        ("d_scale_q", C.c_void_p), ("d_scale_k", C.c_void_p), ("d_scale_v", C.c_void_p), ("q_scale_s", C.c_void_p),
        ("q_scale_o", C.c_void_p), ("d_scale_s", C.c_void_p),
        ("d_scale_q_host", C.c_float), ("d_scale_k_host", C.c_float), ("d_scale_v_host", C.c_float),
        ("q_scale_s_host", C.c_float), ("q_scale_o_host", C.c_float), ("d_scale_s_host", C.c_float),
        ("d_scale_s_given", C.c_int),
        ("m_out", C.c_void_p), ("linv_out", C.c_void_p), ("amax_s", C.c_void_p), ("amax_o", C.c_void_p),
        ("force_plain", C.c_int), ("stream", C.c_void_p),
    ]


def _bind():
    lib = C.CDLL(_LIB_PATH, mode=C.RTLD_GLOBAL)
    lib.b200q_strerror.restype = C.c_char_p
    lib.b200q_strerror.argtypes = [C.c_int]
    lib.b200q_last_cuda_error.restype = C.c_char_p
    lib.b200q_device_status.argtypes = [C.POINTER(C.c_int)]
    lib.b200q_launch_count.restype = C.c_uint64
    lib.b200q_sizeof_args.restype = C.c_size_t
    lib.b200q_sizeof_args.argtypes = [C.c_int]
    lib.b200q_selftest_wait_timeout.argtypes = [C.c_int, C.c_void_p]
    lib.b200q_cast_to_fp8.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_float, C.c_int,
                                      C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64,
                                      C.c_int, C.c_void_p]
    lib.b200q_cast_to_fp8_hybrid.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int,
                                             C.c_void_p, C.c_float, C.c_int, C.c_int64, C.c_void_p, C.c_int, C.c_uint64,
                                             C.c_uint64, C.c_uint64, C.c_int, C.c_void_p]
    lib.b200q_cast_from_fp8.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_float, C.c_int,
                                        C.c_int64, C.c_int64, C.c_void_p]
    lib.b200q_dequant_int4.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                       C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]
    lib.b200q_fp8_gemm.argtypes = [C.POINTER(GemmArgs)]
    lib.b200q_fp8_sdpa_fwd.argtypes = [C.POINTER(SdpaArgs)]
    lib.b200q_tp_reduce_bcast.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_void_p]
    lib.b200q_gptq_repack.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64,
                                      C.c_void_p]
    lib.b200q_w4a16_gemm.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                     C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_int64,
                                     C.c_void_p, C.c_size_t, C.c_void_p]
    lib.b200q_w4a16_gemm_noalloc.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                             C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_int64,
                                             C.c_void_p]
    lib.b200q_softmax_fp8.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_float, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.b200q_sum_fp8_workspace_bytes.restype = C.c_size_t
    lib.b200q_sum_fp8_workspace_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int64]
    lib.b200q_sum_fp8.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_size_t,
                                  C.c_void_p]
    lib.b200q_in_place_interleave.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
    lib.b200q_amax.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p]
    lib.b200q_scale_from_amax.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_void_p]
    lib.b200q_amax_history_update.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                              C.c_float, C.c_int, C.c_int, C.c_void_p]
    lib.b200q_w4a16_workspace_bytes.restype = C.c_size_t
    lib.b200q_w4a16_workspace_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int64]
    lib.b200q_swiglu_cast_fp8.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_float,
                                          C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
    return lib


lib = _bind()


class B200QError(RuntimeError):
    pass


def check(rc: int, what: str = "b200q") -> None:
    if rc != 0:
        msg = lib.b200q_strerror(rc).decode()
        if rc == -3:
            msg += " -- " + lib.b200q_last_cuda_error().decode()
        raise B200QError(f"{what}: {msg} ({rc})")


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def launch_count() -> int:
    return int(lib.b200q_launch_count())


def device_status() -> int:
    """Synchronise and return the device status word (0 = every bounded wait completed)."""
    code = C.c_int(0)
    rc = lib.b200q_device_status(C.byref(code))
    if rc not in (0, -5):
        check(rc, "b200q_device_status")
    return code.value


def cast_to_fp8(x, out_dtype, scale=None, scale_mode=None, amax=False, stochastic=False, seed=1234, offset=0,
                first_index=0, mul_in_fp32=False, rows=None, cols=None):
    """Direct C-ABI call.  scale: None | float | fp32 CUDA tensor (mode inferred: 1 element ->
    SCALAR_DEV, else `scale_mode` must be given).  Returns (out, amax or None)."""
    assert x.is_cuda and x.is_contiguous()
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    am = torch.empty((), dtype=torch.float32, device=x.device) if amax else None
    sdev, shost, mode = None, 1.0, BCAST_NONE
    if isinstance(scale, (int, float)):
        shost, mode = float(scale), BCAST_SCALAR_HOST
    elif scale is not None:
        sdev = scale
        mode = scale_mode if scale_mode is not None else BCAST_SCALAR_DEV
    if rows is None:
        rows, cols = 1, x.numel()
    check(lib.b200q_cast_to_fp8(ptr(x), DTYPE[x.dtype], ptr(out), DTYPE[out_dtype], ptr(sdev), shost, mode, rows, cols,
                                ptr(am), ROUND_STOCHASTIC if stochastic else ROUND_RNE, seed, offset, first_index,
                                CAST_MUL_IN_FP32 if mul_in_fp32 else 0, stream_ptr()), "b200q_cast_to_fp8")
    return out, am


def cast_from_fp8(x8, out_dtype, scale=None, scale_mode=None, rows=None, cols=None):
    assert x8.is_cuda and x8.is_contiguous()
    out = torch.empty(x8.shape, dtype=out_dtype, device=x8.device)
    sdev, shost, mode = None, 1.0, BCAST_NONE
    if isinstance(scale, (int, float)):
        shost, mode = float(scale), BCAST_SCALAR_HOST
    elif scale is not None:
        sdev = scale
        mode = scale_mode if scale_mode is not None else BCAST_SCALAR_DEV
    if rows is None:
        rows, cols = 1, x8.numel()
    check(lib.b200q_cast_from_fp8(ptr(x8), DTYPE[x8.dtype], ptr(out), DTYPE[out_dtype], ptr(sdev), shost, mode, rows,
                                  cols, stream_ptr()), "b200q_cast_from_fp8")
    return out


def fp8_gemm_nt(a8, b8, out_dtype=torch.bfloat16, a_scale=None, b_scale=None, bias=None, out=None,
                force_generic=False, route=None, b_static=False):
    """out[M][N] = a8[M][K] . b8[N][K]^T with scalar (float) a_scale, per-column fp32 CUDA b_scale [N]
    (or float), optional per-column bias [N]: the projection-GEMM form, straight through the C ABI."""
    M, K = a8.shape
    N = b8.shape[0]
    g = GemmArgs()
    if route is not None:
        # (pointers, rows per block, row offset inside a block): block i = m // rows of the result
        # goes to pointers[i] (bf16 [.., N], possibly another GPU's memory); nothing is returned
        ptrs, rows, offset = route
        for i, q in enumerate(ptrs):
            g.route_out[i] = q
        g.route_count, g.route_rows, g.route_row_offset = len(ptrs), rows, offset
        g.out, g.out_dtype, g.ldo = ptrs[0], BF16, N
    elif out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a8.device)
    g.A, g.B = a8.data_ptr(), b8.data_ptr()
    g.a_dtype, g.b_dtype = DTYPE[a8.dtype], DTYPE[b8.dtype]
    g.trans_a, g.trans_b = 0, 1
    g.M, g.N, g.K, g.lda, g.ldb = M, N, K, a8.stride(0), b8.stride(0)
    g.batch = 1
    if route is None:
        g.out, g.out_dtype, g.ldo = out.data_ptr(), DTYPE[out.dtype], out.stride(0)
    for name, s in (("a", a_scale), ("b", b_scale)):
        if s is None:
            setattr(g, name + "_scale_mode", BCAST_NONE)
        elif isinstance(s, (int, float)):
            setattr(g, name + "_scale_mode", BCAST_SCALAR_HOST)
            setattr(g, name + "_scale_host", float(s))
        else:
            setattr(g, name + "_scale", s.data_ptr())
            setattr(g, name + "_scale_mode", BCAST_SCALAR_DEV if s.numel() == 1 else BCAST_PER_COL)
    if bias is not None:
        g.bias, g.bias_dtype, g.bias_mode = bias.data_ptr(), DTYPE[bias.dtype], BCAST_PER_COL
    g.force_generic = 1 if force_generic else 0
    g.b_static = 1 if b_static else 0  # the weights are not being written: see b200q_gemm_args.b_static
    g.stream = torch.cuda.current_stream().cuda_stream
    check(lib.b200q_fp8_gemm(C.byref(g)), "b200q_fp8_gemm")
    return out


def tp_reduce_bcast(stage, out_ptrs, me, rows, d):
    """b200q_tp_reduce_bcast on the current stream; out_ptrs = every rank's output buffer address."""
    arr = (C.c_void_p * len(out_ptrs))(*out_ptrs)
    check(lib.b200q_tp_reduce_bcast(ptr(stage), arr, len(out_ptrs), me, rows, d, stream_ptr()), "b200q_tp_reduce_bcast")
