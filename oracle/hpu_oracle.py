"""CPU oracle for the quantized-inference operator family (TEST INFRASTRUCTURE ONLY).

This module is a checker, not a product path: only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it.  It restates, on
the host CPU with torch float8 dtypes, the semantics that the reference fixes
for ``torch.ops.hpu.{cast_to_fp8_v2, cast_from_fp8, fp8_gemm_v2,
convert_from_int4, convert_from_uint4}``.  The reference itself holds no
arithmetic for these operators (each one only appends a node to a graph that a
closed kernel library executes), so every function below follows the argument
plumbing of the reference's C++ and the CPU emulation that the reference's own
tests compare the device against:

* ``hpu_ops/backend/fp8_ops.cpp:29-53``   scale / scale_shape validation
* ``hpu_ops/backend/fp8_ops.cpp:63-96``   scale tensor reshape, scalar and list scales
* ``hpu_ops/backend/fp8_ops.cpp:105-119`` rounding-mode choice (RNE / stochastic)
* ``hpu_ops/backend/fp8_ops.cpp:170-258`` cast_to_fp8_v2 (dtype checks, amax shape)
* ``hpu_ops/backend/fp8_ops.cpp:262-308`` cast_from_fp8
* ``hpu_ops/backend/fp8_ops.cpp:370-496`` fp8_gemm_v2 (operand order, accumulate check)
* ``hpu_ops/common/batched_matmul_output_shape.cpp:34-88`` matmul output shape rules
* ``hpu_ops/backend/int4_ops.cpp:22-56``  convert_from_{int4,uint4}
* ``tests/pytest_working/any_mode/test_hpu_fp8_ops_any_mode.py:85-87`` expected value of a
  cast: ``simulateFp8Precision(input * scale.to(dtype))`` -- the product is
  formed and rounded in the INPUT dtype before the fp8 rounding
* ``tests/pytest_working/any_mode/test_hpu_fp8_ops_any_mode.py:220-243`` saturation to +-max
* ``tests/pytest_working/any_mode/test_hpu_convert_from_int4.py:41-71,119-132`` nibble order
  (LSB first), packed / unpacked zero points

Pinning: the RNE cast is checked against golden vectors produced by the
reference's own ``tests/pytest_working/fp8_utils.py::simulateFp8Precision``
(imported from the reference tree by ``tests/golden/make_golden.py``; the
vectors are committed under ``tests/golden/``).  Stochastic-rounding bit
patterns, NaN/Inf handling and the GEMM summation order are pinned by no
reference test; for those the definitions in this file are the contract.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Union

import numpy as np
import torch

FP8_DTYPES = (torch.float8_e5m2, torch.float8_e4m3fn)
FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}
# (mantissa bits, biased fp32 exponent of the smallest normal, log2 of the subnormal quantum)
_FP8_FMT = {torch.float8_e4m3fn: (3, 127 - 6, -9), torch.float8_e5m2: (2, 127 - 14, -16)}

ScaleArg = Union[None, float, Sequence[float], torch.Tensor]


def dtype_name(dt: torch.dtype) -> str:
    """c10 spelling of a dtype as it appears in the reference's error strings."""
    return {
        torch.float8_e5m2: "Float8_e5m2",
        torch.float8_e4m3fn: "Float8_e4m3fn",
        torch.float32: "Float",
        torch.bfloat16: "BFloat16",
    }.get(dt, str(dt))


# --------------------------------------------------------------------------- scales
def validate_scale_shape(scale: ScaleArg, scale_shape) -> None:
    """fp8_ops.cpp:29-53 -- element-count check, skipped for None / float scales."""
    if scale is None or isinstance(scale, (float, int)) or scale_shape is None:
        return
    n = scale.numel() if isinstance(scale, torch.Tensor) else len(scale)
    m = 1
    for d in scale_shape:
        m *= int(d)
    if n != m:
        raise RuntimeError(
            f"Number of scale elements ({n}) is not equal to number of scale_shape elements ({m})."
        )


def resolve_scale(scale: ScaleArg, scale_shape=None) -> Optional[torch.Tensor]:
    """Return the scale as a tensor ready to broadcast, or None.

    fp8_ops.cpp:63-74: a tensor with more than one element is reshaped to
    scale_shape when the two differ.  fp8_ops.cpp:85-96: a float becomes a
    constant, a float list becomes a constant tensor of shape scale_shape.
    """
    validate_scale_shape(scale, scale_shape)
    if scale is None:
        return None
    if isinstance(scale, (float, int)):
        return torch.tensor(float(scale), dtype=torch.float32)
    if isinstance(scale, torch.Tensor):
        s = scale.detach().cpu()
        if s.numel() > 1 and scale_shape is not None and list(s.shape) != list(scale_shape):
            s = s.reshape(list(scale_shape))
        return s
    s = torch.tensor([float(v) for v in scale], dtype=torch.float32)
    if scale_shape is not None:
        s = s.reshape(list(scale_shape))
    return s


# --------------------------------------------------------------------------- Philox + SR
_PHILOX_M0 = np.uint64(0xD2511F53)
_PHILOX_M1 = np.uint64(0xCD9E8D57)
_PHILOX_W0 = 0x9E3779B9
_PHILOX_W1 = 0xBB67AE85
_U32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(counter_lo: np.ndarray, seed: int, offset: int = 0) -> np.ndarray:
    """Philox4x32-10.  counter = (c & 2^32-1, c >> 32, offset lo, offset hi), key = seed.

    counter_lo: uint64 array of 64-bit block counters.  Returns uint32 [n, 4].
    """
    c = counter_lo.astype(np.uint64)
    c0 = c & _U32
    c1 = c >> np.uint64(32)
    c2 = np.full_like(c0, np.uint64(offset & 0xFFFFFFFF))
    c3 = np.full_like(c0, np.uint64((offset >> 32) & 0xFFFFFFFF))
    k0 = seed & 0xFFFFFFFF
    k1 = (seed >> 32) & 0xFFFFFFFF
    for r in range(10):
        p0 = _PHILOX_M0 * c0
        p1 = _PHILOX_M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _U32
        hi1, lo1 = p1 >> np.uint64(32), p1 & _U32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ np.uint64(k0)), lo1, (hi0 ^ c3 ^ np.uint64(k1)), lo0
        k0 = (k0 + _PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def philox_random_bits(n: int, seed: int, offset: int, first_index: int, bits: int) -> np.ndarray:
    """`bits` (8 or 16) random bits per element, as uint64.  128-bit Philox block b = i // (128 / bits)
    serves elements i = b * (128 / bits) ...; inside the block the elements take consecutive bytes
    (bits = 8) or 16-bit halves (bits = 16) in little-endian order of the four 32-bit words."""
    per = 128 // bits
    idx = np.arange(first_index, first_index + n, dtype=np.uint64)
    blocks = idx // np.uint64(per)
    ub, inv = np.unique(blocks, return_inverse=True)
    w = philox4x32_10(ub, seed, offset).astype(np.uint64)  # [nb, 4]
    e = (idx % np.uint64(per)).astype(np.int64)
    per_word = 32 // bits
    word = w[inv, e // per_word]
    return (word >> ((e % per_word).astype(np.uint64) * np.uint64(bits))) & np.uint64((1 << bits) - 1)


def stochastic_round_to_fp8(v32: torch.Tensor, dtype: torch.dtype, seed: int, offset: int = 0,
                            first_index: int = 0, rand_bits: int = 16) -> torch.Tensor:
    """Stochastic rounding of an fp32 tensor (the scaled product) to fp8.

    |v| is rounded to one of its two fp8 neighbours; it moves away from zero with probability
    (|v| - lo) / (hi - lo), resolved to `rand_bits` random bits per element.  rand_bits is 8 when
    the product is a bf16 value (bf16 input, product formed in bf16: 8 bits resolve every bf16
    mantissa exactly in the normal range) and 16 otherwise.  Bit-level definition, with
    d = 23 - (fp8 mantissa bits), g = d - 16, Emin = exponent of the smallest normal fp8 value and
    r = the element's random bits (philox_random_bits):
        a   = min(|v|, max)                         NaN -> byte 0x7F
        sub = a < 2^Emin;   u = a + 2^Emin if sub else a        (fp32 addition)
        r_d = (r >> (8 - g)) << 16                  if rand_bits == 8 and not sub
              (r << (d - rand_bits)) + (1 << (d - rand_bits - 1))   otherwise
        bits(u) = (bits(u) + r_d) with the low d bits cleared
        result  = min(u - 2^Emin if sub else u, max), sign restored
    Values between 0 and the smallest subnormal therefore also round stochastically (the
    reference's default "SFTZ" behaviour, scripts/env_flags.yaml:753-758).
    """
    mbits, emin_biased, _ = _FP8_FMT[dtype]
    d = 23 - mbits
    g = d - 16
    mx = np.float32(FP8_MAX[dtype])
    flat = v32.detach().to(torch.float32).contiguous().reshape(-1)
    n = flat.numel()
    v = flat.numpy()
    bits = v.view(np.uint32)
    neg = (bits & np.uint32(0x80000000)) != 0
    isnan = np.isnan(v)
    a = np.minimum(np.abs(np.where(isnan, np.float32(0), v)), mx).astype(np.float32)
    min_normal = np.float32(2.0 ** (emin_biased - 127))
    sub = a < min_normal
    u = np.where(sub, (a + min_normal).astype(np.float32), a).astype(np.float32)
    r = philox_random_bits(n, seed, offset, first_index, rand_bits)
    wide = (r << np.uint64(d - rand_bits)) + np.uint64(1 << (d - rand_bits - 1))
    if rand_bits == 8:
        r_d = np.where(sub, wide, (r >> np.uint64(8 - g)) << np.uint64(16))
    else:
        r_d = wide
    ub = u.view(np.uint32).astype(np.uint64)
    ub = (ub + r_d) & ~np.uint64((1 << d) - 1)
    res = (ub & _U32).astype(np.uint32).view(np.float32)
    res = np.where(sub, (res - min_normal).astype(np.float32), res)
    res = np.minimum(res, mx).astype(np.float32)
    res = np.where(neg, -res, res).astype(np.float32)
    out8 = torch.from_numpy(res.copy()).to(dtype)  # exact: every value is representable
    if isnan.any():
        nanbyte = torch.full((n,), 0x7F, dtype=torch.uint8)
        out8 = torch.where(torch.from_numpy(isnan.copy()), nanbyte, out8.view(torch.uint8)).view(dtype)
    return out8.reshape(v32.shape)


# --------------------------------------------------------------------------- casts
def _rne_to_fp8(v32: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Saturating round-half-to-even: clamp to +-max in fp32, then convert; never inf.
    Every NaN becomes the byte 0x7F (sign and payload dropped: CPUs and GPUs do not agree on
    the sign of a NaN that went through a multiply, so the contract is the canonical NaN)."""
    mx = FP8_MAX[dtype]
    out = v32.clamp(-mx, mx).to(dtype)
    nan = torch.isnan(v32)
    if nan.any():
        out = torch.where(nan, torch.full_like(out.view(torch.uint8), 0x7F), out.view(torch.uint8)).view(dtype)
    return out


def cast_to_fp8_v2(input: torch.Tensor, scale: ScaleArg = None, stochastic_rounding: bool = False,
                   is_amax: bool = False, dtype: torch.dtype = None, scale_shape=None, *,
                   mul_in_fp32: bool = False, seed: int = 1234, offset: int = 0, first_index: int = 0):
    """(out, amax) = cast_to_fp8_v2(...)   -- fp8_ops.cpp:192-258.

    out  = fp8(input * scale), same shape as input.
    amax = max|input| of the unscaled input as a 0-dim fp32 tensor when is_amax,
           else an empty fp32 tensor of shape [0] (fp8_ops.cpp:170-178).
    The product is formed in the input dtype (scale cast to it first) unless
    mul_in_fp32 is set, in which case it is formed in fp32 with the fp32 scale.
    """
    if dtype is None:
        raise RuntimeError("cast_to_fp8_v2: dtype is required")
    x = input.detach().cpu()
    is_fp8_in = x.dtype in FP8_DTYPES
    if not (is_fp8_in or x.dtype in (torch.float32, torch.bfloat16)):
        raise RuntimeError(
            "CastToFp8V2 input dtype must be one of [float, bfloat16, float8_e5m2, float8_e4m3fn].")
    if is_fp8_in:
        if is_amax:
            raise RuntimeError("CastToFp8V2 must have no amax for float8.")
        if x.dtype != dtype:
            raise RuntimeError(
                "CastToFp8V2 input and output must have the same dtype for float8, but are "
                f"{dtype_name(x.dtype)} and {dtype_name(dtype)}")
    s = resolve_scale(scale, scale_shape)
    amax = x.float().abs().max().to(torch.float32) if (is_amax and x.numel()) else (
        torch.zeros((), dtype=torch.float32) if is_amax else torch.empty(0, dtype=torch.float32))
    if is_fp8_in:
        return x.clone(), amax
    if s is None:
        y32 = x.float()
    elif mul_in_fp32:
        y32 = x.float() * s.float()
    else:
        y32 = (x * s.to(x.dtype)).float()
    mx = FP8_MAX[dtype]
    if stochastic_rounding:
        rand_bits = 8 if (x.dtype == torch.bfloat16 and not mul_in_fp32) else 16
        out = stochastic_round_to_fp8(y32, dtype, seed, offset, first_index, rand_bits)
    else:
        out = _rne_to_fp8(y32, dtype)
    return out, amax


def cast_to_fp8_hybrid(input, scale_152=None, scale_143=None, stochastic_rounding: bool = False, is_amax: bool = False, *,
                       mul_in_fp32: bool = False, seed: int = 1234, offset: int = 0):
    """(e5m2, e4m3, amax) -- hpu_ops/backend/cast_to_fp8_hybrid_gen.cpp:39-100.  Stochastic rounding
    applies to the e5m2 output only: the reference test compares the e4m3 output with the RNE
    emulation even when stochastic rounding is on (test_hpu_fp8_ops_any_mode.py:331-338)."""
    if input.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("CastToFp8Hybrid input must be of float or bfloat16 dtype.")
    o152, amax = cast_to_fp8_v2(input, scale_152, stochastic_rounding, is_amax, torch.float8_e5m2,
                                mul_in_fp32=mul_in_fp32, seed=seed, offset=offset)
    o143, _ = cast_to_fp8_v2(input, scale_143, False, False, torch.float8_e4m3fn, mul_in_fp32=mul_in_fp32)
    return o152, o143, amax


def cast_from_fp8(input: torch.Tensor, scale: ScaleArg, out_dtype: torch.dtype, scale_shape=None):
    """out = T(input) * scale.to(T), rounded once in T  -- fp8_ops.cpp:265-308 and
    test_hpu_fp8_ops_any_mode.py:85-87."""
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("CastFromFp8 output dtype must be equal to float or bfloat16.")
    s = resolve_scale(scale, scale_shape)
    y = input.detach().cpu().to(out_dtype)
    return y if s is None else y * s.to(out_dtype)


# --------------------------------------------------------------------------- gemm
def matmul_out_shape(shape_a, shape_b, trans_a: bool, trans_b: bool):
    """batched_matmul_output_shape.cpp:34-88 (torch.matmul rules with transposes)."""
    ra, rb = len(shape_a), len(shape_b)
    out = []
    ca = cb = 0
    if rb > 1:
        out.append(shape_b[rb - 2 if trans_b else rb - 1])
        cb = rb - 1 if trans_b else rb - 2
    if ra > 1:
        out.append(shape_a[ra - 1 if trans_a else ra - 2])
        ca = ra - 2 if trans_a else ra - 1
    if shape_a[ca] != shape_b[cb]:
        raise RuntimeError(
            f"Common dimension sizes of matmul inputs should be the same. Got {shape_a[ca]} and {shape_b[cb]}")
    mr = max(ra, rb)
    for i in range(3, mr + 1):
        da = 1 if i > ra else shape_a[ra - i]
        db = 1 if i > rb else shape_b[rb - i]
        if da != db and da != 1 and db != 1:
            raise RuntimeError(
                f"Batch dimension {mr - i} of matmul inputs should be the same or at least one of them "
                f"should be equal to 1. Got {da} and {db}")
        out.append(da if da == db else da * db)
    return list(reversed(out))


def fp8_gemm_v2(A, trans_A, B, trans_B, D, out_dtype, A_scale_inv: ScaleArg = None,
                B_scale_inv: ScaleArg = None, bias=None, accumulate: bool = False, B_scale_shape=None):
    """out = (op(A) @ op(B)) * A_scale_inv * B_scale_inv [+ bias] [+ D]  -- fp8_ops.cpp:403-496.
    fp32 accumulation; scales, bias and D applied in fp32; one rounding to out_dtype."""
    if accumulate and D is None:
        raise RuntimeError(
            "Accumulation tensor must be provided at index 4 for Fp8GemmV2, when accumulate is true")
    matmul_out_shape(list(A.shape), list(B.shape), trans_A, trans_B)
    a = A.detach().cpu().float()
    b = B.detach().cpu().float()
    if trans_A and a.dim() >= 2:
        a = a.transpose(-2, -1)
    if trans_B and b.dim() >= 2:
        b = b.transpose(-2, -1)
    acc = torch.matmul(a, b)
    sa = resolve_scale(A_scale_inv, None)
    sb = resolve_scale(B_scale_inv, B_scale_shape)
    if sa is not None:
        acc = acc * sa.float()
    if sb is not None:
        acc = acc * sb.float()
    if bias is not None:
        acc = acc + bias.detach().cpu().float()
    if accumulate:
        acc = acc + D.detach().cpu().float()
    return acc.to(out_dtype)


# --------------------------------------------------------------------------- int4
def pack_nibbles(values: torch.Tensor) -> torch.Tensor:
    """Pack 4-bit values (any integer tensor, last dim a multiple of 8) into int32,
    element 8p+i of the last dim -> bits [4i, 4i+4) of word p (LSB first), the
    format of test_hpu_convert_from_int4.py:41-71."""
    v = (values.to(torch.int64) & 0xF).reshape(*values.shape[:-1], values.shape[-1] // 8, 8)
    sh = torch.arange(8, dtype=torch.int64) * 4
    w = (v << sh).sum(-1)
    w = torch.where(w >= 2 ** 31, w - 2 ** 32, w)
    return w.to(torch.int32)


def unpack_nibbles(packed: torch.Tensor, signed: bool) -> torch.Tensor:
    w = packed.detach().cpu().to(torch.int64) & 0xFFFFFFFF
    sh = torch.arange(8, dtype=torch.int64) * 4
    v = (w.unsqueeze(-1) >> sh) & 0xF
    if signed:
        v = torch.where(v > 7, v - 16, v)
    return v.reshape(*packed.shape[:-1], packed.shape[-1] * 8)


def _expand_groups(t: torch.Tensor, out_shape) -> torch.Tensor:
    """[.., K/g, N] -> [.., K, N] by repeating each row g times (grouped GPTQ scales)."""
    if list(t.shape) == list(out_shape):
        return t
    if t.dim() >= 2 and t.dim() == len(out_shape) and t.shape[-1] == out_shape[-1] \
            and out_shape[-2] % t.shape[-2] == 0 and list(t.shape[:-2]) == list(out_shape[:-2]):
        return t.repeat_interleave(out_shape[-2] // t.shape[-2], dim=-2)
    return t.expand(out_shape)


def convert_from_4bit(input, scale, zero_point, out_dtype, signed: bool):
    """out = (q - zero_point) * scale   -- int4_ops.cpp:22-56.
    Packed int32 zero points are unpacked like the input and subtracted exactly as
    integers; float zero points are subtracted in out_dtype.  Every float
    operation is rounded in out_dtype (test_hpu_convert_from_int4.py:128-132)."""
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("convert_from_int4 output dtype must be float or bfloat16.")
    q = unpack_nibbles(input, signed)
    oshape = list(q.shape)
    s = _expand_groups(scale.detach().cpu().to(out_dtype), oshape)
    if zero_point is None:
        sub = q.to(out_dtype)
    elif zero_point.dtype == torch.int32:
        zp = _expand_groups(unpack_nibbles(zero_point, signed), oshape)
        sub = (q - zp).to(out_dtype)
    else:
        zp = _expand_groups(zero_point.detach().cpu().to(out_dtype), oshape)
        sub = q.to(out_dtype) - zp
    return sub * s


def convert_from_int4(input, scale, zero_point, out_dtype):
    return convert_from_4bit(input, scale, zero_point, out_dtype, True)


def convert_from_uint4(input, scale, zero_point, out_dtype):
    return convert_from_4bit(input, scale, zero_point, out_dtype, False)


def dequant_kpacked(qweight, scales, qzeros, out_dtype=torch.bfloat16):
    """Dequantise weights packed along K (AutoGPTQ layout): qweight int32 [K/8, N], row
    8p+i of W = nibble i of qweight[p]; scales [K/g, N]; qzeros int32 [K/g, N/8]
    packed along N (or None)."""
    w = unpack_nibbles(qweight.t().contiguous(), False).t().contiguous()  # [K, N]
    K, N = w.shape
    s = _expand_groups(scales.detach().cpu().to(out_dtype), [K, N])
    if qzeros is None:
        return w.to(out_dtype) * s
    zp = _expand_groups(unpack_nibbles(qzeros, False), [K, N])
    return (w - zp).to(out_dtype) * s


def w4a16_gemm(x, qweight, scales, qzeros, out_dtype=torch.bfloat16, k_packed=False):
    """x @ W with W = convert_from_uint4(...) rounded to bf16; fp32 accumulation.
    Contract by composition (the reference fuses the two nodes in its graph compiler)."""
    if k_packed:
        w = dequant_kpacked(qweight, scales, qzeros, torch.bfloat16)
    else:
        w = convert_from_uint4(qweight, scales, qzeros, torch.bfloat16)
    return torch.matmul(x.detach().cpu().float(), w.float()).to(out_dtype)


# --------------------------------------------------------------------------- TP MLP
def fp8_swiglu_mlp(x_bf16, wg8, wu8, wd8, sg_inv, su_inv, sd_inv, x_scale, act_scale):
    """FP8 SwiGLU MLP on one device: the composition the tensor-parallel path must match.
    x_bf16 [T, d]; w*8 e4m3 [out, in]; s*_inv per-output-channel fp32; x_scale / act_scale
    per-tensor fp32 scalars."""
    x8, _ = cast_to_fp8_v2(x_bf16, x_scale, False, False, torch.float8_e4m3fn)
    xs_inv = 1.0 / float(x_scale)
    g = fp8_gemm_v2(x8, False, wg8, True, None, torch.bfloat16, xs_inv, sg_inv, None, False, [1, sg_inv.numel()])
    u = fp8_gemm_v2(x8, False, wu8, True, None, torch.bfloat16, xs_inv, su_inv, None, False, [1, su_inv.numel()])
    h = (torch.nn.functional.silu(g.float()) * u.float()).to(torch.bfloat16)
    h8, _ = cast_to_fp8_v2(h, act_scale, False, False, torch.float8_e4m3fn)
    return fp8_gemm_v2(h8, False, wd8, True, None, torch.bfloat16, 1.0 / float(act_scale), sd_inv, None, False,
                       [1, sd_inv.numel()])


# ---------------------------------------------------------------------------- softmax_fp8 / sum_fp8 / interleave
def softmax_fp8(input, dim, input_scale=None, output_scale=None, inv_attn_heads=None, fused_add=None):
    """hpu_ops/backend/softmax_fp8_gen.cpp:65-160.  ``x = input * inv_attn_heads * input_scale +
    fused_add`` in fp32, softmax over the last dimension, result rounded to bf16; with scales the
    output is ``e4m3(bf16(y * output_scale))`` (saturating), without them bf16.  The checks and
    their messages are the reference's (lines 90-125)."""
    if input.dtype not in (torch.bfloat16, torch.float8_e4m3fn):
        raise RuntimeError("Input tensor must be of torch.bfloat16 or torch.float8_e4m3fn dtype.")
    if (input_scale is None) != (output_scale is None):
        raise RuntimeError("Output and input scales must be both given or None")
    if input.dtype == torch.float8_e4m3fn and input_scale is None:
        raise RuntimeError("If Input is of torch.float8_e4m3fn dtype then input scale must be given.")
    if fused_add is not None and input_scale is None:
        raise RuntimeError("FusedAdd available only for Float8 output, but input scale is not given.")
    dim = dim % input.dim()
    if dim != input.dim() - 1 and fused_add is not None:
        raise RuntimeError("softmax_fp8: fused_add needs dim = -1")
    f32 = lambda v: torch.as_tensor(v, dtype=torch.float32).reshape(())  # noqa: E731
    pre = torch.ones((), dtype=torch.float32)
    if inv_attn_heads is not None:
        pre = pre * f32(inv_attn_heads)
    if input_scale is not None:
        pre = pre * f32(input_scale)
    x = input.float() * pre
    if fused_add is not None:
        x = x + fused_add.float()
    y = torch.softmax(x, dim).to(torch.bfloat16)
    if input_scale is None:
        return y
    z = (y.float() * f32(output_scale)).to(torch.bfloat16).float()
    return _rne_to_fp8(z, torch.float8_e4m3fn)


def sum_fp8(input, dim=None, keepdim=False, out_dtype=None):
    """hpu_ops/backend/fp8_ops_gen.cpp:20-49: sum of an fp8 tensor over ``dim`` (all dimensions when
    None), accumulated in wider precision; ``out_dtype`` None keeps the input's fp8 format
    (rounded to nearest even, saturating)."""
    if input.dtype not in FP8_MAX:
        raise RuntimeError("sum_fp8: input must be float8_e5m2 or float8_e4m3fn")
    dims = list(range(input.dim())) if dim is None or (isinstance(dim, (list, tuple)) and len(dim) == 0) else dim
    s = torch.sum(input.to(torch.float64), dims, keepdim).to(torch.float32)
    od = out_dtype or input.dtype
    return _rne_to_fp8(s, od) if od in FP8_MAX else s.to(od)


def conv2d_fp8(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, out_dtype=None, scale_input=None,
               scale_weight=None):
    """hpu_ops/backend/fp8_ops.cpp:547-705: ``conv2d(input, weight) * scale_input * scale_weight + bias``
    on fp8 operands, fp32 accumulation, result in ``out_dtype`` (bf16 when None)."""
    if input.dim() != 4 or weight.dim() != 4:
        raise RuntimeError("Input and weight must be 4D tensors")
    if bias is not None and (bias.dim() != 1 or bias.shape[0] != weight.shape[0]):
        raise RuntimeError("Bias must be 1D tensor with size equal to weight dim0")
    for sc in (scale_input, scale_weight):
        if isinstance(sc, torch.Tensor) and sc.numel() != 1:
            raise RuntimeError("Multi-element scale tensors are not supported yet.")
    od = out_dtype or torch.bfloat16
    y = torch.nn.functional.conv2d(input.to(torch.float64), weight.to(torch.float64), None, stride, padding, dilation, groups).float()
    f32 = lambda v: torch.ones((), dtype=torch.float32) if v is None else torch.as_tensor(v, dtype=torch.float32).reshape(())  # noqa: E731
    y = (y * f32(scale_input)) * f32(scale_weight)
    if bias is not None:
        y = y + bias.float().reshape(1, -1, 1, 1)
    return y.to(od)


def in_place_interleave(input):
    """hpu_ops/backend/fp8_ops.cpp:498-545 with the semantics its test pins
    (test_hpu_fp8_ops_any_mode.py:795-824): row j of the 4-D input becomes row j // 4."""
    if input.dim() != 4:
        raise RuntimeError("Input has to be a 4D tensor.")
    if input.shape[0] % 4:
        raise RuntimeError("Batch size has to be a multiple of 4.")
    return torch.index_select(input, 0, torch.arange(input.shape[0]) // 4)


# ---------------------------------------------------------------------------- FP8 scale management
def scale_from_amax(amax: torch.Tensor, prev_scale: torch.Tensor, fp8_max: float, pow2: bool = True,
                    margin: int = 0) -> torch.Tensor:
    """habana_kernels/lazy_optimizer_kernels.cpp:113-121: ``exp = floor(log2(fp8_max / amax))``,
    ``sf = pow(2, exp)``, ``scale = where(amax > 0, sf, scale)`` -- all in fp32.

    The exponent is taken exactly (``frexp`` of the fp32 quotient), where the reference evaluates
    ``log2`` in floating point: the two agree except when the quotient lies within rounding
    distance below a power of two, where a rounded ``log2`` returns the next integer.
    ``pow2=False`` gives the plain quotient divided by ``2**margin`` (current scaling without
    the power-of-two restriction)."""
    a = amax.detach().float().reshape(())
    prev = prev_scale.detach().float().reshape(())
    if not bool(a > 0):
        return prev.clone()
    q = torch.tensor(fp8_max, dtype=torch.float32) / a
    if pow2:
        if bool(torch.isinf(q)):
            return q
        _, e = torch.frexp(q)  # q = m * 2**e, m in [0.5, 1)
        return torch.ldexp(torch.tensor(1.0, dtype=torch.float32), e - 1).float()
    return torch.ldexp(q, torch.tensor(-int(margin))).float()


def cast_moment_to_fp8(moment: torch.Tensor, prev_scale: torch.Tensor, dtype: torch.dtype, seed: int, offset: int = 0):
    """CastMomentToFp8WithScale (lazy_optimizer_kernels.cpp:113-126): amax of the moment ->
    power-of-two scale (kept when the amax is 0) -> stochastic cast with that scale and
    ``scale_shape = [1]``.  Returns (fp8 tensor, new scale)."""
    amax = moment.detach().abs().max().float() if moment.numel() else torch.zeros(())
    scale = scale_from_amax(amax, prev_scale, FP8_MAX[dtype], True)
    out, _ = cast_to_fp8_v2(moment, scale.reshape(1), True, False, dtype, [1], seed=seed, offset=offset)
    return out, scale


def amax_history_update(history: torch.Tensor, pos: int, new_amax: torch.Tensor, prev_scale: torch.Tensor, use_max: bool,
                        fp8_max: float, pow2: bool = True, margin: int = 0):
    """Delayed scaling: write the new amax into the ring, reduce it (max over the ring, or the
    newest entry), derive the scale as ``scale_from_amax``.  Returns (history, scale)."""
    h = history.detach().float().clone()
    h[pos] = new_amax.detach().float().reshape(())
    a = h.abs().max() if use_max else h[pos].abs()
    return h, scale_from_amax(a, prev_scale, fp8_max, pow2, margin)


def rel_frobenius(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().cpu().double()
    b = b.detach().cpu().double()
    return float((a - b).norm() / max(b.norm(), 1e-30))


# ---------------------------------------------------------------------------- FP8 SDPA (forward)
SDPA_MASKED = -1.0e30  # what a masked-out score is set to (finite: exp gives exactly 0)


def fp8_sdpa_recomp_fwd(q, k, v, attention_mask=None, p=0.0, scale=None, is_causal=False, requires_backward=False,
                        softmax_mode="None", d_scale_q=None, d_scale_k=None, d_scale_v=None, q_scale_s=None,
                        q_scale_o=None, d_scale_s=None, is_amax_s=False, is_amax_o=False, valid_seq_len=None,
                        seq_padding_type="None"):
    """hpu::fp8_sdpa_recomp_fwd (habana_kernels/kernels_register.cpp:2525; node built in
    hpu_ops/backend/sdpa_gen.cpp:820-1000; Python caller
    python_packages/habana_frameworks/torch/hpex/kernels/Fp8FusedSDPA.py:70-160), forward only, no
    dropout.  The reference's arithmetic lives in its closed kernel library; what its test checks
    the result against is plain attention on the unquantised tensors
    (tests/pytest_working/any_mode/FusedSDPA/test_hpu_sdpa_fp8.py:292-320, atol 0.4 for fp8 runs).
    This restatement fixes the quantisation points the way the B200 kernel has them:

        S  = (q8 @ k8^T) * (d_scale_q * d_scale_k * scale)  [+ mask]  [causal: key <= query]
        m  = rowmax(S);  Pt = exp(S - m);  l = rowsum(Pt)                       (fp32)
        P8 = e4m3(Pt * q_scale_s)                       (q_scale_s absent = 1: Pt is in [0, 1])
        O  = (P8 @ v8) * (d_scale_s * d_scale_v) / l    (d_scale_s absent = 1 / q_scale_s)
        out = bf16(O), or e4m3(O * q_scale_o) when q_scale_o is given
        amax_s = max softmax probability = max over rows of 1 / l;  amax_o = max |O|

    Returns (out, m, linv, seed, amax_s, amax_o) with the reference's shapes
    (sdpa_gen.cpp:600-702): m / linv are [..., L, 1] bf16 when requires_backward, else [1]."""
    if p != 0.0:
        raise RuntimeError("fp8_sdpa_recomp_fwd: dropout is not supported")
    if valid_seq_len is not None:
        raise RuntimeError("fp8_sdpa_recomp_fwd: valid_seq_len is not supported")
    f = lambda s, d: float(d if s is None else (s.reshape(-1)[0] if isinstance(s, torch.Tensor) else s))  # noqa: E731
    dq, dk, dv = f(d_scale_q, 1.0), f(d_scale_k, 1.0), f(d_scale_v, 1.0)
    qs = f(q_scale_s, 1.0)
    ds = f(d_scale_s, 1.0 / qs)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    c = torch.tensor(dq, dtype=torch.float32) * torch.tensor(dk, dtype=torch.float32) * torch.tensor(float(scale), dtype=torch.float32)
    s = torch.matmul(q.float(), k.float().transpose(-2, -1)) * c
    L, S = q.shape[-2], k.shape[-2]
    if attention_mask is not None:
        if attention_mask.dtype == torch.bool:
            s = s.masked_fill(~attention_mask, SDPA_MASKED)
        else:
            s = s + attention_mask.float()
    if is_causal:
        keep = torch.ones(L, S, dtype=torch.bool).tril(0)
        s = s.masked_fill(~keep, SDPA_MASKED)
    m = s.amax(dim=-1, keepdim=True)
    pt = torch.exp2((s - m) * 1.4426950408889634)
    l = pt.sum(dim=-1, keepdim=True)
    p8 = _rne_to_fp8((pt * qs).clamp(max=448.0), torch.float8_e4m3fn)
    o = torch.matmul(p8.float(), v.float()) * (torch.tensor(ds, dtype=torch.float32) * torch.tensor(dv, dtype=torch.float32)) / l
    if q_scale_o is not None:
        out = _rne_to_fp8((o * f(q_scale_o, 1.0)).clamp(-448.0, 448.0), torch.float8_e4m3fn)
    else:
        out = o.to(torch.bfloat16)
    one = torch.zeros(1, dtype=torch.float32)
    amax_s = (1.0 / l).max().reshape(1).float() if is_amax_s else one
    amax_o = o.abs().max().reshape(1).float() if is_amax_o else one
    if requires_backward:
        m_out, linv = m.to(torch.bfloat16), (1.0 / l).to(torch.bfloat16)
    else:
        m_out, linv = torch.zeros(1, dtype=torch.bfloat16), torch.zeros(1, dtype=torch.bfloat16)
    return out, m_out, linv, torch.zeros(1, dtype=torch.int32), amax_s, amax_o
