"""Generate the golden fixtures in this directory from the reference's own test helpers.

Run once, in a container that has the reference tree, with its path as the argument (or in the
environment variable ``REFERENCE_ROOT``):  ``python tests/golden/make_golden.py REFERENCE_ROOT``.
Nothing at test time reads the reference tree; only the ``.npz`` files written
here are used.

Sources (all under ``tests/pytest_working/`` of the reference):

* ``fp8_utils.py`` is plain torch and is imported as is; its
  ``simulateFp8Precision`` (lines 58-79) is the bit-level round-to-nearest-even
  that the reference tests assert device results against with ``torch.equal``.
* ``any_mode/test_hpu_convert_from_int4.py`` imports the Gaudi runtime at module
  level, so it cannot be imported.  Its packing helpers and its AutoGPTQ
  pack / unpack / dequantise functions (lines 41-71 and 140-247) are pure
  numpy / torch: they are pulled out of the parsed module by name and executed
  unchanged, with a no-op stand-in for the ``htcore.mark_step()`` calls.
"""
import ast
import math
import os
import sys

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT", "")
if not os.path.isdir(os.path.join(REF, "tests", "pytest_working")):
    sys.exit("usage: make_golden.py REFERENCE_ROOT  (the checkout of the reference repository)")
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(REF, "tests", "pytest_working"))

import fp8_utils  # noqa: E402  (the reference's file)


def _bits(t):
    """fp32 / bf16 tensor -> numpy integer view (bf16 has no numpy dtype)."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.view(torch.int32).numpy()


def golden_cast():
    """Inputs and expected values of test_cast_to_fp8_v2 / test_cast_to_fp8_v2_scales
    (test_hpu_fp8_ops_any_mode.py:48-87,142-147,205-217): input = cat(rand*30+10, -that),
    expected low-precision value = simulateFp8Precision(input * scale.to(dtype)),
    expected round trip = that * (1/scale).to(dtype)."""
    out = {}
    g = torch.Generator().manual_seed(0xC001A1)
    rng = np.random.RandomState(0xC001A1 & 0xFFFFFFF)
    cases = []
    for dtype in (torch.float32, torch.bfloat16):
        cases.append(("tensor", (64, 48), dtype, None))
    for axis in (0, 1):
        cases.append(("channel", (16, 24, 8), torch.bfloat16, axis))
        cases.append(("channel", (16, 24, 8), torch.float32, axis))
    idx = 0
    for mode, shape, dtype, axis in cases:
        for fp8 in fp8_utils.fp8_dtypes:
            pos = torch.rand(shape, dtype=dtype, generator=g) * 30 + 10
            x = torch.cat((pos, -pos))
            if mode == "tensor":
                scale = torch.tensor(1.3)
            else:
                scale = torch.tensor((rng.rand(x.shape[-1 - axis]) * 2.0 + 0.5).astype(np.float32))
                scale = torch.unsqueeze(scale, axis)
            low = fp8_utils.simulateFp8Precision(x * scale.to(dtype), fp8)
            back = low * scale.reciprocal().to(dtype)
            k = f"c{idx}"
            out[k + "_x"] = _bits(x)
            out[k + "_scale"] = scale.numpy()
            out[k + "_low"] = _bits(low)
            out[k + "_back"] = _bits(back)
            out[k + "_meta"] = np.array([str(dtype), str(fp8), mode, str(axis)])
            idx += 1
    out["n"] = np.array(idx)
    np.savez_compressed(os.path.join(HERE, "cast_rne.npz"), **out)
    print("cast_rne.npz:", idx, "cases")


def golden_hybrid():
    """Inputs and expected values of test_cast_to_fp8_hybrid (test_hpu_fp8_ops_any_mode.py:266-346):
    scales 1.3 (e5m2) and 0.7 (e4m3), expected = simulateFp8Precision(input * scale.to(dtype))."""
    out = {}
    g = torch.Generator().manual_seed(0xC001A1 + 1)
    idx = 0
    for shape, dtype in (((64, 48), torch.float32), ((64, 48), torch.bfloat16), ((16, 24, 8), torch.bfloat16)):
        pos = torch.rand(shape, dtype=dtype, generator=g) * 30 + 10
        x = torch.cat((pos, -pos))
        s152, s143 = torch.tensor(1.3), torch.tensor(0.7)
        low152 = fp8_utils.simulateFp8Precision(x * s152.to(dtype), torch.float8_e5m2)
        low143 = fp8_utils.simulateFp8Precision(x * s143.to(dtype), torch.float8_e4m3fn)
        k = f"h{idx}"
        out[k + "_x"] = _bits(x)
        out[k + "_low152"] = _bits(low152)
        out[k + "_low143"] = _bits(low143)
        out[k + "_back152"] = _bits(low152 * s152.reciprocal().to(dtype))
        out[k + "_back143"] = _bits(low143 * s143.reciprocal().to(dtype))
        out[k + "_meta"] = np.array([str(dtype)])
        idx += 1
    out["n"] = np.array(idx)
    np.savez_compressed(os.path.join(HERE, "hybrid.npz"), **out)
    print("hybrid.npz:", idx, "cases")


def golden_gemm():
    """Operands of test_fp8_gemm_v2 (test_hpu_fp8_ops_any_mode.py:352-484): A [24,12] and
    B [24,36] = rand*10+30, per-tensor scales 0.9*max/amax, trans_A=True; expected =
    A^T @ B (+bias) (+out) in the test dtype.  The reference tolerance is 15 %
    (integer-truncated), lines 471-473."""
    out = {}
    g = torch.Generator().manual_seed(0xC001A1)
    idx = 0
    for dtype in (torch.float32, torch.bfloat16):
        for fp8 in fp8_utils.fp8_dtypes:
            A = torch.rand((24, 12), dtype=dtype, generator=g) * 10 + 30.0
            B = torch.rand((24, 36), dtype=dtype, generator=g) * 10 + 30.0
            bias = torch.rand((12, 36), dtype=dtype, generator=g) * 10 + 30.0
            sA = fp8_utils.FP8_MAX[fp8] / torch.max(torch.abs(A)).to(torch.float)
            sB = fp8_utils.FP8_MAX[fp8] / torch.max(torch.abs(B)).to(torch.float)
            ref = torch.matmul(A.transpose(-2, -1), B)
            k = f"g{idx}"
            out[k + "_A"] = A.float().numpy()
            out[k + "_B"] = B.float().numpy()
            out[k + "_bias"] = bias.float().numpy()
            out[k + "_sA"] = sA.numpy()
            out[k + "_sB"] = sB.numpy()
            out[k + "_ref"] = ref.float().numpy()
            out[k + "_meta"] = np.array([str(dtype), str(fp8)])
            idx += 1
    out["n"] = np.array(idx)
    np.savez_compressed(os.path.join(HERE, "gemm_small.npz"), **out)
    print("gemm_small.npz:", idx, "cases")


class _NoHpu:
    @staticmethod
    def mark_step():
        pass


def _load_int4_helpers():
    path = os.path.join(REF, "tests", "pytest_working", "any_mode", "test_hpu_convert_from_int4.py")
    tree = ast.parse(open(path).read())
    want = {"pack_1d", "pack_int4_into_int32", "pack_tensor", "pack_cuda_old", "unpack_weight_cuda",
            "unpack_zeros_cuda_old", "get_weight_cuda_old", "gen_quant4", "prepare_data"}
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in want]
    ns = {"torch": torch, "np": np, "math": math, "htcore": _NoHpu}
    exec(compile(ast.Module(body=body, type_ignores=[]), path, "exec"), ns)
    return ns


def golden_int4():
    ns = _load_int4_helpers()
    out = {}
    # (1) test_convert_from_int4 (lines 74-137): shapes (10,) and (4,6,4), both variants,
    #     packed / unpacked / no zero point, random scales.
    g = torch.Generator().manual_seed(0xC001A1)
    idx = 0
    for packed_shape in ((10,), (4, 6, 4)):
        real = list(packed_shape)
        real[-1] *= 8
        for variant in ("int4", "uint4"):
            for zp_kind in ("packed", "unpacked", "none"):
                for od in (torch.float32, torch.bfloat16):
                    sub_dtype = od
                    if zp_kind == "packed":
                        sub_dtype = torch.int8 if variant == "int4" else torch.uint8
                    q = torch.randint(0, 16, real, dtype=torch.int, generator=g)
                    packed = torch.tensor(ns["pack_int4_into_int32"](q, packed_shape), dtype=torch.int)
                    if variant == "int4":
                        q = torch.where(q > 7, q - 16, q)
                    q = q.to(sub_dtype)
                    scale = (torch.randn(real, generator=g) * 50.0).to(od)
                    zp_in = None
                    zp = torch.tensor(0.0)
                    if zp_kind == "packed":
                        zp = torch.randint(1, 5, real, dtype=torch.int, generator=g)
                        if variant == "uint4":
                            zp = torch.where(zp > q, 0, zp)
                        zp_in = torch.tensor(ns["pack_int4_into_int32"](zp, packed_shape), dtype=torch.int)
                        zp = zp.to(sub_dtype)
                        sub = (q - zp).to(od)
                    elif zp_kind == "unpacked":
                        zp = (torch.randn(real, generator=g) * 5.0).to(od)
                        zp_in = zp
                        sub = q - zp
                    else:
                        sub = q - zp.to(od) if od == torch.float32 else (q - zp).to(od)
                    res = sub * scale
                    k = f"u{idx}"
                    out[k + "_packed"] = packed.numpy()
                    out[k + "_scale"] = scale.float().numpy()
                    if zp_in is not None:
                        out[k + "_zp"] = zp_in.numpy() if zp_in.dtype == torch.int32 else zp_in.float().numpy()
                    out[k + "_ref"] = res.float().numpy()
                    out[k + "_meta"] = np.array([variant, zp_kind, str(od)])
                    idx += 1
    out["n_unit"] = np.array(idx)

    # (2) test_convert_from_int4_AutoGPTQ (lines 398-476): 64x64, group 16, uint4.
    torch.manual_seed(0xC001A1)
    bits, group, K, N = 4, 16, 64, 64
    wf = torch.tensor(list(range(0, 32, bits)), dtype=torch.int32).unsqueeze(0)
    gi = 0
    for od in (torch.float32, torch.bfloat16):
        for (is_zp, packed_zp) in ((False, True), (True, False), (True, True)):
            for zv, sv, iv in (("range", "rand", "normal"), ("8", "range", "range"), ("1", "1", "7"),
                               ("0", "range_int", "1"), ("range", "rand", "0")):
                inp, scale, zeros = ns["prepare_data"](K, N, group, bits, "uint4", od, is_zp, packed_zp, iv, sv, zv)
                qw, qz, cs = ns["pack_cuda_old"](inp, scale.T, zeros.T, -1, K, N, group, bits)
                if iv == "0":
                    qw = torch.zeros_like(qw)
                # the reference's host-side repack to the operator layout (lines 380-395)
                weight = ns["unpack_weight_cuda"](qw, bits, wf, group, False)
                op_qweight = ns["pack_tensor"](weight)
                zeros_u = ns["unpack_zeros_cuda_old"](qz, cs, bits, wf, False)
                op_qzeros = ns["pack_tensor"](zeros_u)
                expect = ns["get_weight_cuda_old"](is_zp, bits, qw, qz, cs, group)
                k = f"a{gi}"
                out[k + "_gptq_qweight"] = qw.numpy()
                out[k + "_gptq_qzeros"] = qz.numpy()
                out[k + "_qweight"] = op_qweight.numpy()
                out[k + "_qzeros"] = op_qzeros.numpy()
                out[k + "_scale"] = cs.to(od).float().numpy()
                out[k + "_ref"] = expect.float().numpy()
                out[k + "_meta"] = np.array([str(od), str(is_zp), zv, sv, iv])
                gi += 1
    out["n_gptq"] = np.array(gi)
    np.savez_compressed(os.path.join(HERE, "int4.npz"), **out)
    print("int4.npz:", idx, "unit cases,", gi, "gptq cases")


if __name__ == "__main__":
    golden_cast()
    golden_hybrid()
    golden_gemm()
    golden_int4()
