"""The CPU oracle against the golden vectors made from the reference's own test helpers
(tests/golden/make_golden.py) and against the values the reference tests state in text."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import hpu_oracle as O

_DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16,
       "torch.float8_e5m2": torch.float8_e5m2, "torch.float8_e4m3fn": torch.float8_e4m3fn}


def _from_bits(a, dtype):
    t = torch.from_numpy(a.copy())
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t.view(torch.float32)


def test_cast_rne_matches_reference_emulation():
    z = np.load(os.path.join(GOLDEN, "cast_rne.npz"))
    for i in range(int(z["n"])):
        k = f"c{i}"
        dtype, fp8 = _DT[z[k + "_meta"][0]], _DT[z[k + "_meta"][1]]
        x = _from_bits(z[k + "_x"], dtype)
        scale = torch.from_numpy(z[k + "_scale"])
        low = _from_bits(z[k + "_low"], dtype)
        back = _from_bits(z[k + "_back"], dtype)
        out, amax = O.cast_to_fp8_v2(x, scale, False, True, fp8, list(scale.shape) if scale.dim() else None)
        assert out.dtype == fp8 and out.shape == x.shape
        assert torch.equal(out.to(dtype), low), k
        assert amax.dim() == 0 and amax == x.abs().max().float()
        rt = O.cast_from_fp8(out, scale.reciprocal(), dtype, list(scale.shape) if scale.dim() else None)
        assert torch.equal(rt, back), k
        # list / float overloads agree with the tensor overload
        if scale.dim() == 0:
            o2, _ = O.cast_to_fp8_v2(x, float(scale), False, False, fp8)
        else:
            o2, _ = O.cast_to_fp8_v2(x, scale.flatten().tolist(), False, False, fp8, list(scale.shape))
        assert torch.equal(o2.view(torch.uint8), out.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("stochastic", [False, True])
def test_cast_saturates(dtype, stochastic):
    # test_hpu_fp8_ops_any_mode.py:220-243
    for fp8, vals in ((torch.float8_e5m2, [100000, 60000, -60000, -100000]),
                      (torch.float8_e4m3fn, [1000, 500, -500, -1000])):
        x = torch.tensor(vals, dtype=dtype)
        mx = torch.finfo(fp8).max
        out, amax = O.cast_to_fp8_v2(x, torch.tensor(1.0), stochastic, False, fp8)
        assert out.float().tolist() == [mx, mx, -mx, -mx]
        assert amax.numel() == 0 and amax.shape == (0,)


def test_te_rounding_values():
    # test_hpu_fp8_te.py:96-155: 18.5 rounds to 20 (e5m2) / 18 (e4m3) under RNE.
    x = torch.full((8,), 18.5)
    assert O.cast_to_fp8_v2(x, None, False, False, torch.float8_e5m2)[0].float().unique().tolist() == [20.0]
    assert O.cast_to_fp8_v2(x, None, False, False, torch.float8_e4m3fn)[0].float().unique().tolist() == [18.0]


def test_fp8_passthrough_and_errors():
    x = (torch.rand(16, 24, 8) * 30 + 10).to(torch.float8_e5m2)
    out, amax = O.cast_to_fp8_v2(x, None, False, False, torch.float8_e5m2)
    assert torch.equal(out.view(torch.uint8), x.view(torch.uint8)) and amax.numel() == 0
    with pytest.raises(RuntimeError, match="CastToFp8V2 must have no amax for float8."):
        O.cast_to_fp8_v2(x, None, False, True, torch.float8_e5m2)
    with pytest.raises(RuntimeError, match="but are Float8_e5m2 and Float8_e4m3fn"):
        O.cast_to_fp8_v2(x, None, False, False, torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="input dtype must be one of"):
        O.cast_to_fp8_v2(x.to(torch.float16), None, False, False, torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match=r"Number of scale elements \(3\) is not equal to number of scale_shape"):
        O.cast_to_fp8_v2(x.float(), [1.0, 2.0, 3.0], False, False, torch.float8_e4m3fn, [1, 8])
    with pytest.raises(RuntimeError, match="CastFromFp8 output dtype must be equal to float or bfloat16."):
        O.cast_from_fp8(x, None, torch.float16)


def test_gemm_golden():
    z = np.load(os.path.join(GOLDEN, "gemm_small.npz"))
    for i in range(int(z["n"])):
        k = f"g{i}"
        dtype, fp8 = _DT[z[k + "_meta"][0]], _DT[z[k + "_meta"][1]]
        A = torch.from_numpy(z[k + "_A"]).to(dtype)
        B = torch.from_numpy(z[k + "_B"]).to(dtype)
        bias = torch.from_numpy(z[k + "_bias"]).to(dtype)
        sA, sB = torch.from_numpy(z[k + "_sA"]), torch.from_numpy(z[k + "_sB"])
        ref = torch.from_numpy(z[k + "_ref"])
        A8, _ = O.cast_to_fp8_v2(A, sA, False, False, fp8)
        B8, _ = O.cast_to_fp8_v2(B, sB, False, False, fp8)
        D = torch.full(ref.shape, 1000.0, dtype=dtype)
        for use_bias in (False, True):
            for acc in (False, True):
                r = O.fp8_gemm_v2(A8, True, B8, False, D, dtype, sA.reciprocal(), sB.reciprocal(),
                                  bias if use_bias else None, acc)
                e = ref + (bias.float() if use_bias else 0) + (D.float() if acc else 0)
                pd = torch.abs(((r.float() - e) / e) * 100).to(torch.int)
                assert int(pd.max()) <= 15  # the reference's bound
                assert O.rel_frobenius(r, e) < 0.08
    with pytest.raises(RuntimeError, match="Accumulation tensor must be provided at index 4"):
        O.fp8_gemm_v2(A8, True, B8, False, None, dtype, None, None, None, True)


def test_matmul_shape_rules():
    assert O.matmul_out_shape([2, 1, 4, 2], [1, 3, 4, 8], True, False) == [2, 3, 2, 8]
    assert O.matmul_out_shape([4, 2], [3, 4, 8], True, False) == [3, 2, 8]
    assert O.matmul_out_shape([10], [10], False, False) == []
    assert O.matmul_out_shape([2, 10], [10], False, False) == [2]
    assert O.matmul_out_shape([8], [2, 4, 8, 16], False, False) == [2, 4, 16]
    assert O.matmul_out_shape([8], [2, 4, 16, 8], False, True) == [2, 4, 16]
    with pytest.raises(RuntimeError, match="Common dimension sizes of matmul inputs should be the same. Got 5 and 4"):
        O.matmul_out_shape([3, 5], [4, 6], False, False)
    with pytest.raises(RuntimeError, match="Batch dimension 0 of matmul inputs"):
        O.matmul_out_shape([2, 3, 5], [3, 5, 6], False, False)


def test_int4_golden():
    z = np.load(os.path.join(GOLDEN, "int4.npz"))
    for i in range(int(z["n_unit"])):
        k = f"u{i}"
        variant, zp_kind, od = z[k + "_meta"]
        od = _DT[od]
        packed = torch.from_numpy(z[k + "_packed"])
        scale = torch.from_numpy(z[k + "_scale"]).to(od)
        zp = None
        if zp_kind == "packed":
            zp = torch.from_numpy(z[k + "_zp"])
        elif zp_kind == "unpacked":
            zp = torch.from_numpy(z[k + "_zp"]).to(od)
        fn = O.convert_from_int4 if variant == "int4" else O.convert_from_uint4
        r = fn(packed, scale, zp, od)
        assert r.dtype == od and list(r.shape) == list(packed.shape[:-1]) + [packed.shape[-1] * 8]
        assert torch.equal(r.float(), torch.from_numpy(z[k + "_ref"])), (k, variant, zp_kind, od)
    for i in range(int(z["n_gptq"])):
        k = f"a{i}"
        od = _DT[z[k + "_meta"][0]]
        is_zp = z[k + "_meta"][1] == "True"
        qw = torch.from_numpy(z[k + "_qweight"])
        qz = torch.from_numpy(z[k + "_qzeros"])
        sc = torch.from_numpy(z[k + "_scale"]).to(od)
        ref = torch.from_numpy(z[k + "_ref"])
        r = O.convert_from_uint4(qw, sc, qz if is_zp else None, od)
        assert torch.equal(r.float(), ref), (k, list(z[k + "_meta"]))


def test_pack_roundtrip_and_nibble_order():
    q = torch.arange(16).repeat(3)[:40].reshape(1, 40)
    p = O.pack_nibbles(q)
    assert p.dtype == torch.int32 and p.shape == (1, 5)
    assert p[0, 0].item() == 0x76543210
    assert torch.equal(O.unpack_nibbles(p, False), q)
    assert O.unpack_nibbles(p, True)[0, 8:16].tolist() == [-8, -7, -6, -5, -4, -3, -2, -1]


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10.
    r = O.philox4x32_10(np.array([0], dtype=np.uint64), 0, 0)[0]
    assert [hex(v) for v in r] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]


def test_stochastic_rounding_properties():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1 << 16, generator=g) * 3
    for fp8 in O.FP8_DTYPES:
        a, _ = O.cast_to_fp8_v2(x, None, True, False, fp8, seed=1234)
        b, _ = O.cast_to_fp8_v2(x, None, True, False, fp8, seed=1234)
        c, _ = O.cast_to_fp8_v2(x, None, True, False, fp8, seed=99)
        rne, _ = O.cast_to_fp8_v2(x, None, False, False, fp8)
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
        assert not torch.equal(a.view(torch.uint8), c.view(torch.uint8))
        assert not torch.equal(a.view(torch.uint8), rne.view(torch.uint8))
        af = a.float()
        # each output is one of the two neighbours of x: never further than one fp8 step
        lo = torch.minimum(af, rne.float())
        assert torch.all((af - x).abs() <= (x.abs() * 2.0 ** -(2 if fp8 == torch.float8_e5m2 else 3)) + 2.0 ** -9)
        err = (af - x).double()
        sigma = err.std().item() / (x.numel() ** 0.5)
        assert abs(err.mean().item()) < 3 * sigma + 1e-12
        # chunks of the tensor cast with first_index reproduce the whole-tensor bytes
        h = x.numel() // 2
        p1, _ = O.cast_to_fp8_v2(x[h:], None, True, False, fp8, seed=1234, first_index=h)
        assert torch.equal(p1.view(torch.uint8), a.view(torch.uint8)[h:])


def test_sftz_below_min_subnormal():
    # test_hpu_fp8_ops_any_mode.py:246-263 (xfail there): values between 0 and the smallest
    # e5m2 subnormal round to either of them, and the mean is preserved.
    v = 2.0 ** -16 / 3.0
    x = torch.full((100, 100), v, dtype=torch.bfloat16)
    r, _ = O.cast_to_fp8_v2(x, None, True, False, torch.float8_e5m2)
    assert r.float().unique().tolist() == [0.0, 2.0 ** -16]
    assert abs(r.float().mean().item() - float(x[0, 0])) < 0.1 * v


def test_hybrid_golden():
    z = np.load(os.path.join(GOLDEN, "hybrid.npz"))
    for i in range(int(z["n"])):
        k = f"h{i}"
        dtype = _DT[z[k + "_meta"][0]]
        x = _from_bits(z[k + "_x"], dtype)
        o152, o143, amax = O.cast_to_fp8_hybrid(x, torch.tensor(1.3), torch.tensor(0.7), False, True)
        assert torch.equal(o152.to(dtype), _from_bits(z[k + "_low152"], dtype))
        assert torch.equal(o143.to(dtype), _from_bits(z[k + "_low143"], dtype))
        assert amax == x.abs().max().float()
        s152, s143, a0 = O.cast_to_fp8_hybrid(x, torch.tensor(1.3), torch.tensor(0.7), True, False)
        assert torch.equal(s143.view(torch.uint8), o143.view(torch.uint8))      # e4m3 stays RNE
        assert not torch.equal(s152.view(torch.uint8), o152.view(torch.uint8)) and a0.numel() == 0
