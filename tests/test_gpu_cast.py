"""cast_to_fp8_v2 / cast_from_fp8 on the GPU against the CPU oracle: FP8 bytes and amax
bit-exact, stochastic rounding bit-exact against the oracle's Philox definition and unbiased.
Cases mirror tests/pytest_working/any_mode/test_hpu_fp8_ops_any_mode.py of the reference."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import hpu_oracle as O

pytestmark = pytest.mark.gpu
FP8 = [torch.float8_e5m2, torch.float8_e4m3fn]
_DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16,
       "torch.float8_e5m2": torch.float8_e5m2, "torch.float8_e4m3fn": torch.float8_e4m3fn}


@pytest.fixture(scope="module")
def ops():
    import b200_hpu_ops
    assert torch.cuda.is_available()
    return b200_hpu_ops


def _bytes(t):
    return t.cpu().view(torch.uint8)


def _from_bits(a, dtype):
    t = torch.from_numpy(a.copy())
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t.view(torch.float32)


def test_golden_rne_through_cuda(ops):
    """Reference-emulation vectors (simulateFp8Precision) through the CUDA operators."""
    z = np.load(os.path.join(GOLDEN, "cast_rne.npz"))
    for i in range(int(z["n"])):
        k = f"c{i}"
        dtype, fp8 = _DT[z[k + "_meta"][0]], _DT[z[k + "_meta"][1]]
        x = _from_bits(z[k + "_x"], dtype)
        scale = torch.from_numpy(z[k + "_scale"])
        shape = list(scale.shape) if scale.dim() else None
        out, amax = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), scale.cuda(), False, True, fp8, shape)
        assert torch.equal(out.cpu().to(dtype), _from_bits(z[k + "_low"], dtype)), k
        assert amax.dim() == 0 and amax.cpu() == x.abs().max().float()
        back = torch.ops.hpu.cast_from_fp8(out, scale.reciprocal().cuda(), dtype, shape)
        assert torch.equal(back.cpu(), _from_bits(z[k + "_back"], dtype)), k
        if scale.dim() == 0:
            o2, a2 = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), float(scale), False, False, fp8)
            b2 = torch.ops.hpu.cast_from_fp8(o2, 1.0 / float(scale), dtype)
        else:
            o2, a2 = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), scale.flatten().tolist(), False, False, fp8, shape)
            b2 = torch.ops.hpu.cast_from_fp8(o2, scale.reciprocal().flatten().tolist(), dtype, shape)
        assert torch.equal(_bytes(o2), _bytes(out)) and a2.numel() == 0 and tuple(a2.shape) == (0,)
        assert torch.equal(b2.cpu(), back.cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fp8", FP8)
@pytest.mark.parametrize("n", [1, 7, 15, 16, 17, 8191, (1 << 20) + 3])
def test_sizes_and_tails_bit_exact(ops, dtype, fp8, n):
    g = torch.Generator().manual_seed(n)
    x = (torch.randn(n, generator=g) * 20).to(dtype)
    for scale in (None, 0.37):
        out, amax = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), scale, False, True, fp8)
        ref, ramax = O.cast_to_fp8_v2(x, scale, False, True, fp8)
        assert torch.equal(_bytes(out), _bytes(ref))
        assert amax.cpu() == ramax
        back = torch.ops.hpu.cast_from_fp8(out, None if scale is None else 1 / scale, dtype)
        assert torch.equal(back.cpu(), O.cast_from_fp8(ref, None if scale is None else 1 / scale, dtype))


@pytest.mark.parametrize("fp8", FP8)
def test_all_fp8_codes_roundtrip(ops, fp8):
    codes = torch.arange(256, dtype=torch.uint8).view(fp8)
    for dt in (torch.float32, torch.bfloat16):
        up = torch.ops.hpu.cast_from_fp8(codes.cuda(), None, dt).cpu()
        ref = O.cast_from_fp8(codes, None, dt)
        nan = torch.isnan(ref.float())   # NaN payloads are not part of the contract
        assert torch.equal(torch.isnan(up.float()), nan)
        it = torch.int32 if dt == torch.float32 else torch.int16
        assert torch.equal(up.view(it)[~nan], ref.view(it)[~nan])
        finite = torch.isfinite(ref.float())
        down, _ = torch.ops.hpu.cast_to_fp8_v2(up.cuda(), None, False, False, fp8)
        assert torch.equal(_bytes(down)[finite], _bytes(codes)[finite])
    # fp8 -> fp8 pass-through
    same, am = torch.ops.hpu.cast_to_fp8_v2(codes.cuda(), None, False, False, fp8)
    assert torch.equal(_bytes(same), _bytes(codes)) and am.numel() == 0


@pytest.mark.parametrize("fp8", FP8)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ties_specials_subnormals(ops, fp8, dtype):
    codes = torch.arange(256, dtype=torch.uint8).view(fp8).float()
    vals = codes[torch.isfinite(codes)].sort().values
    mids = (vals[:-1] + vals[1:]) / 2  # every RNE tie
    mx = torch.finfo(fp8).max
    tiny = 2.0 ** (-9 if fp8 == torch.float8_e4m3fn else -16)
    extra = torch.tensor([mx, -mx, mx * 1.03, -mx * 1.03, mx * 2, 1e30, -1e30, float("inf"), -float("inf"),
                          float("nan"), -float("nan"), 0.0, -0.0, tiny, tiny / 2, tiny / 2 * 1.01, tiny * 0.49,
                          -tiny / 2, tiny * 1.5, tiny * 2.5, 1e-30, -1e-30])
    x = torch.cat([vals, mids, torch.nextafter(mids, mids + 1), torch.nextafter(mids, mids - 1), extra]).to(dtype)
    for scale in (None, 1.0, 3.0):
        out, amax = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), scale, False, True, fp8)
        ref, ramax = O.cast_to_fp8_v2(x, scale, False, True, fp8)
        assert torch.equal(_bytes(out), _bytes(ref))
        assert torch.isnan(amax.cpu()) and torch.isnan(ramax)  # NaN in the input propagates
    xf = x[torch.isfinite(x.float())]
    _, amax = torch.ops.hpu.cast_to_fp8_v2(xf.cuda(), None, False, True, fp8)
    assert amax.cpu() == xf.float().abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("stochastic", [True, False])
@pytest.mark.parametrize("big", [True, False])
@pytest.mark.parametrize("fp8", FP8)
def test_out_of_range_saturates(ops, dtype, stochastic, big, fp8):
    # test_hpu_fp8_ops_any_mode.py:220-243
    vals = [100000, 60000, -60000, -100000] if fp8 == torch.float8_e5m2 else [1000, 500, -500, -1000]
    x = torch.tensor(vals, dtype=dtype)
    mx = torch.finfo(fp8).max
    exp = torch.tensor([mx, mx, -mx, -mx])
    if big:
        x = x.expand(800, 4).reshape(80, 40)
        exp = exp.expand(800, 4).reshape(80, 40)
    r, _ = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), torch.tensor(1.0).cuda(), stochastic, False, fp8)
    assert torch.equal(r.cpu().float(), exp)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fp8", FP8)
def test_scale_shapes(ops, dtype, fp8):
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(6, 32, 48, generator=g) * 10).to(dtype)
    xc = x.cuda()
    cases = [
        (torch.rand(48, generator=g) + 0.5, [1, 48]),         # per last dim
        (torch.rand(48, generator=g) + 0.5, None),            # [48] broadcasts the same way
        (torch.rand(6, generator=g) + 0.5, [6, 1, 1]),        # per leading dim
        (torch.rand(32, generator=g) + 0.5, [32, 1]),         # middle dim: mixed pattern
        (torch.rand(6, 32, 48, generator=g) + 0.5, None),     # element-wise
        (torch.rand(32 * 48, generator=g) + 0.5, [32, 48]),   # trailing block, reshaped
        (torch.rand(1, generator=g) + 0.5, None),
    ]
    for s, shape in cases:
        out, amax = torch.ops.hpu.cast_to_fp8_v2(xc, s.cuda(), False, True, fp8, shape)
        ref, ramax = O.cast_to_fp8_v2(x, s, False, True, fp8, shape)
        assert torch.equal(_bytes(out), _bytes(ref)), (list(s.shape), shape)
        assert amax.cpu() == ramax
        back = torch.ops.hpu.cast_from_fp8(out, s.reciprocal().cuda(), dtype, shape)
        assert torch.equal(back.cpu(), O.cast_from_fp8(ref, s.reciprocal(), dtype, shape))
        if s.numel() > 1:
            o2, _ = torch.ops.hpu.cast_to_fp8_v2(xc, s.flatten().tolist(), False, False, fp8,
                                                 shape if shape is not None else list(s.shape))
            assert torch.equal(_bytes(o2), _bytes(ref))
    # a bf16 scale tensor is accepted too
    s = (torch.rand(48, generator=g) + 0.5).to(torch.bfloat16)
    out, _ = torch.ops.hpu.cast_to_fp8_v2(xc, s.cuda(), False, False, fp8, [1, 48])
    assert torch.equal(_bytes(out), _bytes(O.cast_to_fp8_v2(x, s, False, False, fp8, [1, 48])[0]))


def test_unaligned_and_noncontiguous_views(ops):
    g = torch.Generator().manual_seed(9)
    base = (torch.randn(4099, generator=g) * 5).to(torch.bfloat16)
    x = base.cuda()[3:]            # 6-byte offset: not 16-byte aligned
    out, amax = torch.ops.hpu.cast_to_fp8_v2(x, 0.5, False, True, torch.float8_e4m3fn)
    ref, ramax = O.cast_to_fp8_v2(base[3:], 0.5, False, True, torch.float8_e4m3fn)
    assert torch.equal(_bytes(out), _bytes(ref)) and amax.cpu() == ramax
    m = (torch.randn(64, 96, generator=g) * 5).to(torch.float32)
    xt = m.cuda().t()              # non-contiguous
    out, _ = torch.ops.hpu.cast_to_fp8_v2(xt, None, False, False, torch.float8_e5m2)
    assert torch.equal(_bytes(out), _bytes(O.cast_to_fp8_v2(m.t(), None, False, False, torch.float8_e5m2)[0]))
    o8 = out[:, 1:]                # fp8 view with odd offset into cast_from_fp8
    back = torch.ops.hpu.cast_from_fp8(o8, 2.0, torch.bfloat16)
    assert torch.equal(back.cpu(), O.cast_from_fp8(out.cpu()[:, 1:], 2.0, torch.bfloat16))


def test_mul_in_fp32_mode(ops):
    g = torch.Generator().manual_seed(11)
    x = (torch.rand(1 << 16, generator=g) * 30 + 10).to(torch.bfloat16)
    try:
        ops.set_cast_mul_in_fp32(True)
        out, _ = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), 1.3, False, False, torch.float8_e4m3fn)
    finally:
        ops.set_cast_mul_in_fp32(False)
    ref32, _ = O.cast_to_fp8_v2(x, 1.3, False, False, torch.float8_e4m3fn, mul_in_fp32=True)
    ref, _ = O.cast_to_fp8_v2(x, 1.3, False, False, torch.float8_e4m3fn)
    assert torch.equal(_bytes(out), _bytes(ref32))
    assert not torch.equal(_bytes(ref32), _bytes(ref))  # the two definitions really differ
    out, _ = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), 1.3, False, False, torch.float8_e4m3fn)
    assert torch.equal(_bytes(out), _bytes(ref))


def test_errors_match_reference_strings(ops):
    # test_hpu_fp8_ops_any_mode.py:179-202 and fp8_ops.cpp:29-53,201-215,276-278
    x8 = torch.rand(16, 24, 8).to(torch.float8_e5m2).cuda()
    with pytest.raises(RuntimeError, match="CastToFp8V2 must have no amax for float8."):
        torch.ops.hpu.cast_to_fp8_v2(x8, None, False, True, torch.float8_e5m2)
    with pytest.raises(RuntimeError, match="CastToFp8V2 input and output must have the same dtype for float8, "
                                           "but are Float8_e5m2 and Float8_e4m3fn"):
        torch.ops.hpu.cast_to_fp8_v2(x8, None, False, False, torch.float8_e4m3fn)
    with pytest.raises(RuntimeError, match="CastToFp8V2 input dtype must be one of"):
        torch.ops.hpu.cast_to_fp8_v2(torch.zeros(4, dtype=torch.float16).cuda(), None, False, False, torch.float8_e5m2)
    xf = torch.zeros(4, 8).cuda()
    with pytest.raises(RuntimeError, match=r"Number of scale elements \(3\) is not equal to number of scale_shape "
                                           r"elements \(8\)"):
        torch.ops.hpu.cast_to_fp8_v2(xf, [1.0, 2.0, 3.0], False, False, torch.float8_e5m2, [1, 8])
    with pytest.raises(RuntimeError, match="CastFromFp8 output dtype must be equal to float or bfloat16."):
        torch.ops.hpu.cast_from_fp8(x8, None, torch.float16)
    with pytest.raises(RuntimeError):  # dtype=None default: a missing dtype is an error
        torch.ops.hpu.cast_to_fp8_v2(xf)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fp8", FP8)
def test_stochastic_rounding_bit_exact_and_unbiased(ops, dtype, fp8):
    g = torch.Generator().manual_seed(21)
    n = (1 << 20) + 5
    x = (torch.randn(n, generator=g) * 4).to(dtype)
    x[:64] = x[:64] * 1e-4   # reach the subnormal range of both formats
    for scale in (None, 1.7):
        ops.set_sr_seed(1234)
        out, amax = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), scale, True, True, fp8)
        ref, _ = O.cast_to_fp8_v2(x, scale, True, True, fp8, seed=1234, offset=0)
        assert torch.equal(_bytes(out), _bytes(ref))
        assert amax.cpu() == x.float().abs().max()
        out2, _ = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), scale, True, False, fp8)   # next offset
        ref2, _ = O.cast_to_fp8_v2(x, scale, True, False, fp8, seed=1234, offset=1)
        assert torch.equal(_bytes(out2), _bytes(ref2))
        assert not torch.equal(_bytes(out2), _bytes(out))
        rne, _ = O.cast_to_fp8_v2(x, scale, False, False, fp8)
        assert not torch.equal(_bytes(out), _bytes(rne))
    # unbiasedness: mean of the dequantised result within 3 sigma of the mean of the input
    ops.set_sr_seed(1234)
    out, _ = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), None, True, False, fp8)
    err = (out.cpu().float() - x.float()).double()
    sigma = err.std().item() / n ** 0.5
    assert abs(err.mean().item()) < 3 * sigma
    # reference test bound (test_hpu_fp8_ops_any_mode.py:126-128): within rtol 0.26 of the RNE result
    big = x.float().abs() > 1e-2
    rne, _ = O.cast_to_fp8_v2(x, None, False, False, fp8)
    assert torch.allclose(out.cpu().float()[big], rne.float()[big], rtol=0.26, atol=0.0)


def test_sftz_below_min_subnormal(ops):
    v = 2.0 ** -16 / 3.0
    x = torch.full((100, 100), v, dtype=torch.bfloat16)
    ops.set_sr_seed(7)
    r, _ = torch.ops.hpu.cast_to_fp8_v2(x.cuda(), None, True, False, torch.float8_e5m2)
    rc = r.cpu().float()
    assert rc.unique().tolist() == [0.0, 2.0 ** -16]
    assert abs(rc.mean().item() - float(x[0, 0])) < 0.1 * v
    assert torch.equal(_bytes(r), _bytes(O.cast_to_fp8_v2(x, None, True, False, torch.float8_e5m2, seed=7)[0]))


def test_sr_chunks_reproduce_whole_tensor_via_abi(ops):
    """Sharding a tensor over ranks must not change the bytes: element i always uses the
    Philox word of its global index (first_index argument of the C ABI)."""
    from b200_hpu_ops import abi
    g = torch.Generator().manual_seed(31)
    x = (torch.randn(1 << 18, generator=g) * 3).to(torch.bfloat16).cuda()
    whole, _ = abi.cast_to_fp8(x, torch.float8_e5m2, 2.0, stochastic=True, seed=99)
    parts = []
    step = x.numel() // 8
    for r in range(8):
        p, _ = abi.cast_to_fp8(x[r * step:(r + 1) * step].contiguous(), torch.float8_e5m2, 2.0, stochastic=True,
                               seed=99, first_index=r * step)
        parts.append(p)
    assert torch.equal(_bytes(torch.cat(parts)), _bytes(whole))
    ref, _ = O.cast_to_fp8_v2(x.cpu(), 2.0, True, False, torch.float8_e5m2, seed=99)
    assert torch.equal(_bytes(whole), _bytes(ref))


@pytest.mark.parametrize("n", [1 << 24])
def test_full_size_properties(ops, n):
    """At benchmark size the oracle is too slow to run in full: check a strided sample bit-exactly
    and size-independent properties (idempotent round trip, amax equals torch's)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(n, device="cuda", generator=g, dtype=torch.float32).to(torch.bfloat16)
    x[::1000] = 50.0
    s = 448.0 / 50.0
    out, amax = torch.ops.hpu.cast_to_fp8_v2(x, s, False, True, torch.float8_e4m3fn)
    assert amax.item() == x.float().abs().max().item() == 50.0
    back = torch.ops.hpu.cast_from_fp8(out, 1 / s, torch.bfloat16)
    again, _ = torch.ops.hpu.cast_to_fp8_v2(torch.ops.hpu.cast_from_fp8(out, None, torch.bfloat16), None, False,
                                            False, torch.float8_e4m3fn)
    assert torch.equal(_bytes(again), _bytes(out))  # fp8 -> bf16 -> fp8 is the identity
    idx = torch.arange(0, n, 4099, device="cuda")
    ref, _ = O.cast_to_fp8_v2(x[idx].cpu(), s, False, False, torch.float8_e4m3fn)
    assert torch.equal(_bytes(out[idx]), _bytes(ref))
    assert torch.equal(back[idx].cpu(), O.cast_from_fp8(ref, 1 / s, torch.bfloat16))


def test_swiglu_cast(ops):
    g = torch.Generator().manual_seed(41)
    gate = torch.randn(64, 256, generator=g).to(torch.bfloat16)
    up = torch.randn(64, 256, generator=g).to(torch.bfloat16)
    out, amax = torch.ops.b200q.swiglu_cast_fp8(gate.cuda(), up.cuda(), 37.0, True)
    h = (torch.nn.functional.silu(gate.float()) * up.float()).to(torch.bfloat16)
    ref, ramax = O.cast_to_fp8_v2(h, 37.0, False, True, torch.float8_e4m3fn)
    # expf on the device and in torch's CPU kernels may differ in the last fp32 bit, which can move
    # a bf16 rounding: allow a one-code difference on a handful of elements
    a, b = _bytes(out).int(), _bytes(ref).int()
    assert (a - b).abs().max() <= 1 and (a != b).float().mean() < 2e-3
    assert abs(amax.item() - ramax.item()) <= 2 ** -7 * ramax.item()


def test_hybrid_cast_matches_reference_emulation_and_oracle(ops):
    """cast_to_fp8_hybrid (test_hpu_fp8_ops_any_mode.py:266-352): golden vectors from the reference's
    emulation, then scale / stochastic / amax variants against the oracle."""
    z = np.load(os.path.join(GOLDEN, "hybrid.npz"))
    for i in range(int(z["n"])):
        k = f"h{i}"
        dtype = _DT[z[k + "_meta"][0]]
        x = _from_bits(z[k + "_x"], dtype)
        s152, s143 = torch.tensor(1.3), torch.tensor(0.7)
        o152, o143, amax = torch.ops.hpu.cast_to_fp8_hybrid(x.cuda(), s152.cuda(), s143.cuda(), False, True)
        assert o152.dtype == torch.float8_e5m2 and o143.dtype == torch.float8_e4m3fn
        assert torch.equal(o152.cpu().to(dtype), _from_bits(z[k + "_low152"], dtype))
        assert torch.equal(o143.cpu().to(dtype), _from_bits(z[k + "_low143"], dtype))
        assert amax.dim() == 0 and amax.cpu() == x.abs().max().float()
        b152 = torch.ops.hpu.cast_from_fp8(o152, s152.reciprocal().cuda(), dtype)
        b143 = torch.ops.hpu.cast_from_fp8(o143, s143.reciprocal().cuda(), dtype)
        assert torch.equal(b152.cpu(), _from_bits(z[k + "_back152"], dtype))
        assert torch.equal(b143.cpu(), _from_bits(z[k + "_back143"], dtype))
    g = torch.Generator().manual_seed(3)
    for dtype in (torch.float32, torch.bfloat16):
        x = (torch.randn((1 << 18) + 7, generator=g) * 20).to(dtype)
        for s5, s4 in ((None, None), (torch.tensor(2.5), None), (torch.tensor(0.3), torch.tensor(4.0))):
            for sr in (False, True):
                ops.set_sr_seed(1234)
                o152, o143, amax = torch.ops.hpu.cast_to_fp8_hybrid(x.cuda(), _c(s5), _c(s4), sr, False)
                r152, r143, _ = O.cast_to_fp8_hybrid(x, s5, s4, sr, False, seed=1234, offset=0)
                assert torch.equal(_bytes(o152), _bytes(r152)) and torch.equal(_bytes(o143), _bytes(r143))
                assert amax.numel() == 0
    with pytest.raises(RuntimeError, match="CastToFp8Hybrid input must be of float or bfloat16 dtype."):
        torch.ops.hpu.cast_to_fp8_hybrid(torch.zeros(4, dtype=torch.float16).cuda(), None, None, False, False)


def _c(t):
    return None if t is None else t.cuda()
