"""FP8 scale management: amax pass, amax -> scale, the reference's CastMomentToFp8WithScale
composition (habana_kernels/lazy_optimizer_kernels.cpp:113-126) and delayed scaling, CUDA
against the oracle (bit-exact) and the oracle against the reference's own ATen formula."""
import math

import pytest
import torch

from oracle import hpu_oracle as O

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


@pytest.fixture(scope="module")
def ops():
    import b200_hpu_ops
    assert torch.cuda.is_available()
    return b200_hpu_ops


def _reference_formula(amax, prev, fp8_max):
    """The four ATen calls of the reference, on CPU tensors."""
    exp = torch.floor(torch.log2(fp8_max / amax))
    sf = torch.pow(2.0, exp)
    return torch.where(amax > 0.0, sf, prev)


def test_oracle_scale_matches_reference_formula():
    g = torch.Generator().manual_seed(11)
    for fp8_max in (448.0, 57344.0):
        # log-uniform amax values; quotients near a power of two are left to the test below
        amax = torch.exp(torch.rand(4000, generator=g) * 40 - 20).float()
        for a in amax:
            q = fp8_max / float(a)
            if abs(math.log2(q) - round(math.log2(q))) < 1e-5:
                continue
            want = _reference_formula(a, torch.tensor(7.0), fp8_max)
            got = O.scale_from_amax(a, torch.tensor(7.0), fp8_max)
            assert torch.equal(want, got), (float(a), float(want), float(got))
    zero = torch.tensor(0.0)
    assert float(O.scale_from_amax(zero, torch.tensor(7.0), 448.0)) == 7.0
    assert float(_reference_formula(zero, torch.tensor(7.0), 448.0)) == 7.0


def test_oracle_scale_exact_at_powers_of_two():
    """fp8_max / amax an exact power of two, and one ulp below it."""
    for k in range(-20, 20):
        a = torch.tensor(448.0 / 2.0 ** k)
        assert float(O.scale_from_amax(a, torch.tensor(1.0), 448.0)) == 2.0 ** k
        a_up = torch.nextafter(a, torch.tensor(float("inf")))  # quotient just below 2^k
        assert float(O.scale_from_amax(a_up, torch.tensor(1.0), 448.0)) == 2.0 ** (k - 1)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [0, 1, 7, 8, 1000, 4096, (1 << 20) + 3])
def test_amax_matches_torch(ops, dtype, n):
    g = torch.Generator().manual_seed(n + 1)
    x = (torch.randn(n, generator=g) * 3).to(dtype)
    if n > 100:
        x[n // 3] = -77.5
    got = torch.ops.b200q.amax(x.cuda()).cpu()
    want = x.abs().max().float() if n else torch.zeros(())
    assert got.shape == () and torch.equal(got, want)
    if n > 8:
        x[n // 2] = float("nan")
        assert torch.isnan(torch.ops.b200q.amax(x.cuda())).item()


@pytest.mark.gpu
def test_scale_from_amax_bit_exact(ops):
    g = torch.Generator().manual_seed(5)
    vals = torch.exp(torch.rand(300, generator=g) * 60 - 30).float().tolist()
    vals += [0.0, 448.0, 448.0 / 8, float(torch.nextafter(torch.tensor(56.0), torch.tensor(1e9))), 1e-38, 3e38, float("nan")]
    for fp8_max in (448.0, 57344.0):
        for pow2, margin in ((True, 0), (False, 0), (False, 2)):
            for a in vals:
                amax = torch.tensor(a, dtype=torch.float32)
                scale = torch.tensor([3.0], device="cuda")
                torch.ops.b200q.scale_from_amax_(scale, amax.cuda(), fp8_max, pow2, margin)
                want = O.scale_from_amax(amax, torch.tensor(3.0), fp8_max, pow2, margin)
                assert torch.equal(scale.cpu().reshape(()), want), (a, fp8_max, pow2, margin, float(scale), float(want))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [E4M3, E5M2])
@pytest.mark.parametrize("src", [torch.bfloat16, torch.float32])
def test_cast_moment_to_fp8(ops, dtype, src):
    g = torch.Generator().manual_seed(3)
    m = (torch.randn(257, 129, generator=g) * 1e-3).to(src)
    ops.set_sr_seed(99)
    scale = torch.ones(1, device="cuda")
    out = torch.ops.b200q.cast_moment_to_fp8(m.cuda(), scale, dtype)
    want, want_scale = O.cast_moment_to_fp8(m, torch.ones(1), dtype, seed=99)
    assert torch.equal(scale.cpu().reshape(()), want_scale)
    assert torch.equal(out.cpu().view(torch.uint8), want.view(torch.uint8))
    # the scale is a power of two that maps the amax into the top binade of the format
    amax = m.abs().max().float()
    assert O.FP8_MAX[dtype] / 2 < float(amax * scale.cpu()) <= O.FP8_MAX[dtype]
    # an all-zero moment keeps the scale
    scale2 = torch.full((1,), 4.0, device="cuda")
    out0 = torch.ops.b200q.cast_moment_to_fp8(torch.zeros(64, dtype=src).cuda(), scale2, dtype)
    assert float(scale2) == 4.0 and int(out0.view(torch.uint8).max()) == 0


@pytest.mark.gpu
def test_delayed_and_current_scaling(ops):
    from b200_hpu_ops.scaling import DelayedScaling, current_scaling_cast

    g = torch.Generator().manual_seed(8)
    ds = DelayedScaling("cuda", E4M3, history_len=4)
    hist, scale, pos = torch.zeros(4), torch.ones(()), 0
    for step in range(7):
        x = (torch.randn(1000, generator=g) * (0.5 + step)).to(torch.bfloat16)
        out = ds.cast(x.cuda())
        want, amax = O.cast_to_fp8_v2(x, scale.reshape(1), False, True, E4M3, [1])
        assert torch.equal(out.cpu().view(torch.uint8), want.view(torch.uint8)), step
        hist, scale = O.amax_history_update(hist, pos, amax, scale, True, 448.0)
        pos = (pos + 1) % 4
        assert torch.equal(ds.history.cpu(), hist) and torch.equal(ds.scale.cpu().reshape(()), scale), step
    x = (torch.randn(4099, generator=g) * 5).to(torch.bfloat16)
    out, s, amax = current_scaling_cast(x.cuda(), E4M3)
    ws = O.scale_from_amax(x.abs().max().float(), torch.ones(()), 448.0)
    want, _ = O.cast_to_fp8_v2(x, ws.reshape(1), False, False, E4M3, [1])
    assert torch.equal(s.cpu().reshape(()), ws) and torch.equal(out.cpu().view(torch.uint8), want.view(torch.uint8))
    assert ops.device_status() == 0
